"""Seeded synthetic tensors with the shapes and value distributions of the
benchmark configurations.  They stand in for real GGUF model files, which are
not available offline; nothing here reproduces any model's data.

All generators take a ``numpy.random.Generator`` (or a seed) and return numpy
arrays in the on-disk byte formats:

* Q4_K super-block, 144 B / 256 weights: fp16 d, fp16 dmin, 12 B of packed
  6-bit scales and mins, 128 B of nibbles (bench/bpd_quant.c:15-22 of the
  reference).
* Q8_0 block, 34 B / 32 weights: fp16 scale, 32 int8 (bench/bpd_cpu.c:3886-3890).
"""
import numpy as np

Q4K_BYTES, Q4K_ELEMS = 144, 256
Q80_BYTES, Q80_ELEMS = 34, 32
Q8K_BYTES = 292

# Mistral-7B-shaped layer: (name, rows N, cols K)
MISTRAL_LAYER = (
    ("wq", 4096, 4096), ("wk", 1024, 4096), ("wv", 1024, 4096), ("wo", 4096, 4096),
    ("w1", 14336, 4096), ("w3", 14336, 4096), ("w2", 4096, 14336),
)
# Llama-70B-shaped layer and output head
LLAMA70B_LAYER = (
    ("wq", 8192, 8192), ("wk", 1024, 8192), ("wv", 1024, 8192), ("wo", 8192, 8192),
    ("w1", 28672, 8192), ("w3", 28672, 8192), ("w2", 8192, 28672),
)
LLAMA70B_HEAD = ("head", 128256, 8192)


def _rng(seed_or_rng):
    if isinstance(seed_or_rng, np.random.Generator):
        return seed_or_rng
    return np.random.default_rng(seed_or_rng)


def q4k_blocks(n_blocks, rng, d_sigma=0.02):
    """n_blocks random super-blocks: d, dmin = fp16(|N(0, d_sigma)|); the other
    140 bytes uniform, which is the same distribution as 6-bit scales/mins
    uniform on 0..63 and nibbles uniform on 0..15."""
    rng = _rng(rng)
    raw = rng.integers(0, 256, size=(n_blocks, Q4K_BYTES), dtype=np.uint8)
    dd = np.abs(rng.normal(0.0, d_sigma, size=(n_blocks, 2))).astype(np.float16)
    raw[:, 0:4] = dd.view(np.uint8).reshape(n_blocks, 4)
    return raw.reshape(-1)


def q4k_matrix(rows, cols, rng):
    assert cols % Q4K_ELEMS == 0
    return q4k_blocks(rows * (cols // Q4K_ELEMS), rng)


def pack_q4k_scales(sc, mn):
    """Inverse of the 6-bit unpack (bench/bpd_quant.c:56-62): sc, mn are
    [..., 8] integer arrays with values 0..63; returns [..., 12] uint8."""
    sc = np.asarray(sc, dtype=np.uint8)
    mn = np.asarray(mn, dtype=np.uint8)
    out = np.zeros(sc.shape[:-1] + (12,), np.uint8)
    out[..., 0:4] = sc[..., 0:4] | ((sc[..., 4:8] >> 4) << 6)
    out[..., 4:8] = mn[..., 0:4] | ((mn[..., 4:8] >> 4) << 6)
    out[..., 8:12] = (sc[..., 4:8] & 15) | ((mn[..., 4:8] & 15) << 4)
    return out


def q8_0_matrix(rows, cols, rng, scale_sigma=0.01):
    """rows x cols Q8_0 weights: scale fp16(|N(0, scale_sigma)|), int8 uniform
    on [-127, 127]."""
    rng = _rng(rng)
    assert cols % Q80_ELEMS == 0
    nb = rows * (cols // Q80_ELEMS)
    raw = np.empty((nb, Q80_BYTES), np.uint8)
    sc = np.abs(rng.normal(0.0, scale_sigma, size=nb)).astype(np.float16)
    raw[:, 0:2] = sc.view(np.uint8).reshape(nb, 2)
    raw[:, 2:] = rng.integers(-127, 128, size=(nb, Q80_ELEMS), dtype=np.int8).view(np.uint8)
    return raw.reshape(-1)


def activations(n, rng, rows=None):
    rng = _rng(rng)
    shape = (n,) if rows is None else (rows, n)
    return rng.standard_normal(shape, dtype=np.float32)


def q4k_row_bytes(cols):
    return cols // Q4K_ELEMS * Q4K_BYTES


def q8_0_row_bytes(cols):
    return cols // Q80_ELEMS * Q80_BYTES


def gemv_bytes_q4k(rows, cols, tokens=1):
    """Algorithmic bytes of one Q4_K GEMV/GEMM: quantized weights + fp32
    activations in + fp32 outputs out."""
    return rows * q4k_row_bytes(cols) + tokens * cols * 4 + tokens * rows * 4


def gemv_bytes_q8_0(rows, cols, tokens=1):
    return rows * q8_0_row_bytes(cols) + tokens * cols * 4 + tokens * rows * 4

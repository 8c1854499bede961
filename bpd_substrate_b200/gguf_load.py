"""Minimal GGUF reader: maps the quantized tensors of a model file straight to device shards.

The walk over header, metadata and tensor table follows the reference's own reader
(bench/verify_quant_gpu.py:56-89) and the block sizes its manifest emitter lists
(lib/gguf_emit_manifest.pl:130-142).  GGUF files carry Q4_K in ggml's nibble order (chunk il of a
super-block: bytes 32*il..32*il+31 hold sub-block 2*il in their low nibbles and 2*il+1 in their high
nibbles), the C-ABI of this library's default in the order of bench/bpd_quant.c:68-72 (sub-block j:
bytes 16*j..16*j+15, elements 0..15 low, 16..31 high).  A loader can either keep the file's order and
pass ``layout=1`` to the kernels that take it, or repack once at load with
:func:`repack_q4k_ggml_to_bpd`, which only moves nibbles (scales and mins stay where they are).
"""
import mmap
import struct
from dataclasses import dataclass

import numpy as np

MAGIC = b"GGUF"
# ggml type id -> (elements per block, bytes per block)
BLOCK_INFO = {
    0: (1, 4), 1: (1, 2),                                      # F32, F16
    2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34), 9: (32, 36),       # Q4_0 Q4_1 Q5_0 Q5_1 Q8_0 Q8_1
    10: (256, 84), 11: (256, 110), 12: (256, 144), 13: (256, 176), 14: (256, 210), 15: (256, 292),   # Q2_K .. Q8_K
    24: (1, 1), 25: (1, 2), 26: (1, 4), 27: (1, 8), 28: (1, 8), 30: (1, 2),              # I8 I16 I32 I64 F64 BF16
}
TYPE_F32, TYPE_F16, TYPE_Q8_0, TYPE_Q4_K = 0, 1, 8, 12
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_STRING, _ARRAY = 8, 9


@dataclass
class TensorInfo:
    name: str
    dims: tuple          # ggml order: dims[0] is the contiguous (column) dimension
    type: int
    offset: int          # from the start of the data section
    nbytes: int

    @property
    def rows(self):
        n = 1
        for d in self.dims[1:]:
            n *= d
        return n

    @property
    def row_bytes(self):
        per, size = BLOCK_INFO[self.type]
        return self.dims[0] // per * size


class GgufFile:
    """Header, metadata and tensor table of a GGUF file; tensor bytes are read through a memory map."""

    def __init__(self, path, keep_arrays_up_to=4096):
        self.path = path
        self._fh = open(path, "rb")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        m, self._at = self._map, 0
        if m[:4] != MAGIC:
            raise ValueError(f"{path}: not a GGUF file")
        self._at = 4
        self.version = self._u32()
        if self.version < 2:
            raise ValueError(f"{path}: GGUF version {self.version} (64-bit counts start with version 2)")
        n_tensors, n_kv = self._u64(), self._u64()
        self.metadata = {}
        for _ in range(n_kv):
            key = self._str()
            self.metadata[key] = self._value(self._u32(), keep_arrays_up_to)
        self.tensors = {}
        for _ in range(n_tensors):
            name = self._str()
            dims = tuple(self._u64() for _ in range(self._u32()))
            ttype, offset = self._u32(), self._u64()
            if ttype not in BLOCK_INFO:
                raise ValueError(f"{path}: tensor {name} has ggml type {ttype}, not in the block-size table")
            per, size = BLOCK_INFO[ttype]
            if dims and dims[0] % per:
                raise ValueError(f"{path}: tensor {name}: {dims[0]} columns are not whole blocks of {per}")
            count = 1
            for d in dims:
                count *= d
            self.tensors[name] = TensorInfo(name, dims, ttype, offset, count // per * size)
        align = int(self.metadata.get("general.alignment", 32))
        self.data_start = (self._at + align - 1) // align * align
        for t in self.tensors.values():
            if self.data_start + t.offset + t.nbytes > len(m):
                raise ValueError(f"{path}: tensor {t.name} runs past the end of the file")

    # ---- primitive reads
    def _unpack(self, fmt):
        size = struct.calcsize(fmt)
        v = struct.unpack_from(fmt, self._map, self._at)[0]
        self._at += size
        return v

    def _u32(self):
        return self._unpack("<I")

    def _u64(self):
        return self._unpack("<Q")

    def _str(self):
        n = self._u64()
        s = self._map[self._at:self._at + n].decode("utf-8", errors="replace")
        self._at += n
        return s

    def _value(self, vtype, keep):
        if vtype in _SCALAR:
            return self._unpack(_SCALAR[vtype])
        if vtype == _STRING:
            return self._str()
        if vtype == _ARRAY:
            etype, count = self._u32(), self._u64()
            if etype in _SCALAR:
                fmt = _SCALAR[etype]
                size = struct.calcsize(fmt)
                if count <= keep:
                    out = [struct.unpack_from(fmt, self._map, self._at + i * size)[0] for i in range(count)]
                else:
                    out = f"<{count} values skipped>"
                self._at += count * size
                return out
            if etype == _STRING:
                out = [self._str() for _ in range(count)]
                return out if count <= keep else f"<{count} strings skipped>"
            raise ValueError(f"{self.path}: array of type {etype}")
        raise ValueError(f"{self.path}: metadata value type {vtype}")

    # ---- tensor data
    def raw(self, name, row_begin=0, row_end=None):
        """uint8 view of rows [row_begin, row_end) of a tensor (a contiguous byte range)."""
        t = self.tensors[name]
        row_end = t.rows if row_end is None else row_end
        if not (0 <= row_begin <= row_end <= t.rows):
            raise ValueError(f"{name}: rows [{row_begin}, {row_end}) outside 0..{t.rows}")
        begin = self.data_start + t.offset + row_begin * t.row_bytes
        return np.frombuffer(self._map, np.uint8, (row_end - row_begin) * t.row_bytes, begin)

    def to_device(self, lib, name, rank=0, world=1, repack=False):
        """Uploads rank's row shard of a 2-D weight; returns (device pointer, rows, cols, ggml type,
        nibble layout to pass to the kernels: 0 after a repack or for non-Q4_K, 1 for Q4_K as stored)."""
        t = self.tensors[name]
        if t.rows % world:
            raise ValueError(f"{name}: {t.rows} rows do not divide over {world} ranks")
        per = t.rows // world
        data = self.raw(name, rank * per, (rank + 1) * per)
        layout = 0
        if t.type == TYPE_Q4_K:
            if repack:
                data = repack_q4k_ggml_to_bpd(data)
            else:
                layout = 1
        data = np.ascontiguousarray(data)
        ptr = lib.bpdq_alloc(max(16, data.nbytes))
        if not ptr:
            raise MemoryError(f"{name}: device allocation of {data.nbytes} bytes failed")
        lib.bpdq_h2d(ptr, data.ctypes.data, data.nbytes)
        return ptr, per, t.dims[0], t.type, layout

    def close(self):
        try:
            self._map.close()
        except BufferError:
            pass            # arrays returned by raw() still look into the map: it goes when they do
        self._fh.close()


def _q4k_nibbles_in_element_order(qs, order):
    """qs uint8 [n_blocks, 128] -> values 0..15 [n_blocks, 256] in element order."""
    lo, hi = qs & 15, qs >> 4
    n = qs.shape[0]
    if order == "ggml":       # chunk il: bytes 32il..32il+31 -> elements 64il+l (low), 64il+32+l (high)
        return np.concatenate([lo.reshape(n, 4, 32), hi.reshape(n, 4, 32)], axis=2).reshape(n, 256)
    # C-ABI order: sub-block j: bytes 16j..16j+15 -> elements 32j+k (low), 32j+16+k (high)
    return np.concatenate([lo.reshape(n, 8, 16), hi.reshape(n, 8, 16)], axis=2).reshape(n, 256)


def _q4k_pack(values, order):
    n = values.shape[0]
    if order == "ggml":
        v = values.reshape(n, 4, 2, 32)
    else:
        v = values.reshape(n, 8, 2, 16)
    return (v[:, :, 0, :] | (v[:, :, 1, :] << 4)).reshape(n, 128).astype(np.uint8)


def repack_q4k_ggml_to_bpd(raw):
    """Q4_K super-blocks in ggml's nibble order -> the C-ABI order; header and scales untouched."""
    blocks = np.array(raw, np.uint8).reshape(-1, 144)
    blocks[:, 16:] = _q4k_pack(_q4k_nibbles_in_element_order(blocks[:, 16:], "ggml"), "bpd")
    return blocks.reshape(-1)


def repack_q4k_bpd_to_ggml(raw):
    """The inverse of :func:`repack_q4k_ggml_to_bpd`."""
    blocks = np.array(raw, np.uint8).reshape(-1, 144)
    blocks[:, 16:] = _q4k_pack(_q4k_nibbles_in_element_order(blocks[:, 16:], "bpd"), "ggml")
    return blocks.reshape(-1)


# ---- Q8_0 rows <-> the tensor-core tiles of bpd_qmatmul_q8_0_tiles_cuda (a permutation of bytes)
Q8_TILE_ROWS, Q8_TILE_UNIT = 128, 128 * 34


def repack_q8_0_to_tiles(raw, rows, cols):
    """Q8_0 rows [rows][cols/32][34] -> units [row tile][block][4352]: the 128x32 int8 quants with element
    (r, k) at (k/16)*2048 + (r/8)*128 + (r%8)*16 + k%16, then the 128 fp16 scales.  Rows of the last tile
    beyond ``rows`` are zero.  Host twin of bpd_repack_q8_0_tiles_cuda, for loaders that repack before upload."""
    nb = cols // 32
    tiles = -(-rows // Q8_TILE_ROWS)
    src = np.zeros((tiles * Q8_TILE_ROWS, nb, 34), np.uint8)
    src[:rows] = np.asarray(raw, np.uint8).reshape(rows, nb, 34)
    src = src.reshape(tiles, 16, 8, nb, 34)                       # [tile][r/8][r%8][block][byte]
    out = np.empty((tiles, nb, Q8_TILE_UNIT), np.uint8)
    quants = src[..., 2:].reshape(tiles, 16, 8, nb, 2, 16)         # [tile][r/8][r%8][block][k/16][k%16]
    out[:, :, :4096] = quants.transpose(0, 3, 4, 1, 2, 5).reshape(tiles, nb, 4096)
    out[:, :, 4096:] = src[..., :2].reshape(tiles, 128, nb, 2).transpose(0, 2, 1, 3).reshape(tiles, nb, 256)
    return out.reshape(-1)


def repack_tiles_to_q8_0(tiles_raw, rows, cols):
    """The inverse of :func:`repack_q8_0_to_tiles`."""
    nb = cols // 32
    tiles = -(-rows // Q8_TILE_ROWS)
    units = np.asarray(tiles_raw, np.uint8).reshape(tiles, nb, Q8_TILE_UNIT)
    out = np.empty((tiles, 16, 8, nb, 34), np.uint8)
    quants = units[:, :, :4096].reshape(tiles, nb, 2, 16, 8, 16)   # [tile][block][k/16][r/8][r%8][k%16]
    out[..., 2:] = quants.transpose(0, 3, 4, 1, 2, 5).reshape(tiles, 16, 8, nb, 32)
    out[..., :2] = units[:, :, 4096:].reshape(tiles, nb, 16, 8, 2).transpose(0, 2, 3, 1, 4)
    return out.reshape(tiles * Q8_TILE_ROWS, nb * 34)[:rows].reshape(-1)


# ---- Q4_K re-tiled in groups of 16 rows for the int8 MMA (host twin of bpd_repack_q4k_rg16_cuda)

Q4K_RG_ROWS, Q4K_RG_UNIT = 16, 16 * 144


def repack_q4k_to_rg16(raw, rows, cols):
    """Q4_K rows [rows][cols/256][144] -> units [row group][super-block][2304]: the 16 block headers (16 bytes
    each), then for q = 0..3 and lane L = 0..31 (g = L / 4, t = L % 4) 16 bytes = word t of sub-block 2q of rows g
    and g + 8, then of sub-block 2q + 1 (word t of sub-block j = bytes 16 + 16 j + 4 t .. + 3 of the block).  Rows
    beyond ``rows`` are zero.  A pure permutation of the bytes."""
    nb = cols // 256
    groups = -(-rows // Q4K_RG_ROWS)
    src = np.zeros((groups * Q4K_RG_ROWS, nb, 144), np.uint8)
    src[:rows] = np.asarray(raw, np.uint8).reshape(rows, nb, 144)
    src = src.reshape(groups, 2, 8, nb, 144)                                   # [G][row / 8][g][b][byte]
    out = np.empty((groups, nb, Q4K_RG_UNIT), np.uint8)
    out[:, :, :256] = src[..., :16].reshape(groups, 16, nb, 16).transpose(0, 2, 1, 3).reshape(groups, nb, 256)
    words = src[..., 16:].reshape(groups, 2, 8, nb, 4, 2, 4, 4)                # [G][hi][g][b][q][j & 1][t][byte]
    # target order inside a unit: [q][g][t][j & 1][hi][byte]
    out[:, :, 256:] = words.transpose(0, 3, 4, 2, 6, 5, 1, 7).reshape(groups, nb, 2048)
    return out.reshape(-1)


def repack_rg16_to_q4k(tiles_raw, rows, cols):
    """The inverse of :func:`repack_q4k_to_rg16`."""
    nb = cols // 256
    groups = -(-rows // Q4K_RG_ROWS)
    units = np.asarray(tiles_raw, np.uint8).reshape(groups, nb, Q4K_RG_UNIT)
    out = np.empty((groups, 2, 8, nb, 144), np.uint8)
    out[..., :16] = units[:, :, :256].reshape(groups, nb, 2, 8, 16).transpose(0, 2, 3, 1, 4)
    words = units[:, :, 256:].reshape(groups, nb, 4, 8, 4, 2, 2, 4)            # [G][b][q][g][t][j & 1][hi][byte]
    out[..., 16:] = words.transpose(0, 6, 3, 1, 2, 5, 4, 7).reshape(groups, 2, 8, nb, 128)
    return out.reshape(groups * Q4K_RG_ROWS, nb * 144)[:rows].reshape(-1)

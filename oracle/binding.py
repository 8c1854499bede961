"""ctypes access to the CPU checker.  TEST INFRASTRUCTURE ONLY.

Two things are loaded here and nothing else in the repository may load them
except the tests, the smoke check and the bench's CPU-baseline leg:

* ``oracle/_build/libbpdq_oracle.so`` -- this repository's restatement
  (``bpdq_oracle.c``), wrapped by :class:`Oracle` with numpy in/out;
* ``oracle/_ref/*.so`` -- the reference's own C files compiled unmodified
  (``make -C oracle ref``), wrapped by :func:`load_ref`.  These exist only
  where the reference tree was present at build time, or where the prebuilt
  files travelled with the working copy.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "_build", "libbpdq_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")

Q4K_BYTES, Q80_BYTES, Q8K_BYTES = 144, 34, 292


def build(ref_root=None):
    """Compile the restatement; also the reference files when their tree exists."""
    subprocess.check_call(["make", "-s", "-C", HERE, "all"])
    # the reference checkout: named by the environment, else a directory "reference" beside this repository
    root = ref_root or os.environ.get("BPD_REFERENCE_ROOT") or os.path.join(os.path.dirname(HERE), os.pardir, "reference")
    if os.path.isdir(os.path.join(root, "bench")):
        subprocess.check_call(["make", "-s", "-C", HERE, "ref", "REF=" + root])
        import shutil
        if shutil.which("nvcc"):      # the reference's own GPU kernels, as a second baseline and checker on a GPU box
            subprocess.check_call(["make", "-s", "-C", HERE, "refgpu", "REF=" + root])


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _u8(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.uint8
    return a


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class Oracle:
    """numpy front end of bpdq_oracle.c; layout 0 = C-ABI nibble order, 1 = ggml order."""

    def __init__(self, path=ORACLE_SO):
        if not os.path.exists(path):
            build()
        self.lib = lib = C.CDLL(path)
        vp, i, l = C.c_void_p, C.c_int, C.c_long
        lib.orc_f16_to_f32.argtypes = [C.c_uint16]
        lib.orc_f16_to_f32.restype = C.c_float
        lib.orc_f32_to_f16.argtypes = [C.c_float]
        lib.orc_f32_to_f16.restype = C.c_uint16
        lib.orc_q4k_scales.argtypes = [vp, vp, vp]
        lib.orc_dequant_q4k.argtypes = [vp, vp, l, i]
        lib.orc_qmatmul_q4k.argtypes = [vp, vp, vp, i, i, i]
        lib.orc_qmatmul_q4k_f64.argtypes = [vp, vp, vp, i, i, i]
        lib.orc_qmm_q4k.argtypes = [vp, vp, vp, i, i, i, i]
        lib.orc_dequant_q8_0.argtypes = [vp, vp, l]
        lib.orc_embed_lookup_q8_0.argtypes = [vp, vp, vp, i, i]
        lib.orc_quant_q8_0.argtypes = [vp, vp, l]
        lib.orc_q8_0_block_dots.argtypes = [vp, vp, vp, l]
        lib.orc_qdot_q8_0.argtypes = [vp, vp, i]
        lib.orc_qdot_q8_0.restype = C.c_float
        lib.orc_qdot_q8_0_f64.argtypes = [vp, vp, i]
        lib.orc_qdot_q8_0_f64.restype = C.c_double
        lib.orc_qmatmul_q8_0.argtypes = [vp, vp, vp, i, i, i]
        lib.orc_qmatmul_q8_0.restype = i
        lib.orc_qmatmul_q8_0_f64.argtypes = [vp, vp, vp, i, i, i]
        lib.orc_qmatmul_q8_0_f64.restype = i
        lib.orc_quant_q8_K.argtypes = [vp, vp, l]
        lib.orc_dequant_q8_K.argtypes = [vp, vp, l]
        lib.orc_q4k_q8k_subdots.argtypes = [vp, vp, vp, i, i, i]
        lib.orc_qmatmul_q4k_q8k.argtypes = [vp, vp, vp, vp, i, i, i]
        lib.orc_qmm_q4k_q8k.argtypes = [vp, vp, vp, vp, i, i, i, i]
        lib.orc_qmm_q4k_q8k.restype = i
        lib.orc_qmm_q4k_q8k_ints.argtypes = [vp, vp, vp, i, i, i, i]
        lib.orc_qmm_q4k_q8k_ints.restype = i
        lib.orc_qmatmul_q8_0_lanes.argtypes = [vp, vp, vp, i, i, i]
        lib.orc_vecmat_f32.argtypes = [vp, vp, vp, i, i]
        lib.orc_rms_norm_f64.argtypes = [vp, vp, vp, i, i, C.c_float]
        f = C.c_float
        lib.orc_rmsnorm_llama.argtypes = [vp, vp, vp, i, i, f]
        lib.orc_rope_norm_freqs.argtypes = [vp, vp, vp, vp, i, i, i, i, f]
        lib.orc_kv_cache_write.argtypes = [vp, vp, vp, i, i, i]
        lib.orc_gqa_attn.argtypes = [vp, vp, vp, vp, i, i, i, i, i, f, i]
        lib.orc_argmax_rows.argtypes = [vp, vp, i, i]
        lib.orc_llama_block.argtypes = [vp, vp, vp, vp, i, i, vp, vp, vp, vp, vp, vp]
        lib.orc_llama_forward.argtypes = [vp, i, vp, vp, vp, i, vp, vp, vp, vp]
        lib.orc_llama_forward.restype = i

    # -- fp16
    def f16_to_f32(self, h):
        return self.lib.orc_f16_to_f32(int(h))

    def f32_to_f16(self, v):
        return self.lib.orc_f32_to_f16(float(v))

    # -- Q4_K
    def q4k_scales(self, s12):
        s12 = _u8(s12)
        sc, mn = np.zeros(8, np.uint8), np.zeros(8, np.uint8)
        self.lib.orc_q4k_scales(_p(s12), _p(sc), _p(mn))
        return sc, mn

    def dequant_q4k(self, q, layout=0):
        q = _u8(q)
        nb = q.size // Q4K_BYTES
        out = np.empty(nb * 256, np.float32)
        self.lib.orc_dequant_q4k(_p(q), _p(out), nb, layout)
        return out

    def qmatmul_q4k(self, qw, x, M, K, layout=0):
        qw, x = _u8(qw), _f32(x)
        out = np.empty(M, np.float32)
        self.lib.orc_qmatmul_q4k(_p(qw), _p(x), _p(out), M, K, layout)
        return out

    def qmatmul_q4k_f64(self, qw, x, M, K, layout=0):
        qw, x = _u8(qw), _f32(x)
        out = np.empty(M, np.float64)
        self.lib.orc_qmatmul_q4k_f64(_p(qw), _p(x), _p(out), M, K, layout)
        return out

    def qmm_q4k(self, qA, B, M, N, K, layout=0):
        qA, B = _u8(qA), _f32(B)
        out = np.empty((M, N), np.float32)
        self.lib.orc_qmm_q4k(_p(qA), _p(B), _p(out), M, N, K, layout)
        return out

    # -- Q8_0
    def dequant_q8_0(self, raw):
        raw = _u8(raw)
        nb = raw.size // Q80_BYTES
        out = np.empty(nb * 32, np.float32)
        self.lib.orc_dequant_q8_0(_p(raw), _p(out), nb)
        return out

    def embed_lookup_q8_0(self, table, ids, embed_dim):
        table = _u8(table)
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        out = np.empty((ids.size, embed_dim), np.float32)
        self.lib.orc_embed_lookup_q8_0(_p(table), _p(ids), _p(out), ids.size, embed_dim)
        return out

    def quant_q8_0(self, x):
        x = _f32(x).ravel()
        y = np.zeros(x.size // 32 * Q80_BYTES, np.uint8)
        self.lib.orc_quant_q8_0(_p(x), _p(y), x.size)
        return y

    def q8_0_block_dots(self, w, a):
        w, a = _u8(w), _u8(a)
        nb = w.size // Q80_BYTES
        out = np.empty(nb, np.int32)
        self.lib.orc_q8_0_block_dots(_p(w), _p(a), _p(out), nb)
        return out

    def qdot_q8_0(self, w, a):
        w, a = _u8(w), _u8(a)
        return self.lib.orc_qdot_q8_0(_p(w), _p(a), w.size // Q80_BYTES)

    def qmatmul_q8_0(self, W, X, M, N, K):
        W, X = _u8(W), _f32(X)
        out = np.empty((M, N), np.float32)
        assert self.lib.orc_qmatmul_q8_0(_p(W), _p(X), _p(out), M, N, K) == 0
        return out

    def qmatmul_q8_0_f64(self, W, X, M, N, K):
        W, X = _u8(W), _f32(X)
        out = np.empty((M, N), np.float64)
        assert self.lib.orc_qmatmul_q8_0_f64(_p(W), _p(X), _p(out), M, N, K) == 0
        return out

    # -- Q8_K and the Q4_K x Q8_K dot (builder-defined)
    def quant_q8_K(self, x):
        x = _f32(x).ravel()
        y = np.zeros(x.size // 256 * Q8K_BYTES, np.uint8)
        self.lib.orc_quant_q8_K(_p(x), _p(y), x.size)
        return y

    def dequant_q8_K(self, y):
        y = _u8(y)
        nb = y.size // Q8K_BYTES
        out = np.empty(nb * 256, np.float32)
        self.lib.orc_dequant_q8_K(_p(y), _p(out), nb)
        return out

    def q4k_q8k_subdots(self, qw, xq, M, K, layout=0):
        qw, xq = _u8(qw), _u8(xq)
        out = np.empty((M, K // 256, 8), np.int32)
        self.lib.orc_q4k_q8k_subdots(_p(qw), _p(xq), _p(out), M, K, layout)
        return out

    def qmatmul_q4k_q8k(self, qw, xq, M, K, layout=0):
        """Returns (fp32 sequential result, binary64 result)."""
        qw, xq = _u8(qw), _u8(xq)
        out, out64 = np.empty(M, np.float32), np.empty(M, np.float64)
        self.lib.orc_qmatmul_q4k_q8k(_p(qw), _p(xq), _p(out), _p(out64), M, K, layout)
        return out, out64

    def qmm_q4k_q8k(self, qw, X, T, M, K, layout=0):
        """X [T][K] fp32 -> (out [T][M] fp32, out64 [T][M])."""
        qw, X = _u8(qw), _f32(X)
        out, out64 = np.empty((T, M), np.float32), np.empty((T, M), np.float64)
        assert self.lib.orc_qmm_q4k_q8k(_p(qw), _p(X), _p(out), _p(out64), T, M, K, layout) == 0
        return out, out64

    def qmm_q4k_q8k_ints(self, qw, X, T, M, K, layout=0):
        """X [T][K] fp32 -> int32 [T][M][K/256][2]: the exact (isum, msum) of every super-block."""
        qw, X = _u8(qw), _f32(X)
        ints = np.empty((T, M, K // 256, 2), np.int32)
        assert self.lib.orc_qmm_q4k_q8k_ints(_p(qw), _p(X), _p(ints), T, M, K, layout) == 0
        return ints

    def qmatmul_q8_0_lanes(self, Wq, Xq, m_weight, m_tokens, K):
        """Q8_0 x Q8_0 with the eight-lane fp32 order of the reference's AVX tile kernels:
        out [m_tokens][m_weight]."""
        Wq, Xq = _u8(Wq), _u8(Xq)
        out = np.empty((m_tokens, m_weight), np.float32)
        self.lib.orc_qmatmul_q8_0_lanes(_p(Wq), _p(Xq), _p(out), m_weight, m_tokens, K)
        return out

    # -- fp32 dispatch ops
    def vecmat_f32(self, a, b, k, n):
        a, b = _f32(a), _f32(b)
        out = np.empty(n, np.float32)
        self.lib.orc_vecmat_f32(_p(a), _p(b), _p(out), k, n)
        return out

    def rms_norm(self, x, w, rows, cols, eps):
        x, w = _f32(x), _f32(w)
        out = np.empty((rows, cols), np.float32)
        self.lib.orc_rms_norm_f64(_p(x), _p(w), _p(out), rows, cols, eps)
        return out


    # -- Q8_0 Llama forward.  `weights` and `cfg` are ctypes structs with the layout of
    # bench/bpd_cpu.c:5537-5588 whose pointers are HOST memory; the caches are updated in place.
    def llama_forward(self, weights, cfg, token_ids, pos_ids, kv_pos, k_cache, v_cache):
        return llama_forward_with(self.lib.orc_llama_forward, weights, cfg, token_ids, pos_ids, kv_pos, k_cache, v_cache)


def llama_forward_with(fn, weights, cfg, token_ids, pos_ids, kv_pos, k_cache, v_cache):
    """Calls a CPU forward (the checker's or the compiled reference's: same signature) and returns
    (logits [n, vocab], argmax tokens [n])."""
    token_ids = np.ascontiguousarray(token_ids, np.int32)
    pos_ids = np.ascontiguousarray(pos_ids, np.int32)
    n = token_ids.size
    logits = np.empty((n, cfg.vocab_size), np.float32)
    tokens = np.empty(n, np.int64)
    fn(_p(token_ids), n, C.byref(weights), C.byref(cfg), _p(pos_ids), kv_pos, _p(k_cache), _p(v_cache), _p(logits), _p(tokens))
    return logits, tokens


def ref_available(name="bpd_quant.so"):
    return os.path.exists(os.path.join(REF_DIR, name))


def load_ref(name):
    """Load one of the compiled reference libraries with the argtypes its own
    callers declare (bench/verify_quant_gpu.py:27-30, tests/verify_f16_fix.py:18-28,
    bench/test_gemm_q8_0_tiles.py:40-70)."""
    lib = C.CDLL(os.path.join(REF_DIR, name))
    vp, i = C.c_void_p, C.c_int
    if name == "bpd_quant_gpu.so":
        # bench/verify_quant_gpu.py:33-42 of the reference
        lib.bpd_dequant_q4k_gpu.argtypes = [vp, vp, i]
        lib.bpd_qmatmul_q4k_gpu.argtypes = [vp, vp, vp, i, i]
        lib.qgpu_sync.argtypes = []
    elif name == "bpd_quant.so":
        lib.bpd_dequant_q4k.argtypes = [vp, vp, i]
        lib.bpd_qmatmul_q4k.argtypes = [vp, vp, vp, i, i]
        lib.bpd_qmm_q4k.argtypes = [vp, vp, vp, i, i, i]
    else:
        lib.bpd_dequant_q8_0_cpu.argtypes = [vp, vp, i]
        lib.bpd_quant_q8_0_cpu.argtypes = [vp, vp, i]
        lib.bpd_qdot_q8_0_q8_0_cpu.argtypes = [vp, vp, i]
        lib.bpd_qdot_q8_0_q8_0_cpu.restype = C.c_float
        lib.bpd_qmatmul_q8_0_cpu.argtypes = [vp, vp, vp, i, i, i]
        lib.bpd_qmatmul_q8_0_llamafile_cpu.argtypes = [vp, vp, vp, i, i, i]
        lib.bpd_qmatmul_q8_0_dispatch_cpu.argtypes = [vp, vp, vp, i, i, i]
        lib.bpd_embed_lookup_q8_0_cpu.argtypes = [vp, vp, vp, i, i]
        f = C.c_float
        lib.bpd_rmsnorm_llama_cpu.argtypes = [vp, vp, vp, i, i, f]
        lib.bpd_rope_norm_freqs_cpu.argtypes = [vp, vp, vp, vp, i, i, i, i, f]
        lib.bpd_kv_cache_write_f16_cpu.argtypes = [vp, vp, vp, i, i, i, i]
        lib.bpd_gqa_attn_cpu.argtypes = [vp, vp, vp, vp, i, i, i, i, i, f, i]
        lib.bpd_argmax_dim_cpu.argtypes = [vp, vp, i, i, i]
        lib.bpd_llama_forward_cpu.argtypes = [vp, i, vp, vp, vp, i, vp, vp, vp, vp]
        for rm in (1, 2, 4):
            for rn in (1, 2, 4):
                getattr(lib, f"bpd_gemm_q8_0_{rm}_{rn}_cpu").argtypes = [vp, vp, i, i, i, vp, i]
    return lib

"""Pins the CPU checker (oracle/bpdq_oracle.c): against the known-answer cases the reference's
own tests hold, against fixtures produced by the reference's C code (tests/golden), and --
where the compiled reference is present -- against that code directly."""
import hashlib
import os
import struct

import numpy as np
import pytest

from bpd_substrate_b200 import synth
from oracle import binding

GOLD = os.path.join(os.path.dirname(__file__), "golden")
needs_ref = pytest.mark.skipif(not binding.ref_available(), reason="compiled reference not present")


def u32(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


# ---- fp16 conversions (tests/check_f16_algorithm.py:85-117 of the reference: all 65536 values)

def test_f16_to_f32_all_values(oracle):
    h = np.arange(65536, dtype=np.uint16)
    want = h.view(np.float16).astype(np.float32)
    got = np.array([oracle.f16_to_f32(int(v)) for v in h], dtype=np.float32)
    nan = np.isnan(want)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(u32(got)[~nan], u32(want)[~nan])
    assert np.array_equal(np.signbit(got[nan]), np.signbit(want[nan]))


def test_f32_to_f16_round_to_nearest_even(oracle):
    rng = np.random.default_rng(1)
    vals = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 20000).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001,
                  2.0 ** -14, 6.1e-5, 5.96e-8, 2.98e-8, 2.9802322e-8, np.inf, -np.inf], dtype=np.float32),
        np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float32)[:0x7C00],
    ])
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = np.array([oracle.f32_to_f16(float(v)) for v in vals], dtype=np.uint16)
    assert np.array_equal(got, want)


# ---- known answers from tests/verify_f16_fix.py

def test_kat_subnormal_scale_dequant(oracle):
    """verify_f16_fix.py:99-117 -- scale bits 0x0001 (2^-24), quants 1..32."""
    raw = np.zeros(34, np.uint8)
    raw[0] = 1
    raw[2:] = np.arange(1, 33, dtype=np.uint8)
    want = (np.arange(1, 33, dtype=np.float32) * np.float32(2.0 ** -24))
    assert np.array_equal(u32(oracle.dequant_q8_0(raw)), u32(want))


def test_kat_subnormal_block_00c2(oracle):
    """tests/check_dequant_subnormal.py -- scale bits 0x00c2, 32 ones."""
    raw = np.zeros(34, np.uint8)
    raw[0], raw[1] = 0xC2, 0x00
    raw[2:] = 1
    want = np.full(32, np.float32(0xC2 * 2.0 ** -24))
    assert np.array_equal(u32(oracle.dequant_q8_0(raw)), u32(want))


def py_qdot(w, a, nb):
    """Sequential mirror used by verify_f16_fix.py:61-75 (float32 running sum)."""
    s = np.float32(0.0)
    for b in range(nb):
        wb, ab = w[34 * b:34 * b + 34], a[34 * b:34 * b + 34]
        sumi = int(np.dot(wb[2:].view(np.int8).astype(np.int64), ab[2:].view(np.int8).astype(np.int64)))
        wd = wb[:2].view(np.float16).astype(np.float32)[0]
        ad = ab[:2].view(np.float16).astype(np.float32)[0]
        s = np.float32(s + np.float32(np.float32(sumi) * np.float32(wd * ad)))
    return s


def test_kat_qdot_with_subnormal_block(oracle):
    """verify_f16_fix.py:119-144 -- 64 blocks of ones, block 0 with scale 0x0001."""
    nb = 64
    W = np.zeros(nb * 34, np.uint8)
    A = np.zeros(nb * 34, np.uint8)
    for b in range(nb):
        W[34 * b:34 * b + 2] = [0x00, 0x3C]
        A[34 * b:34 * b + 2] = [0x00, 0x3C]
        W[34 * b + 2:34 * b + 34] = 1
        A[34 * b + 2:34 * b + 34] = 1
    W[0:2] = [0x01, 0x00]
    got = np.float32(oracle.qdot_q8_0(W, A))
    assert u32([got])[0] == u32([py_qdot(W, A, nb)])[0]


def test_kat_matmul_seed7(oracle):
    """verify_f16_fix.py:146-201 -- M=2, N=8, K=256, np.random.seed(7)."""
    np.random.seed(7)
    M, N, K = 2, 8, 256
    X = (np.random.randn(M, K).astype(np.float32) * 0.3).astype(np.float32)
    Wf = (np.random.randn(N, K).astype(np.float32) * 0.5).astype(np.float32)
    Wq = np.concatenate([oracle.quant_q8_0(Wf[n]) for n in range(N)])
    Xq = np.concatenate([oracle.quant_q8_0(X[m]) for m in range(M)])
    got = oracle.qmatmul_q8_0(Wq, X, M, N, K)
    rb = K // 32 * 34
    want = np.array([[py_qdot(Wq[n * rb:(n + 1) * rb], Xq[m * rb:(m + 1) * rb], K // 32) for n in range(N)]
                     for m in range(M)], dtype=np.float32)
    assert np.array_equal(u32(got), u32(want))


# ---- fixtures produced by the reference's C code

def test_golden_q4k_small(oracle):
    g = np.load(os.path.join(GOLD, "q4k_small.npz"))
    M, K, N = g["shape"]
    assert np.array_equal(u32(oracle.dequant_q4k(g["q"], 0)), g["dequant"])
    assert np.array_equal(u32(oracle.qmatmul_q4k(g["W"], g["x"], M, K)), g["gemv"])
    assert np.array_equal(u32(oracle.qmm_q4k(g["W"], g["B"], M, N, K)), g["gemm"])


def test_golden_q4k_full_tensor(oracle):
    g = np.load(os.path.join(GOLD, "q4k_dequant_14336x4096.npz"))
    nb = int(g["n_blocks"][0])
    q = synth.q4k_blocks(nb, int(g["seed"][0]))
    assert hashlib.sha256(q.tobytes()).hexdigest() == str(g["input_sha256"][0])
    out = oracle.dequant_q4k(q, 0)
    assert hashlib.sha256(out.tobytes()).hexdigest() == str(g["output_sha256"][0])
    assert np.array_equal(u32(out[::int(g["sample_stride"][0])]), g["sample"])


def test_golden_q8_0_small(oracle):
    g = np.load(os.path.join(GOLD, "q8_0_small.npz"))
    Mt, Nw, Kq = g["shape"]
    assert np.array_equal(u32(oracle.dequant_q8_0(g["W"])), g["dequant"])
    assert np.array_equal(oracle.quant_q8_0(g["X"]), g["Xq"])
    got = oracle.qmatmul_q8_0(g["W"], g["X"], Mt, Nw, Kq)
    assert np.array_equal(u32(got), g["matmul_scalar"].reshape(Mt, Nw))
    # the AVX tile path sums in another order: same integers, fp32 within 1e-5 norm-wise
    avx = g["matmul_avx_tiles"].view(np.float32).reshape(Mt, Nw)
    assert np.max(np.abs(avx - got)) / np.max(np.abs(got)) <= 1e-5


def test_golden_q8_0_avx_tiles(oracle):
    """The eight-lane restatement of the AVX tile kernels (bench/bpd_gemm_q8_0_cpu.c:32-207) gives the
    bits the compiled AVX build produced: dispatcher, bpd_qmatmul_q8_0_llamafile_cpu and three single
    tiles, on 37 weight rows x 7 activation rows (all nine tile shapes occur)."""
    g = np.load(os.path.join(GOLD, "q8_0_avx_tiles.npz"))
    mw, mt, K = (int(v) for v in g["shape"])
    assert np.array_equal(oracle.quant_q8_0(g["X"]), g["Xq"])
    got = oracle.qmatmul_q8_0_lanes(g["W"], g["Xq"], mw, mt, K)
    assert np.array_equal(u32(got), g["dispatch"])
    assert np.array_equal(u32(got), g["llamafile"])
    rb = K // 32 * 34
    for rm, rn in ((4, 4), (2, 1), (1, 2)):
        tile = oracle.qmatmul_q8_0_lanes(g["W"][3 * rb:(3 + rm) * rb], g["Xq"][rb:(1 + rn) * rb], rm, rn, K)
        assert np.array_equal(u32(tile), g[f"tile_{rm}_{rn}"][:, :rm])
    # the small fixture's dispatcher output too
    s = np.load(os.path.join(GOLD, "q8_0_small.npz"))
    Mt, Nw, Kq = (int(v) for v in s["shape"])
    assert np.array_equal(u32(oracle.qmatmul_q8_0_lanes(s["W"], s["Xq"], Nw, Mt, Kq)), s["matmul_avx_tiles"].reshape(Mt, Nw))


def test_golden_q8_0_gemv_4096(oracle):
    g = np.load(os.path.join(GOLD, "q8_0_gemv_4096x4096.npz"))
    W = synth.q8_0_matrix(4096, 4096, int(g["w_seed"][0]))
    assert hashlib.sha256(W.tobytes()).hexdigest() == str(g["input_sha256"][0])
    x = synth.activations(4096, int(g["x_seed"][0]))
    assert np.array_equal(u32(oracle.qmatmul_q8_0(W, x, 1, 4096, 4096)), g["out"])


# ---- the compiled reference itself, where present

@pytest.mark.skipif(not binding.ref_available("bpd_cpu_avx.so"), reason="compiled reference (AVX build) not present")
def test_lane_order_restatement_equals_compiled_avx_dispatcher(oracle):
    ra = binding.load_ref("bpd_cpu_avx.so")
    rng = np.random.default_rng(5)
    for mw, mt, K in ((7, 5, 256), (33, 3, 1024), (4, 4, 64), (1, 1, 32), (130, 9, 4096)):
        W = synth.q8_0_matrix(mw, K, rng)
        xq = oracle.quant_q8_0(synth.activations(K, rng, rows=mt))
        out = np.empty((mt, mw), np.float32)
        ra.bpd_qmatmul_q8_0_dispatch_cpu(W.ctypes.data, xq.ctypes.data, out.ctypes.data, mw, mt, K)
        assert np.array_equal(u32(out), u32(oracle.qmatmul_q8_0_lanes(W, xq, mw, mt, K))), (mw, mt, K)


@needs_ref
def test_checker_equals_compiled_reference_q4k(oracle):
    ref = binding.load_ref("bpd_quant.so")
    for seed, nb in ((1, 1), (2, 777)):
        q = synth.q4k_blocks(nb, seed)
        out = np.empty(nb * 256, np.float32)
        ref.bpd_dequant_q4k(q.ctypes.data, out.ctypes.data, nb)
        assert np.array_equal(u32(out), u32(oracle.dequant_q4k(q, 0)))
    M, K, N = 9, 2048, 5
    W, x = synth.q4k_matrix(M, K, 3), synth.activations(K, 4)
    y = np.empty(M, np.float32)
    ref.bpd_qmatmul_q4k(W.ctypes.data, x.ctypes.data, y.ctypes.data, M, K)
    assert np.array_equal(u32(y), u32(oracle.qmatmul_q4k(W, x, M, K)))
    B = synth.activations(N, 5, rows=K)
    Cm = np.empty((M, N), np.float32)
    ref.bpd_qmm_q4k(W.ctypes.data, B.ctypes.data, Cm.ctypes.data, M, N, K)
    assert np.array_equal(u32(Cm), u32(oracle.qmm_q4k(W, B, M, N, K)))


@needs_ref
def test_checker_equals_compiled_reference_q8_0(oracle):
    ref = binding.load_ref("bpd_cpu.so")
    W = synth.q8_0_matrix(24, 1024, 6)
    X = synth.activations(1024, 7, rows=3)
    deq = np.empty(24 * 1024, np.float32)
    ref.bpd_dequant_q8_0_cpu(W.ctypes.data, deq.ctypes.data, 24 * 32)
    assert np.array_equal(u32(deq), u32(oracle.dequant_q8_0(W)))
    Xq = np.zeros(3 * 32 * 34, np.uint8)
    ref.bpd_quant_q8_0_cpu(X.ctypes.data, Xq.ctypes.data, 3 * 1024)
    assert np.array_equal(Xq, oracle.quant_q8_0(X))
    out = np.empty((3, 24), np.float32)
    ref.bpd_qmatmul_q8_0_cpu(W.ctypes.data, X.ctypes.data, out.ctypes.data, 3, 24, 1024)
    assert np.array_equal(u32(out), u32(oracle.qmatmul_q8_0(W, X, 3, 24, 1024)))
    ids = np.array([5, 0, 23, 5], np.int32)
    emb = np.empty((4, 1024), np.float32)
    ref.bpd_embed_lookup_q8_0_cpu(W.ctypes.data, ids.ctypes.data, emb.ctypes.data, 4, 1024)
    assert np.array_equal(u32(emb), u32(oracle.embed_lookup_q8_0(W, ids, 1024)))


# ---- structure of the Q4_K format and of the builder-defined Q8_K / Q4_K x Q8_K pieces

def test_scale_pack_unpack_roundtrip(oracle):
    rng = np.random.default_rng(8)
    for _ in range(200):
        sc, mn = rng.integers(0, 64, 8), rng.integers(0, 64, 8)
        got_sc, got_mn = oracle.q4k_scales(synth.pack_q4k_scales(sc, mn))
        assert np.array_equal(got_sc, sc) and np.array_equal(got_mn, mn)


def test_ggml_nibble_order_differs_only_by_permutation_of_nibbles(oracle):
    """Same scales, other element order: re-packing the nibbles maps one layout onto the other."""
    q = synth.q4k_blocks(5, 9).reshape(5, 144).copy()
    a = oracle.dequant_q4k(q.reshape(-1), 1).reshape(5, 256)
    # build the C-ABI-order block that holds the same element values
    nib = np.empty((5, 256), np.uint8)
    qs = q[:, 16:]
    for c in range(4):
        nib[:, 64 * c:64 * c + 32] = qs[:, 32 * c:32 * c + 32] & 15
        nib[:, 64 * c + 32:64 * c + 64] = qs[:, 32 * c:32 * c + 32] >> 4
    r = q.copy()
    for j in range(8):
        r[:, 16 + 16 * j:32 + 16 * j] = nib[:, 32 * j:32 * j + 16] | (nib[:, 32 * j + 16:32 * j + 32] << 4)
    b = oracle.dequant_q4k(r.reshape(-1), 0).reshape(5, 256)
    assert np.array_equal(u32(a), u32(b))


def test_ggml_nibble_order_matches_gguf_package(oracle):
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    q = synth.q4k_blocks(64, 10)
    want = quants.dequantize(q.reshape(64, 144), gguf.GGMLQuantizationType.Q4_K).astype(np.float32).reshape(-1)
    assert np.array_equal(u32(oracle.dequant_q4k(q, 1)), u32(want))


def test_q8_K_quantizer_properties(oracle):
    rng = np.random.default_rng(11)
    x = synth.activations(256 * 9, rng)
    x[256:512] = 0
    y = oracle.quant_q8_K(x).reshape(9, 292)
    d = y[:, :4].copy().view(np.float32).reshape(9)
    qs = y[:, 4:260].view(np.int8).astype(np.int32)
    bs = y[:, 260:].copy().view(np.int16).reshape(9, 16)
    amax = np.abs(x.reshape(9, 256)).max(axis=1)
    assert np.array_equal(u32(d), u32(amax / np.float32(127.0)))
    assert np.array_equal(bs, qs.reshape(9, 16, 16).sum(axis=2))
    assert np.abs(qs).max() <= 127 and (qs[1] == 0).all()
    deq = oracle.dequant_q8_K(y.reshape(-1)).reshape(9, 256)
    assert (np.abs(deq - x.reshape(9, 256)) <= d[:, None] * 0.5000001 + 1e-30).all()


def test_q4k_q8k_dot_equals_dequantized_product(oracle):
    """The W4A8 result equals (dequantized weights) . (dequantized activations) up to fp error."""
    M, K = 7, 1024
    W, x = synth.q4k_matrix(M, K, 12), synth.activations(K, 13)
    xq = oracle.quant_q8_K(x)
    _, ref64 = oracle.qmatmul_q4k_q8k(W, xq, M, K)
    wd = oracle.dequant_q4k(W, 0).astype(np.float64).reshape(M, K)
    xd = oracle.dequant_q8_K(xq).astype(np.float64)
    # the only difference: each dequantized weight carries one fp32 rounding (2^-24 relative)
    assert np.max(np.abs(ref64 - wd @ xd)) / np.max(np.abs(wd @ xd)) < 1e-6
    dots = oracle.q4k_q8k_subdots(W, xq, M, K)
    assert dots.shape == (M, K // 256, 8) and np.abs(dots).max() <= 15 * 127 * 32

"""Q8_0 kernels against the CPU checker and the reference-made fixtures, through the C ABI."""
import os

import numpy as np
import pytest

from bpd_substrate_b200 import synth
from tests.util import Dev, assert_bits_equal, normwise

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
TOL = 1e-5   # norm-wise, fp32 GEMV outputs


def gpu_matmul(lib, W, X, M, N, K):
    dW, dX, dO = Dev(lib, W), Dev(lib, X), Dev(lib, nbytes=M * N * 4, fill=0xFF)
    assert lib.bpd_qmatmul_q8_0_cuda(dW.ptr, dX.ptr, dO.ptr, M, N, K, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    return dO.read(np.float32).reshape(M, N)


@pytest.mark.parametrize("nb", [1, 7, 64, 4097])
def test_dequant_bit_exact(lib, oracle, nb):
    raw = synth.q8_0_matrix(1, nb * 32, 50 + nb)
    raw[0:2] = [0x01, 0x00]                     # subnormal fp16 scale (tests/verify_f16_fix.py:99-117)
    dR, dO = Dev(lib, raw), Dev(lib, nbytes=nb * 128 + 64, fill=0x7F)
    assert lib.bpd_dequant_q8_0_cuda(dR.ptr, dO.ptr, nb, None) == 0
    lib.bpdq_sync()
    out = dO.read(np.uint8)
    assert (out[nb * 128:] == 0x7F).all()
    assert_bits_equal(out[:nb * 128].view(np.float32), oracle.dequant_q8_0(raw))


def test_dequant_every_fp16_scale(lib, oracle):
    nb = 65536
    raw = np.zeros((nb, 34), np.uint8)
    raw[:, 0:2] = np.arange(nb, dtype=np.uint16).view(np.uint8).reshape(nb, 2)
    raw[:, 2:] = np.random.default_rng(1).integers(-127, 128, (nb, 32), dtype=np.int8).view(np.uint8)
    raw = raw.reshape(-1)
    dR, dO = Dev(lib, raw), Dev(lib, nbytes=nb * 128)
    assert lib.bpd_dequant_q8_0_cuda(dR.ptr, dO.ptr, nb, None) == 0
    lib.bpdq_sync()
    assert_bits_equal(dO.read(np.float32), oracle.dequant_q8_0(raw))


@pytest.mark.parametrize("n", [32, 96, 4096, 32 * 1001])
def test_quantizer_bytes_identical(lib, oracle, n):
    rng = np.random.default_rng(n)
    x = synth.activations(n, rng)
    x[:32] = 0.0                                 # all-zero block
    if n > 64:
        x[40] = 0.5 * np.abs(x[32:64]).max() / 127 * 1.0   # a value near a rounding tie
    dX, dY = Dev(lib, x), Dev(lib, nbytes=n // 32 * 34 + 16, fill=0xAB)
    assert lib.bpd_quant_q8_0_cuda(dX.ptr, dY.ptr, n, None) == 0
    lib.bpdq_sync()
    y = dY.read(np.uint8)
    assert (y[n // 32 * 34:] == 0xAB).all()
    assert np.array_equal(y[:n // 32 * 34], oracle.quant_q8_0(x))


def test_block_dots_exact(lib, oracle):
    w = synth.q8_0_matrix(3, 4096, 5)
    a = oracle.quant_q8_0(synth.activations(3 * 4096, 6))
    dW, dA, dD = Dev(lib, w), Dev(lib, a), Dev(lib, nbytes=3 * 128 * 4)
    assert lib.bpd_q8_0_block_dots_cuda(dW.ptr, dA.ptr, dD.ptr, 3 * 128, None) == 0
    lib.bpdq_sync()
    assert np.array_equal(dD.read(np.int32), oracle.q8_0_block_dots(w, a))


@pytest.mark.parametrize("M,N,K", [(1, 64, 4096), (1, 37, 256), (3, 50, 1024), (1, 19, 14336), (2, 33, 96), (1, 5, 32),
                                   (1, 300, 8192)])
def test_matmul_matches_checker(lib, oracle, M, N, K):
    rng = np.random.default_rng(M * 1000 + N + K)
    W = synth.q8_0_matrix(N, K, rng)
    X = synth.activations(K, rng, rows=M)
    got = gpu_matmul(lib, W, X, M, N, K)
    assert normwise(got, oracle.qmatmul_q8_0_f64(W, X, M, N, K)) <= TOL
    assert normwise(got, oracle.qmatmul_q8_0(W, X, M, N, K)) <= TOL


def test_gemv_4096_against_reference_fixture(lib):
    g = np.load(os.path.join(GOLD, "q8_0_gemv_4096x4096.npz"))
    W = synth.q8_0_matrix(4096, 4096, int(g["w_seed"][0]))
    x = synth.activations(4096, int(g["x_seed"][0]))
    got = gpu_matmul(lib, W, x, 1, 4096, 4096)
    assert normwise(got, g["out"].view(np.float32).reshape(1, 4096)) <= TOL


def test_small_fixture_from_reference(lib):
    g = np.load(os.path.join(GOLD, "q8_0_small.npz"))
    Mt, Nw, Kq = (int(v) for v in g["shape"])
    got = gpu_matmul(lib, g["W"], g["X"], Mt, Nw, Kq)
    assert normwise(got, g["matmul_scalar"].view(np.float32).reshape(Mt, Nw)) <= TOL
    dX, dY = Dev(lib, g["X"]), Dev(lib, nbytes=g["Xq"].size)
    assert lib.bpd_quant_q8_0_cuda(dX.ptr, dY.ptr, Mt * Kq, None) == 0
    lib.bpdq_sync()
    assert np.array_equal(dY.read(np.uint8), g["Xq"])


def test_embed_lookup(lib, oracle):
    table = synth.q8_0_matrix(40, 512, 8)
    ids = np.array([3, 39, 0, 3, 17], np.int32)
    dT, dI, dO = Dev(lib, table), Dev(lib, ids), Dev(lib, nbytes=5 * 512 * 4)
    assert lib.bpd_embed_lookup_q8_0_cuda(dT.ptr, dI.ptr, dO.ptr, 5, 512, None) == 0
    lib.bpdq_sync()
    assert_bits_equal(dO.read(np.float32).reshape(5, 512), oracle.embed_lookup_q8_0(table, ids, 512))


def test_vecmat_shaped_entry(lib, oracle):
    K, N = 4096, 48
    W, x = synth.q8_0_matrix(N, K, 9), synth.activations(K, 10)
    dW, dX, dO = Dev(lib, W), Dev(lib, x), Dev(lib, nbytes=N * 4)
    lib.gpu_vecmat_q8_0(dX.ptr, dW.ptr, dO.ptr, K, N)
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    assert normwise(dO.read(np.float32), oracle.qmatmul_q8_0_f64(W, x, 1, N, K)[0]) <= TOL


def test_llamafile_and_dispatch_twins_give_the_avx_reference_bits(lib, oracle):
    """bpd_qmatmul_q8_0_dispatch_cuda / _llamafile_cuda (bench/bpd_gemm_q8_0_cpu.c:159-207, bench/bpd_cpu.c:4428-4459):
    the fixture written by the reference's AVX build, bit for bit; per-block integers are exact by construction
    (test_block_dots) and the eight fp32 lanes are added in the reference's order."""
    g = np.load(os.path.join(GOLD, "q8_0_avx_tiles.npz"))
    mw, mt, K = (int(v) for v in g["shape"])
    dW, dX, dXq = Dev(lib, g["W"]), Dev(lib, g["X"]), Dev(lib, g["Xq"])
    dO = Dev(lib, nbytes=mt * mw * 4, fill=0xFF)
    assert lib.bpd_qmatmul_q8_0_dispatch_cuda(dW.ptr, dXq.ptr, dO.ptr, mw, mt, K, None) == 0
    lib.bpdq_sync()
    assert np.array_equal(dO.read(np.uint32).reshape(mt, mw), g["dispatch"])
    lib.bpdq_memset_async(dO.ptr, 0xFF, dO.nbytes, None)
    assert lib.bpd_qmatmul_q8_0_llamafile_cuda(dW.ptr, dX.ptr, dO.ptr, mw, mt, K, None) == 0
    lib.bpdq_sync()
    assert np.array_equal(dO.read(np.uint32).reshape(mt, mw), g["llamafile"])
    assert lib.bpdq_last_status() == 0
    # within the stated bar of the sequential-order product as well
    assert normwise(dO.read(np.float32).reshape(mt, mw), oracle.qmatmul_q8_0_f64(g["W"], g["X"], mt, mw, K)) <= TOL


@pytest.mark.parametrize("rm", [1, 2, 4])
@pytest.mark.parametrize("rn", [1, 2, 4])
def test_tile_twins(lib, oracle, rm, rn):
    """The nine bpd_gemm_q8_0_{RM}_{RN}_cuda entries: strided tile in, out[j*ldc + i], cells outside the
    tile untouched; equal to the lane-order checker (three of them also to the reference-made fixture)."""
    g = np.load(os.path.join(GOLD, "q8_0_avx_tiles.npz"))
    mw, mt, K = (int(v) for v in g["shape"])
    rb = K // 32 * 34
    dW, dXq = Dev(lib, g["W"]), Dev(lib, g["Xq"])
    ldc = 8
    dO = Dev(lib, nbytes=rn * ldc * 4, fill=0xFF)
    fn = getattr(lib, f"bpd_gemm_q8_0_{rm}_{rn}_cuda")
    assert fn(dW.ptr + 3 * rb, dXq.ptr + rb, K // 32, rb, rb, dO.ptr, ldc, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    got = dO.read(np.uint32).reshape(rn, ldc)
    want = oracle.qmatmul_q8_0_lanes(g["W"][3 * rb:(3 + rm) * rb], g["Xq"][rb:(1 + rn) * rb], rm, rn, K)
    assert np.array_equal(got[:, :rm], want.view(np.uint32))
    assert (got[:, rm:] == 0xFFFFFFFF).all()
    if f"tile_{rm}_{rn}" in g.files:
        assert np.array_equal(got[:, :rm], g[f"tile_{rm}_{rn}"][:, :rm])


def test_dispatch_twin_large_ragged(lib, oracle):
    mw, mt, K = 1001, 13, 4096
    rng = np.random.default_rng(77)
    W = synth.q8_0_matrix(mw, K, rng)
    Xq = oracle.quant_q8_0(synth.activations(K, rng, rows=mt))
    dW, dXq, dO = Dev(lib, W), Dev(lib, Xq), Dev(lib, nbytes=mt * mw * 4, fill=0xFF)
    assert lib.bpd_qmatmul_q8_0_dispatch_cuda(dW.ptr, dXq.ptr, dO.ptr, mw, mt, K, None) == 0
    lib.bpdq_sync()
    assert np.array_equal(dO.read(np.uint32).reshape(mt, mw), oracle.qmatmul_q8_0_lanes(W, Xq, mw, mt, K).view(np.uint32))
    assert lib.bpd_qmatmul_q8_0_dispatch_cuda(dW.ptr, dXq.ptr, dO.ptr, mw, mt, 100, None) == -1
    assert lib.bpd_qmatmul_q8_0_dispatch_cuda(dW.ptr + 1, dXq.ptr, dO.ptr, mw, mt, K, None) == -2
    lib.bpdq_clear_status()


def test_embed_lookup_refuses_out_of_range_ids(lib, oracle):
    """A token id outside the table is not looked up: its output row keeps its bytes, the other rows are
    right, and the status reports -4 (no read outside the table happens)."""
    table = synth.q8_0_matrix(40, 512, 8)
    ids = np.array([3, 40, 0, -1, 17], np.int32)
    dT, dI, dO = Dev(lib, table), Dev(lib, ids), Dev(lib, nbytes=5 * 512 * 4, fill=0xCD)
    lib.bpdq_clear_status()
    assert lib.bpd_embed_lookup_q8_0_vocab_cuda(dT.ptr, dI.ptr, dO.ptr, 5, 512, 40, None) == 0
    lib.bpdq_sync()
    got = dO.read(np.float32).reshape(5, 512)
    assert lib.bpdq_last_status() == -4 and lib.bpdq_device_error_word() == 21
    lib.bpdq_clear_status()
    want = oracle.embed_lookup_q8_0(table, np.array([3, 0, 0, 0, 17], np.int32), 512)
    for t in (0, 2, 4):
        assert_bits_equal(got[t], want[t])
    for t in (1, 3):
        assert (got[t].view(np.uint32) == 0xCDCDCDCD).all()
    # the reference-shaped entry has no table size: negative ids are still refused
    lib.bpdq_memset_async(dO.ptr, 0xCD, dO.nbytes, None)
    dI2 = Dev(lib, np.array([3, 39, 0, -5, 17], np.int32))
    assert lib.bpd_embed_lookup_q8_0_cuda(dT.ptr, dI2.ptr, dO.ptr, 5, 512, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == -4
    lib.bpdq_clear_status()
    assert (dO.read(np.uint32).reshape(5, 512)[3] == 0xCDCDCDCD).all()


def test_stream_of_q8_0_products(lib, oracle):
    """40 independent Q8_0 products (several shapes, own vectors) as one persistent launch: the bits of
    bpd_qmatmul_q8_0_cuda product by product, and the checker's binary64 result within the bar."""
    from bpd_substrate_b200 import capi
    rng = np.random.default_rng(66)
    kinds = [(300, 4096), (64, 1024), (17, 14336), (500, 256), (128, 8192)]
    Ws = [synth.q8_0_matrix(m, k, rng) for m, k in kinds]
    dWs = [Dev(lib, w) for w in Ws]
    shapes = [kinds[j % len(kinds)] for j in range(40)]
    xs = [synth.activations(k, rng) for _, k in shapes]
    dXs = [Dev(lib, x) for x in xs]
    outs = [Dev(lib, nbytes=m * 4, fill=0xFF) for m, _ in shapes]
    n = len(shapes)
    descs = (capi.GemvDesc * n)(*[capi.GemvDesc(dWs[j % len(kinds)].ptr, dXs[j].ptr, outs[j].ptr, m, k)
                                  for j, (m, k) in enumerate(shapes)])
    nbytes = lib.bpdq_gemv_stream_q8_0_workspace_bytes(n, descs)
    ws = Dev(lib, nbytes=nbytes, fill=0xCD)
    h = lib.bpdq_gemv_stream_create_q8_0(n, descs, ws.ptr, nbytes)
    assert h
    for run in (lib.bpdq_gemv_stream_run, lib.bpdq_gemv_stream_run_ready):
        for o in outs:
            lib.bpdq_memset_async(o.ptr, 0xFF, o.nbytes, None)
        assert run(h, None) == 0
        lib.bpdq_sync()
        assert lib.bpdq_last_status() == 0
        for j, (m, k) in enumerate(shapes):
            got = outs[j].read(np.float32)
            single = gpu_matmul(lib, Ws[j % len(kinds)], xs[j], 1, m, k)[0]
            assert np.array_equal(got.view(np.uint32), single.view(np.uint32)), j
            if j < 10:
                assert normwise(got, oracle.qmatmul_q8_0_f64(Ws[j % len(kinds)], xs[j], 1, m, k)[0]) <= TOL
    lib.bpdq_gemv_stream_destroy(h)

"""Q4_K re-tiled in groups of 16 rows: the permutation (host and device, both ways, bit for bit) and the
many-token product on it against the CPU checker -- exact integers, fp32 outputs within 1e-5 norm-wise."""
import numpy as np
import pytest

from bpd_substrate_b200 import capi, gguf_load, synth
from tests.util import Dev, normwise

TOL = 1e-5


def test_host_repack_is_an_invertible_permutation():
    for rows, cols in ((16, 256), (37, 512), (5, 1024), (130, 768)):
        raw = synth.q4k_matrix(rows, cols, rows + cols)
        tiles = gguf_load.repack_q4k_to_rg16(raw, rows, cols)
        assert tiles.size == -(-rows // 16) * (cols // 256) * 2304
        assert np.array_equal(gguf_load.repack_rg16_to_q4k(tiles, rows, cols), raw)
        # a permutation: the multiset of bytes is kept (plus the zero rows of the last group)
        assert np.array_equal(np.bincount(tiles, minlength=256)[1:], np.bincount(raw, minlength=256)[1:])
    # spot check of the documented formula: word t of sub-block j of row r
    rows, cols = 32, 512
    raw = synth.q4k_matrix(rows, cols, 9)
    tiles = gguf_load.repack_q4k_to_rg16(raw, rows, cols).reshape(2, 2, 2304)
    src = raw.reshape(rows, 2, 144)
    for G, b, q, L, e in ((0, 0, 0, 0, 0), (1, 1, 3, 31, 3), (0, 1, 2, 13, 1), (1, 0, 1, 6, 2)):
        g, t, j, row = L >> 2, L & 3, 2 * q + (e >> 1), G * 16 + (L >> 2) + 8 * (e & 1)
        at = 256 + 512 * q + 16 * L + 4 * e
        assert np.array_equal(tiles[G, b, at:at + 4], src[row, b, 16 + 16 * j + 4 * t:16 + 16 * j + 4 * t + 4])
    assert np.array_equal(tiles[1, 0, 16 * 5:16 * 6], src[21, 0, :16])


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols", [(16, 256), (37, 512), (1000, 4096), (14336, 4096)])
def test_device_repack_equals_host_repack_and_inverts(lib, rows, cols):
    raw = synth.q4k_matrix(rows, cols, rows)
    nbytes = lib.bpd_q4k_rg16_bytes(rows, cols)
    want = gguf_load.repack_q4k_to_rg16(raw, rows, cols)
    assert nbytes == want.size
    dR, dT, dB = Dev(lib, raw), Dev(lib, nbytes=nbytes, fill=0xEE), Dev(lib, nbytes=raw.size, fill=0xDD)
    assert lib.bpd_repack_q4k_rg16_cuda(dR.ptr, dT.ptr, rows, cols, None) == 0
    assert lib.bpd_unrepack_q4k_rg16_cuda(dT.ptr, dB.ptr, rows, cols, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    assert np.array_equal(dT.read(np.uint8), want)
    assert np.array_equal(dB.read(np.uint8), raw)


def _retiled(lib, W, N, K):
    dR = Dev(lib, W)
    dT = Dev(lib, nbytes=lib.bpd_q4k_rg16_bytes(N, K))
    assert lib.bpd_repack_q4k_rg16_cuda(dR.ptr, dT.ptr, N, K, None) == 0
    lib.bpdq_sync()
    return dT


@pytest.mark.gpu
@pytest.mark.parametrize("T,N,K", [(1, 16, 256), (2, 40, 512), (5, 300, 1024), (8, 128, 4096), (9, 64, 768), (16, 500, 2048),
                                   (17, 96, 256), (32, 260, 4096), (33, 1280, 1792), (64, 2000, 1024), (65, 48, 512),
                                   (130, 100, 768), (8, 1024, 28672), (16, 3584, 8192)])
def test_product_on_retiled_weights(lib, oracle, T, N, K):
    """All token-tile widths (8, 16, 32, 64), more than 64 tokens (two and three passes), ragged row groups, K of one
    super-block and of 112 (chunks shorter than the ring's chunk size at the end), more CTA tiles than SMs."""
    rng = np.random.default_rng(T * 13 + N + K)
    W = synth.q4k_matrix(N, K, rng)
    X = synth.activations(K, rng, rows=T)
    dT, dX = _retiled(lib, W, N, K), Dev(lib, X)
    dO = Dev(lib, nbytes=T * N * 4, fill=0xFF)
    nb = K // 256
    dI = Dev(lib, nbytes=T * N * nb * 8, fill=0xEE)
    assert lib.bpd_qmm_q4k_q8k_rg16_ints_cuda(dT.ptr, dX.ptr, dO.ptr, dI.ptr, T, N, K, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    _, ref64 = oracle.qmm_q4k_q8k(W, X, T, N, K)
    assert np.array_equal(dI.read(np.int32).reshape(T, N, nb, 2), oracle.qmm_q4k_q8k_ints(W, X, T, N, K))
    got = dO.read(np.float32).reshape(T, N)
    assert normwise(got, ref64) <= TOL
    # the plain entry and the caller-workspace entry: same bits
    for entry in ("plain", "ws"):
        dO2 = Dev(lib, nbytes=T * N * 4, fill=0xFF)
        if entry == "plain":
            assert lib.bpd_qmm_q4k_q8k_rg16_cuda(dT.ptr, dX.ptr, dO2.ptr, T, N, K, None) == 0
        else:
            nbytes = lib.bpdq_qmm_q4k_q8k_rg16_workspace_bytes(T, K)
            ws = Dev(lib, nbytes=nbytes, fill=0xAB)
            assert lib.bpd_qmm_q4k_q8k_rg16_ws_cuda(dT.ptr, dX.ptr, dO2.ptr, T, N, K, ws.ptr, nbytes, None) == 0
        lib.bpdq_sync()
        assert lib.bpdq_last_status() == 0
        assert np.array_equal(dO2.read(np.uint32), got.view(np.uint32).ravel()), entry


@pytest.mark.gpu
def test_retiled_product_has_the_bits_of_the_row_layout_tensor_core_kernel(lib):
    """Same arithmetic in the same order as bpd_qmm_q4k_q8k_mma_cuda on the original rows."""
    T, N, K = 24, 520, 2048
    rng = np.random.default_rng(3)
    W, X = synth.q4k_matrix(N, K, rng), synth.activations(K, rng, rows=T)
    dW, dX, dT = Dev(lib, W), Dev(lib, X), _retiled(lib, W, N, K)
    a, b = Dev(lib, nbytes=T * N * 4, fill=0xFF), Dev(lib, nbytes=T * N * 4, fill=0xFF)
    assert lib.bpd_qmm_q4k_q8k_mma_cuda(dW.ptr, dX.ptr, a.ptr, T, N, K, None) == 0
    assert lib.bpd_qmm_q4k_q8k_rg16_cuda(dT.ptr, dX.ptr, b.ptr, T, N, K, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    assert np.array_equal(a.read(np.uint32), b.read(np.uint32))


@pytest.mark.gpu
@pytest.mark.parametrize("tokens", [1, 8, 20])
def test_stream_of_products_on_retiled_weights(lib, oracle, tokens):
    """Several independent products per persistent launch (two share an activation matrix; 140 products = two
    launches), run twice: against the checker, and the same bits both times."""
    rng = np.random.default_rng(50 + tokens)
    kinds = [(448, 1024), (128, 1024), (40, 4096), (260, 256), (96, 2048)]
    shapes = [kinds[j % len(kinds)] for j in range(140)]
    Ws = [synth.q4k_matrix(m, k, rng) for m, k in kinds]
    dTs = [_retiled(lib, Ws[j], m, k) for j, (m, k) in enumerate(kinds)]
    Xs, dXs = [], []
    for j, (m, k) in enumerate(shapes):
        if j == 6:                              # same matrix and same X as product 1 (K = 1024)
            Xs.append(Xs[1]); dXs.append(dXs[1])
        else:
            Xs.append(synth.activations(k, rng, rows=tokens)); dXs.append(Dev(lib, Xs[-1]))
    outs = [Dev(lib, nbytes=tokens * m * 4, fill=0xFF) for m, _ in shapes]
    n = len(shapes)
    descs = (capi.GemvDesc * n)(*[capi.GemvDesc(dTs[j % len(kinds)].ptr, dXs[j].ptr, outs[j].ptr, m, k)
                                  for j, (m, k) in enumerate(shapes)])
    nbytes = lib.bpdq_gemm_rg16_stream_workspace_bytes(n, descs, tokens)
    ws = Dev(lib, nbytes=nbytes, fill=0xCD)
    h = lib.bpdq_gemm_rg16_stream_create(n, descs, tokens, ws.ptr, nbytes)
    assert h and lib.bpdq_gemm_rg16_stream_launches(h) == 4
    first = None
    for rep in range(2):
        assert lib.bpdq_gemm_rg16_stream_run(h, None) == 0
        lib.bpdq_sync()
        assert lib.bpdq_last_status() == 0
        got = [o.read(np.float32) for o in outs]
        if first is None:
            first = got
            refs = {}
            for j, (m, k) in enumerate(shapes):
                key = (j % len(kinds), id(Xs[j]))
                if key not in refs:
                    refs[key] = oracle.qmm_q4k_q8k(Ws[j % len(kinds)], Xs[j], tokens, m, k)[1]
                assert normwise(got[j].reshape(tokens, m), refs[key]) <= TOL, j
        else:
            for j in range(n):
                assert np.array_equal(got[j].view(np.uint32), first[j].view(np.uint32)), j
        for o in outs:
            lib.bpdq_memset_async(o.ptr, 0xFF, o.nbytes, None)
    lib.bpdq_gemm_rg16_stream_destroy(h)
    assert not lib.bpdq_gemm_rg16_stream_create(n, descs, 65, ws.ptr, nbytes)
    assert not lib.bpdq_gemm_rg16_stream_create(n, descs, tokens, ws.ptr, 1024)
    lib.bpdq_clear_status()


@pytest.mark.gpu
def test_rejects_bad_arguments(lib):
    d = Dev(lib, nbytes=1 << 16)
    assert lib.bpd_qmm_q4k_q8k_rg16_cuda(d.ptr, d.ptr, d.ptr, 4, 16, 100, None) == -1
    assert lib.bpd_qmm_q4k_q8k_rg16_cuda(d.ptr + 8, d.ptr, d.ptr, 4, 16, 256, None) == -2
    assert lib.bpd_qmm_q4k_q8k_rg16_cuda(None, d.ptr, d.ptr, 4, 16, 256, None) == -1
    assert lib.bpd_repack_q4k_rg16_cuda(d.ptr, d.ptr + 4, 16, 256, None) == -2
    assert lib.bpd_q4k_rg16_bytes(16, 100) == 0
    lib.bpdq_clear_status()

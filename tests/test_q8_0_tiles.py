"""Q8_0 re-tiled for the tensor cores: the permutation (host and device, both directions) and the tcgen05
product against the scalar reference arithmetic, bit for bit, through the C ABI."""
import numpy as np
import pytest

from bpd_substrate_b200 import gguf_load, synth
from tests.util import Dev, assert_bits_equal


def tiles_by_formula(raw, rows, cols):
    """Independent restatement of the layout: one byte at a time from the documented index formula."""
    nb = cols // 32
    src = np.asarray(raw, np.uint8).reshape(rows, nb, 34)
    tiles = -(-rows // 128)
    out = np.zeros((tiles, nb, 4352), np.uint8)
    for n in range(rows):
        t, r = divmod(n, 128)
        for b in range(nb):
            out[t, b, 4096 + 2 * r:4096 + 2 * r + 2] = src[n, b, :2]
            for k in range(32):
                out[t, b, (k // 16) * 2048 + (r // 8) * 128 + (r % 8) * 16 + k % 16] = src[n, b, 2 + k]
    return out.reshape(-1)


@pytest.mark.parametrize("rows,cols", [(1, 32), (130, 96), (256, 64)])
def test_host_repack_follows_the_formula_and_inverts(rows, cols):
    raw = synth.q8_0_matrix(rows, cols, rows + cols)
    tiles = gguf_load.repack_q8_0_to_tiles(raw, rows, cols)
    assert np.array_equal(tiles, tiles_by_formula(raw, rows, cols))
    assert np.array_equal(gguf_load.repack_tiles_to_q8_0(tiles, rows, cols), raw)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols", [(1, 32), (128, 4096), (200, 96), (1000, 2048)])
def test_device_repack_equals_host_and_round_trips(lib, rows, cols):
    raw = synth.q8_0_matrix(rows, cols, 3 * rows + cols)
    nbytes = lib.bpd_q8_0_tiles_bytes(rows, cols)
    assert nbytes == -(-rows // 128) * (cols // 32) * 4352
    dR, dT, dB = Dev(lib, raw), Dev(lib, nbytes=nbytes, fill=0xEE), Dev(lib, nbytes=raw.nbytes + 16, fill=0x55)
    assert lib.bpd_repack_q8_0_tiles_cuda(dR.ptr, dT.ptr, rows, cols, None) == 0
    assert lib.bpd_unrepack_q8_0_tiles_cuda(dT.ptr, dB.ptr, rows, cols, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    assert np.array_equal(dT.read(np.uint8), gguf_load.repack_q8_0_to_tiles(raw, rows, cols))
    back = dB.read(np.uint8)
    assert np.array_equal(back[:raw.nbytes], raw)
    assert (back[raw.nbytes:] == 0x55).all()


def tiles_matmul(lib, W, X, M, N, K, host_repack=False):
    if host_repack:
        dT = Dev(lib, gguf_load.repack_q8_0_to_tiles(W, N, K))
    else:
        dW, dT = Dev(lib, W), Dev(lib, nbytes=lib.bpd_q8_0_tiles_bytes(N, K))
        assert lib.bpd_repack_q8_0_tiles_cuda(dW.ptr, dT.ptr, N, K, None) == 0
    dX, dO = Dev(lib, X), Dev(lib, nbytes=M * N * 4 + 64, fill=0xFF)
    assert lib.bpd_qmatmul_q8_0_tiles_cuda(dT.ptr, dX.ptr, dO.ptr, M, N, K, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    out = dO.read(np.uint8)
    assert (out[M * N * 4:] == 0xFF).all()
    return out[:M * N * 4].view(np.float32).reshape(M, N)


# tokens below, at and above each token tile (16, 32, 64) and beyond one tile; rows below and across
# row tiles; blocks per row below, at and not a multiple of the ring's four-block stages
SHAPES = [(1, 128, 32), (5, 200, 96), (16, 256, 4096), (17, 100, 160), (32, 384, 1024), (33, 130, 2048),
          (64, 512, 4096), (70, 300, 992), (130, 256, 512)]


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_product_is_the_scalar_reference_bit_for_bit(lib, oracle, M, N, K):
    rng = np.random.default_rng(M * 131 + N * 7 + K)
    W = synth.q8_0_matrix(N, K, rng)
    X = synth.activations(K, rng, rows=M)
    X[0, :32] = 0.0                              # an all-zero activation block
    got = tiles_matmul(lib, W, X, M, N, K)
    assert_bits_equal(got, oracle.qmatmul_q8_0(W, X, M, N, K).reshape(M, N))


@pytest.mark.gpu
def test_gemv_4096_equals_the_reference_made_fixture(lib):
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "q8_0_gemv_4096x4096.npz"))
    W = synth.q8_0_matrix(4096, 4096, int(g["w_seed"][0]))
    x = synth.activations(4096, int(g["x_seed"][0]))
    got = tiles_matmul(lib, W, x.reshape(1, -1), 1, 4096, 4096)
    assert np.array_equal(got.view(np.uint32).ravel(), g["out"].ravel())


@pytest.mark.gpu
def test_product_on_host_repacked_weights_and_repeats(lib, oracle):
    M, N, K = 48, 640, 4096
    W = synth.q8_0_matrix(N, K, 9)
    X = synth.activations(K, 10, rows=M)
    want = oracle.qmatmul_q8_0(W, X, M, N, K).reshape(M, N)
    first = tiles_matmul(lib, W, X, M, N, K, host_repack=True)
    assert_bits_equal(first, want)
    assert_bits_equal(tiles_matmul(lib, W, X, M, N, K), first)


@pytest.mark.gpu
def test_product_equals_the_row_layout_kernel_within_its_tolerance(lib):
    M, N, K = 8, 512, 4096
    W = synth.q8_0_matrix(N, K, 21)
    X = synth.activations(K, 22, rows=M)
    dW, dX, dO = Dev(lib, W), Dev(lib, X), Dev(lib, nbytes=M * N * 4)
    assert lib.bpd_qmatmul_q8_0_cuda(dW.ptr, dX.ptr, dO.ptr, M, N, K, None) == 0
    lib.bpdq_sync()
    rows = dO.read(np.float32).reshape(M, N)
    got = tiles_matmul(lib, W, X, M, N, K)
    assert np.abs(got - rows).max() <= 1e-5 * np.abs(rows).max()


@pytest.mark.gpu
def test_bad_arguments_are_rejected(lib):
    d = Dev(lib, nbytes=1 << 16)
    try:
        assert lib.bpd_qmatmul_q8_0_tiles_cuda(d.ptr, d.ptr, d.ptr, 1, 128, 48, None) != 0      # K not whole blocks
        assert lib.bpd_qmatmul_q8_0_tiles_cuda(d.ptr + 8, d.ptr, d.ptr, 1, 128, 32, None) != 0  # tiles not 16-byte aligned
        assert lib.bpd_qmatmul_q8_0_tiles_cuda(None, d.ptr, d.ptr, 1, 128, 32, None) != 0
        assert lib.bpd_repack_q8_0_tiles_cuda(d.ptr, d.ptr + 4, 128, 32, None) != 0
        assert lib.bpd_q8_0_tiles_bytes(128, 48) == 0
        assert lib.bpd_qmatmul_q8_0_tiles_cuda(d.ptr, d.ptr, d.ptr, 0, 128, 32, None) == 0      # nothing to do
    finally:
        lib.bpdq_clear_status()

"""Batched Q4_K x Q8_K product (many tokens): the int8 tensor-core kernel against the checker."""
import numpy as np
import pytest

from bpd_substrate_b200 import synth
from tests.util import Dev, normwise

pytestmark = pytest.mark.gpu
TOL = 1e-5


def run(lib, entry, W, X, T, N, K):
    dW, dX, dO = Dev(lib, W), Dev(lib, X), Dev(lib, nbytes=T * N * 4, fill=0xFF)
    if entry == "mma":
        rc = lib.bpd_qmm_q4k_q8k_mma_cuda(dW.ptr, dX.ptr, dO.ptr, T, N, K, None)
    elif entry == "tc5":
        rc = lib.bpd_qmm_q4k_q8k_tc5_cuda(dW.ptr, dX.ptr, dO.ptr, T, N, K, None)
    else:
        rc = lib.bpd_qmm_q4k_q8k_cuda(dW.ptr, dX.ptr, dO.ptr, T, N, K, 0, 0, None, None)
    assert rc == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    return dO.read(np.float32).reshape(T, N)


@pytest.mark.parametrize("T,N,K", [(16, 128, 256), (16, 300, 1024), (9, 64, 4096), (33, 112, 512), (64, 260, 4096),
                                   (1, 40, 256), (70, 100, 768), (130, 48, 256)])
def test_mma_kernel_matches_checker(lib, oracle, T, N, K):
    rng = np.random.default_rng(T * 7 + N + K)
    W = synth.q4k_matrix(N, K, rng)
    X = synth.activations(K, rng, rows=T)
    got = run(lib, "mma", W, X, T, N, K)
    ref32, ref64 = oracle.qmm_q4k_q8k(W, X, T, N, K)
    assert normwise(got, ref64) <= TOL


@pytest.mark.parametrize("T,N,K", [(16, 128, 256), (9, 300, 768), (32, 384, 1024), (64, 512, 4096), (40, 1000, 2048),
                                   (100, 256, 512), (1, 128, 256), (64, 14336 // 8, 4096),
                                   (48, 256, 8192), (16, 130, 4096), (33, 1280, 14336 // 2)])
def test_tcgen05_kernel_matches_checker(lib, oracle, T, N, K):
    """The TMEM-accumulator kernel: same integers, same tolerance; partial last row tile included,
    and K split over 1, 2, 4 and 8 ranges (few row tiles, many super-blocks per row)."""
    rng = np.random.default_rng(T * 11 + N + K)
    W = synth.q4k_matrix(N, K, rng)
    X = synth.activations(K, rng, rows=T)
    got = run(lib, "tc5", W, X, T, N, K)
    _, ref64 = oracle.qmm_q4k_q8k(W, X, T, N, K)
    assert normwise(got, ref64) <= TOL


def test_tcgen05_split_k_repeats_bit_for_bit(lib):
    """Ranges of K are summed in a fixed order by whichever unit arrives last, and the arrival counters
    reset themselves: back-to-back calls on one stream give identical bits."""
    T, N, K = 40, 384, 8192
    rng = np.random.default_rng(12)
    W = synth.q4k_matrix(N, K, rng)
    X = synth.activations(K, rng, rows=T)
    dW, dX = Dev(lib, W), Dev(lib, X)
    outs = [Dev(lib, nbytes=T * N * 4, fill=0xFF) for _ in range(4)]
    for o in outs:
        assert lib.bpd_qmm_q4k_q8k_tc5_cuda(dW.ptr, dX.ptr, o.ptr, T, N, K, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    first = outs[0].read(np.uint32)
    for o in outs[1:]:
        assert np.array_equal(first, o.read(np.uint32))


def test_tcgen05_kernel_rejects_short_matrices(lib):
    d = Dev(lib, nbytes=64 * 144 + 4096)
    assert lib.bpd_qmm_q4k_q8k_tc5_cuda(d.ptr, d.ptr, d.ptr, 16, 64, 256, None) == -3
    lib.bpdq_clear_status()


def test_dispatcher_agrees_across_token_counts(lib, oracle):
    """1..4 tokens (dp4a kernel), 16 and 64 tokens (tensor cores): each token's row equals the
    checker, whatever kernel produced it."""
    N, K = 96, 2048
    rng = np.random.default_rng(5)
    W = synth.q4k_matrix(N, K, rng)
    X = synth.activations(K, rng, rows=64)
    _, ref64 = oracle.qmm_q4k_q8k(W, X, 64, N, K)
    for T in (1, 4, 16, 64):
        got = run(lib, "dispatch", W, X[:T], T, N, K)
        assert normwise(got, ref64[:T]) <= TOL, T


def test_dispatcher_large_matrix_many_tokens(lib, oracle):
    """2^25 weights and 33 tokens: the size from which the dispatcher hands the product to the
    tcgen05 kernel; the result must not depend on that choice."""
    T, N, K = 33, 8192, 4096
    rng = np.random.default_rng(8)
    W = synth.q4k_matrix(N, K, rng)
    X = synth.activations(K, rng, rows=T)
    got = run(lib, "dispatch", W, X, T, N, K)
    via_mma = run(lib, "mma", W, X, T, N, K)
    _, ref64 = oracle.qmm_q4k_q8k(W, X, T, N, K)
    assert normwise(got, ref64) <= TOL
    assert normwise(got, via_mma) <= TOL


def test_gpu_matmul_q4k_entry(lib, oracle):
    T, N, K = 24, 80, 1024
    rng = np.random.default_rng(6)
    W, X = synth.q4k_matrix(N, K, rng), synth.activations(K, rng, rows=T)
    dW, dX, dO = Dev(lib, W), Dev(lib, X), Dev(lib, nbytes=T * N * 4)
    lib.gpu_matmul_q4k(dX.ptr, dW.ptr, dO.ptr, T, N, K)
    lib.gpu_sync()
    assert lib.bpdq_last_status() == 0
    assert normwise(dO.read(np.float32).reshape(T, N), oracle.qmm_q4k_q8k(W, X, T, N, K)[1]) <= TOL

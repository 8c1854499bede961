"""Q4_K weights x fp32 activations (the reference's own GEMV/GEMM semantics) on the GPU."""
import os

import numpy as np
import pytest

from bpd_substrate_b200 import synth
from tests.util import Dev, normwise

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")
TOL = 1e-5   # norm-wise max|d|/max|ref| against the reference's CPU result


@pytest.mark.parametrize("M,K", [(1, 256), (12, 1024), (64, 4096), (33, 14336), (100, 512)])
def test_gemv_matches_reference_order_within_tolerance(lib, oracle, M, K):
    W, x = synth.q4k_matrix(M, K, 60 + M), synth.activations(K, 61 + K)
    dW, dX, dO = Dev(lib, W), Dev(lib, x), Dev(lib, nbytes=M * 4, fill=0xFF)
    lib.bpd_qmatmul_q4k_gpu(dW.ptr, dX.ptr, dO.ptr, M, K)
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    got = dO.read(np.float32)
    assert normwise(got, oracle.qmatmul_q4k(W, x, M, K)) <= TOL        # the reference's sequential fp32 sum
    assert normwise(got, oracle.qmatmul_q4k_f64(W, x, M, K)) <= TOL    # and the binary64 sum


def test_gemv_and_gemm_against_reference_fixture(lib):
    g = np.load(os.path.join(GOLD, "q4k_small.npz"))
    M, K, N = (int(v) for v in g["shape"])
    dW, dX, dO = Dev(lib, g["W"]), Dev(lib, g["x"]), Dev(lib, nbytes=M * 4)
    assert lib.bpd_qmatmul_q4k_gpu_st(dW.ptr, dX.ptr, dO.ptr, M, K, None) == 0
    lib.bpdq_sync()
    assert normwise(dO.read(np.float32), g["gemv"].view(np.float32)) <= TOL
    dB, dC = Dev(lib, g["B"]), Dev(lib, nbytes=M * N * 4)
    assert lib.bpd_qmm_q4k_cuda(dW.ptr, dB.ptr, dC.ptr, M, N, K, None) == 0
    lib.bpdq_sync()
    assert normwise(dC.read(np.float32).reshape(M, N), g["gemm"].view(np.float32).reshape(M, N)) <= TOL


@pytest.mark.parametrize("N", [1, 4, 5, 9])
def test_gemm_columns(lib, oracle, N):
    M, K = 20, 1024
    W, B = synth.q4k_matrix(M, K, 70), synth.activations(N, 71, rows=K)
    dW, dB, dC = Dev(lib, W), Dev(lib, B), Dev(lib, nbytes=M * N * 4, fill=0xFF)
    assert lib.bpd_qmm_q4k_cuda(dW.ptr, dB.ptr, dC.ptr, M, N, K, None) == 0
    lib.bpdq_sync()
    assert normwise(dC.read(np.float32).reshape(M, N), oracle.qmm_q4k(W, B, M, N, K)) <= TOL

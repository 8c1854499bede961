"""fp32 decode-dispatch operators (the gpu_* surface) against numpy / the CPU checker."""
import numpy as np
import pytest

from tests.util import Dev, normwise

pytestmark = pytest.mark.gpu


def test_vecmat(lib, oracle):
    rng = np.random.default_rng(1)
    for k, n in ((64, 32), (4096, 1000), (257, 33), (1, 5)):
        a = rng.standard_normal(k, dtype=np.float32)
        b = rng.standard_normal((k, n), dtype=np.float32)
        dA, dB, dC = Dev(lib, a), Dev(lib, b), Dev(lib, nbytes=n * 4, fill=0xFF)
        lib.gpu_vecmat(dA.ptr, dB.ptr, dC.ptr, k, n)
        lib.gpu_sync()
        want = a.astype(np.float64) @ b.astype(np.float64)
        assert normwise(dC.read(np.float32), want) <= 1e-5
        if k <= 257:
            assert normwise(dC.read(np.float32), oracle.vecmat_f32(a, b, k, n)) <= 1e-5


def test_rms_norm(lib, oracle):
    rng = np.random.default_rng(2)
    for rows, cols in ((1, 4096), (3, 2048), (2, 100)):
        x = rng.standard_normal((rows, cols), dtype=np.float32)
        w = rng.standard_normal(cols, dtype=np.float32)
        dX, dW, dO = Dev(lib, x), Dev(lib, w), Dev(lib, nbytes=rows * cols * 4)
        lib.gpu_rms_norm(dX.ptr, dW.ptr, dO.ptr, rows, cols, 1e-5)
        lib.gpu_sync()
        got = dO.read(np.float32).reshape(rows, cols)
        assert np.allclose(got, oracle.rms_norm(x, w, rows, cols, 1e-5), rtol=2e-6, atol=1e-7)


def test_elementwise(lib):
    rng = np.random.default_rng(3)
    n = 14336 + 3
    a, b = rng.standard_normal(n, dtype=np.float32) * 4, rng.standard_normal(n, dtype=np.float32)
    dA, dB, dO = Dev(lib, a), Dev(lib, b), Dev(lib, nbytes=n * 4)
    lib.gpu_add(dA.ptr, dB.ptr, dO.ptr, n)
    lib.gpu_sync()
    assert np.array_equal(dO.read(np.float32), a + b)
    lib.gpu_mul(dA.ptr, dB.ptr, dO.ptr, n)
    lib.gpu_sync()
    assert np.array_equal(dO.read(np.float32), a * b)
    lib.gpu_silu(dA.ptr, dO.ptr, n)
    lib.gpu_sync()
    want = a.astype(np.float64) / (1.0 + np.exp(-a.astype(np.float64)))
    assert np.allclose(dO.read(np.float32), want, rtol=2e-6, atol=1e-7)
    assert lib.bpdq_last_status() == 0


def test_matmul(lib):
    rng = np.random.default_rng(4)
    M, N, K = 5, 70, 130
    A, B = rng.standard_normal((M, K), dtype=np.float32), rng.standard_normal((K, N), dtype=np.float32)
    dA, dB, dC = Dev(lib, A), Dev(lib, B), Dev(lib, nbytes=M * N * 4)
    for fn in (lib.gpu_matmul, lib.gpu_matmul_opt):
        fn(dA.ptr, dB.ptr, dC.ptr, M, N, K)
        lib.gpu_sync()
        assert normwise(dC.read(np.float32).reshape(M, N), A.astype(np.float64) @ B.astype(np.float64)) <= 1e-5

"""The allocation-free batched GEMV entry point (collected last on purpose).

Some callers cannot call cudaMalloc when they need a result: a plugin whose host application
owns all device memory, code in a region where the device-wide synchronization of cudaMalloc
and cudaFree is not acceptable, a latency-bound loop.  For them
``bpd_qmatmul_q4k_q8k_batch_static_cuda`` keeps its scratch (the quantized activations) in a
fixed array inside the library.  Here it is called twice in a row through the C ABI and must
return exactly what the ordinary entry point returns, and refuse a call that needs more scratch
than the array holds."""
import numpy as np
import pytest

from bpd_substrate_b200 import capi, synth
from tests.util import Dev, normwise

pytestmark = pytest.mark.gpu


def _problem(lib, shapes, seed):
    rng = np.random.default_rng(seed)
    Ws = [synth.q4k_matrix(m, k, rng) for m, k in shapes]
    xs = [synth.activations(k, rng) for _, k in shapes]
    dW, dX = [Dev(lib, w) for w in Ws], [Dev(lib, x) for x in xs]
    return Ws, xs, dW, dX


def _run(lib, entry, shapes, dW, dX):
    outs = [Dev(lib, nbytes=m * 4, fill=0xFF) for m, _ in shapes]
    descs = (capi.GemvDesc * len(shapes))()
    for j, (m, k) in enumerate(shapes):
        descs[j] = capi.GemvDesc(dW[j].ptr, dX[j].ptr, outs[j].ptr, m, k)
    assert getattr(lib, entry)(len(shapes), descs, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    return [o.read(np.float32) for o in outs]


def test_static_scratch_matches_ordinary_entry_twice_in_a_row(lib, oracle):
    shapes_a = [(64, 4096), (16, 4096), (40, 14336), (7, 256)]
    shapes_b = [(33, 8192), (50, 4096)]          # a second, different call reuses the same array
    for call, (shapes, seed) in enumerate(((shapes_a, 501), (shapes_b, 502))):
        Ws, xs, dW, dX = _problem(lib, shapes, seed)
        want = _run(lib, "bpd_qmatmul_q4k_q8k_batch_cuda", shapes, dW, dX)
        got = _run(lib, "bpd_qmatmul_q4k_q8k_batch_static_cuda", shapes, dW, dX)
        for j, (m, k) in enumerate(shapes):
            assert np.array_equal(got[j].view(np.uint32), want[j].view(np.uint32)), (call, j)
            _, ref64 = oracle.qmatmul_q4k_q8k(Ws[j], oracle.quant_q8_K(xs[j]), m, k)
            assert normwise(got[j], ref64) <= 1e-5, (call, j)


def test_static_scratch_rejects_oversized_calls(lib):
    cap = lib.bpdq_batch_static_capacity()
    assert cap == 256 * 1024
    k = 28672
    n = 9                                              # 9 x 28672 activations need 291,456 bytes of records
    d = Dev(lib, nbytes=16 * (k // 256) * 144)
    x = Dev(lib, nbytes=k * 4)
    o = Dev(lib, nbytes=64)
    descs = (capi.GemvDesc * n)(*[capi.GemvDesc(d.ptr, x.ptr, o.ptr, 16, k) for _ in range(n)])
    assert lib.bpdq_batch_workspace_bytes(n, descs) > cap
    assert lib.bpd_qmatmul_q4k_q8k_batch_static_cuda(n, descs, None) == -3
    lib.bpdq_clear_status()

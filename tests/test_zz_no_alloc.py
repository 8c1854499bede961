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


def test_static_scratch_allocates_nothing_and_takes_many_descriptors(lib, oracle):
    """Twelve products in one call (more than one launch holds: their records sit side by side in the
    fixed array), with the driver's free-memory reading unchanged across the calls."""
    import ctypes as C
    shapes = [(24 + 3 * j, 4096 if j % 3 else 1024) for j in range(12)]
    Ws, xs, dW, dX = _problem(lib, shapes, 503)
    want = _run(lib, "bpd_qmatmul_q4k_q8k_batch_cuda", shapes, dW, dX)
    outs = [Dev(lib, nbytes=m * 4, fill=0xFF) for m, _ in shapes]
    descs = (capi.GemvDesc * len(shapes))(*[capi.GemvDesc(dW[j].ptr, dX[j].ptr, outs[j].ptr, m, k)
                                            for j, (m, k) in enumerate(shapes)])
    assert lib.bpd_qmatmul_q4k_q8k_batch_static_cuda(len(shapes), descs, None) == 0   # first call: set-up done
    lib.bpdq_sync()
    free0, free1 = C.c_size_t(0), C.c_size_t(0)
    assert lib.bpdq_mem_info(C.byref(free0), None) == 0
    for _ in range(3):
        assert lib.bpd_qmatmul_q4k_q8k_batch_static_cuda(len(shapes), descs, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_mem_info(C.byref(free1), None) == 0
    assert free1.value == free0.value
    assert lib.bpdq_last_status() == 0
    for j in range(len(shapes)):
        assert np.array_equal(outs[j].read(np.uint32), want[j].view(np.uint32)), j
    # a malformed descriptor is an argument error whatever the size of the call
    bad = (capi.GemvDesc * 1)(capi.GemvDesc(dW[0].ptr, dX[0].ptr, outs[0].ptr, 4, 100))
    assert lib.bpd_qmatmul_q4k_q8k_batch_static_cuda(1, bad, None) == -1
    lib.bpdq_clear_status()


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

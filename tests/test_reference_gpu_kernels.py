"""The reference's own CUDA kernels (bench/bpd_quant_gpu.cu: k_dequant_q4k, k_qmatmul_q4k), compiled unmodified for
sm_100a, beside this library's drop-ins for the same two entry points on the same device buffers: results compared
(dequantization bit for bit, the fp32-activation GEMV norm-wise) and both timed with CUDA events on the legacy
default stream, which is where the reference launches.  The timings are printed as one JSON line (run with -s)."""
import json

import numpy as np
import pytest

from bpd_substrate_b200 import synth
from oracle import binding
from tests.util import Dev, assert_bits_equal, normwise

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not binding.ref_available("bpd_quant_gpu.so"), reason="compiled reference GPU library not present")]


def _time(lib, fn, iters=20):
    e0, e1 = lib.bpdq_event_create(), lib.bpdq_event_create()
    for _ in range(3):
        fn()
    lib.bpdq_sync()
    lib.bpdq_event_record(e0, None)
    for _ in range(iters):
        fn()
    lib.bpdq_event_record(e1, None)
    us = lib.bpdq_event_elapsed_ms(e0, e1) / iters * 1e3
    lib.bpdq_event_destroy(e0)
    lib.bpdq_event_destroy(e1)
    return us


def test_reference_gpu_kernels_beside_the_drop_ins(lib, oracle):
    ref = binding.load_ref("bpd_quant_gpu.so")
    N, K = 14336, 4096
    nb = N * (K // 256)
    W = synth.q4k_matrix(N, K, 1000)
    x = synth.activations(K, 1005)
    # 19 copies of the weights (627 MB, beyond L2) so that no launch finds its input cached
    copies = [Dev(lib, W) for _ in range(19)]
    dx = Dev(lib, x)
    out_ref, out_mine = Dev(lib, nbytes=nb * 1024, fill=0xFF), Dev(lib, nbytes=nb * 1024, fill=0xEE)
    y_ref, y_mine = Dev(lib, nbytes=N * 4, fill=0xFF), Dev(lib, nbytes=N * 4, fill=0xEE)
    prev = lib.bpdq_get_stream()
    lib.bpdq_set_stream(None)
    try:
        ref.bpd_dequant_q4k_gpu(copies[0].ptr, out_ref.ptr, nb)
        lib.bpd_dequant_q4k_gpu(copies[0].ptr, out_mine.ptr, nb)
        ref.bpd_qmatmul_q4k_gpu(copies[0].ptr, dx.ptr, y_ref.ptr, N, K)
        lib.bpd_qmatmul_q4k_gpu(copies[0].ptr, dx.ptr, y_mine.ptr, N, K)
        lib.bpdq_sync()
        assert lib.bpdq_last_status() == 0
        assert_bits_equal(out_mine.read(np.float32), out_ref.read(np.float32))
        a, b = y_mine.read(np.float32), y_ref.read(np.float32)
        exact = oracle.qmatmul_q4k_f64(W, x, N, K)
        assert normwise(a, b) <= 1e-5
        assert normwise(a, exact) <= 1e-5 and normwise(b, exact) <= 1e-5
        i = [0]

        def rot():
            i[0] += 1
            return copies[i[0] % len(copies)].ptr

        t = {
            "reference k_dequant_q4k us": _time(lib, lambda: ref.bpd_dequant_q4k_gpu(rot(), out_ref.ptr, nb)),
            "this library's dequant us": _time(lib, lambda: lib.bpd_dequant_q4k_gpu(rot(), out_mine.ptr, nb)),
            "reference k_qmatmul_q4k us": _time(lib, lambda: ref.bpd_qmatmul_q4k_gpu(rot(), dx.ptr, y_ref.ptr, N, K)),
            "this library's W4A32 GEMV us": _time(lib, lambda: lib.bpd_qmatmul_q4k_gpu(rot(), dx.ptr, y_mine.ptr, N, K)),
        }
        print("\nREFERENCE_GPU_BASELINE " + json.dumps({"shape": [N, K], **{k: round(v, 2) for k, v in t.items()},
                                                        "gemv_norm_err_mine": normwise(a, exact), "gemv_norm_err_reference": normwise(b, exact)}))
    finally:
        lib.bpdq_set_stream(prev)

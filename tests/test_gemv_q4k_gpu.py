"""Q4_K x Q8_K GEMV / small-batch GEMM against the CPU checker, through the C ABI."""
import numpy as np
import pytest

from bpd_substrate_b200 import synth
from tests.util import Dev, normwise

pytestmark = pytest.mark.gpu

TOL = 1e-5  # norm-wise max|d|/max|ref| on the fp32 outputs (the stated bar for GEMV outputs)


def run_gemm(lib, W, X, tokens, M, K, layout=0, xsrc=0, want_dots=False):
    dW, dX = Dev(lib, W), Dev(lib, X)
    dO = Dev(lib, nbytes=tokens * M * 4, fill=0xFF)
    dD = Dev(lib, nbytes=M * (K // 256) * 8 * 4, fill=0xEE) if want_dots else None
    rc = lib.bpd_qmm_q4k_q8k_cuda(dW.ptr, dX.ptr, dO.ptr, tokens, M, K, layout, xsrc,
                                  dD.ptr if dD else None, None)
    assert rc == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    out = dO.read(np.float32).reshape(tokens, M)
    dots = dD.read(np.int32).reshape(M, K // 256, 8) if dD else None
    return out, dots


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("M,K", [(1, 256), (5, 512), (64, 4096), (37, 4096), (24, 14336), (16, 8192),
                                 (9, 28672), (300, 1024), (2, 40960)])
def test_gemv_matches_checker(lib, oracle, M, K, layout):
    rng = np.random.default_rng(100 + M + K)
    W = synth.q4k_matrix(M, K, rng)
    x = synth.activations(K, rng)
    out, dots = run_gemm(lib, W, x, 1, M, K, layout, want_dots=True)
    xq = oracle.quant_q8_K(x)
    ref32, ref64 = oracle.qmatmul_q4k_q8k(W, xq, M, K, layout)
    # integer sub-block dots: bit-exact
    assert np.array_equal(dots, oracle.q4k_q8k_subdots(W, xq, M, K, layout))
    assert normwise(out[0], ref64) <= TOL
    assert normwise(out[0], ref32) <= TOL


@pytest.mark.parametrize("tokens", [2, 3, 4, 7])
def test_small_batch(lib, oracle, tokens):
    M, K = 48, 4096
    rng = np.random.default_rng(7 + tokens)
    W = synth.q4k_matrix(M, K, rng)
    X = synth.activations(K, rng, rows=tokens)
    out, _ = run_gemm(lib, W, X, tokens, M, K)
    ref32, ref64 = oracle.qmm_q4k_q8k(W, X, tokens, M, K)
    assert normwise(out, ref64) <= TOL


def test_prequantized_activations_give_identical_bits(lib, oracle):
    M, K = 40, 4096
    rng = np.random.default_rng(5)
    W = synth.q4k_matrix(M, K, rng)
    x = synth.activations(K, rng)
    out_f, _ = run_gemm(lib, W, x, 1, M, K)
    out_q, _ = run_gemm(lib, W, oracle.quant_q8_K(x), 1, M, K, xsrc=1)
    assert np.array_equal(out_f.view(np.uint32), out_q.view(np.uint32))


def test_quantizer_q8_K_bytes(lib, oracle):
    rng = np.random.default_rng(11)
    x = synth.activations(256 * 37, rng)
    x[256:512] = 0.0            # an all-zero block: scale 0, quants 0
    x[1000] = 1e-30
    dX = Dev(lib, x)
    dY = Dev(lib, nbytes=37 * 292, fill=0xAA)
    assert lib.bpd_quant_q8_K_cuda(dX.ptr, dY.ptr, x.size, None) == 0
    lib.bpdq_sync()
    assert np.array_equal(dY.read(np.uint8), oracle.quant_q8_K(x))


def test_bad_arguments_are_rejected(lib):
    d = Dev(lib, nbytes=4096)
    assert lib.bpd_qmatmul_q4k_q8k_cuda(d.ptr, d.ptr, d.ptr, 4, 100, None) == -1   # K not a multiple of 256
    assert lib.bpd_qmatmul_q4k_q8k_cuda(d.ptr + 4, d.ptr, d.ptr, 4, 256, None) == -2  # misaligned weights
    assert lib.bpd_qmatmul_q4k_q8k_cuda(None, d.ptr, d.ptr, 4, 256, None) == -1
    lib.bpdq_clear_status()


def test_grouped_matrices_share_one_launch(lib, oracle):
    """q/k/v-style grouping: three matrices, one activation vector, one launch; every output
    equals the single-matrix launch bit for bit."""
    import ctypes as C
    K = 4096
    Ms = [96, 24, 37]
    rng = np.random.default_rng(21)
    Ws = [synth.q4k_matrix(m, K, rng) for m in Ms]
    x = synth.activations(K, rng)
    dWs = [Dev(lib, w) for w in Ws]
    dOs = [Dev(lib, nbytes=m * 4, fill=0xFF) for m in Ms]
    dX = Dev(lib, x)
    wp = (C.c_void_p * 3)(*[d.ptr for d in dWs])
    op = (C.c_void_p * 3)(*[d.ptr for d in dOs])
    mp = (C.c_int * 3)(*Ms)
    assert lib.bpd_qmatmul_q4k_q8k_multi_cuda(3, wp, op, mp, dX.ptr, K, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    xq = oracle.quant_q8_K(x)
    for W, m, dO in zip(Ws, Ms, dOs):
        single, _ = run_gemm(lib, W, x, 1, m, K)
        got = dO.read(np.float32)
        assert np.array_equal(got.view(np.uint32), single[0].view(np.uint32))
        assert normwise(got, oracle.qmatmul_q4k_q8k(W, xq, m, K)[1]) <= TOL


def test_many_launches_leave_scheduler_clean(lib, oracle):
    """The tile-scheduler words are reused round robin; 200 launches in a row stay correct."""
    M, K = 333, 4096
    rng = np.random.default_rng(77)
    W = synth.q4k_matrix(M, K, rng)
    x = synth.activations(K, rng)
    dW, dX, dO = Dev(lib, W), Dev(lib, x), Dev(lib, nbytes=M * 4, fill=0xFF)
    first = None
    for i in range(200):
        assert lib.bpd_qmatmul_q4k_q8k_cuda(dW.ptr, dX.ptr, dO.ptr, M, K, None) == 0
        if i in (0, 63, 64, 199):
            lib.bpdq_sync()
            got = dO.read(np.float32)
            first = got if first is None else first
            assert np.array_equal(got.view(np.uint32), first.view(np.uint32))
    assert lib.bpdq_last_status() == 0
    assert normwise(first, oracle.qmatmul_q4k_q8k(W, oracle.quant_q8_K(x), M, K)[1]) <= TOL


def test_batched_independent_products(lib, oracle):
    """Seven products of different shapes, each with its own vector (two share one), in one call."""
    import ctypes as C
    from bpd_substrate_b200 import capi
    shapes = [(40, 4096), (9, 4096), (9, 4096), (33, 4096), (70, 4096), (70, 4096), (21, 14336), (5, 256), (3, 28672)]
    rng = np.random.default_rng(91)
    Ws = [synth.q4k_matrix(m, k, rng) for m, k in shapes]
    xs = [synth.activations(k, rng) for _, k in shapes]
    dWs, dXs = [Dev(lib, w) for w in Ws], [Dev(lib, x) for x in xs]
    dOs = [Dev(lib, nbytes=m * 4, fill=0xFF) for m, _ in shapes]
    share = {2: 1}                      # product 2 reads product 1's vector
    descs = (capi.GemvDesc * len(shapes))()
    for j, (m, k) in enumerate(shapes):
        descs[j] = capi.GemvDesc(dWs[j].ptr, dXs[share.get(j, j)].ptr, dOs[j].ptr, m, k)
    assert lib.bpd_qmatmul_q4k_q8k_batch_cuda(len(shapes), descs, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    first = []
    for j, (m, k) in enumerate(shapes):
        x = xs[share.get(j, j)]
        _, ref64 = oracle.qmatmul_q4k_q8k(Ws[j], oracle.quant_q8_K(x), m, k)
        got = dOs[j].read(np.float32)
        first.append(got)
        assert normwise(got, ref64) <= TOL, (j, m, k)
    # with caller-owned scratch (activations quantized once by a separate kernel): same bits
    ws_bytes = lib.bpdq_batch_workspace_bytes(len(shapes), descs)
    ws = Dev(lib, nbytes=ws_bytes, fill=0xCD)
    for d in dOs:
        lib.bpdq_memset_async(d.ptr, 0xFF, d.nbytes, None)
    assert lib.bpd_qmatmul_q4k_q8k_batch_ws_cuda(len(shapes), descs, ws.ptr, ws_bytes, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    for j in range(len(shapes)):
        assert np.array_equal(dOs[j].read(np.float32).view(np.uint32), first[j].view(np.uint32)), j


def test_batched_rejects_bad_descriptors(lib):
    from bpd_substrate_b200 import capi
    d = Dev(lib, nbytes=4096)
    descs = (capi.GemvDesc * 1)(capi.GemvDesc(d.ptr, d.ptr, d.ptr, 4, 100))
    assert lib.bpd_qmatmul_q4k_q8k_batch_cuda(1, descs, None) == -1
    descs = (capi.GemvDesc * 1)(capi.GemvDesc(d.ptr + 8, d.ptr, d.ptr, 4, 256))
    assert lib.bpd_qmatmul_q4k_q8k_batch_cuda(1, descs, None) == -2
    lib.bpdq_clear_status()


def test_stream_of_products_equals_batched_entries(lib):
    """bpdq_gemv_stream_*: 19 products of mixed shapes (several phases, some sharing a vector) in one
    persistent launch give the bits of the batched entry, run after run."""
    from bpd_substrate_b200 import capi
    rng = np.random.default_rng(77)
    shapes = [(96, 4096), (40, 4096), (40, 4096), (130, 2048), (64, 14336), (7, 256), (300, 4096), (33, 14336),
              (512, 1024), (96, 4096), (18, 8192), (200, 4096), (1, 256), (64, 14336), (128, 4096), (90, 512),
              (256, 4096), (31, 14336), (77, 4096)]
    Ws = [Dev(lib, synth.q4k_matrix(m, k, rng)) for m, k in shapes]
    xs = {}
    for j, (m, k) in enumerate(shapes):
        if j in (1, 2):           # two products on one vector
            xs[j] = xs.setdefault(1, Dev(lib, synth.activations(k, rng)))
        else:
            xs[j] = Dev(lib, synth.activations(k, rng))
    n = len(shapes)

    def run(entry):
        outs = [Dev(lib, nbytes=m * 4, fill=0xFF) for m, _ in shapes]
        descs = (capi.GemvDesc * n)(*[capi.GemvDesc(Ws[j].ptr, xs[j].ptr, outs[j].ptr, m, k) for j, (m, k) in enumerate(shapes)])
        ws_bytes = lib.bpdq_batch_workspace_bytes(n, descs)
        ws = Dev(lib, nbytes=ws_bytes)
        if entry in ("stream", "stream-ready"):
            h = lib.bpdq_gemv_stream_create(n, descs, ws.ptr, ws_bytes)
            assert h and lib.bpdq_gemv_stream_launches(h) == 2
            for _ in range(3):
                assert (lib.bpdq_gemv_stream_run if entry == "stream" else lib.bpdq_gemv_stream_run_ready)(h, None) == 0
            lib.bpdq_sync()
            lib.bpdq_gemv_stream_destroy(h)
        else:
            assert lib.bpd_qmatmul_q4k_q8k_batch_ws_cuda(n, descs, ws.ptr, ws_bytes, None) == 0
            lib.bpdq_sync()
        assert lib.bpdq_last_status() == 0
        return [o.read(np.uint32) for o in outs]

    a, b, c = run("batch"), run("stream"), run("stream-ready")
    for j in range(n):
        assert np.array_equal(a[j], b[j]), j
        assert np.array_equal(a[j], c[j]), j
    assert not lib.bpdq_gemv_stream_create(0, None, None, 0)
    lib.bpdq_clear_status()


def test_layer_set_schedules_and_host_step_agree(lib, oracle):
    """The dispatch host layer on a small layer set: every schedule writes the same outputs, they
    match the checker, and a step from host buffers (copies pipelined with the GEMVs over three
    streams) returns them unchanged."""
    from bpd_substrate_b200.dispatch import LayerSet
    shapes = (("wq", 256, 512), ("wk", 64, 512), ("wv", 64, 512), ("wo", 256, 512), ("w1", 384, 512), ("w3", 384, 512),
              ("w2", 256, 1536))
    ls = LayerSet(shapes, n_layers=5, seed=31, lib=lib)
    try:
        rng = np.random.default_rng(4)
        x_all = rng.standard_normal(ls.x_bytes // 4, dtype=np.float32)
        ls.upload_activations(x_all)
        results = {}
        for schedule in ("separate", "grouped", "batched", "persistent"):
            lib.bpdq_memset_async(ls.d_out, 0xFF, ls.o_bytes, ls.stream)
            ls.step(schedule)
            results[schedule] = ls.download_outputs()
        # grouped launches share the first member's activation vector: compare the members that read their own
        for layer in range(ls.n_layers):
            for m, (_, rows, cols) in enumerate(shapes):
                want = oracle.qmatmul_q4k_q8k(ls.host_weight(layer, m), oracle.quant_q8_K(ls.activation_slice(x_all, layer, m)),
                                              rows, cols)[1]
                for schedule in ("separate", "batched", "persistent"):
                    assert normwise(ls.output_slice(results[schedule], layer, m), want) <= 1e-5, (schedule, layer, m)
        assert np.array_equal(results["batched"].view(np.uint32), results["persistent"].view(np.uint32))
        # host step: pinned buffers, three streams
        x_host, o_host = lib.bpdq_host_alloc(ls.x_bytes), lib.bpdq_host_alloc(ls.o_bytes)
        import ctypes as C
        C.memmove(x_host, x_all.ctypes.data, ls.x_bytes)
        for chunks in (1, 3, 5):
            C.memset(o_host, 0xFF, ls.o_bytes)
            ls.step_host(x_host, o_host, "batched", chunks=chunks)
            got = np.frombuffer((C.c_char * ls.o_bytes).from_address(o_host), np.uint32).copy()
            assert np.array_equal(got, results["batched"].view(np.uint32)), chunks
        lib.bpdq_host_free(x_host)
        lib.bpdq_host_free(o_host)
        assert lib.bpdq_last_status() == 0
    finally:
        ls.close()


def test_product_chained_behind_its_producer_with_programmatic_launch(lib, oracle):
    """The activation vector of a batched product is the OUTPUT of the launch just ahead of it (itself a
    product kernel, which lets its dependents start early).  The stream-ordered entries (_ws and the
    allocation-free one) must read the finished vector: same bits with programmatic launch on and off,
    and equal to the checker fed the first product's output."""
    from bpd_substrate_b200 import capi
    K0, K1, M = 2048, 4096, 300
    rng = np.random.default_rng(55)
    W0, W1 = synth.q4k_matrix(K1, K0, rng), synth.q4k_matrix(M, K1, rng)
    x0 = synth.activations(K0, rng)
    dW0, dW1, dx0 = Dev(lib, W0), Dev(lib, W1), Dev(lib, x0)
    results = {}
    for pdl in (1, 0):
        lib.bpdq_set_tuning(0, 0, 0, 0, pdl)
        for entry in ("ws", "static"):
            mid = Dev(lib, nbytes=K1 * 4, fill=0xFF)      # poisoned: a stale read shows
            out = Dev(lib, nbytes=M * 4, fill=0xFF)
            d0 = (capi.GemvDesc * 1)(capi.GemvDesc(dW0.ptr, dx0.ptr, mid.ptr, K1, K0))
            d1 = (capi.GemvDesc * 1)(capi.GemvDesc(dW1.ptr, mid.ptr, out.ptr, M, K1))
            nbytes = lib.bpdq_batch_workspace_bytes(1, d0) + lib.bpdq_batch_workspace_bytes(1, d1)
            ws = Dev(lib, nbytes=nbytes)
            for rep in range(20):                           # back to back: the overlap window is open every time
                assert lib.bpd_qmatmul_q4k_q8k_batch_ws_cuda(1, d0, ws.ptr, nbytes, None) == 0
                if entry == "ws":
                    assert lib.bpd_qmatmul_q4k_q8k_batch_ws_cuda(1, d1, ws.ptr, nbytes, None) == 0
                else:
                    assert lib.bpd_qmatmul_q4k_q8k_batch_static_cuda(1, d1, None) == 0
            lib.bpdq_sync()
            assert lib.bpdq_last_status() == 0
            results[(pdl, entry)] = (mid.read(np.float32), out.read(np.float32))
    lib.bpdq_set_tuning(0, 0, 0, 0, 1)
    mid_ref, out_ref = results[(0, "ws")]
    for key, (mid, out) in results.items():
        assert np.array_equal(mid.view(np.uint32), mid_ref.view(np.uint32)), key
        assert np.array_equal(out.view(np.uint32), out_ref.view(np.uint32)), key
    _, want = oracle.qmatmul_q4k_q8k(W1, oracle.quant_q8_K(mid_ref), M, K1)
    assert normwise(out_ref, want) <= TOL


def test_long_stream_many_phases_and_two_launches(lib, oracle):
    """150 products (two persistent launches of 75) whose activation records fill the two shared-memory record
    buffers many times over: every consumer warp passes through every phase, with and without tiles of its own
    (several products have fewer tiles than there are warps).  Checked against the CPU checker product by product."""
    from bpd_substrate_b200 import capi
    rng = np.random.default_rng(314)
    kinds = [(700, 4096), (40, 4096), (3, 14336), (260, 1024), (1, 256), (90, 8192), (33, 28672)]
    base = {kk: synth.q4k_matrix(m, k, rng) for kk, (m, k) in enumerate(kinds)}
    shapes, Ws, xs = [], [], []
    for j in range(150):
        kk = j % len(kinds)
        shapes.append(kinds[kk])
        Ws.append(np.roll(base[kk], 144 * (j // len(kinds) + 1)))
        xs.append(synth.activations(kinds[kk][1], rng))
    dW, dX = [Dev(lib, w) for w in Ws], [Dev(lib, x) for x in xs]
    outs = [Dev(lib, nbytes=m * 4, fill=0xFF) for m, _ in shapes]
    n = len(shapes)
    descs = (capi.GemvDesc * n)(*[capi.GemvDesc(dW[j].ptr, dX[j].ptr, outs[j].ptr, m, k) for j, (m, k) in enumerate(shapes)])
    ws_bytes = lib.bpdq_batch_workspace_bytes(n, descs)
    ws = Dev(lib, nbytes=ws_bytes, fill=0xCD)
    h = lib.bpdq_gemv_stream_create(n, descs, ws.ptr, ws_bytes)
    assert h and lib.bpdq_gemv_stream_launches(h) == 4
    first = None
    for rep in range(3):
        assert lib.bpdq_gemv_stream_run_ready(h, None) == 0
        lib.bpdq_sync()
        assert lib.bpdq_last_status() == 0
        got = [o.read(np.float32) for o in outs]
        if first is None:
            first = got
            for j, (m, k) in enumerate(shapes):
                _, ref64 = oracle.qmatmul_q4k_q8k(Ws[j], oracle.quant_q8_K(xs[j]), m, k)
                assert normwise(got[j], ref64) <= TOL, (j, m, k)
        else:
            for j in range(n):
                assert np.array_equal(got[j].view(np.uint32), first[j].view(np.uint32)), (rep, j)
        for o in outs:
            lib.bpdq_memset_async(o.ptr, 0xFF, o.nbytes, None)
    lib.bpdq_gemv_stream_destroy(h)
    # rows of K = 28672 arrive in two pieces per ring turn: still the bits of the batched entry
    for j in (6, 13):
        m, k = shapes[j]
        o = Dev(lib, nbytes=m * 4, fill=0xFF)
        one = (capi.GemvDesc * 1)(capi.GemvDesc(dW[j].ptr, dX[j].ptr, o.ptr, m, k))
        assert lib.bpd_qmatmul_q4k_q8k_batch_cuda(1, one, None) == 0
        lib.bpdq_sync()
        assert np.array_equal(o.read(np.uint32), first[j].view(np.uint32)), j
    # too small a workspace is refused
    assert not lib.bpdq_gemv_stream_create(n, descs, ws.ptr, 1024)
    lib.bpdq_clear_status()


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5])
def test_stream_of_random_shapes(lib, oracle, seed):
    """Seeded random launches of the persistent kernel: 1-40 products, 1-600 rows, 1-65 super-blocks per row
    (65 = rows that arrive in two pieces), some products sharing a vector.  Every output against the CPU checker,
    and the launch repeated gives the same bits."""
    from bpd_substrate_b200 import capi
    rng = np.random.default_rng(1000 + seed)
    n = int(rng.integers(1, 41))
    ks = [256, 512, 1024, 2048, 4096, 8192, 14336, 65 * 256]
    shapes = [(int(rng.integers(1, 601)), int(ks[rng.integers(0, len(ks))])) for _ in range(n)]
    hW = [synth.q4k_matrix(m, k, rng) for m, k in shapes]
    hx, dx = [], []
    for j, (m, k) in enumerate(shapes):
        share = [i for i in range(j) if shapes[i][1] == k]
        if share and rng.random() < 0.3:
            i = share[0]
            hx.append(hx[i])
            dx.append(dx[i])
        else:
            hx.append(synth.activations(k, rng))
            dx.append(Dev(lib, hx[-1]))
    dW = [Dev(lib, w) for w in hW]
    outs = [Dev(lib, nbytes=m * 4, fill=0xFF) for m, _ in shapes]
    descs = (capi.GemvDesc * n)(*[capi.GemvDesc(dW[j].ptr, dx[j].ptr, outs[j].ptr, m, k) for j, (m, k) in enumerate(shapes)])
    ws_bytes = lib.bpdq_batch_workspace_bytes(n, descs)
    ws = Dev(lib, nbytes=ws_bytes, fill=0xAB)
    h = lib.bpdq_gemv_stream_create(n, descs, ws.ptr, ws_bytes)
    assert h
    assert lib.bpdq_gemv_stream_run(h, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    first = [o.read(np.float32) for o in outs]
    for j, (m, k) in enumerate(shapes):
        _, ref64 = oracle.qmatmul_q4k_q8k(hW[j], oracle.quant_q8_K(hx[j]), m, k)
        assert normwise(first[j], ref64) <= TOL, (seed, j, m, k)
    for o in outs:
        lib.bpdq_memset_async(o.ptr, 0xFF, o.nbytes, None)
    assert lib.bpdq_gemv_stream_run(h, None) == 0
    lib.bpdq_sync()
    for j in range(n):
        assert np.array_equal(outs[j].read(np.uint32), first[j].view(np.uint32)), (seed, j)
    lib.bpdq_gemv_stream_destroy(h)

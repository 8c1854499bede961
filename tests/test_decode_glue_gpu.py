"""Decode glue: record producers fused with rms_norm / SwiGLU, products over records with the
residual add as their epilogue, and the dependent per-layer chain built from them.

Each fused step must give the same bits as the separate calls it replaces (whose arithmetic is
checked against the CPU checker elsewhere); the records themselves are checked against the
checker's Q8_K quantizer, integer for integer."""
import numpy as np
import pytest

from bpd_substrate_b200 import capi, synth
from bpd_substrate_b200.dispatch import DecodeChain
from tests.util import Dev, normwise

pytestmark = pytest.mark.gpu


def decode_records(raw, K):
    """records -> (int8 [K], int sums of 32 [K/32], fp32 scale per 256 [K/256])."""
    rec = np.asarray(raw, np.uint8)[: K // 128 * 144].reshape(K // 128, 144)
    q = rec[:, :128].copy().view(np.int8).reshape(K)
    sums = rec[:, 128:136].copy().view(np.int16).reshape(K // 32).astype(np.int64)
    d = rec[:, 136:140].copy().view(np.float32).reshape(K // 128)
    assert np.array_equal(d[0::2].view(np.uint32), d[1::2].view(np.uint32))   # both halves carry the block scale
    return q, sums, d[0::2]


def decode_q8k(blocks, K):
    """the checker's 292-byte blocks -> the same triple."""
    b = np.asarray(blocks, np.uint8).reshape(K // 256, 292)
    d = b[:, :4].copy().view(np.float32).reshape(K // 256)
    q = b[:, 4:260].copy().view(np.int8).reshape(K)
    bs = b[:, 260:292].copy().view(np.int16).reshape(K // 16).astype(np.int64)
    return q, bs[0::2] + bs[1::2], d


def records_of(lib, x):
    K = x.size
    dX, dR = Dev(lib, x), Dev(lib, nbytes=lib.bpdq_records_bytes(K), fill=0xEE)
    assert lib.bpd_quant_q8k_records_cuda(dX.ptr, dR.ptr, K, None) == 0
    lib.bpdq_sync()
    return dR.read(np.uint8)


@pytest.mark.parametrize("K", [256, 4096, 14336])
def test_records_match_checker_quantizer(lib, oracle, K):
    rng = np.random.default_rng(K)
    x = rng.standard_normal(K, dtype=np.float32) * 3
    if K > 256:
        x[K // 2: K // 2 + 256] = 0.0      # an all-zero block: scale 0, multiplier 0
    assert lib.bpdq_records_bytes(K) == K // 128 * 144
    q, sums, d = decode_records(records_of(lib, x), K)
    q_ref, sums_ref, d_ref = decode_q8k(oracle.quant_q8_K(x), K)
    assert np.array_equal(q, q_ref)
    assert np.array_equal(sums, sums_ref)
    assert np.array_equal(d.view(np.uint32), d_ref.view(np.uint32))


@pytest.mark.parametrize("rows,K", [(1, 4096), (3, 512), (2, 14336)])
def test_rmsnorm_records_equal_separate_calls(lib, rows, K):
    rng = np.random.default_rng(rows * K)
    x = rng.standard_normal((rows, K), dtype=np.float32) * 5
    w = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    dX, dW, dH = Dev(lib, x), Dev(lib, w), Dev(lib, nbytes=rows * K * 4)
    rb = lib.bpdq_records_bytes(K)
    dR = Dev(lib, nbytes=rows * rb, fill=0xEE)
    assert lib.bpd_rmsnorm_q8k_records_cuda(dX.ptr, dW.ptr, dR.ptr, rows, K, 1e-5, None) == 0
    lib.gpu_rms_norm(dX.ptr, dW.ptr, dH.ptr, rows, K, 1e-5)
    lib.bpdq_sync()
    h = dH.read(np.float32).reshape(rows, K)
    fused = dR.read(np.uint8).reshape(rows, rb)
    for r in range(rows):
        assert np.array_equal(fused[r], records_of(lib, h[r])), r


def test_swiglu_records_equal_separate_calls(lib):
    K = 14336
    rng = np.random.default_rng(77)
    g = rng.standard_normal(K, dtype=np.float32) * 6
    g[:8] = [-200.0, 200.0, -90.0, 90.0, 0.0, -0.0, 1e-30, -1e-30]     # exp overflow/underflow ends
    u = rng.standard_normal(K, dtype=np.float32) * 2
    dG, dU, dT = Dev(lib, g), Dev(lib, u), Dev(lib, nbytes=K * 4)
    dR = Dev(lib, nbytes=lib.bpdq_records_bytes(K), fill=0xEE)
    assert lib.bpd_swiglu_q8k_records_cuda(dG.ptr, dU.ptr, dR.ptr, K, None) == 0
    lib.gpu_silu(dG.ptr, dT.ptr, K)
    lib.gpu_mul(dT.ptr, dU.ptr, dT.ptr, K)
    lib.bpdq_sync()
    assert np.array_equal(dR.read(np.uint8), records_of(lib, dT.read(np.float32)))


def test_products_over_records_and_residual_epilogue(lib, oracle):
    K = 2048
    shapes = [(96, K), (40, K), (130, K)]
    rng = np.random.default_rng(31)
    x = rng.standard_normal(K, dtype=np.float32)
    Ws = [synth.q4k_matrix(m, k, rng) for m, k in shapes]
    prev = [rng.standard_normal(m, dtype=np.float32) * 100 for m, _ in shapes]
    dX, dWs = Dev(lib, x), [Dev(lib, w) for w in Ws]
    dR = Dev(lib, nbytes=lib.bpdq_records_bytes(K))
    assert lib.bpd_quant_q8k_records_cuda(dX.ptr, dR.ptr, K, None) == 0
    # the separate path: each product through the batched entry (its own quantizer launch)
    plain = []
    ws = Dev(lib, nbytes=lib.bpdq_records_bytes(K) + 4096)
    for (m, k), dW in zip(shapes, dWs):
        dO = Dev(lib, nbytes=m * 4, fill=0xFF)
        d = (capi.GemvDesc * 1)(capi.GemvDesc(dW.ptr, dX.ptr, dO.ptr, m, k))
        assert lib.bpd_qmatmul_q4k_q8k_batch_ws_cuda(1, d, ws.ptr, ws.nbytes, None) == 0
        lib.bpdq_sync()
        plain.append(dO.read(np.float32))
    xq = oracle.quant_q8_K(x)
    for (m, k), W, got in zip(shapes, Ws, plain):
        _, ref64 = oracle.qmatmul_q4k_q8k(W, xq, m, k)
        assert normwise(got, ref64) <= 1e-5
    # one launch over the records: overwrite, accumulate, overwrite
    outs = [Dev(lib, p) for p in prev]
    descs = (capi.GemvDesc * 3)(*[capi.GemvDesc(dW.ptr, None, o.ptr, m, k) for (m, k), dW, o in zip(shapes, dWs, outs)])
    assert lib.bpd_qmatmul_q4k_records_cuda(3, descs, dR.ptr, 0b010, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    for j, (o, p, pl) in enumerate(zip(outs, prev, plain)):
        want = p + pl if j == 1 else pl
        assert np.array_equal(o.read(np.float32).view(np.uint32), want.astype(np.float32).view(np.uint32)), j


def test_products_over_records_reject_bad_calls(lib):
    d = Dev(lib, nbytes=1 << 16)
    descs = (capi.GemvDesc * 2)(capi.GemvDesc(d.ptr, None, d.ptr, 8, 256), capi.GemvDesc(d.ptr, None, d.ptr, 8, 512))
    assert lib.bpd_qmatmul_q4k_records_cuda(2, descs, d.ptr, 0, None) == -1      # different K
    assert lib.bpd_qmatmul_q4k_records_cuda(0, descs, d.ptr, 0, None) == -1
    assert lib.bpd_qmatmul_q4k_records_cuda(1, descs, None, 0, None) == -1
    assert lib.bpd_quant_q8k_records_cuda(d.ptr, d.ptr, 100, None) == -1
    assert lib.bpd_swiglu_q8k_records_cuda(d.ptr, d.ptr + 4, d.ptr, 256, None) == -2
    lib.bpdq_clear_status()


@pytest.fixture(scope="module")
def chain(lib):
    c = DecodeChain(hidden=512, kv=256, ffn=1024, n_layers=3, seed=11, lib=lib)
    yield c
    c.close()


def test_chain_fused_equals_reference_call_sequence(chain):
    """4 and 8 launches per layer against the reference's 13-call sequence on the same weights: same
    bits, directly enqueued and replayed from a CUDA graph."""
    rng = np.random.default_rng(5)
    x0 = rng.standard_normal(chain.hidden, dtype=np.float32)
    results = []
    for mode in ("chain-separate", "chain4", "chain", "chain-persistent", "chain-graph", "chain-persistent", "persistent-graph"):
        chain.set_state(x0)
        if mode.endswith("-graph"):
            which = "chain" if mode == "chain-graph" else "chain-persistent"
            chain.capture(which)         # (the capture's warm-up runs advance the state: reset it)
            chain.set_state(x0)
            chain.step(which)
        else:
            chain.enqueue_token(mode)
        results.append(chain.get_state())
        assert chain.lib.bpdq_last_status() == 0
    assert np.isfinite(results[0]).all()
    for other in results[1:]:
        assert np.array_equal(results[0].view(np.uint32), other.view(np.uint32))
    assert [chain.launches_per_token(m) for m in ("chain", "chain4", "chain-separate")] == [24, 12, 39]


def test_chain_wide_rows(lib):
    """Rows of 32 super-blocks: the product kernels take two rows per tile, and the one-launch program pairs ONE
    row of the gate matrix with the same row of the up matrix per tile.  Same bits as the 13-call sequence."""
    c = DecodeChain(hidden=8192, kv=256, ffn=1024, n_layers=2, seed=12, lib=lib)
    try:
        x0 = np.random.default_rng(6).standard_normal(c.hidden, dtype=np.float32)
        results = []
        for mode in ("chain-separate", "chain", "chain-persistent", "chain-persistent"):
            c.set_state(x0)
            c.enqueue_token(mode)
            results.append(c.get_state())
            assert lib.bpdq_last_status() == 0
        assert np.isfinite(results[0]).all()
        for other in results[1:]:
            assert np.array_equal(results[0].view(np.uint32), other.view(np.uint32))
    finally:
        c.close()


@pytest.mark.parametrize("tile_bytes,stages,warps", [(4096, 2, 4), (8192, 3, 8), (9216, 4, 6), (2048, 2, 16), (9216, 2, 11)])
def test_ring_geometries_give_the_same_bits(lib, tile_bytes, stages, warps):
    """Other tile sizes, ring depths and warp counts (bpdq_set_tuning) change how often a warp's ring wraps and which
    warp folds which rows, not the results: the dependent chain in its launch-per-step, fused and one-launch forms and
    a stream of independent products give the bits of the default geometry."""
    rng = np.random.default_rng(21)
    c = DecodeChain(hidden=1024, kv=256, ffn=2816, n_layers=2, seed=13, lib=lib)
    shapes = [(300, 1024), (64, 4096), (1, 256), (130, 2816), (77, 4096)]
    Ws = [Dev(lib, synth.q4k_matrix(m, k, rng)) for m, k in shapes]
    xs = [Dev(lib, synth.activations(k, rng)) for _, k in shapes]
    x0 = rng.standard_normal(c.hidden, dtype=np.float32)

    def run_all():
        got = []
        for mode in ("chain", "chain4", "chain-persistent"):
            if c.program:
                lib.bpdq_chain_destroy(c.program)
                c.program = None
            c.set_state(x0)
            c.enqueue_token(mode)
            got.append(c.get_state().view(np.uint32))
        outs = [Dev(lib, nbytes=m * 4, fill=0xFF) for m, _ in shapes]
        n = len(shapes)
        descs = (capi.GemvDesc * n)(*[capi.GemvDesc(Ws[j].ptr, xs[j].ptr, outs[j].ptr, m, k) for j, (m, k) in enumerate(shapes)])
        ws_bytes = lib.bpdq_batch_workspace_bytes(n, descs)
        ws = Dev(lib, nbytes=ws_bytes)
        h = lib.bpdq_gemv_stream_create(n, descs, ws.ptr, ws_bytes)
        assert h
        assert lib.bpdq_gemv_stream_run(h, None) == 0
        lib.bpdq_sync()
        lib.bpdq_gemv_stream_destroy(h)
        got += [o.read(np.uint32) for o in outs]
        assert lib.bpdq_last_status() == 0
        return got

    try:
        want = run_all()
        for other in want[1:3]:
            assert np.array_equal(want[0], other)
        lib.bpdq_set_tuning(tile_bytes, stages, 0, warps, -1)
        got = run_all()
        for a, b in zip(want, got):
            assert np.array_equal(a, b)
    finally:
        lib.bpdq_set_tuning(8192, 2, 0, 16, -1)     # the library's defaults
        c.close()


def records_as_q8k(raw, K):
    """The 144-byte records of a vector as the checker's 292-byte Q8_K blocks (group sums recomputed from the
    int8 values; the records' own sums are compared with them by the caller)."""
    q, sums, d = decode_records(raw, K)
    out = np.zeros((K // 256, 292), np.uint8)
    out[:, :4] = d.astype(np.float32).view(np.uint8).reshape(K // 256, 4)
    out[:, 4:260] = q.view(np.uint8).reshape(K // 256, 256)
    out[:, 260:292] = q.reshape(K // 16, 16).astype(np.int16).sum(axis=1, dtype=np.int16).view(np.uint8).reshape(K // 256, 32)
    assert np.array_equal(sums, q.reshape(K // 32, 32).astype(np.int64).sum(axis=1))
    return out.reshape(-1)


def check_quantized(raw, K, want64):
    """Records against a vector known in binary64: the scale is max|v|/127 to fp32 accuracy and every int8 is
    within half a step (plus rounding slack) of v * 127/max|v|."""
    q, _, d = decode_records(raw, K)
    v = np.asarray(want64, np.float64).reshape(K // 256, 256)
    amax = np.abs(v).max(axis=1)
    assert np.allclose(d, amax / 127.0, rtol=2e-6, atol=0)
    scaled = v * (127.0 / np.where(amax > 0, amax, 1.0))[:, None]
    assert np.max(np.abs(q.reshape(K // 256, 256) - scaled)) <= 0.5 + 2e-3


def test_chain_layer_step_by_step_against_checker(chain, oracle):
    """One layer of the dependent chain, every step compared with the checker FROM IDENTICAL INPUTS (each CPU
    step starts from what the device produced for the step before): the quantized records integer by
    integer, each product and residual add to 1e-5 norm-wise.  Then the whole token through
    DecodeChain("chain") must equal this step-by-step run bit for bit."""
    lib, b, r = chain.lib, chain.buf, chain.rec
    H, KV, F, eps = chain.hidden, chain.kv, chain.ffn, chain.eps
    rng = np.random.default_rng(6)
    x0 = rng.standard_normal(H, dtype=np.float32)
    chain.set_state(x0)
    layer = 0

    def read(ptr, n):
        out = np.empty(n, np.float32)
        lib.bpdq_sync()
        lib.bpdq_d2h(out.ctypes.data, ptr, out.nbytes)
        return out

    def read_rec(ptr, K):
        out = np.empty(K // 128 * 144, np.uint8)
        lib.bpdq_sync()
        lib.bpdq_d2h(out.ctypes.data, ptr, out.nbytes)
        return out

    def prod(m, blocks):
        _, rows, cols = chain.shapes[m]
        return oracle.qmatmul_q4k_q8k(chain.host_weight(layer, m), blocks, rows, cols)[1]

    def norm64(x, w):
        x = x.astype(np.float64)
        return x / np.sqrt(np.mean(x * x) + eps) * w.astype(np.float64)

    # 1. rms_norm -> records
    capi.check(lib.bpd_rmsnorm_q8k_records_cuda(b["x"], chain.norm_ptr(layer, 0), r["h"], 1, H, eps, None))
    rec_h = read_rec(r["h"], H)
    check_quantized(rec_h, H, norm64(x0, chain.norm_host[layer, 0]))
    # 2. q, k, v from the device's records
    capi.check(lib.bpd_qmatmul_q4k_records_cuda(3, chain._descs(layer, (0, 1, 2), ("q", "k", "v")), r["h"], 0, None))
    blocks_h = records_as_q8k(rec_h, H)
    q = read(b["q"], H)
    assert normwise(q, prod(0, blocks_h)) <= 1e-5
    assert normwise(read(b["k"], KV), prod(1, blocks_h)) <= 1e-5
    assert normwise(read(b["v"], KV), prod(2, blocks_h)) <= 1e-5
    # 3. records of q: the checker's quantizer byte for byte
    capi.check(lib.bpd_quant_q8k_records_cuda(b["q"], r["q"], H, None))
    blocks_q = records_as_q8k(read_rec(r["q"], H), H)
    assert np.array_equal(blocks_q, oracle.quant_q8_K(q))
    # 4. x += wo . q
    capi.check(lib.bpd_qmatmul_q4k_records_cuda(1, chain._descs(layer, (3,), ("x",)), r["q"], 1, None))
    x1 = read(b["x"], H)
    assert normwise(x1, x0.astype(np.float64) + prod(3, blocks_q)) <= 1e-5
    # 5. second norm, gate and up
    capi.check(lib.bpd_rmsnorm_q8k_records_cuda(b["x"], chain.norm_ptr(layer, 1), r["h"], 1, H, eps, None))
    rec_h2 = read_rec(r["h"], H)
    check_quantized(rec_h2, H, norm64(x1, chain.norm_host[layer, 1]))
    capi.check(lib.bpd_qmatmul_q4k_records_cuda(2, chain._descs(layer, (4, 5), ("gate", "up")), r["h"], 0, None))
    blocks_h2 = records_as_q8k(rec_h2, H)
    g, u = read(b["gate"], F), read(b["up"], F)
    assert normwise(g, prod(4, blocks_h2)) <= 1e-5
    assert normwise(u, prod(5, blocks_h2)) <= 1e-5
    # 6. silu(gate) * up -> records
    capi.check(lib.bpd_swiglu_q8k_records_cuda(b["gate"], b["up"], r["act"], F, None))
    rec_a = read_rec(r["act"], F)
    g64, u64 = g.astype(np.float64), u.astype(np.float64)
    check_quantized(rec_a, F, g64 / (1.0 + np.exp(-g64)) * u64)
    # 7. x += w2 . act
    capi.check(lib.bpd_qmatmul_q4k_records_cuda(1, chain._descs(layer, (6,), ("x",)), r["act"], 1, None))
    x2 = read(b["x"], H)
    assert normwise(x2, x1.astype(np.float64) + prod(6, records_as_q8k(rec_a, F))) <= 1e-5
    assert lib.bpdq_last_status() == 0
    # the chain itself: same bits as the steps above for its first layer (run one layer's worth by comparing
    # a fresh single-layer chain over the same weights)
    one = DecodeChain(hidden=H, kv=KV, ffn=F, n_layers=1, seed=11, lib=lib)
    try:
        assert all(np.array_equal(one.host_weight(0, m), chain.host_weight(0, m)) for m in range(7))
        assert np.array_equal(one.norm_host[0], chain.norm_host[0])
        one.set_state(x0)
        one.enqueue_token("chain")
        assert np.array_equal(one.get_state().view(np.uint32), x2.view(np.uint32))
    finally:
        one.close()


@pytest.mark.parametrize("prologue", [0, 1, 2])
def test_fused_product_equals_records_path(lib, prologue):
    """bpd_qmatmul_q4k_fused_cuda against the producer kernel + product over records, shapes of the
    benchmark's layer (K = 4096 and 14336, several matrices per launch, residual on one of them)."""
    K = 14336 if prologue == 2 else 4096
    shapes = [(4096, K)] if prologue == 2 else [(1024, K), (4096, K), (260, K)]
    rng = np.random.default_rng(40 + prologue)
    a = rng.standard_normal(K, dtype=np.float32) * 4
    b = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32) if prologue == 1 else rng.standard_normal(K, dtype=np.float32)
    Ws = [synth.q4k_matrix(m, k, rng) for m, k in shapes]
    prev = [rng.standard_normal(m, dtype=np.float32) * 50 for m, _ in shapes]
    dA, dB, dWs = Dev(lib, a), Dev(lib, b), [Dev(lib, w) for w in Ws]
    dR = Dev(lib, nbytes=lib.bpdq_records_bytes(K))
    mask = 0b001
    got = []
    for fused in (False, True):
        outs = [Dev(lib, p) for p in prev]
        descs = (capi.GemvDesc * len(shapes))(*[capi.GemvDesc(dW.ptr, None, o.ptr, m, k)
                                                for (m, k), dW, o in zip(shapes, dWs, outs)])
        if fused:
            assert lib.bpd_qmatmul_q4k_fused_cuda(len(shapes), descs, prologue, dA.ptr, dB.ptr if prologue else None,
                                                  1e-5, mask, None) == 0
        else:
            if prologue == 0:
                assert lib.bpd_quant_q8k_records_cuda(dA.ptr, dR.ptr, K, None) == 0
            elif prologue == 1:
                assert lib.bpd_rmsnorm_q8k_records_cuda(dA.ptr, dB.ptr, dR.ptr, 1, K, 1e-5, None) == 0
            else:
                assert lib.bpd_swiglu_q8k_records_cuda(dA.ptr, dB.ptr, dR.ptr, K, None) == 0
            assert lib.bpd_qmatmul_q4k_records_cuda(len(shapes), descs, dR.ptr, mask, None) == 0
        lib.bpdq_sync()
        assert lib.bpdq_last_status() == 0
        got.append([o.read(np.uint32) for o in outs])
    for x, y in zip(*got):
        assert np.array_equal(x, y)

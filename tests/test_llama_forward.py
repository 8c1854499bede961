"""Q8_0 Llama forward (bench/bpd_cpu.c:5608-5798 of the reference).

CPU part: the checker's restatement against the fixture that the compiled reference produced
(tests/golden/llama_tiny.npz, bit for bit) and, where the compiled reference is present, step by
step.  GPU part: bpd_llama_forward_cuda against fixture and checker.  The device's cosf / sinf / expf
and the tree-shaped sums differ from libm's in the last bits, so the GPU comparison is norm-wise; the
integer and format steps (f16 cache write, argmax, quantization inside the products) are exact."""
import numpy as np
import pytest

from bpd_substrate_b200 import capi, llama
from oracle import binding
from tests.golden.make_golden import LLAMA_TINY, LLAMA_TINY_SEED, LLAMA_TINY_STEPS
from tests.util import normwise

import os

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "llama_tiny.npz")
needs_ref = pytest.mark.skipif(not binding.ref_available("bpd_cpu.so"), reason="compiled reference not present")


def u32(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)


def f16_as_f32(a):
    return np.asarray(a, np.uint16).view(np.float16).astype(np.float32)


@pytest.fixture(scope="module")
def tiny():
    cfg = llama.make_config(**LLAMA_TINY)
    return llama.SyntheticLlama(cfg, seed=LLAMA_TINY_SEED)


def run_steps(forward, model):
    """prefill + two decode steps; returns {name: (logits, tokens)}, caches updated by `forward`."""
    out, kv_pos = {}, 0
    for name, toks in LLAMA_TINY_STEPS:
        pos = np.arange(kv_pos, kv_pos + len(toks), dtype=np.int32)
        out[name] = forward(toks, pos, kv_pos)
        kv_pos += len(toks)
    return out


def test_checker_forward_equals_reference_fixture(oracle, tiny):
    g = np.load(GOLDEN)
    w, keep = tiny.host_structs()
    k, v = tiny.kv_cache()
    got = run_steps(lambda t, p, kp: oracle.llama_forward(w, tiny.cfg, t, p, kp, k, v), tiny)
    for name, (logits, tokens) in got.items():
        assert np.array_equal(u32(logits), g[f"{name}_logits"]), name
        assert np.array_equal(tokens, g[f"{name}_tokens"]), name
    assert np.array_equal(k, g["k_cache"]) and np.array_equal(v, g["v_cache"])
    assert np.count_nonzero(k[:, 7:]) == 0          # only the seven positions fed so far are written


@needs_ref
def test_checker_steps_equal_compiled_reference(oracle):
    ref = binding.load_ref("bpd_cpu.so")
    rng = np.random.default_rng(3)
    T, H, HKV, D, S = 3, 4, 2, 32, 12
    x = rng.standard_normal((T, H * D), dtype=np.float32)
    w = (1 + 0.1 * rng.standard_normal(H * D)).astype(np.float32)
    a, b = np.empty_like(x), np.empty_like(x)
    ref.bpd_rmsnorm_llama_cpu(x.ctypes.data, w.ctypes.data, a.ctypes.data, T, H * D, 1e-5)
    oracle.lib.orc_rmsnorm_llama(x.ctypes.data, w.ctypes.data, b.ctypes.data, T, H * D, 1e-5)
    assert np.array_equal(u32(a), u32(b))
    pos = np.array([4, 5, 9], np.int32)
    ff = (1 + rng.random(D // 2)).astype(np.float32)
    for freqs, n_dims in ((ff, D), (None, D - 8)):
        fp = freqs.ctypes.data if freqs is not None else None
        ref.bpd_rope_norm_freqs_cpu(x.ctypes.data, a.ctypes.data, pos.ctypes.data, fp, T, H, D, n_dims, 500000.0)
        oracle.lib.orc_rope_norm_freqs(x.ctypes.data, b.ctypes.data, pos.ctypes.data, fp, T, H, D, n_dims, 500000.0)
        assert np.array_equal(u32(a), u32(b))
    src = rng.standard_normal((T, HKV * D), dtype=np.float32) * 3
    src[0, :4] = [1e-7, 65520.0, -7e4, 6.1e-5]      # underflow, overflow to inf, f16 subnormal range
    ca, cb = np.zeros((S, HKV * D), np.uint16), np.zeros((S, HKV * D), np.uint16)
    ref.bpd_kv_cache_write_f16_cpu(ca.ctypes.data, src.ctypes.data, pos.ctypes.data, T, HKV, D, S)
    oracle.lib.orc_kv_cache_write(cb.ctypes.data, src.ctypes.data, pos.ctypes.data, T, HKV * D, 1)
    assert np.array_equal(ca, cb)
    q = rng.standard_normal((T, H * D), dtype=np.float32)
    kk = rng.standard_normal((S, HKV * D), dtype=np.float32)
    vv = rng.standard_normal((S, HKV * D), dtype=np.float32)
    ref.bpd_gqa_attn_cpu(q.ctypes.data, kk.ctypes.data, vv.ctypes.data, a.ctypes.data, T, S, H, HKV, D, 0.25, 2)
    oracle.lib.orc_gqa_attn(q.ctypes.data, kk.ctypes.data, vv.ctypes.data, b.ctypes.data, T, S, H, HKV, D, 0.25, 2)
    assert np.array_equal(u32(a), u32(b))
    z = rng.standard_normal((5, 33), dtype=np.float32)
    z[1, 7] = z[1, 20] = 9.0                        # a tie: the lower index wins
    ia, ib = np.empty(5, np.int64), np.empty(5, np.int64)
    ref.bpd_argmax_dim_cpu(z.ctypes.data, ia.ctypes.data, 5, 33, 1)
    oracle.lib.orc_argmax_rows(z.ctypes.data, ib.ctypes.data, 5, 33)
    assert np.array_equal(ia, ib) and ia[1] == 7


# --------------------------------------------------------------------------- GPU

@pytest.mark.gpu
@pytest.mark.parametrize("retiled", [False, True])
def test_forward_tiny_against_reference_fixture(lib, tiny, retiled):
    """retiled: the prefill's products run on the re-tiled copies of the matrices (tensor cores)."""
    g = np.load(GOLDEN)
    dev = llama.DeviceLlama(tiny, lib)
    try:
        if retiled:
            dev.retile()
        got = run_steps(dev.forward, tiny)
        for name, (logits, tokens) in got.items():
            want = g[f"{name}_logits"].view(np.float32)
            assert normwise(logits, want) <= 2e-5, name
            assert np.array_equal(tokens, g[f"{name}_tokens"]), name
        k, v = dev.read_cache()
        # the cached K and V are f16 roundings of values that agree to ~1e-6: equal up to one f16 step here and there
        for mine, ref in ((k, g["k_cache"]), (v, g["v_cache"])):
            assert np.count_nonzero(mine[:, 7:]) == 0
            a, b = f16_as_f32(mine), f16_as_f32(ref)
            assert np.max(np.abs(a - b)) <= 2e-3 * np.max(np.abs(b))
            assert np.mean(mine == ref) > 0.99
    finally:
        dev.close()


@pytest.mark.gpu
def test_steps_against_checker(lib, oracle):
    """Every step of the block on device pointers against the checker's restatement of it, from
    identical inputs (so no quantization sits between the two sides)."""
    from tests.util import Dev
    rng = np.random.default_rng(21)
    T, H, HKV, D, S = 5, 8, 2, 64, 40
    E = H * D
    x = rng.standard_normal((T, E), dtype=np.float32) * 2
    w = (1 + 0.1 * rng.standard_normal(E)).astype(np.float32)
    dX, dW, dO = Dev(lib, x), Dev(lib, w), Dev(lib, nbytes=x.nbytes)
    want = np.empty_like(x)
    # rms_norm
    assert lib.bpd_rmsnorm_llama_cuda(dX.ptr, dW.ptr, dO.ptr, T, E, 1e-5, None) == 0
    oracle.lib.orc_rmsnorm_llama(x.ctypes.data, w.ctypes.data, want.ctypes.data, T, E, 1e-5)
    lib.bpdq_sync()
    assert np.array_equal(u32(dO.read(np.float32)), u32(want).ravel())
    # rotary embedding: full and partial rotation, with and without frequency factors, in place
    pos = np.array([0, 3, 17, 38, 39], np.int32)
    ff = (1 + 3 * rng.random(D // 2)).astype(np.float32)
    dP, dF = Dev(lib, pos), Dev(lib, ff)
    for freqs, n_dims in ((ff, D), (None, 48), (ff, 0)):
        assert lib.bpd_rope_norm_freqs_cuda(dX.ptr, dO.ptr, dP.ptr, dF.ptr if freqs is not None else None, T, H, D, n_dims,
                                            500000.0, None) == 0
        if n_dims:
            oracle.lib.orc_rope_norm_freqs(x.ctypes.data, want.ctypes.data, pos.ctypes.data,
                                           freqs.ctypes.data if freqs is not None else None, T, H, D, n_dims, 500000.0)
        else:
            want[:] = x
        lib.bpdq_sync()
        got = dO.read(np.float32).reshape(T, E)
        assert np.mean(u32(got) == u32(want)) > 0.995 and normwise(got, want) <= 1e-6
    # KV-cache writes: f16 rounding is exact, including the overflow and subnormal ends
    src = rng.standard_normal((T, HKV * D), dtype=np.float32) * 3
    src[0, :6] = [1e-7, 65520.0, -7e4, 6.1e-5, 5.96e-8, -2.98e-8]
    dS = Dev(lib, src)
    for f16 in (1, 0):
        cache = np.zeros((S, HKV * D), np.uint16 if f16 else np.float32)
        dC = Dev(lib, cache)
        fn = lib.bpd_kv_cache_write_f16_cuda if f16 else lib.bpd_kv_cache_write_cuda
        assert fn(dC.ptr, dS.ptr, dP.ptr, T, HKV, D, S, None) == 0
        oracle.lib.orc_kv_cache_write(cache.ctypes.data, src.ctypes.data, pos.ctypes.data, T, HKV * D, f16)
        lib.bpdq_sync()
        assert np.array_equal(dC.read(cache.dtype).reshape(cache.shape), cache)
    # attention over a partly filled cache, fp32 and f16 caches
    q = rng.standard_normal((T, E), dtype=np.float32)
    kk = rng.standard_normal((S, HKV * D), dtype=np.float32)
    vv = rng.standard_normal((S, HKV * D), dtype=np.float32)
    dQ = Dev(lib, q)
    for f16 in (0, 1):
        if f16:
            kh, vh = kk.astype(np.float16), vv.astype(np.float16)
            kk, vv = kh.astype(np.float32), vh.astype(np.float32)
            dK, dV = Dev(lib, kh), Dev(lib, vh)
        else:
            dK, dV = Dev(lib, kk), Dev(lib, vv)
        assert lib.bpd_gqa_attn_cuda(dQ.ptr, dK.ptr, dV.ptr, dO.ptr, T, S, H, HKV, D, 0.125, 30, f16, None) == 0
        oracle.lib.orc_gqa_attn(q.ctypes.data, kk.ctypes.data, vv.ctypes.data, want.ctypes.data, T, S, H, HKV, D, 0.125, 30)
        lib.bpdq_sync()
        got = dO.read(np.float32).reshape(T, E)
        assert np.mean(u32(got) == u32(want)) > 0.99 and normwise(got, want) <= 1e-6
    # SwiGLU and argmax
    g = rng.standard_normal(E * T, dtype=np.float32) * 5
    g[:4] = [-120.0, 120.0, 0.0, -0.0]
    dG = Dev(lib, g)
    assert lib.bpd_swiglu_fuse_cuda(dG.ptr, dX.ptr, dO.ptr, T * E, None) == 0
    lib.bpdq_sync()
    with np.errstate(over="ignore"):
        ref = (g / (np.float32(1) + np.exp(-g.astype(np.float64)).astype(np.float32))) * x.ravel()
    got = dO.read(np.float32)
    assert np.mean(u32(got) == u32(ref)) > 0.995 and normwise(got, ref) <= 1e-6
    z = rng.standard_normal((6, 1001), dtype=np.float32)
    z[2, 40] = z[2, 900] = 7.0
    dZ, dI = Dev(lib, z), Dev(lib, nbytes=6 * 8)
    assert lib.bpd_argmax_dim_cuda(dZ.ptr, dI.ptr, 6, 1001, 1, None) == 0
    lib.bpdq_sync()
    idx = dI.read(np.int64)
    assert np.array_equal(idx, np.argmax(z, axis=1)) and idx[2] == 40
    assert lib.bpdq_last_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("f16,retiled", [(1, False), (0, False), (1, True), (0, True)])
def test_forward_larger_model_against_checker(lib, oracle, f16, retiled):
    """Shapes that take the fast Q8_0 kernel (K multiple of 256), GQA group of 4, partial rotary
    dimension, both cache types; prefill of 9 tokens and three single-token steps.

    The products agree with the checker to ~1e-6 (a different order of the fp32 sums), and every
    product re-quantizes its input to int8: per 512-element vector a few percent chance that one
    rounding flips, which is a ~1e-3 difference downstream and, through the KV cache, in every later
    token.  The bound on whole-forward logits allows for such flips and for nothing structural (a
    wrong step, weight or position is an O(1) difference); the steps themselves are checked tightly
    in test_steps_against_checker."""
    cfg = llama.make_config(n_layers=3, n_heads=8, n_kv_heads=2, head_dim=64, ffn_dim=1024, vocab_size=777, max_seq_len=40,
                            rope_dim=48, kv_cache_f16=f16)
    model = llama.SyntheticLlama(cfg, seed=5 + f16, rope_freqs=bool(f16))
    w, keep = model.host_structs()
    k, v = model.kv_cache()
    dev = llama.DeviceLlama(model, lib)
    try:
        if retiled:
            dev.retile()
        rng = np.random.default_rng(9)
        kv_pos = 0
        for n in (9, 1, 1, 1):
            toks = rng.integers(0, cfg.vocab_size, n).astype(np.int32)
            pos = np.arange(kv_pos, kv_pos + n, dtype=np.int32)
            want_logits, want_tok = oracle.llama_forward(w, cfg, toks, pos, kv_pos, k, v)
            logits, tok = dev.forward(toks, pos, kv_pos)
            assert normwise(logits, want_logits) <= 2e-2, (n, kv_pos)
            # argmax may only differ where the two best logits are closer than the numerical difference
            for r in np.flatnonzero(tok != want_tok):
                assert abs(want_logits[r, tok[r]] - want_logits[r, want_tok[r]]) <= 2e-2 * np.abs(want_logits[r]).max()
            kv_pos += n
    finally:
        dev.close()


@pytest.mark.gpu
def test_forward_rejects_bad_configurations(lib, tiny):
    import ctypes as C
    from bpd_substrate_b200 import capi
    dev = llama.DeviceLlama(tiny, lib)
    try:
        bad = llama.make_config(**LLAMA_TINY)
        bad.max_seq_len = 4                       # prefill of five tokens does not fit
        d = lib.bpdq_alloc(4096)
        args = (d, 5, C.byref(dev.weights))
        assert lib.bpd_llama_forward_cuda(*args, C.byref(bad), d, 0, dev.d_k, dev.d_v, d, d, None) == -3
        bad = llama.make_config(**LLAMA_TINY)
        bad.n_kv_heads = 3                        # heads do not divide
        assert lib.bpd_llama_forward_cuda(*args, C.byref(bad), d, 0, dev.d_k, dev.d_v, d, d, None) == -1
        assert lib.bpd_llama_forward_cuda(None, 5, C.byref(dev.weights), C.byref(tiny.cfg), d, 0, dev.d_k, dev.d_v, d, d, None) == -1
        lib.bpdq_free(d)
        lib.bpdq_clear_status()
        assert capi.check(0) == 0
    finally:
        dev.close()


def _block_by_twins(lib, dev, layer, d_x, d_pos, n, kv_pos, d_k, d_v, scr):
    """One block as the sequence of separate entry points (the reference's call order, bench/bpd_cpu.c:5608-5738)."""
    c, lw = dev.cfg, dev.layers[layer]
    E, H, HKV, D, F = c.embed_dim, c.n_heads, c.n_kv_heads, c.head_dim, c.ffn_dim
    row = HKV * D
    s1, s2, s3, sv = scr
    ok = lambda rc: capi.check(rc)
    ok(lib.bpd_rmsnorm_llama_cuda(d_x, lw.attn_norm_w, s1, n, E, c.rms_eps, None))
    ok(lib.bpd_qmatmul_q8_0_cuda(lw.w_q, s1, s2, n, H * D, E, None))
    ok(lib.bpd_qmatmul_q8_0_cuda(lw.w_k, s1, s3, n, row, E, None))
    ok(lib.bpd_qmatmul_q8_0_cuda(lw.w_v, s1, sv, n, row, E, None))
    ff = dev.weights.rope_freqs
    ok(lib.bpd_rope_norm_freqs_cuda(s2, s2, d_pos, ff, n, H, D, c.rope_dim, c.rope_base, None))
    ok(lib.bpd_rope_norm_freqs_cuda(s3, s3, d_pos, ff, n, HKV, D, c.rope_dim, c.rope_base, None))
    write = lib.bpd_kv_cache_write_f16_cuda if c.kv_cache_f16 else lib.bpd_kv_cache_write_cuda
    ok(write(d_k, s3, d_pos, n, HKV, D, c.max_seq_len, None))
    ok(write(d_v, sv, d_pos, n, HKV, D, c.max_seq_len, None))
    ok(lib.bpd_gqa_attn_cuda(s2, d_k, d_v, s1, n, c.max_seq_len, H, HKV, D, 1.0 / np.sqrt(np.float32(D)), kv_pos,
                             c.kv_cache_f16, None))
    ok(lib.bpd_qmatmul_q8_0_cuda(lw.w_o, s1, s2, n, E, H * D, None))
    lib.gpu_add(d_x, s2, d_x, n * E)
    ok(lib.bpd_rmsnorm_llama_cuda(d_x, lw.ffn_norm_w, s1, n, E, c.rms_eps, None))
    ok(lib.bpd_qmatmul_q8_0_cuda(lw.w_gate, s1, s2, n, F, E, None))
    ok(lib.bpd_qmatmul_q8_0_cuda(lw.w_up, s1, s3, n, F, E, None))
    ok(lib.bpd_swiglu_fuse_cuda(s2, s3, s2, n * F, None))
    ok(lib.bpd_qmatmul_q8_0_cuda(lw.w_down, s2, s1, n, E, F, None))
    lib.gpu_add(d_x, s1, d_x, n * E)


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1, 6])
def test_block_and_forward_equal_their_separate_steps_bit_for_bit(lib, n):
    """The block fuses steps into shared launches (rotary embedding of q and k with the cache stores, residual
    adds with the norms that follow them, products that share an input); the forward also fuses across blocks.
    Both must give the bits of the separate entry points called in the reference's order."""
    import ctypes as C
    from tests.util import Dev
    cfg = llama.make_config(n_layers=2, n_heads=8, n_kv_heads=2, head_dim=64, ffn_dim=1024, vocab_size=300, max_seq_len=24,
                            rope_dim=48, kv_cache_f16=1)
    model = llama.SyntheticLlama(cfg, seed=77)
    dev = llama.DeviceLlama(model, lib)
    try:
        E, F, row = cfg.embed_dim, cfg.ffn_dim, cfg.n_kv_heads * cfg.head_dim
        kv_pos = 5
        rng = np.random.default_rng(n)
        toks = rng.integers(0, cfg.vocab_size, n).astype(np.int32)
        pos = np.arange(kv_pos, kv_pos + n, dtype=np.int32)
        kc, vc = model.kv_cache()
        kc[:, :kv_pos] = rng.standard_normal((cfg.n_layers, kv_pos, row)).astype(np.float16).view(np.uint16)
        vc[:, :kv_pos] = rng.standard_normal((cfg.n_layers, kv_pos, row)).astype(np.float16).view(np.uint16)
        d_tok, d_pos = Dev(lib, toks), Dev(lib, pos)
        scr = [Dev(lib, nbytes=4 * n * max(E, F)) for _ in range(4)]
        ptrs = [d.ptr for d in scr]
        layer_bytes = kc[0].nbytes

        def run(kind):
            d_k, d_v, d_x = Dev(lib, kc), Dev(lib, vc), Dev(lib, nbytes=4 * n * E)
            d_logits = Dev(lib, nbytes=4 * n * cfg.vocab_size)
            if kind == "forward":
                capi.check(lib.bpd_llama_forward_cuda(d_tok.ptr, n, C.byref(dev.weights), C.byref(cfg), d_pos.ptr, kv_pos, d_k.ptr,
                                                      d_v.ptr, d_logits.ptr, None, None))
            else:
                capi.check(lib.bpd_embed_lookup_q8_0_cuda(dev.weights.token_embd, d_tok.ptr, d_x.ptr, n, E, None))
                for layer in range(cfg.n_layers):
                    lk, lv = d_k.ptr + layer * layer_bytes, d_v.ptr + layer * layer_bytes
                    if kind == "blocks":
                        capi.check(lib.bpd_llama_block_cuda(d_x.ptr, C.byref(dev.layers[layer]), C.byref(cfg), d_pos.ptr, n, kv_pos,
                                                            lk, lv, ptrs[0], ptrs[1], ptrs[2], dev.weights.rope_freqs, None))
                    else:
                        _block_by_twins(lib, dev, layer, d_x.ptr, d_pos.ptr, n, kv_pos, lk, lv, ptrs)
                capi.check(lib.bpd_rmsnorm_llama_cuda(d_x.ptr, dev.weights.output_norm_w, ptrs[0], n, E, cfg.rms_eps, None))
                capi.check(lib.bpd_qmatmul_q8_0_cuda(dev.weights.output_w, ptrs[0], d_logits.ptr, n, cfg.vocab_size, E, None))
            lib.bpdq_sync()
            assert lib.bpdq_last_status() == 0
            return d_logits.read(np.uint32), d_k.read(np.uint16), d_v.read(np.uint16)

        want = run("twins")
        for kind in ("blocks", "forward"):
            got = run(kind)
            for a, b, what in zip(got, want, ("logits", "k cache", "v cache")):
                assert np.array_equal(a, b), (kind, what, int(np.count_nonzero(a != b)))
    finally:
        dev.close()


@pytest.mark.gpu
def test_indices_from_device_memory_are_checked(lib, tiny):
    """A position outside [0, max_seq_len) is not stored, a token id outside [0, vocab_size) is not looked
    up: the cache keeps its bytes, nothing outside it is touched, and the status says -4.  (The
    reference's CPU code would index out of bounds.)"""
    import ctypes as C
    from tests.util import Dev
    c = tiny.cfg
    row = c.n_kv_heads * c.head_dim
    rng = np.random.default_rng(3)
    src = rng.standard_normal((3, row)).astype(np.float32)
    pos = np.array([2, c.max_seq_len, -1], np.int32)             # one good row, two without a home
    d_src, d_pos = Dev(lib, src), Dev(lib, pos)
    # the cache sits inside a larger poisoned buffer, so that a stray write would show on either side
    guard = 4096
    for f16, fn in ((1, lib.bpd_kv_cache_write_f16_cuda), (0, lib.bpd_kv_cache_write_cuda)):
        esz = 2 if f16 else 4
        nbytes = c.max_seq_len * row * esz
        buf = Dev(lib, nbytes=nbytes + 2 * guard, fill=0xA5)
        lib.bpdq_clear_status()
        assert fn(buf.ptr + guard, d_src.ptr, d_pos.ptr, 3, c.n_kv_heads, c.head_dim, c.max_seq_len, None) == 0
        lib.bpdq_sync()
        assert lib.bpdq_last_status() == -4 and lib.bpdq_device_error_word() == 20
        lib.bpdq_clear_status()
        raw = buf.read(np.uint8)
        body = raw[guard:guard + nbytes].reshape(c.max_seq_len, row * esz)
        assert (raw[:guard] == 0xA5).all() and (raw[guard + nbytes:] == 0xA5).all()
        want = src[0].astype(np.float16).view(np.uint8) if f16 else src[0].view(np.uint8)
        assert np.array_equal(body[2], want)
        assert (np.delete(body, 2, axis=0) == 0xA5).all()
    # the whole forward: a bad token id and a bad position
    dev = llama.DeviceLlama(tiny, lib)
    try:
        n = 2
        d = {k: Dev(lib, v) for k, v in dict(tok=np.array([5, c.vocab_size], np.int32), pos=np.array([0, 1], np.int32),
                                             badpos=np.array([0, c.max_seq_len + 3], np.int32),
                                             oktok=np.array([5, 6], np.int32)).items()}
        logits, out = Dev(lib, nbytes=4 * n * c.vocab_size), Dev(lib, nbytes=8 * n)
        for tok, pos_key in (("tok", "pos"), ("oktok", "badpos")):
            lib.bpdq_clear_status()
            assert lib.bpd_llama_forward_cuda(d[tok].ptr, n, C.byref(dev.weights), C.byref(dev.cfg), d[pos_key].ptr, 0,
                                              dev.d_k, dev.d_v, logits.ptr, out.ptr, dev.stream) == 0
            assert lib.bpdq_stream_sync(dev.stream) == 0
            assert lib.bpdq_last_status() == -4
        lib.bpdq_clear_status()
    finally:
        dev.close()


@pytest.mark.gpu
def test_forward_with_caller_owned_workspace(lib, tiny):
    """bpd_llama_forward_ws_cuda: same bits as the plain entry, prefill on re-tiled weights included; a
    workspace that is too small is refused before anything runs."""
    import ctypes as C
    from tests.util import Dev
    c = tiny.cfg
    toks = np.array([3, 17, 95, 0, 42], np.int32)
    pos = np.arange(5, dtype=np.int32)
    results = []
    for use_ws in (False, True):
        dev = llama.DeviceLlama(tiny, lib)
        try:
            dev.retile()
            d_tok, d_pos = Dev(lib, toks), Dev(lib, pos)
            logits, out = Dev(lib, nbytes=4 * 5 * c.vocab_size, fill=0xFF), Dev(lib, nbytes=8 * 5)
            if use_ws:
                nbytes = lib.bpdq_llama_forward_workspace_bytes(C.byref(dev.cfg), 5)
                assert nbytes > 0
                ws = Dev(lib, nbytes=nbytes, fill=0xEE)
                assert lib.bpd_llama_forward_ws_cuda(d_tok.ptr, 5, C.byref(dev.weights), C.byref(dev.tiles), C.byref(dev.cfg),
                                                     d_pos.ptr, 0, dev.d_k, dev.d_v, logits.ptr, out.ptr, ws.ptr, 1024,
                                                     dev.stream) == -3
                lib.bpdq_clear_status()
                rc = lib.bpd_llama_forward_ws_cuda(d_tok.ptr, 5, C.byref(dev.weights), C.byref(dev.tiles), C.byref(dev.cfg),
                                                   d_pos.ptr, 0, dev.d_k, dev.d_v, logits.ptr, out.ptr, ws.ptr, nbytes, dev.stream)
            else:
                rc = lib.bpd_llama_forward_tiles_cuda(d_tok.ptr, 5, C.byref(dev.weights), C.byref(dev.tiles), C.byref(dev.cfg),
                                                      d_pos.ptr, 0, dev.d_k, dev.d_v, logits.ptr, out.ptr, dev.stream)
            assert rc == 0
            assert lib.bpdq_stream_sync(dev.stream) == 0
            assert lib.bpdq_last_status() == 0
            results.append((logits.read(np.uint32), out.read(np.int64)))
        finally:
            dev.close()
    assert np.array_equal(results[0][0], results[1][0]) and np.array_equal(results[0][1], results[1][1])

"""Timings of the secondary configurations (the benchmark line itself comes from bench.py).

    python measure.py            # prints one JSON object per configuration
    python measure.py --llama-decode [LAYERS]
                                                    # Q8_0 Llama forward, 8B-shaped layers: ms per decoded token
    python measure.py --llama-prefill [LAYERS] [TOKENS]
                                                    # the same layers, a prefill: rows against re-tiled weights
    python measure.py --q8-tiles [N K]
                                                    # Q8_0 many-token product on re-tiled weights (tcgen05)
                                                    # beside the row-layout kernel, 1..512 tokens
    python measure.py --q8-tiles-once TOKENS [N K]
                                                    # five launches of the re-tiled product: a small case for a profiler
    python measure.py --w4a32-once [N K]           # five launches of the fp32-activation GEMV: a small case for a profiler
    python measure.py --gemm-once tc5 64 [N K]
                                                    # five launches of one many-token product (kernel
                                                    # tc5 | mma | rg16 | dispatch): a small case for a profiler

Cold-HBM protocol: every timed launch reads a different copy of its weights, with enough
copies that the working set is several times the L2 size, so no launch finds its inputs
cached.  Times are CUDA events on the launching stream around `iters` launches.
"""
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from bpd_substrate_b200 import capi, synth  # noqa: E402

PEAK_FALLBACK = 6650.0


def _peak():
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["hbm_gbs"])
    except Exception:
        return PEAK_FALLBACK


class Timer:
    def __init__(self, lib):
        self.lib = lib
        self.stream = lib.bpdq_stream_create()
        self.e0, self.e1 = lib.bpdq_event_create(), lib.bpdq_event_create()

    def run(self, fn, iters, warm=3):
        lib = self.lib
        for i in range(warm):
            fn(i)
        lib.bpdq_stream_sync(self.stream)
        lib.bpdq_event_record(self.e0, self.stream)
        for i in range(iters):
            fn(i)
        lib.bpdq_event_record(self.e1, self.stream)
        return lib.bpdq_event_elapsed_ms(self.e0, self.e1) / iters * 1e3   # microseconds


def _dev(lib, arr):
    p = lib.bpdq_alloc(arr.nbytes)
    lib.bpdq_h2d(p, arr.ctypes.data, arr.nbytes)
    return p


def _copies(nbytes, target=600e6):
    return max(2, int(target // nbytes) + 1)


def gemm_once(lib, kernel, tokens, N=14336, K=4096, launches=5):
    """One Q4_K x Q8_K product, a few launches, nothing else on the device."""
    entry = {"tc5": lib.bpd_qmm_q4k_q8k_tc5_cuda, "mma": lib.bpd_qmm_q4k_q8k_mma_cuda,
             "rg16": lib.bpd_qmm_q4k_q8k_rg16_cuda}.get(kernel)
    w = _dev(lib, synth.q4k_matrix(N, K, 1))
    if kernel == "rg16":            # the product on weights re-tiled in groups of 16 rows
        t = lib.bpdq_alloc(lib.bpd_q4k_rg16_bytes(N, K))
        capi.check(lib.bpd_repack_q4k_rg16_cuda(w, t, N, K, None))
        lib.bpdq_sync()
        lib.bpdq_free(w)
        w = t
    x = _dev(lib, synth.activations(K, 2, rows=tokens))
    o = lib.bpdq_alloc(tokens * N * 4)
    for _ in range(launches):
        if entry is not None:
            capi.check(entry(w, x, o, tokens, N, K, None))
        else:
            capi.check(lib.bpd_qmm_q4k_q8k_cuda(w, x, o, tokens, N, K, 0, 0, None, None))
    lib.bpdq_sync()
    status = lib.bpdq_last_status()
    for p in (w, x, o):
        lib.bpdq_free(p)
    print(json.dumps({"gemm_once": kernel, "tokens": tokens, "N": N, "K": K, "status": status}))
    return 0 if status == 0 else 1


def w4a32_once(lib, N=14336, K=4096, launches=5):
    """The fp32-activation GEMV drop-in (bpd_qmatmul_q4k_gpu's kernel), a few launches: a small case for a profiler."""
    w = _dev(lib, synth.q4k_matrix(N, K, 1))
    x = _dev(lib, synth.activations(K, 2))
    o = lib.bpdq_alloc(N * 4)
    for _ in range(launches):
        capi.check(lib.bpd_qmatmul_q4k_gpu_st(w, x, o, N, K, None))
    lib.bpdq_sync()
    status = lib.bpdq_last_status()
    for p in (w, x, o):
        lib.bpdq_free(p)
    print(json.dumps({"w4a32_once": True, "N": N, "K": K, "status": status}))
    return 0 if status == 0 else 1


def llama_prefill(lib, n_layers=4, tokens=128):
    """Prefill of `tokens` tokens through `n_layers` 8B-shaped Q8_0 layers, on the rows (one pass over each
    matrix per token) and on the re-tiled copies (one pass on the tensor cores)."""
    import ctypes as C
    from bpd_substrate_b200 import llama
    cfg = llama.make_config(n_layers=n_layers, n_heads=32, n_kv_heads=8, head_dim=128, ffn_dim=14336, vocab_size=32000,
                            max_seq_len=max(256, tokens))
    model = llama.SyntheticLlama(cfg, seed=3)
    dev = llama.DeviceLlama(model, lib)
    tm = Timer(lib)
    toks = np.arange(tokens, dtype=np.int32) % cfg.vocab_size
    pos = np.arange(tokens, dtype=np.int32)
    d_tok, d_pos = _dev(lib, toks), _dev(lib, pos)
    d_logits, d_out = lib.bpdq_alloc(4 * tokens * cfg.vocab_size), lib.bpdq_alloc(8 * tokens)
    dev.retile()
    res = {}
    for name, tiles in (("rows", None), ("tiles", C.byref(dev.tiles))):
        def step(i):
            capi.check(lib.bpd_llama_forward_tiles_cuda(d_tok, tokens, C.byref(dev.weights), tiles, C.byref(cfg), d_pos, 0, dev.d_k,
                                                        dev.d_v, d_logits, d_out, tm.stream))
        res[name] = tm.run(step, 5, warm=2) / 1e3
    print(json.dumps(dict(config=f"Q8_0 Llama prefill, {n_layers} layers of 8B shape + 32000-row head, {tokens} tokens",
                          rows_ms=round(res["rows"], 3), tiles_ms=round(res["tiles"], 3),
                          tiles_tokens_per_s=round(tokens / res["tiles"] * 1e3), weight_bytes=model.weight_bytes(),
                          status=lib.bpdq_last_status())), flush=True)
    dev.close()
    return 0 if lib.bpdq_last_status() == 0 else 1


def q8_tiles(lib, N=14336, K=4096, token_counts=(1, 4, 16, 32, 64, 128, 512)):
    """Times bpd_qmatmul_q8_0_tiles_cuda against bpd_qmatmul_q8_0_cuda (one pass over the rows per
    token) on cold weights; prints one JSON object per token count."""
    tm = Timer(lib)
    s = tm.stream
    peak = _peak()
    W = synth.q8_0_matrix(N, K, 1)
    n = _copies(W.nbytes)
    rows = [_dev(lib, W) for _ in range(n)]
    tiles = []
    for r in rows:
        t = lib.bpdq_alloc(lib.bpd_q8_0_tiles_bytes(N, K))
        capi.check(lib.bpd_repack_q8_0_tiles_cuda(r, t, N, K, s))
        tiles.append(t)
    for tokens in token_counts:
        x = _dev(lib, synth.activations(K, 2, rows=tokens))
        o = lib.bpdq_alloc(tokens * N * 4)
        us_t = tm.run(lambda i: lib.bpd_qmatmul_q8_0_tiles_cuda(tiles[i % n], x, o, tokens, N, K, s), 30)
        us_r = tm.run(lambda i: lib.bpd_qmatmul_q8_0_cuda(rows[i % n], x, o, tokens, N, K, s), 30 if tokens <= 16 else 5)
        nbytes = W.nbytes + tokens * (K + N) * 4
        print(json.dumps(dict(config=f"Q8_0 x Q8_0 {N}x{K}, {tokens} tokens", tiles_us=round(us_t, 2), rows_us=round(us_r, 2),
                              algorithmic_bytes=nbytes, tiles_gbs=round(nbytes / us_t / 1e3, 1),
                              tiles_pct_of_measured_peak=round(100 * nbytes / us_t / 1e3 / peak, 1),
                              tiles_tera_int8_macs_per_s=round(tokens * N * K / us_t / 1e6, 2),
                              status=lib.bpdq_last_status())), flush=True)
        lib.bpdq_free(x)
        lib.bpdq_free(o)
    for p in rows + tiles:
        lib.bpdq_free(p)
    return 0 if lib.bpdq_last_status() == 0 else 1


def q8_tiles_once(lib, tokens, N=14336, K=4096, launches=5):
    w = _dev(lib, synth.q8_0_matrix(N, K, 1))
    t = lib.bpdq_alloc(lib.bpd_q8_0_tiles_bytes(N, K))
    capi.check(lib.bpd_repack_q8_0_tiles_cuda(w, t, N, K, None))
    x = _dev(lib, synth.activations(K, 2, rows=tokens))
    o = lib.bpdq_alloc(tokens * N * 4)
    for _ in range(launches):
        capi.check(lib.bpd_qmatmul_q8_0_tiles_cuda(t, x, o, tokens, N, K, None))
    lib.bpdq_sync()
    status = lib.bpdq_last_status()
    for p in (w, t, x, o):
        lib.bpdq_free(p)
    print(json.dumps({"q8_tiles_once": tokens, "N": N, "K": K, "status": status}))
    return 0 if status == 0 else 1


def llama_decode(lib, n_layers=4, steps=32):
    """Single-token steps of bpd_llama_forward_cuda on a synthetic model with Llama-3-8B-shaped layers
    (32 heads, 8 KV heads, head 128, FFN 14336; vocabulary cut to 32000 to keep host generation short),
    f16 KV cache of 256 positions.  Prints ms per token and the bytes that a token must read."""
    import ctypes as C

    from bpd_substrate_b200 import llama
    cfg = llama.make_config(n_layers=n_layers, n_heads=32, n_kv_heads=8, head_dim=128, ffn_dim=14336, vocab_size=32000,
                            max_seq_len=256)
    model = llama.SyntheticLlama(cfg, seed=1)
    dev = llama.DeviceLlama(model, lib)
    n_pre = 8
    dev.forward(np.arange(n_pre, dtype=np.int32), np.arange(n_pre, dtype=np.int32), 0)      # prefill
    d_tok, d_pos = lib.bpdq_alloc(16), lib.bpdq_alloc(16 * (steps + 4))
    d_logits, d_out = lib.bpdq_alloc(4 * cfg.vocab_size), lib.bpdq_alloc(16)
    pos = np.arange(n_pre, n_pre + steps + 4, dtype=np.int32)
    lib.bpdq_h2d(d_pos, pos.ctypes.data, pos.nbytes)
    tok = np.array([5], np.int32)
    lib.bpdq_h2d(d_tok, tok.ctypes.data, 4)
    ev0, ev1 = lib.bpdq_event_create(), lib.bpdq_event_create()

    def step(i):
        capi.check(lib.bpd_llama_forward_cuda(d_tok, 1, C.byref(dev.weights), C.byref(cfg), d_pos + 4 * i, n_pre + i, dev.d_k,
                                              dev.d_v, d_logits, d_out, dev.stream))
    for i in range(4):
        step(i)
    lib.bpdq_stream_sync(dev.stream)
    lib.bpdq_event_record(ev0, dev.stream)
    for i in range(4, 4 + steps):
        step(i)
    lib.bpdq_event_record(ev1, dev.stream)
    ms = lib.bpdq_event_elapsed_ms(ev0, ev1) / steps
    # the same step replayed from a CUDA graph (one position: the arguments are fixed at capture)
    capi.check(lib.bpdq_graph_begin(dev.stream), "graph capture")
    step(4 + steps - 1)
    graph = lib.bpdq_graph_end(dev.stream)
    ms_graph = None
    if graph:
        for _ in range(3):
            capi.check(lib.bpdq_graph_launch(graph, dev.stream))
        lib.bpdq_event_record(ev0, dev.stream)
        for _ in range(steps):
            capi.check(lib.bpdq_graph_launch(graph, dev.stream))
        lib.bpdq_event_record(ev1, dev.stream)
        ms_graph = lib.bpdq_event_elapsed_ms(ev0, ev1) / steps
        lib.bpdq_graph_destroy(graph)
    kv_row = cfg.n_kv_heads * cfg.head_dim
    per_token = (sum(sum(v.nbytes for k, v in layer.items() if k.startswith("w_")) for layer in model.layers)
                 + model.output_w.nbytes + cfg.n_layers * 2 * cfg.max_seq_len * kv_row * 2)
    status = lib.bpdq_last_status()
    print(json.dumps({"config": f"Q8_0 Llama forward, {n_layers} layers of 8B shape, decode", "ms_per_token": round(ms, 4),
                      "ms_per_token_graph": round(ms_graph, 4) if ms_graph else None,
                      "bytes_per_token": per_token, "gbs": round(per_token / (ms_graph or ms) / 1e6, 1),
                      "launches_per_token": 9 * n_layers + 4, "status": status}))
    dev.close()
    return 0 if status == 0 else 1


def main():
    lib = capi.load()
    lib.bpdq_clear_status()
    if len(sys.argv) >= 2 and sys.argv[1] == "--llama-decode":
        return llama_decode(lib, *[int(v) for v in sys.argv[2:3]])
    if len(sys.argv) >= 2 and sys.argv[1] == "--llama-prefill":
        return llama_prefill(lib, *[int(v) for v in sys.argv[2:4]])
    if len(sys.argv) >= 2 and sys.argv[1] == "--q8-tiles":
        return q8_tiles(lib, *[int(v) for v in sys.argv[2:4]])
    if len(sys.argv) >= 3 and sys.argv[1] == "--q8-tiles-once":
        return q8_tiles_once(lib, *[int(v) for v in sys.argv[2:5]])
    if len(sys.argv) >= 2 and sys.argv[1] == "--w4a32-once":
        return w4a32_once(lib, *[int(v) for v in sys.argv[2:4]])
    if len(sys.argv) >= 4 and sys.argv[1] == "--gemm-once":
        extra = [int(v) for v in sys.argv[4:6]]
        return gemm_once(lib, sys.argv[2], int(sys.argv[3]), *extra)
    peak = _peak()
    tm = Timer(lib)
    s = tm.stream
    out = []

    def report(name, us, nbytes, **extra):
        gbs = nbytes / us / 1e3
        rec = dict(config=name, us=round(us, 2), algorithmic_bytes=nbytes, gbs=round(gbs, 1),
                   pct_of_measured_peak=round(100 * gbs / peak, 1), **extra)
        out.append(rec)
        print(json.dumps(rec), flush=True)

    # ---- config 0: Q4_K dequant of a 14336 x 4096 tensor
    nb = 14336 * 16
    q = synth.q4k_blocks(nb, 1000)
    qs = [_dev(lib, q) for _ in range(4)]
    os_ = [lib.bpdq_alloc(nb * 1024) for _ in range(3)]
    us = tm.run(lambda i: lib.bpd_dequant_q4k_gpu_st(qs[i % 4], os_[i % 3], nb, 0, s), 30)
    report("0: Q4_K dequant 14336x4096", us, nb * (144 + 1024), elements_per_s=nb * 256 / us * 1e6)
    for p in qs + os_:
        lib.bpdq_free(p)

    # ---- config 1: Q8_0 GEMV 4096 x 4096 with in-kernel activation quantization
    N = K = 4096
    W = synth.q8_0_matrix(N, K, 1001)
    n = _copies(W.nbytes)
    ws = [_dev(lib, W) for _ in range(n)]
    x, o = _dev(lib, synth.activations(K, 1002)), lib.bpdq_alloc(N * 4)
    us = tm.run(lambda i: lib.bpd_qmatmul_q8_0_cuda(ws[i % n], x, o, 1, N, K, s), 100)
    report("1: Q8_0 GEMV 4096x4096 (single launches back to back)", us, synth.gemv_bytes_q8_0(N, K))
    # the same product the way the benchmark's step is measured: 32 distinct matrices (567 MB, beyond L2), each
    # with its own vector, recorded once into a CUDA graph (programmatic launch edges kept) and replayed
    n32 = 32
    ws32 = ws[:n32] if n >= n32 else ws + [_dev(lib, W) for _ in range(n32 - n)]
    xs32 = [_dev(lib, synth.activations(K, 1100 + j)) for j in range(n32)]
    os32 = [lib.bpdq_alloc(N * 4) for _ in range(n32)]

    def step32(_):
        for j in range(n32):
            lib.bpd_qmatmul_q8_0_cuda(ws32[j], xs32[j], os32[j], 1, N, K, s)
    step32(0)
    lib.bpdq_stream_sync(s)
    lib.bpdq_graph_begin(s)
    step32(0)
    g = lib.bpdq_graph_end(s)
    us = tm.run(lambda i: lib.bpdq_graph_launch(g, s), 50) / n32
    report("1: Q8_0 GEMV 4096x4096 (32 distinct matrices per graph replay, per product)", us, synth.gemv_bytes_q8_0(N, K))
    lib.bpdq_graph_destroy(g)
    # and as ONE persistent launch of the stream kernel in its Q8_0 mode
    descs = (capi.GemvDesc * n32)(*[capi.GemvDesc(ws32[j], xs32[j], os32[j], N, K) for j in range(n32)])
    sbytes = lib.bpdq_gemv_stream_q8_0_workspace_bytes(n32, descs)
    sws = lib.bpdq_alloc(sbytes)
    plan = lib.bpdq_gemv_stream_create_q8_0(n32, descs, sws, sbytes)
    us = tm.run(lambda i: lib.bpdq_gemv_stream_run_ready(plan, s), 50) / n32
    report("1: Q8_0 GEMV 4096x4096 (32 distinct matrices in one persistent launch, per product)", us, synth.gemv_bytes_q8_0(N, K))
    lib.bpdq_gemv_stream_destroy(plan)
    lib.bpdq_free(sws)
    for p in list(set(ws32) | set(ws)) + xs32 + os32 + [x, o]:
        lib.bpdq_free(p)

    # ---- config 3: Q4_K x Q8_K GEMM, N=14336, K=4096, M tokens
    N, K = 14336, 4096
    W = synth.q4k_matrix(N, K, 1003)
    n = _copies(W.nbytes)
    ws = [_dev(lib, W) for _ in range(n)]
    # the same weights re-tiled in groups of 16 rows (one copy of each rotating matrix)
    ts = []
    for w in ws:
        t = lib.bpdq_alloc(lib.bpd_q4k_rg16_bytes(N, K))
        lib.bpd_repack_q4k_rg16_cuda(w, t, N, K, s)
        ts.append(t)
    lib.bpdq_stream_sync(s)
    for M in (1, 4, 8, 16, 32, 64):
        X = _dev(lib, synth.activations(K, 1004, rows=M))
        o = lib.bpdq_alloc(M * N * 4)
        us = tm.run(lambda i: lib.bpd_qmm_q4k_q8k_rg16_cuda(ts[i % n], X, o, M, N, K, s), 50)
        report(f"3: same product on re-tiled weights (k_gemm_q4k_rg16), M={M}", us, synth.gemv_bytes_q4k(N, K, M),
               tflops=round(2.0 * M * N * K / us / 1e6, 2))
        us = tm.run(lambda i: lib.bpd_qmm_q4k_q8k_cuda(ws[i % n], X, o, M, N, K, 0, 0, None, s), 50)
        report(f"3: Q4_K x Q8_K GEMM M={M} N=14336 K=4096", us, synth.gemv_bytes_q4k(N, K, M),
               tflops=round(2.0 * M * N * K / us / 1e6, 2))
        if M >= 16:
            us = tm.run(lambda i: lib.bpd_qmm_q4k_q8k_tc5_cuda(ws[i % n], X, o, M, N, K, s), 50)
            report(f"3: same, tcgen05 kernel, M={M}", us, synth.gemv_bytes_q4k(N, K, M),
                   tflops=round(2.0 * M * N * K / us / 1e6, 2))
            us = tm.run(lambda i: lib.bpd_qmm_q4k_q8k_mma_cuda(ws[i % n], X, o, M, N, K, s), 50)
            report(f"3: same, mma.sync kernel, M={M}", us, synth.gemv_bytes_q4k(N, K, M),
                   tflops=round(2.0 * M * N * K / us / 1e6, 2))
        lib.bpdq_free(X)
        lib.bpdq_free(o)
    # ---- W4A32 drop-in on the same matrix
    x, o = _dev(lib, synth.activations(K, 1005)), lib.bpdq_alloc(N * 4)
    us = tm.run(lambda i: lib.bpd_qmatmul_q4k_gpu_st(ws[i % n], x, o, N, K, s), 20)
    report("W4A32 GEMV 14336x4096 (bpd_qmatmul_q4k_gpu)", us, synth.gemv_bytes_q4k(N, K))
    for p in ws + ts + [x, o]:
        lib.bpdq_free(p)
    status = lib.bpdq_last_status()
    print(json.dumps({"status": status}))
    return 0 if status == 0 else 1


if __name__ == "__main__":
    sys.exit(main())

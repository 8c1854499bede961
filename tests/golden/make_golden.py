#!/usr/bin/env python3
"""Generates tests/golden/*.npz from the reference's own C code.

Run where the reference tree is available (it compiles bench/bpd_quant.c, bench/bpd_cpu.c and
bench/bpd_gemm_q8_0_cpu.c unmodified through oracle/Makefile):

    python tests/golden/make_golden.py

Each fixture holds seeded inputs (or the seed and generator arguments when the input is
large), and what the reference returned for them: full outputs for small cases, SHA-256 of
the output bytes plus a strided sample for large ones.  The GPU box has no reference tree, so
the tests compare against these files.
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from bpd_substrate_b200 import synth  # noqa: E402
from oracle import binding  # noqa: E402


# the tiny Llama of the forward-pass fixture (shared with tests/test_llama_forward.py)
LLAMA_TINY = dict(n_layers=2, n_heads=4, n_kv_heads=2, head_dim=32, ffn_dim=256, vocab_size=96, max_seq_len=16)
LLAMA_TINY_SEED = 77
LLAMA_TINY_STEPS = (("prefill", [3, 17, 95, 0, 42]), ("step1", [7]), ("step2", [64]))


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def avx_tiles_fixture(ra):
    """The tile dispatcher and three single tiles of the AVX build on ragged shapes (every RM x RN
    combination occurs in 37 weight rows x 7 activation rows)."""
    rng = np.random.default_rng(4250)
    mw, mt, K = 37, 7, 1024
    W = synth.q8_0_matrix(mw, K, rng)
    X = synth.activations(K, rng, rows=mt)
    rb = K // 32 * 34
    Xq = np.zeros(mt * rb, np.uint8)
    ra.bpd_quant_q8_0_cpu(X.ctypes.data, Xq.ctypes.data, mt * K)
    disp = np.empty((mt, mw), np.float32)
    ra.bpd_qmatmul_q8_0_dispatch_cpu(W.ctypes.data, Xq.ctypes.data, disp.ctypes.data, mw, mt, K)
    lf = np.empty((mt, mw), np.float32)
    ra.bpd_qmatmul_q8_0_llamafile_cpu(W.ctypes.data, X.ctypes.data, lf.ctypes.data, mw, mt, K)
    tiles = {}
    for rm, rn in ((4, 4), (2, 1), (1, 2)):
        o = np.zeros((rn, 8), np.float32)          # ldc = 8
        getattr(ra, f"bpd_gemm_q8_0_{rm}_{rn}_cpu")(W.ctypes.data + 3 * rb, Xq.ctypes.data + rb, K // 32, rb, rb,
                                                     o.ctypes.data, 8)
        tiles[f"tile_{rm}_{rn}"] = o.view(np.uint32)
    np.savez_compressed(os.path.join(HERE, "q8_0_avx_tiles.npz"), W=W, X=X, Xq=Xq, dispatch=disp.view(np.uint32),
                        llamafile=lf.view(np.uint32), shape=np.array([mw, mt, K]), **tiles)


def main():
    binding.build()
    rq = binding.load_ref("bpd_quant.so")
    rc = binding.load_ref("bpd_cpu.so")        # scalar Q8_0 paths (the reference's default -O2 build)
    ra = binding.load_ref("bpd_cpu_avx.so")    # AVX1 Q8_0 paths + the tile dispatcher

    # ---- Q4_K dequant, small: inputs and all outputs
    nb = 48
    q = synth.q4k_blocks(nb, 4242)
    out = np.empty(nb * 256, np.float32)
    rq.bpd_dequant_q4k(q.ctypes.data, out.ctypes.data, nb)
    # ---- Q4_K W4A32 GEMV and GEMM, small
    M, K, N = 12, 1024, 3
    W = synth.q4k_matrix(M, K, 4243)
    x = synth.activations(K, 4244)
    y = np.empty(M, np.float32)
    rq.bpd_qmatmul_q4k(W.ctypes.data, x.ctypes.data, y.ctypes.data, M, K)
    B = synth.activations(N, 4245, rows=K)
    Cm = np.empty((M, N), np.float32)
    rq.bpd_qmm_q4k(W.ctypes.data, B.ctypes.data, Cm.ctypes.data, M, N, K)
    np.savez_compressed(os.path.join(HERE, "q4k_small.npz"), q=q, dequant=out.view(np.uint32),
                        W=W, x=x, gemv=y.view(np.uint32), B=B, gemm=Cm.view(np.uint32), shape=np.array([M, K, N]))

    # ---- Q4_K dequant of the whole benchmark tensor (14336 x 4096): hash + strided sample
    nb = 14336 * 16
    q = synth.q4k_blocks(nb, 1000)
    out = np.empty(nb * 256, np.float32)
    rq.bpd_dequant_q4k(q.ctypes.data, out.ctypes.data, nb)
    np.savez_compressed(os.path.join(HERE, "q4k_dequant_14336x4096.npz"), seed=np.array([1000]), n_blocks=np.array([nb]),
                        input_sha256=np.array([sha(q)]), output_sha256=np.array([sha(out)]),
                        sample_stride=np.array([65537]), sample=out[::65537].view(np.uint32))

    # ---- Q8_0: dequant, quantize, dot, matmul (scalar build), dispatcher (AVX build)
    rng = np.random.default_rng(4246)
    Nw, Kq, Mt = 8, 256, 2
    Wq = synth.q8_0_matrix(Nw, Kq, rng)
    Wq[0:2] = [0x01, 0x00]            # subnormal fp16 scale in the first block (tests/verify_f16_fix.py:99-117)
    Wq[34:36] = [0xC2, 0x00]          # another subnormal (tests/check_dequant_subnormal.py)
    X = (rng.standard_normal((Mt, Kq)) * 0.3).astype(np.float32)
    deq = np.empty(Nw * Kq, np.float32)
    rc.bpd_dequant_q8_0_cpu(Wq.ctypes.data, deq.ctypes.data, Nw * Kq // 32)
    Xq = np.zeros(Mt * Kq // 32 * 34, np.uint8)
    rc.bpd_quant_q8_0_cpu(X.ctypes.data, Xq.ctypes.data, Mt * Kq)
    mm = np.empty((Mt, Nw), np.float32)
    rc.bpd_qmatmul_q8_0_cpu(Wq.ctypes.data, X.ctypes.data, mm.ctypes.data, Mt, Nw, Kq)
    mm_avx = np.empty((Mt, Nw), np.float32)      # out[token*m_weight + row]
    ra.bpd_qmatmul_q8_0_llamafile_cpu(Wq.ctypes.data, X.ctypes.data, mm_avx.ctypes.data, Nw, Mt, Kq)
    np.savez_compressed(os.path.join(HERE, "q8_0_small.npz"), W=Wq, X=X, dequant=deq.view(np.uint32), Xq=Xq,
                        matmul_scalar=mm.view(np.uint32), matmul_avx_tiles=mm_avx.view(np.uint32),
                        shape=np.array([Mt, Nw, Kq]))

    avx_tiles_fixture(ra)

    # ---- Q8_0 GEMV of the benchmark shape 4096 x 4096: hash + sample (scalar build)
    W = synth.q8_0_matrix(4096, 4096, 1001)
    x = synth.activations(4096, 1002)
    y = np.empty((1, 4096), np.float32)
    rc.bpd_qmatmul_q8_0_cpu(W.ctypes.data, x.ctypes.data, y.ctypes.data, 1, 4096, 4096)
    np.savez_compressed(os.path.join(HERE, "q8_0_gemv_4096x4096.npz"), w_seed=np.array([1001]), x_seed=np.array([1002]),
                        input_sha256=np.array([sha(W)]), out=y.view(np.uint32))
    # ---- Q8_0 Llama forward of a tiny synthetic model (bpd_llama_forward_cpu, scalar build): prefill of
    # five tokens, then two single-token steps against the f16 KV cache
    from bpd_substrate_b200 import llama
    cfg = llama.make_config(**LLAMA_TINY)
    model = llama.SyntheticLlama(cfg, seed=LLAMA_TINY_SEED)
    w, keep = model.host_structs()
    k, v = model.kv_cache()
    steps, kv_pos = {}, 0
    for name, toks in LLAMA_TINY_STEPS:
        pos = np.arange(kv_pos, kv_pos + len(toks), dtype=np.int32)
        logits, out = binding.llama_forward_with(rc.bpd_llama_forward_cpu, w, cfg, toks, pos, kv_pos, k, v)
        steps[f"{name}_logits"] = logits.view(np.uint32)
        steps[f"{name}_tokens"] = out
        kv_pos += len(toks)
    np.savez_compressed(os.path.join(HERE, "llama_tiny.npz"), k_cache=k, v_cache=v, **steps)
    del keep
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()

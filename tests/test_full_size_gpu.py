"""The Q4_K x Q8_K kernels against the CPU checker at the benchmark configurations' own sizes.

Small shapes leave parts of the kernels idle: with few tiles every consumer warp of the batched kernel
gets at most one, so its weight ring never wraps; the tensor-core kernels never see more row tiles than
SMs.  Here one whole Mistral-7B-shaped layer goes through ONE batched launch (37,888 rows: every warp
walks its ring slots many times), the 14336 x 4096 product runs at 1, 4, 16 and 64 tokens through every
kernel that can take it, and the row shards of the 70B-shaped model are covered, with the integer part
compared exactly and the fp32 outputs norm-wise.
"""
import numpy as np
import pytest

from bpd_substrate_b200 import capi, synth
from tests.util import Dev, normwise

pytestmark = pytest.mark.gpu
TOL = 1e-5   # norm-wise max|d| / max|ref| on fp32 outputs, against the checker's binary64 sum


def _batched(lib, entry, mats, ws=True):
    """mats: list of (W, x, rows, cols) -> outputs of one call of a batched entry."""
    dW = [Dev(lib, w) for w, _, _, _ in mats]
    dX = [Dev(lib, x) for _, x, _, _ in mats]
    dO = [Dev(lib, nbytes=rows * 4, fill=0xFF) for _, _, rows, _ in mats]
    descs = (capi.GemvDesc * len(mats))(*[capi.GemvDesc(dW[j].ptr, dX[j].ptr, dO[j].ptr, rows, cols)
                                          for j, (_, _, rows, cols) in enumerate(mats)])
    if ws:
        nbytes = lib.bpdq_batch_workspace_bytes(len(mats), descs)
        scratch = Dev(lib, nbytes=nbytes, fill=0xCD)
        assert getattr(lib, entry)(len(mats), descs, scratch.ptr, nbytes, None) == 0
    else:
        assert getattr(lib, entry)(len(mats), descs, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    return [o.read(np.float32) for o in dO]


def test_whole_mistral_layer_in_one_batched_launch(lib, oracle):
    """Benchmark configuration 2, one layer: seven products of full size, each with its own vector, through
    bpd_qmatmul_q4k_q8k_batch_ready_cuda (the bench's entry) and the allocation-free plain entry.  Also
    reports how far the 8-bit activations move the result from the reference's fp32-activation GEMV
    (bpd_qmatmul_q4k, bench/bpd_quant.c:88-109): quantization noise of about 1e-2 norm-wise."""
    rng = np.random.default_rng(2024)
    mats = []
    for _, rows, cols in synth.MISTRAL_LAYER:
        mats.append((synth.q4k_matrix(rows, cols, rng), synth.activations(cols, rng), rows, cols))
    got = _batched(lib, "bpd_qmatmul_q4k_q8k_batch_ready_cuda", mats)
    plain = _batched(lib, "bpd_qmatmul_q4k_q8k_batch_cuda", mats, ws=False)
    worst, dist = 0.0, 0.0
    for j, (W, x, rows, cols) in enumerate(mats):
        ref32, ref64 = oracle.qmatmul_q4k_q8k(W, oracle.quant_q8_K(x), rows, cols)
        e = normwise(got[j], ref64)
        worst = max(worst, e)
        assert e <= TOL, (j, rows, cols, e)
        assert normwise(got[j], ref32) <= TOL
        assert np.array_equal(got[j].view(np.uint32), plain[j].view(np.uint32)), j
        # distance to the reference's own W4A32 result on the same inputs
        w4a32 = oracle.qmatmul_q4k_f64(W, x, rows, cols)
        dist = max(dist, normwise(got[j], w4a32))
    print(f"\nconfig 2 layer: worst norm-wise error vs checker {worst:.2e}; distance to the W4A32 GEMV {dist:.2e}")
    assert 1e-4 < dist < 5e-2    # int8 activations: visible, and no more than quantization noise


@pytest.mark.parametrize("tokens", [1, 4, 16, 64])
def test_config3_14336x4096_every_kernel(lib, oracle, tokens):
    """Benchmark configuration 3 (N = 14336, K = 4096) at 1, 4, 16, 64 tokens: the dispatcher, the dp4a kernel
    (up to 4 tokens: exact sub-block dots of token 0), the mma.sync kernel, the tcgen05 kernel and the streaming
    kernel on re-tiled weights (exact (isum, msum) of every token, row and super-block)."""
    N, K = 14336, 4096
    rng = np.random.default_rng(300 + tokens)
    W = synth.q4k_matrix(N, K, rng)
    X = synth.activations(K, rng, rows=tokens)
    _, ref64 = oracle.qmm_q4k_q8k(W, X, tokens, N, K)
    ints = oracle.qmm_q4k_q8k_ints(W, X, tokens, N, K)
    dW, dX = Dev(lib, W), Dev(lib, X)

    def run(entry):
        dO = Dev(lib, nbytes=tokens * N * 4, fill=0xFF)
        dI = None
        if entry == "dispatch":
            rc = lib.bpd_qmm_q4k_q8k_cuda(dW.ptr, dX.ptr, dO.ptr, tokens, N, K, 0, 0, None, None)
        elif entry == "dp4a":
            dI = Dev(lib, nbytes=N * (K // 256) * 8 * 4, fill=0xEE)
            rc = lib.bpd_qmm_q4k_q8k_cuda(dW.ptr, dX.ptr, dO.ptr, tokens, N, K, 0, 0, dI.ptr, None)
        else:
            dI = Dev(lib, nbytes=tokens * N * (K // 256) * 2 * 4, fill=0xEE)
            w = dT if entry == "rg16" else dW     # the product on weights re-tiled in groups of 16 rows
            rc = getattr(lib, f"bpd_qmm_q4k_q8k_{entry}_ints_cuda")(w.ptr, dX.ptr, dO.ptr, dI.ptr, tokens, N, K, None)
        assert rc == 0
        lib.bpdq_sync()
        assert lib.bpdq_last_status() == 0
        return dO.read(np.float32).reshape(tokens, N), dI

    dT = Dev(lib, nbytes=lib.bpd_q4k_rg16_bytes(N, K))
    assert lib.bpd_repack_q4k_rg16_cuda(dW.ptr, dT.ptr, N, K, None) == 0

    for entry in ("dispatch", "mma", "tc5", "rg16") + (("dp4a",) if tokens <= 4 else ()):
        out, dI = run(entry)
        assert normwise(out, ref64) <= TOL, entry
        if entry == "dp4a":
            dots = dI.read(np.int32).reshape(N, K // 256, 8)
            assert np.array_equal(dots, oracle.q4k_q8k_subdots(W, oracle.quant_q8_K(X[0]), N, K))
        elif dI is not None:
            assert np.array_equal(dI.read(np.int32).reshape(tokens, N, K // 256, 2), ints), entry


@pytest.mark.parametrize("tokens,N,K", [(5, 300, 1024), (33, 1280, 2048), (64, 4096, 14336 // 2), (100, 256, 512)])
def test_tensor_core_kernels_exact_integers(lib, oracle, tokens, N, K):
    """Ragged shapes (partial row tiles and token tiles, split K, more than 64 tokens): the integer pair of
    every (token, row, super-block) from both tensor-core kernels equals the checker's."""
    rng = np.random.default_rng(tokens + N + K)
    W = synth.q4k_matrix(N, K, rng)
    X = synth.activations(K, rng, rows=tokens)
    ints = oracle.qmm_q4k_q8k_ints(W, X, tokens, N, K)
    _, ref64 = oracle.qmm_q4k_q8k(W, X, tokens, N, K)
    dW, dX = Dev(lib, W), Dev(lib, X)
    for entry in ("mma", "tc5"):
        dO = Dev(lib, nbytes=tokens * N * 4, fill=0xFF)
        dI = Dev(lib, nbytes=ints.nbytes, fill=0xEE)
        assert getattr(lib, f"bpd_qmm_q4k_q8k_{entry}_ints_cuda")(dW.ptr, dX.ptr, dO.ptr, dI.ptr, tokens, N, K, None) == 0
        lib.bpdq_sync()
        assert lib.bpdq_last_status() == 0
        assert np.array_equal(dI.read(np.int32).reshape(ints.shape), ints), entry
        assert normwise(dO.read(np.float32).reshape(tokens, N), ref64) <= TOL, entry


def test_llama70b_row_shards(lib, oracle):
    """Benchmark configuration 4: what one of eight GPUs holds of a 70B-shaped layer (rows / 8 of every matrix;
    K = 8192 and 28672) in one batched launch, and its shard of the output head (16,032 rows)."""
    rng = np.random.default_rng(70)
    world = 8
    mats = []
    for _, rows, cols in synth.LLAMA70B_LAYER:
        r = rows // world
        mats.append((synth.q4k_matrix(r, cols, rng), synth.activations(cols, rng), r, cols))
    got = _batched(lib, "bpd_qmatmul_q4k_q8k_batch_ws_cuda", mats)
    for j, (W, x, rows, cols) in enumerate(mats):
        _, ref64 = oracle.qmatmul_q4k_q8k(W, oracle.quant_q8_K(x), rows, cols)
        assert normwise(got[j], ref64) <= TOL, (j, rows, cols)
    _, rows, cols = synth.LLAMA70B_HEAD
    r = rows // world
    W, x = synth.q4k_matrix(r, cols, rng), synth.activations(cols, rng)
    head = _batched(lib, "bpd_qmatmul_q4k_q8k_batch_ws_cuda", [(W, x, r, cols)])[0]
    assert normwise(head, oracle.qmatmul_q4k_q8k(W, oracle.quant_q8_K(x), r, cols)[1]) <= TOL


def test_llama70b_shard_as_one_persistent_stream(lib, oracle):
    """The same shard through bpdq_gemv_stream_run: the rows of K = 28672 (112 super-blocks) arrive in two pieces per
    row; every output equals the batched entry's bit for bit and the checker's within the bar."""
    rng = np.random.default_rng(72)
    world = 8
    mats = []
    for _, rows, cols in synth.LLAMA70B_LAYER:
        r = rows // world
        mats.append((synth.q4k_matrix(r, cols, rng), synth.activations(cols, rng), r, cols))
    want = _batched(lib, "bpd_qmatmul_q4k_q8k_batch_ws_cuda", mats)
    dW = [Dev(lib, w) for w, _, _, _ in mats]
    dX = [Dev(lib, x) for _, x, _, _ in mats]
    dO = [Dev(lib, nbytes=rows * 4, fill=0xFF) for _, _, rows, _ in mats]
    n = len(mats)
    descs = (capi.GemvDesc * n)(*[capi.GemvDesc(dW[j].ptr, dX[j].ptr, dO[j].ptr, rows, cols)
                                  for j, (_, _, rows, cols) in enumerate(mats)])
    nbytes = lib.bpdq_batch_workspace_bytes(n, descs)
    ws = Dev(lib, nbytes=nbytes, fill=0xCD)
    h = lib.bpdq_gemv_stream_create(n, descs, ws.ptr, nbytes)
    assert h
    assert lib.bpdq_gemv_stream_run(h, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    for j, (W, x, rows, cols) in enumerate(mats):
        got = dO[j].read(np.float32)
        assert np.array_equal(got.view(np.uint32), want[j].view(np.uint32)), j
        assert normwise(got, oracle.qmatmul_q4k_q8k(W, oracle.quant_q8_K(x), rows, cols)[1]) <= TOL, j
    lib.bpdq_gemv_stream_destroy(h)


def test_llama70b_shard_eight_tokens(lib, oracle):
    """Configuration 4 at batch 8: the w1 shard (3584 x 8192) and the w2 shard (1024 x 28672) at eight tokens
    through the dispatcher."""
    rng = np.random.default_rng(71)
    for rows, cols in ((3584, 8192), (1024, 28672)):
        W = synth.q4k_matrix(rows, cols, rng)
        X = synth.activations(cols, rng, rows=8)
        dW, dX, dO = Dev(lib, W), Dev(lib, X), Dev(lib, nbytes=8 * rows * 4, fill=0xFF)
        assert lib.bpd_qmm_q4k_q8k_cuda(dW.ptr, dX.ptr, dO.ptr, 8, rows, cols, 0, 0, None, None) == 0
        lib.bpdq_sync()
        assert lib.bpdq_last_status() == 0
        _, ref64 = oracle.qmm_q4k_q8k(W, X, 8, rows, cols)
        assert normwise(dO.read(np.float32).reshape(8, rows), ref64) <= TOL, (rows, cols)
        # and on the weights re-tiled in groups of 16 rows (what the 8-token sweep of the benchmark runs)
        dT = Dev(lib, nbytes=lib.bpd_q4k_rg16_bytes(rows, cols))
        assert lib.bpd_repack_q4k_rg16_cuda(dW.ptr, dT.ptr, rows, cols, None) == 0
        dI = Dev(lib, nbytes=8 * rows * (cols // 256) * 8, fill=0xEE)
        assert lib.bpd_qmm_q4k_q8k_rg16_ints_cuda(dT.ptr, dX.ptr, dO.ptr, dI.ptr, 8, rows, cols, None) == 0
        lib.bpdq_sync()
        assert lib.bpdq_last_status() == 0
        assert normwise(dO.read(np.float32).reshape(8, rows), ref64) <= TOL, (rows, cols)
        assert np.array_equal(dI.read(np.int32).reshape(8, rows, cols // 256, 2), oracle.qmm_q4k_q8k_ints(W, X, 8, rows, cols))

"""Scratch memory of the compute entries: caller-owned workspaces (*_ws_cuda) and the library's
per-stream blocks behave as include/bpdq.h says -- no state shared between streams, no allocation and
no freed block under a graph, a clear status when a block would have to grow during capture."""
import numpy as np
import pytest

from bpd_substrate_b200 import synth
from tests.util import Dev

pytestmark = pytest.mark.gpu


def _cases():
    rng = np.random.default_rng(900)
    out = []
    for tokens, N, K in ((16, 384, 1024), (40, 256, 2048), (5, 128, 4096), (64, 512, 512)):
        out.append((tokens, N, K, synth.q4k_matrix(N, K, rng), synth.activations(K, rng, rows=tokens)))
    return out


def test_two_streams_interleaved_equal_serial_results(lib):
    """Many-token products issued alternately on two streams, each stream with its own workspace (and, in
    the second round, with the library's own per-stream blocks), give the bits of the same calls made one
    after the other on one stream."""
    cases = _cases()
    dev = [(Dev(lib, W), Dev(lib, X)) for _, _, _, W, X in cases]

    def run(streams, use_ws):
        outs, keep = [], []
        for rep in range(3):
            for i, (tokens, N, K, _, _) in enumerate(cases):
                s = streams[(i + rep) % len(streams)]
                dO = Dev(lib, nbytes=tokens * N * 4, fill=0xFF)
                if use_ws:
                    nbytes = lib.bpdq_qmm_q4k_q8k_workspace_bytes(tokens, N, K)
                    assert nbytes > 0
                    ws = Dev(lib, nbytes=nbytes, fill=0xAB)
                    keep.append(ws)
                    rc = lib.bpd_qmm_q4k_q8k_ws_cuda(dev[i][0].ptr, dev[i][1].ptr, dO.ptr, tokens, N, K, 0, 0, None, ws.ptr,
                                                     nbytes, s)
                else:
                    rc = lib.bpd_qmm_q4k_q8k_cuda(dev[i][0].ptr, dev[i][1].ptr, dO.ptr, tokens, N, K, 0, 0, None, s)
                assert rc == 0
                outs.append(dO)
        lib.bpdq_sync()
        assert lib.bpdq_last_status() == 0
        return [o.read(np.uint32) for o in outs]

    s1, s2 = lib.bpdq_stream_create(), lib.bpdq_stream_create()
    try:
        serial = run([s1], use_ws=True)
        for use_ws in (True, False):
            both = run([s1, s2], use_ws)
            for a, b in zip(serial, both):
                assert np.array_equal(a, b)
    finally:
        lib.bpdq_stream_destroy(s1)
        lib.bpdq_stream_destroy(s2)


def test_workspace_too_small_is_refused(lib):
    tokens, N, K, W, X = _cases()[0]
    dW, dX, dO = Dev(lib, W), Dev(lib, X), Dev(lib, nbytes=tokens * N * 4)
    ws = Dev(lib, nbytes=4096)
    assert lib.bpd_qmm_q4k_q8k_ws_cuda(dW.ptr, dX.ptr, dO.ptr, tokens, N, K, 0, 0, None, ws.ptr, 4096, None) == -3
    assert lib.bpd_qmm_q4k_q8k_ws_cuda(dW.ptr, dX.ptr, dO.ptr, tokens, N, K, 0, 0, None, ws.ptr + 4, 4096, None) == -2
    assert lib.bpd_qmm_q4k_q8k_ws_cuda(dW.ptr, dX.ptr, dO.ptr, tokens, N, K, 0, 0, None, None, 0, None) == -1
    lib.bpdq_clear_status()


def test_scratch_cannot_grow_during_capture_and_graphs_survive_growth(lib):
    """A graph recorded at one size keeps working after a larger call has made the library replace the
    stream's block (the old block stays allocated); a call that would have to grow the block while the
    stream is being captured returns -5 and records nothing."""
    rng = np.random.default_rng(901)
    N, K = 256, 1024
    W = synth.q4k_matrix(N, K, rng)
    X = synth.activations(K, rng, rows=64)
    dW, dX = Dev(lib, W), Dev(lib, X)
    small, big = Dev(lib, nbytes=16 * N * 4, fill=0xFF), Dev(lib, nbytes=64 * N * 4, fill=0xFF)
    s = lib.bpdq_stream_create()
    try:
        # a fresh stream has no block yet: the first call inside a capture cannot create one
        assert lib.bpdq_graph_begin(s) == 0
        assert lib.bpd_qmm_q4k_q8k_mma_cuda(dW.ptr, dX.ptr, small.ptr, 16, N, K, s) == -5
        g0 = lib.bpdq_graph_end(s)
        if g0:
            lib.bpdq_graph_destroy(g0)
        lib.bpdq_clear_status()
        # warm-up outside capture, then the capture succeeds
        assert lib.bpd_qmm_q4k_q8k_mma_cuda(dW.ptr, dX.ptr, small.ptr, 16, N, K, s) == 0
        assert lib.bpdq_stream_sync(s) == 0
        want = small.read(np.uint32)
        assert lib.bpdq_graph_begin(s) == 0
        assert lib.bpd_qmm_q4k_q8k_mma_cuda(dW.ptr, dX.ptr, small.ptr, 16, N, K, s) == 0
        g = lib.bpdq_graph_end(s)
        assert g
        # a much larger product on the same stream replaces the block (1 MiB minimum: ask for more)
        Nb, Kb = 128, 16384
        Wb = Dev(lib, synth.q4k_matrix(Nb, Kb, rng))
        Xb = Dev(lib, synth.activations(Kb, rng, rows=64))
        Ob = Dev(lib, nbytes=64 * Nb * 4)
        assert lib.bpd_qmm_q4k_q8k_mma_cuda(Wb.ptr, Xb.ptr, Ob.ptr, 64, Nb, Kb, s) == 0
        # the graph still holds the old block: replay and compare
        lib.bpdq_memset_async(small.ptr, 0xFF, small.nbytes, s)
        assert lib.bpdq_graph_launch(g, s) == 0
        assert lib.bpdq_stream_sync(s) == 0
        assert np.array_equal(small.read(np.uint32), want)
        lib.bpdq_graph_destroy(g)
        assert lib.bpdq_last_status() == 0
        del big
    finally:
        lib.bpdq_stream_destroy(s)

"""Row sharding + all-gather on two CPU ranks (gloo): the gathered result of per-rank shards
equals the unsharded result bit for bit."""
import os
import socket

import numpy as np
import pytest

from bpd_substrate_b200 import shard, synth


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, tokens, rows, cols, q):
    import torch
    import torch.distributed as dist
    from oracle.binding import Oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        orc = Oracle()
        W = synth.q4k_matrix(rows, cols, 31)
        X = synth.activations(cols, 32, rows=tokens)
        mine = shard.shard_q4k(W, rows, cols, rank, world)
        local, _ = orc.qmm_q4k_q8k(mine, X, tokens, rows // world, cols)
        full = shard.all_gather_outputs(torch.from_numpy(local), tokens, rows)
        want, _ = orc.qmm_q4k_q8k(W, X, tokens, rows, cols)
        ok = np.array_equal(full.numpy().view(np.uint32), want.view(np.uint32))
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("tokens", [1, 3])
def test_two_rank_row_shard_gather(tokens):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, tokens, 64, 512, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    results = dict(q.get(timeout=5) for _ in range(2))
    assert results == {0: True, 1: True}


def test_row_ranges_cover_every_benchmark_shape():
    for shapes in (synth.MISTRAL_LAYER, synth.LLAMA70B_LAYER, (synth.LLAMA70B_HEAD,)):
        for _, rows, cols in shapes:
            for world in (1, 2, 4, 8):
                spans = [shard.row_range(rows, r, world) for r in range(world)]
                assert spans[0][0] == 0 and spans[-1][1] == rows
                assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
                # shards start on 16-byte boundaries (bulk copies need it)
                assert all((lo * synth.q4k_row_bytes(cols)) % 16 == 0 for lo, _ in spans)
    with pytest.raises(ValueError):
        shard.row_range(10, 0, 4)


def test_algorithmic_bytes_match_the_published_arithmetic():
    per_layer = sum(synth.gemv_bytes_q4k(r, c) for _, r, c in synth.MISTRAL_LAYER)
    assert per_layer == 123_011_072 and 32 * per_layer == 3_936_354_304
    assert synth.gemv_bytes_q8_0(4096, 4096) == 17_858_560
    assert [synth.gemv_bytes_q4k(14336, 4096, m) for m in (1, 4, 16, 64)] == [33_103_872, 33_325_056, 34_209_792, 37_748_736]

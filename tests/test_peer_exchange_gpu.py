"""Peer stores in the batched product's epilogue and the per-step flags, as far as one GPU goes: the targets
are buffers of this same device (the kernel path is the same; only the addresses differ on several GPUs).
The several-rank check is `python -m bpd_substrate_b200.peer` under torchrun; it runs here when two GPUs exist."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

from bpd_substrate_b200 import capi, synth
from bpd_substrate_b200.dispatch import LayerSet
from tests.util import Dev

pytestmark = pytest.mark.gpu


def test_results_also_land_in_every_registered_target(lib):
    ls = LayerSet(synth.MISTRAL_LAYER, 2, seed=31)
    try:
        x = np.random.default_rng(5).standard_normal(ls.x_bytes // 4).astype(np.float32)
        ls.upload_activations(x)
        ls.step("batched")
        plain = ls.download_outputs().copy()
        # three targets at different offsets of one arena, as three ranks' gathered buffers would be
        arena = Dev(lib, nbytes=3 * ls.o_bytes + 4096, fill=0xCD)
        targets = (C.c_void_p * 3)(arena.ptr, arena.ptr + ls.o_bytes + 1024, arena.ptr + 2 * ls.o_bytes + 2048)
        assert lib.bpdq_set_peer_outputs(ls.d_out, ls.o_bytes, 3, targets) == 0
        try:
            lib.bpdq_memset_async(ls.d_out, 0, ls.o_bytes, ls.stream)
            ls.step("batched", tag="peers")
        finally:
            assert lib.bpdq_set_peer_outputs(None, 0, 0, None) == 0
        lib.bpdq_stream_sync(ls.stream)
        assert lib.bpdq_last_status() == 0
        assert np.array_equal(ls.download_outputs().view(np.uint32), plain.view(np.uint32))
        raw = arena.read(np.uint8)
        for off in (0, ls.o_bytes + 1024, 2 * ls.o_bytes + 2048):
            assert np.array_equal(raw[off:off + ls.o_bytes].view(np.uint32), plain.view(np.uint32).ravel())
        # the gaps between the targets are untouched
        assert (raw[ls.o_bytes:ls.o_bytes + 1024] == 0xCD).all() and (raw[3 * ls.o_bytes + 2048:] == 0xCD).all()
        # outputs outside the registered range: no peer stores, the launch is the plain one
        ls.step("batched")
        lib.bpdq_stream_sync(ls.stream)
        assert lib.bpdq_last_status() == 0
    finally:
        ls.close()


def test_flags_signal_wait_and_bounded_wait(lib):
    flags = Dev(lib, np.zeros(8, np.uint32))
    slots = (C.c_void_p * 2)(flags.ptr + 4, flags.ptr + 12)
    assert lib.bpdq_peer_signal(slots, 2, 7, None) == 0
    assert lib.bpdq_peer_wait(flags.ptr + 4, 1, 7, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    assert list(flags.read(np.uint32)) == [0, 7, 0, 7, 0, 0, 0, 0]
    # both in one launch: slot i and flag i belong to the same rank
    one = (C.c_void_p * 1)(flags.ptr + 20)
    assert lib.bpdq_peer_signal_wait(one, flags.ptr + 20, 1, 3, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0 and flags.read(np.uint32)[5] == 3
    # flags only grow: an older value is satisfied at once
    assert lib.bpdq_peer_wait(flags.ptr + 4, 1, 5, None) == 0
    lib.bpdq_sync()
    assert lib.bpdq_last_status() == 0
    # a flag that nothing raises: the wait gives up and reports instead of hanging
    try:
        assert lib.bpdq_peer_wait(flags.ptr, 1, 1, None) == 0
        lib.bpdq_sync()
        assert lib.bpdq_last_status() == -4
    finally:
        lib.bpdq_clear_status()
    assert lib.bpdq_peer_signal(slots, 9, 1, None) != 0      # more slots than ranks of a node
    assert lib.bpdq_set_peer_outputs(flags.ptr, 64, 1, (C.c_void_p * 1)(flags.ptr + 4)) != 0   # misaligned target
    lib.bpdq_clear_status()
    handle = (C.c_char * 64)()
    assert lib.bpdq_ipc_export(flags.ptr, handle) == 0 and any(handle.raw)


def test_two_ranks_against_nccl_all_gather():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                          "127.0.0.1", "--master-port", "29533", "-m", "bpd_substrate_b200.peer"], cwd=root, capture_output=True,
                         text=True, timeout=600)
    assert out.returncode == 0 and "selftest: ok" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]

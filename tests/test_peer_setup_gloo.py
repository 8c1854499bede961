"""Set-up of the peer exchange on two CPU ranks (gloo) against a fake of the C library: the address arithmetic of
targets and flag slots, and that a rank whose mapping call fails makes EVERY rank give up together (no rank is
left waiting in a collective call)."""
import ctypes as C
import os
import socket


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


class FakeLib:
    """The entry points PeerExchange calls, on plain integers.  Rank r's allocation sits at (r + 1) << 40; a handle
    is the owner's rank; importing rank o's handle on rank r gives (o + 1) << 40 | r << 32 (a distinct mapping)."""

    def __init__(self, rank, fail_import=False, status=0):
        self.rank, self.fail_import, self.status = rank, fail_import, status
        self.registered, self.signals, self.waits, self.closed, self.freed = None, [], [], [], []

    def bpdq_alloc(self, n):
        self.alloc_bytes = n
        return (self.rank + 1) << 40

    def bpdq_memset_async(self, *a):
        return 0

    def bpdq_stream_sync(self, *a):
        return 0

    def bpdq_ipc_export(self, ptr, handle):
        handle[0] = bytes([self.rank + 1])
        return 0

    def bpdq_ipc_import(self, handle):
        if self.fail_import:
            return None
        owner = handle.raw[0] - 1
        return ((owner + 1) << 40) | (self.rank << 32)

    def bpdq_ipc_close(self, p):
        self.closed.append(p)
        return 0

    def bpdq_free(self, p):
        self.freed.append(p)

    def bpdq_last_status(self):
        return self.status

    def bpdq_clear_status(self):
        pass

    def bpdq_set_peer_outputs(self, base, nbytes, n, targets):
        self.registered = None if not n else (base, nbytes, [targets[i] for i in range(n)])
        return 0

    def bpdq_peer_signal(self, slots, n, value, stream):
        self.signals.append(([slots[i] for i in range(n)], value))
        return 0

    def bpdq_peer_signal_wait(self, slots, flags, n, value, stream):
        self.signals.append(([slots[i] for i in range(n)], value))
        self.waits.append((flags, n, value))
        return 0

    def bpdq_peer_wait(self, flags, n, value, stream):
        self.waits.append((flags, n, value))
        return 0


def _worker(rank, world, port, failing_rank, q, timed_out_rank=-1):
    import torch.distributed as dist
    from bpd_substrate_b200 import capi
    from bpd_substrate_b200.peer import PeerExchange
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lib = FakeLib(rank, fail_import=(rank == failing_rank), status=-4 if rank == timed_out_rank else 0)
        slot = 4096
        try:
            ex = PeerExchange(lib, dist, rank, world, slot)
        except capi.BpdqError as exc:
            q.put((rank, "raised", str(exc), lib.freed, lib.closed))
            return
        own = (rank + 1) << 40
        other = ((2 - rank) << 40) | (rank << 32)        # the other rank's buffer as mapped here
        bases = [own, other] if rank == 0 else [other, own]
        assert ex.bases == bases and lib.alloc_bytes == 2 * world * slot + 256
        ex.register(0x7000, 1)
        assert lib.registered == (0x7000, slot, [b + world * slot + rank * slot for b in bases])
        ex.unregister()
        assert lib.registered is None
        ex.signal(None)
        ex.signal_and_wait(None)
        flags_off = 2 * world * slot
        assert lib.signals == [([b + flags_off + 4 * rank for b in bases], 1), ([b + flags_off + 4 * rank for b in bases], 2)]
        assert lib.waits == [(own + flags_off, world, 2)]
        assert ex.gathered(0) == own and ex.gathered(1) == own + world * slot
        released = ex.close(dist)
        q.put((rank, "ok" if released else "kept", "", lib.freed, lib.closed))
    finally:
        dist.destroy_process_group()


def _run(failing_rank, timed_out_rank=-1):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, failing_rank, q, timed_out_rank)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    return {r[0]: r[1:] for r in (q.get(timeout=5) for _ in range(2))}


def test_targets_and_flag_slots_on_two_ranks():
    res = _run(failing_rank=-1)
    for rank in (0, 1):
        state, _, freed, closed = res[rank]
        assert state == "ok" and freed == [(rank + 1) << 40] and len(closed) == 1


def test_a_failed_mapping_on_one_rank_stops_all_ranks():
    res = _run(failing_rank=1)
    for rank in (0, 1):
        state, message, freed, _ = res[rank]
        assert state == "raised" and "rank 1" in message and "cannot map" in message
        assert freed == [(rank + 1) << 40]          # nothing is left allocated


def test_close_after_a_failed_wait_releases_nothing_on_any_rank():
    """A rank whose bounded flag wait gave up (status -4) cannot know that its peers have stopped storing into its
    buffer: the ranks agree on the host, and then no rank unmaps or frees anything."""
    res = _run(failing_rank=-1, timed_out_rank=1)
    for rank in (0, 1):
        state, _, freed, closed = res[rank]
        assert state == "kept" and freed == [] and closed == []

"""Exchange step of a row-sharded model without a collective: the product kernels of every rank store
their results straight into the gathered buffers of all ranks (peer memory over NVLink), and one flag per
rank and step says when a rank's stores are complete.

One process per GPU; ``dist`` is an initialised ``torch.distributed`` (any backend: it only carries the 64-byte
IPC handles at set-up).  Two gathered buffers alternate by step parity, so that a rank may start writing step
s+1 while another still reads step s; it cannot reach step s+2 before every rank has signalled s+1.

    ex = PeerExchange(lib, dist, rank, world, slot_bytes)      # slot = one rank's outputs of a step
    ex.register(local_out_base, parity); <record or make the step's launches>; ex.unregister()
    ... per step: run the launches recorded for parity = step & 1, then
    ex.signal_and_wait(stream)      # (or ex.signal + ex.wait)    gathered(parity) is complete on this rank

python -m bpd_substrate_b200.peer   (under torchrun, 2 or more GPUs): checks the gathered buffers against an
NCCL all-gather of the same outputs, bit for bit, over several steps.
"""
import ctypes as C

from . import capi


class PeerExchange:
    FLAG_BYTES = 256

    def __init__(self, lib, dist, rank, world, slot_bytes):
        if world > 8:
            raise ValueError("at most 8 ranks (one node)")
        if slot_bytes % 16:
            raise ValueError("a rank's output slot must be a multiple of 16 bytes")
        self.lib, self.rank, self.world, self.slot_bytes = lib, rank, world, slot_bytes
        self.gathered_bytes = world * slot_bytes
        total = 2 * self.gathered_bytes + self.FLAG_BYTES
        self.base, self.bases, self._imported = None, [], []
        # No rank leaves between the collective calls below: a failure is carried to the common verdict at the end,
        # and then every rank raises.
        problem, payload = None, None
        try:
            self.base = lib.bpdq_alloc(total)
            if not self.base:
                raise MemoryError("gathered buffers")
            capi.check(lib.bpdq_memset_async(self.base, 0, total, None))
            capi.check(lib.bpdq_stream_sync(None))
            handle = (C.c_char * 64)()
            capi.check(lib.bpdq_ipc_export(self.base, handle), "bpdq_ipc_export")
            payload = bytes(handle.raw)
        except Exception as exc:
            problem = f"rank {rank}: {exc}"
        handles = [None] * world
        dist.all_gather_object(handles, payload)
        if problem is None and all(h is not None for h in handles):
            for r in range(world):
                if r == rank:
                    self.bases.append(self.base)
                    continue
                p = lib.bpdq_ipc_import((C.c_char * 64).from_buffer_copy(handles[r]))
                if not p:
                    problem = f"rank {rank}: cannot map rank {r}'s gathered buffer (status {lib.bpdq_last_status()})"
                    lib.bpdq_clear_status()
                    break
                self.bases.append(p)
                self._imported.append(p)
        elif problem is None:
            problem = f"rank {rank}: another rank could not export its buffer"
        verdicts = [None] * world
        dist.all_gather_object(verdicts, problem)     # also: every rank has mapped every buffer before anyone stores into one
        if any(v is not None for v in verdicts):
            self.close()
            raise capi.BpdqError("peer exchange set-up failed: " + "; ".join(v for v in verdicts if v))
        flags_off = 2 * self.gathered_bytes
        self.local_flags = self.base + flags_off
        self._slots = (C.c_void_p * world)(*[b + flags_off + 4 * rank for b in self.bases])
        self.step_no = 0

    def gathered(self, parity):
        """This rank's gathered buffer of the given step parity: world slots of slot_bytes."""
        return self.base + parity * self.gathered_bytes

    def register(self, local_out_base, parity):
        """From now on, batched products whose outputs lie in [local_out_base, +slot_bytes) also store their results
        into slot `rank` of every rank's gathered(parity)."""
        targets = (C.c_void_p * self.world)(*[b + parity * self.gathered_bytes + self.rank * self.slot_bytes for b in self.bases])
        capi.check(self.lib.bpdq_set_peer_outputs(local_out_base, self.slot_bytes, self.world, targets), "bpdq_set_peer_outputs")

    def unregister(self):
        capi.check(self.lib.bpdq_set_peer_outputs(None, 0, 0, None))

    def signal(self, stream):
        """After the step's launches on `stream`: raise this rank's flag everywhere."""
        self.step_no += 1
        capi.check(self.lib.bpdq_peer_signal(self._slots, self.world, self.step_no, stream), "bpdq_peer_signal")

    def wait(self, stream):
        """Later work on `stream` starts when every rank has signalled the current step (or the bounded wait gave up:
        bpdq_last_status() then reads -4)."""
        capi.check(self.lib.bpdq_peer_wait(self.local_flags, self.world, self.step_no, stream), "bpdq_peer_wait")

    def signal_and_wait(self, stream):
        """signal() and wait() in one launch."""
        self.step_no += 1
        capi.check(self.lib.bpdq_peer_signal_wait(self._slots, self.local_flags, self.world, self.step_no, stream),
                   "bpdq_peer_signal_wait")

    def close(self, dist=None, stream=None):
        """Collective when ``dist`` is given: every rank finishes its own work, then all ranks agree that nobody will
        store into a peer's buffer any more, and only then are the mappings closed and the buffer freed.  Graphs
        recorded while targets were registered keep storing to those addresses: destroy them before close().  If a rank
        reports a failed wait (status -4: a peer may still be running and storing), nothing is unmapped or freed on any
        rank -- the memory is left to the end of the process rather than pulled away under a peer's stores."""
        lib = self.lib
        lib.bpdq_set_peer_outputs(None, 0, 0, None)
        safe = True
        if dist is not None:
            ok = lib.bpdq_stream_sync(stream) == 0 and lib.bpdq_last_status() == 0
            verdicts = [None] * self.world
            dist.all_gather_object(verdicts, bool(ok))      # also a barrier: every rank's launches have completed
            safe = all(verdicts)
        if not safe:
            self._imported, self.base = [], None
            return False
        for p in self._imported:
            lib.bpdq_ipc_close(p)
        self._imported = []
        if self.base:
            lib.bpdq_free(self.base)
            self.base = None
        return True


def _selftest():
    import os

    import numpy as np
    import torch
    import torch.distributed as dist

    from . import synth
    from .dispatch import LayerSet
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = capi.load()
    capi.check(lib.bpdq_set_device(local))
    ls = LayerSet(synth.MISTRAL_LAYER, 2, seed=100 + rank)
    ex = PeerExchange(lib, dist, rank, world, ls.o_bytes)
    for parity in (0, 1):
        ex.register(ls.d_out, parity)
        ls.capture("batched", tag=parity)
    ex.unregister()
    ok = True
    out_t = torch.empty(ls.o_bytes // 4, dtype=torch.float32, device="cuda")
    want = torch.empty(world * (ls.o_bytes // 4), dtype=torch.float32, device="cuda")
    got = torch.empty_like(want)
    for step in range(6):
        x = np.random.default_rng(1000 * step + rank).standard_normal(ls.x_bytes // 4).astype(np.float32)
        ls.upload_activations(x)
        parity = step & 1
        ls.step("batched", tag=parity)
        if step % 3 == 2:
            ex.signal(ls.stream)
            ex.wait(ls.stream)
        else:
            ex.signal_and_wait(ls.stream)
        capi.check(lib.bpdq_stream_sync(ls.stream))
        lib.bpdq_d2d(out_t.data_ptr(), ls.d_out, ls.o_bytes)
        lib.bpdq_d2d(got.data_ptr(), ex.gathered(parity), world * ls.o_bytes)
        dist.all_gather_into_tensor(want, out_t)
        torch.cuda.synchronize()
        same = bool(torch.equal(got.view(torch.int32), want.view(torch.int32)))
        ok = ok and same and lib.bpdq_last_status() == 0
        dist.barrier()      # nobody overwrites a buffer that another rank is still comparing
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("peer exchange selftest:", "ok" if int(flag.item()) else "MISMATCH", f"({world} ranks, 6 steps)", flush=True)
    ls.close()             # destroys the graphs recorded with peer targets
    ex.close(dist)
    dist.destroy_process_group()
    return 0 if int(flag.item()) else 1


if __name__ == "__main__":
    raise SystemExit(_selftest())

"""Row sharding of quantized weight matrices over the GPUs of one node.

Output rows of a GEMV are independent (out[row] depends on one weight row and the shared
activation vector: bench/bpd_quant.c:93-108 of the reference), so rank g of G owns the
contiguous row range [g*N/G, (g+1)*N/G) of every matrix -- a contiguous byte range of the
quantized tensor -- and the only exchange is an all-gather of the fp32 output slices.

torch.distributed is plumbing here (NCCL on GPUs, gloo in the CPU tests); the shard
arithmetic is plain Python so that it can be tested without a GPU.
"""
import numpy as np

from . import synth


def row_range(rows, rank, world):
    """Rows [lo, hi) owned by `rank`.  Rows must divide evenly (true for every benchmark shape)."""
    if rows % world:
        raise ValueError(f"{rows} rows do not divide over {world} ranks")
    per = rows // world
    return rank * per, (rank + 1) * per


def shard_q4k(weight_bytes, rows, cols, rank, world):
    """The byte range of a [rows][cols] Q4_K matrix that holds `rank`'s rows (a view, no copy)."""
    lo, hi = row_range(rows, rank, world)
    rb = synth.q4k_row_bytes(cols)
    w = np.asarray(weight_bytes).reshape(-1)
    if w.size != rows * rb:
        raise ValueError("weight buffer does not match rows x cols")
    return w[lo * rb:hi * rb]


def shard_q8_0(weight_bytes, rows, cols, rank, world):
    lo, hi = row_range(rows, rank, world)
    rb = synth.q8_0_row_bytes(cols)
    w = np.asarray(weight_bytes).reshape(-1)
    if w.size != rows * rb:
        raise ValueError("weight buffer does not match rows x cols")
    return w[lo * rb:hi * rb]


def gather_layout(tokens, rows, world):
    """After an all-gather of per-rank [tokens][rows/world] slices the buffer is
    [world][tokens][rows/world]; returns the permutation shape to turn it into [tokens][rows]."""
    return (world, tokens, rows // world)


def all_gather_outputs(local_out, tokens, rows, group=None):
    """local_out: torch tensor [tokens][rows/world] (this rank's slice).  Returns [tokens][rows]
    on every rank.  One collective; for tokens == 1 the gathered buffer already is the result."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    local_out = local_out.contiguous().view(-1)
    gathered = torch.empty(world * local_out.numel(), dtype=local_out.dtype, device=local_out.device)
    dist.all_gather_into_tensor(gathered, local_out, group=group)
    if tokens == 1:
        return gathered.view(1, rows)
    return gathered.view(*gather_layout(tokens, rows, world)).permute(1, 0, 2).reshape(tokens, rows)

"""Sharding of the path over the GPUs of one box: one process per GPU, no device-to-device traffic.

Quantising, residual and dequantising are independent per row; a coding batch is independent per rANS segment once
its tables are fixed.  So work is cut by tensor / row-block / segment, every rank reads only its own HBM, and the
only exchange is through the host: histogram counts are summed (exact integers, order-free) before the tables are
normalised, and coded segments are gathered in segment order, so the archive bytes do not depend on the number
of GPUs (the reference keeps its windows, batches and segments independent of the device too,
seedpack/repo3.py:1959-1961).  torch.distributed is the transport (gloo on CPU tensors: a few hundred KB per batch).
"""
import numpy as np
import torch
import torch.distributed as dist


def assign(sizes, world):
    """units (tensors, row blocks, batches) of `sizes` bytes -> rank of each, longest first onto the least loaded
    rank; deterministic, the same on every rank"""
    load = [0] * world
    owner = [0] * len(sizes)
    for i in sorted(range(len(sizes)), key=lambda i: (-sizes[i], i)):
        r = min(range(world), key=lambda r: (load[r], r))
        owner[i] = r
        load[r] += sizes[i]
    return owner


def row_blocks(nrows, row_bytes, world, min_bytes=8 << 20):
    """[(first row, rows)] cutting a tensor into at most `world` row blocks of at least min_bytes (rows are never split:
    the legacy importance quantisers need whole rows)"""
    total = nrows * row_bytes
    parts = max(1, min(world, total // max(min_bytes, 1)))
    base, extra = divmod(nrows, parts)
    out, r0 = [], 0
    for p in range(parts):
        n = base + (1 if p < extra else 0)
        if n:
            out.append((r0, n)); r0 += n
    return out


def segment_range(nseg, rank, world):
    """contiguous share [s0, s1) of a batch's segments for this rank"""
    base, extra = divmod(nseg, world)
    s0 = rank * base + min(rank, extra)
    return s0, s0 + base + (1 if rank < extra else 0)


def sum_counts(counts, group=None):
    """histogram counts of this rank's share -> counts of the whole batch on every rank (int64 sum over the host)"""
    t = torch.from_numpy(np.ascontiguousarray(counts).astype(np.int64))
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t.numpy()


def gather_segments(lens, stream, group=None, dst=0):
    """this rank's segment lengths (uint32 array, in segment order) and their bytes -> on rank `dst` (of the group) the
    lengths and the stream of the whole batch in rank order (ranks own contiguous segment ranges), elsewhere (None, None)"""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return np.asarray(lens, np.uint32), bytes(stream)
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    gathered = [None] * world if rank == dst else None
    dist.gather_object((np.asarray(lens, np.uint32), bytes(stream)), gathered,
                       dst=dist.get_global_rank(group, dst) if group is not None else dst, group=group)
    if rank != dst:
        return None, None
    return np.concatenate([g[0] for g in gathered]), b"".join(g[1] for g in gathered)

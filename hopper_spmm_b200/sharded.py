"""Row-window sharding over the ranks of a torch.distributed job (one process per GPU).

The matrix shards naturally: every 16-row window writes its own rows of C, so rank p converts
and multiplies the contiguous, nnz-balanced row range [cuts[p], cuts[p+1]) with B replicated
and never exchanges data while computing.  The only collective is the optional all-gather of
the row-sharded C.  (The reference is single-GPU; its row windows over CTAs,
src/fp16.cu:86,138, are the decomposition this extends to GPUs.)
"""
from __future__ import annotations

import numpy as np

from . import spmm as _spmm


ROW_CHARGE = 6  # entries a row is charged on top of its own when the ranks' shares are cut

def my_rows(rows: int, row_ptr, world: int, rank: int, row_charge: int = ROW_CHARGE):
    """(cuts, r0, r1): the cuts for `world` ranks, balanced on nnz + row_charge per row, and this
    rank's row range."""
    cuts = _spmm.shard_rows(rows, row_ptr, world, row_charge=row_charge).astype(np.int64)
    return cuts, int(cuts[rank]), int(cuts[rank + 1])


def slice_csr(row_ptr, col_idx, values, r0: int, r1: int):
    """CSR arrays of rows [r0, r1) with row_ptr rebased to zero."""
    lo, hi = int(row_ptr[r0]), int(row_ptr[r1])
    rp = (np.asarray(row_ptr[r0:r1 + 1], dtype=np.int64) - lo).astype(np.uint32)
    return rp, col_idx[lo:hi], values[lo:hi]


def _exchange_row_slices(full, cuts, group=None):
    """Rank p holds rows [cuts[p], cuts[p+1]) of `full`; on return every rank holds all of it.
    The slices may differ in length - rows are cut for equal work, so the rank with the lightest rows
    holds several times the average - and a direct exchange is as slow as that rank's outgoing link
    (eight B200s: 31.6 ms for 8.6 GB of C).  So it runs in two steps: (1) one grouped send/receive moves
    every row that lies outside its holder's EVEN part (part q = rows [q K, (q + 1) K), K = rows // world)
    to the rank whose even part it falls into - such a row crosses one link once; (2) the library's
    in-place all-gather of the even parts, which loads all links alike.  The rows past world * K go to
    everybody in step 1.  Where the busiest rank would send hardly less that way than by sending its
    slice to everybody (two ranks; nearly equal slices with a remainder), step 1 alone does it all."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if world < 2:
        return
    cuts = [int(c) for c in cuts]
    total = cuts[-1]
    part = total // world if full.is_contiguous() else 0   # without whole parts: step 1 alone, everything to everybody
    equal = all(cuts[p + 1] - cuts[p] == part for p in range(world))   # then the all-gather alone does it
    if part and not equal and not two_step_pays(cuts, part):
        part = 0
    whole = part * world
    ops = []

    def piece(lo, hi, op, peer):
        if hi > lo:
            ops.append(dist.P2POp(op, full[lo:hi], dist.get_global_rank(group, peer) if group is not None else peer, group))

    for step in range(1, world):
        # a different peer for every rank at every step, so no rank is everybody's first target
        to, frm = (rank + step) % world, (rank - step) % world
        # what this rank holds of `to`'s even part, then of the tail; what `frm` holds of this rank's
        # even part, then of the tail - sends and receives of a pair in the same order
        piece(max(cuts[rank], part * to), min(cuts[rank + 1], part * (to + 1)), dist.isend, to)
        piece(max(cuts[rank], whole), cuts[rank + 1], dist.isend, to)
        piece(max(cuts[frm], part * rank), min(cuts[frm + 1], part * (rank + 1)), dist.irecv, frm)
        piece(max(cuts[frm], whole), cuts[frm + 1], dist.irecv, frm)
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    if part:
        dist.all_gather_into_tensor(full[:whole], full[part * rank:part * (rank + 1)], group=group)


def two_step_pays(cuts, part) -> bool:
    """Does the busiest rank send at least 15 % less with the two-step exchange of `_exchange_row_slices`
    (its rows outside its even part once, then its even part to everybody) than with the direct one (its
    slice to everybody)?  `cuts`: the world + 1 slice boundaries; `part`: rows of an even part."""
    world = len(cuts) - 1
    direct = max(cuts[p + 1] - cuts[p] for p in range(world)) * (world - 1)
    outside = max((cuts[p + 1] - cuts[p]) - max(0, min(cuts[p + 1], part * (p + 1)) - max(cuts[p], part * p))
                  for p in range(world))
    return (outside + part * (world - 1)) * 1.15 < direct


def allgather_rows(C_local, cuts, group=None):
    """All-gather of a row-sharded C: rank p holds rows [cuts[p], cuts[p+1]).  Works on CUDA
    tensors (NCCL) and CPU tensors (gloo).  Ranges differ in length; every rank's slice goes
    straight into its place in the full-size result, there is no staging copy."""
    import torch
    import torch.distributed as dist
    rank = dist.get_rank(group)
    total = int(cuts[-1])
    full = torch.empty((total, C_local.shape[1]), dtype=C_local.dtype, device=C_local.device)
    full[int(cuts[rank]):int(cuts[rank + 1])].copy_(C_local)
    _exchange_row_slices(full, cuts, group)
    return full


def upload_replicated(B_host, B_dev, group=None):
    """Brings a host B (the same on every rank, pinned) into every rank's B_dev with one trip over
    the host link per element: rank p copies rows [p*K/N, (p+1)*K/N) host -> device and the ranks
    then exchange their parts GPU to GPU.  With N ranks behind one host the replicated operand
    crosses PCIe once instead of N times.  Works on CUDA tensors (NCCL) and CPU tensors (gloo).
    Returns the number of bytes this rank copied from the host."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    K = B_host.shape[0]
    cuts = [K * p // world for p in range(world + 1)]
    mine = B_dev[cuts[rank]:cuts[rank + 1]]
    mine.copy_(B_host[cuts[rank]:cuts[rank + 1]], non_blocking=True)
    if K % world == 0 and B_dev.is_contiguous():
        # equal parts: the library's all-gather, in place (eight B200s: 5.7 ms for 4.3 GB against
        # 6.1 ms for the grouped exchange and 7.1 ms for a loop of broadcasts)
        dist.all_gather_into_tensor(B_dev, mine, group=group)
    else:
        _exchange_row_slices(B_dev, cuts, group)
    return mine.numel() * mine.element_size()

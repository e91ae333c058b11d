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

# The fit behind ROW_CHARGE (default workload, one B200): a rank's product takes about 0.0253 ms per
# million entries plus 0.153 ms per million rows.
_MS_PER_M_ENTRIES = 0.0253


def e2e_row_charge(n: int, c_itemsize: int, host_link_gbs: float = 52.0, row_charge: int = ROW_CHARGE) -> int:
    """Row charge for cuts that balance a rank's whole step when its rows of C go back to the host
    every step: a row then also costs its n * c_itemsize bytes over the rank's host link
    (about 52 GB/s measured device to host), which outweighs the product itself - the cuts
    become nearly equal row counts."""
    ms_per_m_rows = n * c_itemsize / (host_link_gbs * 1e9) * 1e3 * 1e6
    return row_charge + int(round(ms_per_m_rows / _MS_PER_M_ENTRIES))


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


def allgather_rows(C_local, cuts, group=None):
    """All-gather of a row-sharded C: rank p holds rows [cuts[p], cuts[p+1]).  Works on CUDA
    tensors (NCCL) and CPU tensors (gloo).  Ranges differ in length, so every rank broadcasts
    its own slice into the full-size result in place; there is no staging copy."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    total = int(cuts[-1])
    full = torch.empty((total, C_local.shape[1]), dtype=C_local.dtype, device=C_local.device)
    full[int(cuts[rank]):int(cuts[rank + 1])].copy_(C_local)
    work = []
    for p in range(world):
        part = full[int(cuts[p]):int(cuts[p + 1])]
        if part.numel():
            src = dist.get_global_rank(group, p) if group is not None else p
            work.append(dist.broadcast(part, src=src, group=group, async_op=True))
    for w in work:
        w.wait()
    return full


def upload_replicated(B_host, B_dev, group=None):
    """Brings a host B (the same on every rank, pinned) into every rank's B_dev with one trip over
    the host link per element: rank p copies rows [p*K/N, (p+1)*K/N) host -> device and then
    broadcasts them to the other ranks, GPU to GPU.  With N ranks behind one host the replicated
    operand crosses PCIe once instead of N times.  Works on CUDA tensors (NCCL) and CPU tensors
    (gloo).  Returns the number of bytes this rank copied from the host."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    K = B_host.shape[0]
    cuts = [K * p // world for p in range(world + 1)]
    mine = B_dev[cuts[rank]:cuts[rank + 1]]
    mine.copy_(B_host[cuts[rank]:cuts[rank + 1]], non_blocking=True)
    work = []
    for p in range(world):
        part = B_dev[cuts[p]:cuts[p + 1]]
        if part.numel():
            src = dist.get_global_rank(group, p) if group is not None else p
            work.append(dist.broadcast(part, src=src, group=group, async_op=True))
    for w in work:
        w.wait()
    return mine.numel() * mine.element_size()

"""Row-sharded feature tables across the GPUs of one box.

A table that does not fit one GPU (the 1024-d, 100 M-node configuration needs ~410 GB) is block-partitioned by
rows: rank r keeps rows [r * rows_per_shard, (r + 1) * rows_per_shard) in its own HBM.  Every rank exports its
shard with CUDA IPC and opens the others', so each process ends up with one device pointer per shard; the
gather and aggregation kernels then read remote rows with plain peer loads over NVLink, each warp fetching the
rows it needs.  There is no collective on the data path and no multicast object is created.  (The reference
keeps features in host memory and copies the rows of every batch over PCIe, train_fastgl.py:161-184.)
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch.multiprocessing.reductions import reduce_tensor

import fastgl


def rows_per_shard(n_rows: int, world: int) -> int:
    return (n_rows + world - 1) // world


def open_peer_tensors(local: torch.Tensor, group=None) -> list[torch.Tensor]:
    """Collective over ``group``: every rank exports ``local`` (a contiguous CUDA tensor, the same shape on every rank)
    with CUDA IPC and opens the others'; returns one tensor per rank, ``local`` itself at this rank's index.  The
    returned peer tensors are mappings of the peers' memory: drop them (and call ``torch.cuda.ipc_collect()``) before
    the owning processes free it."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if not local.is_cuda or not local.is_contiguous():
        raise RuntimeError("open_peer_tensors needs a contiguous CUDA tensor")
    rebuild, args = reduce_tensor(local)               # CUDA IPC handle of the allocation
    exported = [None] * world
    dist.all_gather_object(exported, (rebuild, args), group=group)
    out = []
    for r, (fn, a) in enumerate(exported):
        if r == rank:
            out.append(local)
        else:
            a = list(a)
            a[6] = local.device.index                   # open the peer's allocation on this rank's device
            out.append(fn(*a))
    dist.barrier(group)
    return out


def share_feature_shards(local_shard: torch.Tensor, n_rows: int, group=None) -> fastgl.ShardedTable:
    """``local_shard``: this rank's float32 [rows_per_shard, dim] block (the last rank may use fewer rows of it).
    Collective over ``group``: returns the table of all ranks' shards as seen from this rank."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if local_shard.dtype != torch.float32 or local_shard.dim() != 2 or not local_shard.is_contiguous():
        raise RuntimeError("local_shard must be a contiguous float32 matrix")
    rps = rows_per_shard(n_rows, world)
    if local_shard.size(0) < min(rps, max(0, n_rows - rank * rps)):
        raise RuntimeError("local_shard has fewer rows than this rank's share")
    shards = open_peer_tensors(local_shard, group)
    return fastgl.ShardedTable(shards, rps, local_shard.size(1), n_rows, local_shard.device, ld=local_shard.stride(0))

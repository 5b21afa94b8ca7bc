"""Two-GPU test of the row-sharded feature table: every rank keeps half of the rows, opens the other half
through CUDA IPC, and gathers / aggregates rows that live on both GPUs with peer loads.  Skipped on boxes with
one GPU.  Ranks are child processes; a rank only leaves between steps (after the final barrier)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port):
    import fastgl
    from fastgl_b200.sharding import rows_per_shard, share_feature_shards
    from oracle import oracle_c as oc

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n, dim = 50_001, 256
        rng = np.random.default_rng(77)                       # the same table on every rank (host side, for checking)
        table = rng.standard_normal((n, dim)).astype(np.float32)
        rps = rows_per_shard(n, world)
        mine = torch.zeros((rps, dim), dtype=torch.float32, device=dev)
        part = table[rank * rps:(rank + 1) * rps]
        mine[: part.shape[0]] = torch.from_numpy(part).to(dev)
        st = share_feature_shards(mine, n)
        ids = np.random.default_rng(100 + rank).integers(0, n, size=20_000).astype(np.int32)
        got = fastgl.gather_rows(st, torch.from_numpy(ids).to(dev))
        assert np.array_equal(got.cpu().numpy(), table[ids])
        # mean aggregation over a random block whose sources live on both GPUs
        n_dst, deg = 3000, 12
        indptr = (np.arange(n_dst + 1) * deg).astype(np.int32)
        src = np.random.default_rng(200 + rank).integers(0, n, size=n_dst * deg).astype(np.int32)
        out = fastgl.aggregate(fastgl.AGG_MEAN, torch.from_numpy(indptr).to(dev), torch.from_numpy(src).to(dev), st, n_dst,
                               zero_deg_passthrough=False)
        ref = oc.aggregate_fwd(oc.MODE_MEAN, indptr, src, table, n_dst, zero_deg_passthrough=False)
        err = float(np.abs(out.cpu().numpy() - ref).max() / np.abs(ref).max())
        assert err <= 1e-5, err
        torch.cuda.synchronize()
        dist.barrier()                                        # nobody unmaps a shard while a peer still reads it
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_feature_table_over_two_gpus():
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)

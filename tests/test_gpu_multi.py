"""Two-GPU tests.  (1) The row-sharded feature table: every rank keeps half of the rows, opens the other half
through CUDA IPC, and gathers / aggregates rows that live on both GPUs with peer loads.  (2) Data-parallel
training over NCCL with the step replayed from CUDA graphs.  Skipped on boxes with one GPU.  Ranks are child
processes.  A rank leaves only through ``_leave_together``: whether its checks passed or raised, it first drains
its own GPU work, waits on a host-side (gloo) barrier until every rank has done the same, drops its mappings of
the peers' memory, waits again, and only then tears down -- so no rank unmaps memory a peer's kernel may still
read, on the failure path as on the success path."""
import datetime
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


def _leave_together(exc, host_group, release=None):
    """Common exit of a rank (see the module docstring); re-raises ``exc`` at the end."""
    try:
        torch.cuda.synchronize()
    finally:
        try:
            dist.barrier(group=host_group)          # every rank's kernels have finished
            if release is not None:
                release()                            # drop this rank's mappings of the peers' memory
            torch.cuda.ipc_collect()
            dist.barrier(group=host_group)          # nobody maps anybody's memory any more
        finally:
            dist.destroy_process_group()
    if exc is not None:
        raise exc


def _worker(rank, world, port):
    import fastgl
    from fastgl_b200.sharding import rows_per_shard, share_feature_shards
    from oracle import oracle_c as oc

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=180))
    held, failure = {}, None
    try:
        n, dim = 50_001, 256
        rng = np.random.default_rng(77)                       # the same table on every rank (host side, for checking)
        table = rng.standard_normal((n, dim)).astype(np.float32)
        rps = rows_per_shard(n, world)
        mine = torch.zeros((rps, dim), dtype=torch.float32, device=dev)
        part = table[rank * rps:(rank + 1) * rps]
        mine[: part.shape[0]] = torch.from_numpy(part).to(dev)
        st = held["table"] = share_feature_shards(mine, n)
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
        # an id beyond the table is reported, not dereferenced (its row comes back as zeros)
        bad = fastgl.gather_rows(st, torch.tensor([0, n, -1, n - 1], dtype=torch.int32, device=dev))
        with pytest.raises(RuntimeError, match="out of range"):
            fastgl.check_status(dev)
        assert np.array_equal(bad.cpu().numpy()[[0, 3]], table[[0, n - 1]]) and not bad[1:3].any()
    except BaseException as e:                                # noqa: BLE001 -- re-raised by _leave_together
        failure = e
    st = None
    _leave_together(failure, dist.group.WORLD, release=held.clear)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_feature_table_over_two_gpus():
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)


def _train_worker(rank, world, port):
    """Two data-parallel ranks.  The step replayed from CUDA graphs must train like the op-by-op step, across an epoch
    boundary with its short last batch, and keep the replicas identical -- with the NCCL all-reduce between two
    graphs, and with the one-launch exchange (peer stores + flags, fused with Adam) that makes the step one graph.
    The two kinds of exchange must agree to rounding."""
    from conftest import make_graph
    from fastgl_b200.layers import GraphSAGE
    from fastgl_b200.trainer import Trainer

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=datetime.timedelta(seconds=180))
    host_group = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=400))
    err = None
    held = {}

    def release():
        for tr in held.values():
            tr.release_peers()
        held.clear()

    try:
        import fastgl
        n = 6000
        indptr, indices = make_graph(n, 14, seed=9, hub=400)
        rng = np.random.default_rng(9)
        feat = torch.from_numpy(rng.standard_normal((n, 100)).astype(np.float32)).to(dev)
        labels = torch.from_numpy(rng.integers(0, 7, n)).to(dev)
        train = torch.from_numpy(np.sort(rng.choice(n, size=n // 2, replace=False)).astype(np.int32)).to(dev)
        runs = {}
        for name, graph, sync in (("eager-nccl", False, "nccl"), ("graph-nccl", True, "nccl"), ("eager-oneshot", False, "oneshot"),
                                  ("graph-oneshot", True, "oneshot")):
            torch.manual_seed(3)
            model = GraphSAGE(100, 32, 7, 3, dropout=0.0).to(dev)
            tr = held[name] = Trainer(torch.from_numpy(indptr).to(dev), torch.from_numpy(indices).to(dev), feat, labels, train,
                                      model, [15, 10, 5], batch_size=256, window=4, cuda_graph=graph, rank=rank, world=world,
                                      grad_sync=sync)
            assert tr.steps_per_epoch() == 6                  # 1500 seeds per rank: five full batches and one of 220
            assert tr.oneshot == (sync == "oneshot")
            losses = tr.run_steps(14, read_loss_each_step=True)
            fastgl.check_status(dev)
            runs[name] = (losses, [p.detach().clone() for p in model.parameters()], tr)
        le, pe, _ = runs["eager-nccl"]
        for name in ("graph-nccl", "eager-oneshot", "graph-oneshot"):
            lg, pg, tg = runs[name]
            if name.startswith("graph"):
                assert tg.graphed is not None and tg.graph_fallbacks <= 2
                assert (tg.graphed.opt_graph is None) == name.endswith("oneshot")   # one graph per step with the exchange inside
            assert np.allclose(le, lg, rtol=1e-4, atol=1e-4), (name, le, lg)
            for a, b in zip(pe, pg):
                assert torch.allclose(a, b, rtol=1e-3, atol=1e-4), name
            flat = torch.cat([p.flatten() for p in pg])
            both = [torch.empty_like(flat) for _ in range(world)]
            dist.all_gather(both, flat)
            assert torch.equal(both[0], both[1]), name        # the replicas stay bit-identical
        # the same average up to the rounding of NCCL's own arithmetic (it scales before it adds)
        for a, b in zip(runs["eager-nccl"][1], runs["eager-oneshot"][1]):
            assert torch.allclose(a, b, rtol=1e-5, atol=1e-6)
    except BaseException as e:                                # noqa: BLE001 -- re-raised by _leave_together
        err = e
    _leave_together(err, host_group, release=release)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_data_parallel_graph_step_over_two_gpus():
    mp.spawn(_train_worker, args=(2, _free_port()), nprocs=2, join=True)

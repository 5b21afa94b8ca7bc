"""CPU tests of the host-side logic around the kernels: synthetic graphs, seed sharding, the Match-Reorder
scheduler, block views, and the data-parallel plumbing on two gloo ranks."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fastgl_b200.block import Block
from fastgl_b200.graphgen import build_csr, rmat_edges, rmat_graph, synthetic_node_data
from fastgl_b200.scheduler import MatchReorder, greedy_order, overlap_matrix
from fastgl_b200.trainer import FlatGrads, shard_seeds


def test_rmat_graph_is_a_valid_symmetric_csr():
    indptr, indices = rmat_graph(5000, 12.0, seed=3)
    n = 5000
    assert indptr.dtype == torch.int64 and indices.dtype == torch.int32
    assert indptr[0] == 0 and indptr[-1] == indices.numel() and bool((indptr[1:] >= indptr[:-1]).all())
    assert 0.8 * n * 12 <= indices.numel() <= n * 12
    assert int(indices.min()) >= 0 and int(indices.max()) < n
    dst = torch.repeat_interleave(torch.arange(n), indptr[1:] - indptr[:-1])
    assert bool((dst != indices.long()).all())                      # no self loops
    fwd = torch.sort(dst * n + indices.long()).values
    bwd = torch.sort(indices.long() * n + dst).values
    assert torch.equal(fwd, bwd)                                    # every edge has its reverse
    again, _ = rmat_graph(5000, 12.0, seed=3)
    assert torch.equal(again, indptr)                               # seeded
    deg = indptr[1:] - indptr[:-1]
    assert int(deg.max()) > 20 * float(deg.float().mean())          # skewed, power-law like


def test_build_csr_keeps_edge_order_within_a_destination():
    src = torch.tensor([5, 1, 7, 2, 9])
    dst = torch.tensor([2, 0, 2, 0, 1])
    indptr, indices = build_csr(3, src, dst)
    assert indptr.tolist() == [0, 2, 3, 5] and indices.tolist() == [1, 2, 9, 5, 7]


def test_relabel_by_degree_is_an_isomorphism_with_hubs_first():
    from fastgl_b200.graphgen import relabel_by_degree, rmat_graph
    indptr, indices = rmat_graph(3000, 9.0, seed=3, device="cpu")
    p2, i2, order, new_of_old = relabel_by_degree(indptr, indices, chunk_edges=1000)
    deg2 = p2[1:] - p2[:-1]
    assert bool((deg2[:-1] >= deg2[1:]).all()) and int(p2[-1]) == int(indptr[-1])
    assert torch.equal(new_of_old[order], torch.arange(3000))
    for v in (0, 1, 17, 1500, 2999):                      # the same neighbours, renamed, in the same order
        old = order[v]
        want = new_of_old[indices[indptr[old]: indptr[old + 1]].long()]
        assert torch.equal(i2[p2[v]: p2[v + 1]].long(), want)


def test_synthetic_node_data_shapes():
    feat, labels, train = synthetic_node_data(1000, 16, 7, 0.1, seed=1)
    assert feat.shape == (1000, 16) and feat.dtype == torch.float32
    assert int(labels.max()) < 7 and train.numel() == 100 and train.dtype == torch.int32
    assert torch.unique(train).numel() == 100


def test_shard_seeds_partitions_the_training_set():
    train = torch.arange(1000, 2003, dtype=torch.int32)
    shards = [shard_seeds(train, r, 4, epoch_seed=9) for r in range(4)]
    assert all(s.numel() == 251 for s in shards)                    # ceil(1003 / 4), padded by wrap-around
    allv = torch.cat(shards)
    assert set(allv.tolist()) == set(train.tolist())
    assert allv.numel() - torch.unique(allv).numel() == 1           # exactly the padding is repeated
    assert not torch.equal(shards[0], shard_seeds(train, 0, 4, epoch_seed=10))


def test_overlap_matrix_and_greedy_order():
    lists = [torch.tensor([0, 1, 2, 3]), torch.tensor([2, 3, 4]), torch.tensor([10, 11]), torch.tensor([3, 4, 5, 6, 10])]
    ov = overlap_matrix(lists, 16, chunk=5)
    assert ov.tolist() == [[4, 2, 0, 1], [2, 3, 0, 2], [0, 0, 2, 1], [1, 2, 1, 5]]
    # match degree (i<j) = |i & j| / |j|: from 0 the best is 1 (2/3), from 1 it is 3 (2/5), then 2
    assert greedy_order(ov, torch.tensor([4, 3, 2, 5])) == [0, 1, 3, 2]
    assert MatchReorder(16).reorder(lists) == [0, 1, 3, 2]
    assert MatchReorder(16).reorder(lists[:2]) == [0, 1]
    # batches without any overlap are still all scheduled exactly once
    disjoint = [torch.tensor([i]) for i in range(5)]
    assert sorted(MatchReorder(8).reorder(disjoint)) == [0, 1, 2, 3, 4]


def test_overlap_of_padded_device_style_node_lists_equals_the_list_version():
    from fastgl_b200.scheduler import MatchReorder, overlap_matrix, overlap_matrix_padded
    rng = np.random.default_rng(8)
    n, W, stride = 5000, 6, 900
    counts = rng.integers(100, stride, size=W)
    nodes = rng.integers(0, n, size=(W, stride)).astype(np.int32)         # stale entries everywhere ...
    lists = []
    for b in range(W):
        ids = rng.choice(n, size=counts[b], replace=False).astype(np.int32)
        nodes[b, : counts[b]] = ids                                          # ... except the first counts[b]
        lists.append(torch.from_numpy(ids))
    want = overlap_matrix(lists, n, chunk=1024)
    got = overlap_matrix_padded(torch.from_numpy(nodes), torch.from_numpy(counts), n, chunk=1500)
    assert torch.equal(got, want)
    m = MatchReorder(n)
    m._pinned = {(0, W): got}
    assert m.order(counts.tolist()) == m.reorder(lists)


def test_block_edges_view_matches_the_csr():
    blk = Block(torch.tensor([0, 2, 2, 5], dtype=torch.int32), torch.tensor([4, 1, 0, 2, 3], dtype=torch.int32), 6, 3)
    src, dst = blk.edges()
    assert dst.tolist() == [0, 0, 2, 2, 2] and src.tolist() == [4, 1, 0, 2, 3]
    assert blk.num_edges() == 5 and blk.num_dst_nodes() == 3 and blk.num_src_nodes() == 6


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ddp_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)                                        # same initial weights on every rank
        model = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Linear(5, 3))
        grads = FlatGrads(model.parameters())
        train = torch.arange(100, dtype=torch.int32)
        mine = shard_seeds(train, rank, world, epoch_seed=1)
        x = torch.randn(8, 6, generator=torch.Generator().manual_seed(100 + rank))
        grads.zero()
        model(x).square().sum().backward()
        local = grads.buffer.clone()
        grads.all_reduce(world)
        gathered = [torch.zeros_like(local) for _ in range(world)]
        dist.all_gather(gathered, local)
        assert torch.allclose(grads.buffer, torch.stack(gathered).mean(0), atol=1e-6)
        assert all(p.grad.data_ptr() >= grads.buffer.data_ptr() for p in model.parameters())   # views of one buffer
        seeds = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(seeds, mine)
        assert set(torch.cat(seeds).tolist()) == set(range(100))
        torch.save(grads.buffer, os.path.join(out_dir, f"g{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_gradient_all_reduce_and_seed_split_on_two_gloo_ranks(tmp_path):
    port = _free_port()
    mp.spawn(_ddp_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    g0, g1 = torch.load(tmp_path / "g0.pt"), torch.load(tmp_path / "g1.pt")
    assert torch.equal(g0, g1)                                      # both ranks hold the same averaged gradient


def test_gcn_order_cost_model():
    """Aggregate-first wins where many gathered rows feed few output rows of a narrower layer (the first layer of
    the 602-d workload); update-first wins where the layer shrinks the rows a lot and the block is not much
    smaller on the destination side."""
    from fastgl_b200.layers import gcn_aggregate_first
    assert gcn_aggregate_first(n_src=233_000, n_dst=11_000, n_edges=281_000, in_dim=602, out_dim=256)
    assert gcn_aggregate_first(n_src=60_000, n_dst=6_000, n_edges=61_000, in_dim=256, out_dim=256)
    assert not gcn_aggregate_first(n_src=1_200, n_dst=1_000, n_edges=400_000, in_dim=1024, out_dim=8)

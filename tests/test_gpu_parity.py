"""GPU parity tests: the CUDA path, called through the ``fastgl`` ops (ctypes -> C ABI), against the CPU
oracle on the same seeded inputs.  Integer results are compared bit for bit; fp32 aggregation within
1e-5 relative to the largest reference magnitude (the tolerance stated for the path)."""
import os

import numpy as np
import pytest
import torch

from conftest import make_graph
from oracle import oracle_c as oc

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hotpath_small.npz")
AGG_RTOL = 1e-5


def dev():
    return torch.device("cuda", 0)


def to_dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.to(dev())


def rel_err(got, ref):
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(np.asarray(got, dtype=np.float64) - ref).max() / max(1e-30, np.abs(ref).max()))


@pytest.fixture(scope="module")
def fastgl():
    import fastgl as mod
    assert torch.cuda.is_available()
    return mod


@pytest.fixture(scope="module")
def graph():
    indptr, indices = make_graph(20000, 16, seed=21, hub=3000)
    return indptr, indices


# ----------------------------------------------------------------------------------------------
# a3
# ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("n_ids,n_nodes", [(0, 5), (1, 1), (1000, 37), (300000, 70000), (5_000_000, 1_000_000)])
def test_cal_deg_and_exclusive_sum(fastgl, n_ids, n_nodes):
    rng = np.random.default_rng(n_ids + 1)
    ids = rng.integers(0, n_nodes, size=n_ids).astype(np.int32)
    deg = fastgl.cal_deg(to_dev(ids), n_nodes)
    ref = oc.cal_deg(ids, n_nodes)
    assert np.array_equal(deg.cpu().numpy(), ref)
    ptr = fastgl.exclusive_sum(deg)
    assert np.array_equal(ptr.cpu().numpy(), oc.exclusive_sum(ref))


def test_exclusive_sum_empty(fastgl):
    out = fastgl.exclusive_sum(torch.zeros(0, dtype=torch.int32, device=dev()))
    assert out.cpu().tolist() == [0]


# ----------------------------------------------------------------------------------------------
# a1
# ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("ptr_dtype", [torch.int32, torch.int64])
@pytest.mark.parametrize("replace", [False, True])
@pytest.mark.parametrize("fanout", [1, 5, 10, 15, 25, 32, 33, 100])
def test_sample_matches_oracle(fastgl, graph, ptr_dtype, replace, fanout):
    indptr, indices = graph
    rng = np.random.default_rng(fanout)
    seeds = rng.choice(len(indptr) - 1, size=3000, replace=False).astype(np.int32)
    seeds[0] = 0  # the hub
    src, dst, ptr, E = fastgl.sample_node_csr(to_dev(indices), to_dev(indptr, ptr_dtype), to_dev(seeds), fanout,
                                              replace=replace, rng_seed=4242, rng_ctr=fanout)
    rptr, rsrc, rdst = oc.sample(indptr, indices, seeds, fanout, replace, rng_seed=4242, rng_ctr=fanout)
    assert E == len(rsrc)
    assert np.array_equal(ptr.cpu().numpy(), rptr)
    assert np.array_equal(src.cpu().numpy(), rsrc)
    assert np.array_equal(dst.cpu().numpy(), rdst)


def test_sample_node_drop_in_signature(fastgl, graph):
    indptr, indices = graph
    seeds = np.arange(100, 612, dtype=np.int32)
    fastgl.seed(12345, 7)
    fastgl.set_sampling(replace=False)
    d_idx = to_dev(indices)
    out = fastgl.sample_node(d_idx, d_idx, to_dev(indptr, torch.int32), to_dev(seeds), len(seeds), 10)
    assert len(out) == 3 and out[2].dtype == torch.int32 and out[2].numel() == 1
    rptr, rsrc, rdst = oc.sample(indptr, indices, seeds, 10, False, rng_seed=12345, rng_ctr=7)
    assert int(out[2].item()) == len(rsrc) == out[0].numel() == out[1].numel()
    assert np.array_equal(out[0].cpu().numpy(), rsrc) and np.array_equal(out[1].cpu().numpy(), rdst)


def test_full_neighbourhood_mode_is_the_csr_itself(fastgl, graph):
    indptr, indices = graph
    deg = np.diff(indptr)
    fan = 100
    seeds = np.nonzero(deg <= fan)[0].astype(np.int32)  # fanout >= degree for every seed
    assert len(seeds) > 15000
    src, _, ptr, E = fastgl.sample_node_csr(to_dev(indices), to_dev(indptr), to_dev(seeds), fan, want_dst=False)
    ref = np.concatenate([indices[indptr[s]:indptr[s + 1]] for s in seeds])
    assert np.array_equal(np.diff(ptr.cpu().numpy()), deg[seeds])
    assert np.array_equal(src.cpu().numpy(), ref)


def test_sample_empty_and_isolated_seeds(fastgl):
    indptr = np.array([0, 0, 2, 2], dtype=np.int64)
    indices = np.array([0, 2], dtype=np.int32)
    src, dst, ptr, E = fastgl.sample_node_csr(to_dev(indices), to_dev(indptr), to_dev(np.array([0, 2, 1, 0], dtype=np.int32)), 4)
    assert E == 2 and ptr.cpu().tolist() == [0, 0, 0, 2, 2]
    assert src.cpu().tolist() == [0, 2] and dst.cpu().tolist() == [1, 1]
    src, dst, ptr, E = fastgl.sample_node_csr(to_dev(indices), to_dev(indptr), torch.zeros(0, dtype=torch.int32, device=dev()), 4)
    assert E == 0 and ptr.cpu().tolist() == [0]


def test_selection_frequency_chi_square_on_gpu(fastgl):
    deg, fanout, trials = 40, 8, 6000
    indptr = np.array([0, deg] + [deg] * deg, dtype=np.int64)
    indices = np.arange(1, deg + 1, dtype=np.int32)
    seeds = np.zeros(trials, dtype=np.int32)
    for replace in (False, True):
        src, _, _, E = fastgl.sample_node_csr(to_dev(indices), to_dev(indptr), to_dev(seeds), fanout, replace=replace,
                                              rng_seed=777, rng_ctr=1, want_dst=False)
        src = src.cpu().numpy()
        assert E == trials * fanout
        counts = np.bincount(src, minlength=deg + 1)[1:]
        expected = trials * fanout / deg
        assert float(((counts - expected) ** 2 / expected).sum()) < 72.1  # chi-square(39), p = 0.001
        if not replace:
            per_seed = src.reshape(trials, fanout)
            assert all(len(set(r.tolist())) == fanout for r in per_seed[:500])


def test_out_of_range_seed_is_reported(fastgl, graph):
    indptr, indices = graph
    seeds = np.array([1, 2, len(indptr) + 5], dtype=np.int32)
    with pytest.raises(RuntimeError, match="out of range"):
        fastgl.sample_node_csr(to_dev(indices), to_dev(indptr), to_dev(seeds), 5)
    # the workspace stays usable
    src, _, _, E = fastgl.sample_node_csr(to_dev(indices), to_dev(indptr), to_dev(seeds[:2]), 5)
    assert E == src.numel()


# ----------------------------------------------------------------------------------------------
# a2
# ----------------------------------------------------------------------------------------------
def check_map_invariants(src_g, dst_g, seeds, src_l, dst_l, uniq):
    S = len(seeds)
    assert np.array_equal(uniq[:S], seeds)                                   # (i)
    pos = {int(v): i for i, v in enumerate(seeds)}
    assert np.array_equal(dst_l, np.array([pos[int(v)] for v in dst_g], dtype=np.int32))  # (ii)
    assert np.array_equal(uniq[src_l], src_g)                                # (iv)
    new = uniq[S:]
    assert len(set(new.tolist())) == len(new) and not (set(new.tolist()) & set(seeds.tolist()))  # (v)
    assert set(new.tolist()) == set(src_g.tolist()) - set(seeds.tolist())


@pytest.mark.parametrize("n_seeds,fanout", [(1, 3), (64, 5), (1024, 5), (6000, 10), (60000, 15)])
def test_map_matches_oracle_first_occurrence_order(fastgl, n_seeds, fanout):
    indptr, indices = make_graph(max(4000, n_seeds * 3), 14, seed=n_seeds, hub=500)
    rng = np.random.default_rng(n_seeds)
    seeds = rng.choice(len(indptr) - 1, size=n_seeds, replace=False).astype(np.int32)
    _, src_g, dst_g = oc.sample(indptr, indices, seeds, fanout, False, rng_seed=3, rng_ctr=1)
    rs, rd, ru = oc.map_edges(src_g, dst_g, seeds)
    fastgl.set_sampling(arrival_order=False)
    d_src, d_dst = to_dev(src_g), to_dev(dst_g)
    out = fastgl.transfer_edge_id(d_src, d_dst, to_dev(seeds), n_seeds, n_seeds + len(src_g),
                                  min(len(indptr) - 1, fanout * n_seeds), len(src_g))
    assert out[0].data_ptr() == d_src.data_ptr() and out[1].data_ptr() == d_dst.data_ptr()  # in place
    assert np.array_equal(out[2].cpu().numpy(), ru)       # (vi) element for element
    assert np.array_equal(out[0].cpu().numpy(), rs)
    assert np.array_equal(out[1].cpu().numpy(), rd)


@pytest.mark.parametrize("n_seeds,fanout", [(64, 5), (6000, 10)])
def test_map_arrival_order_keeps_the_invariants(fastgl, n_seeds, fanout):
    indptr, indices = make_graph(20000, 14, seed=5, hub=500)
    rng = np.random.default_rng(1)
    seeds = rng.choice(len(indptr) - 1, size=n_seeds, replace=False).astype(np.int32)
    _, src_g, dst_g = oc.sample(indptr, indices, seeds, fanout, False, rng_seed=3, rng_ctr=1)
    _, _, ru = oc.map_edges(src_g, dst_g, seeds)
    fastgl.set_sampling(arrival_order=True)
    try:
        out = fastgl.transfer_edge_id(to_dev(src_g), to_dev(dst_g), to_dev(seeds), n_seeds, n_seeds + len(src_g),
                                      fanout * n_seeds, len(src_g))
    finally:
        fastgl.set_sampling(arrival_order=False)
    uniq = out[2].cpu().numpy()
    assert len(uniq) == len(ru)
    check_map_invariants(src_g, dst_g, seeds, out[0].cpu().numpy(), out[1].cpu().numpy(), uniq)


def test_map_without_edges_and_with_repeated_sources(fastgl):
    seeds = np.array([5, 9], dtype=np.int32)
    e = torch.zeros(0, dtype=torch.int32, device=dev())
    out = fastgl.transfer_edge_id(e, e.clone(), to_dev(seeds), 2, 2, 10, 0)
    assert out[2].cpu().tolist() == [5, 9] and out[0].numel() == 0
    src = np.array([7, 7, 7, 5, 7, 11, 11], dtype=np.int32)
    dst = np.array([5, 5, 9, 9, 9, 9, 5], dtype=np.int32)
    out = fastgl.transfer_edge_id(to_dev(src), to_dev(dst), to_dev(seeds), 2, 9, 7, 7)
    assert out[2].cpu().tolist() == [5, 9, 7, 11]
    assert out[0].cpu().tolist() == [2, 2, 2, 0, 2, 3, 3] and out[1].cpu().tolist() == [0, 0, 1, 1, 1, 1, 0]


# ----------------------------------------------------------------------------------------------
# fused multi-hop, multi-mini-batch
# ----------------------------------------------------------------------------------------------
def run_fused_and_compare(fastgl, indptr, indices, seed_lists, fanouts_sampling, replace, n_teams, ptr_dtype=torch.int64,
                          table_slots=0):
    nb = len(seed_lists)
    stride = max(len(s) for s in seed_lists)
    seeds = np.zeros((nb, stride), dtype=np.int32)
    counts = np.zeros(nb, dtype=np.int32)
    for b, s in enumerate(seed_lists):
        seeds[b, :len(s)] = s
        counts[b] = len(s)
    fb = fastgl.sample_map_fused(to_dev(indptr, ptr_dtype), to_dev(indices), to_dev(seeds), to_dev(counts),
                                 fanouts_sampling, replace=replace, arrival_order=False, rng_seed=31337, rng_ctr=800,
                                 n_teams=n_teams, table_slots=table_slots)
    fastgl.check_status()
    L = len(fanouts_sampling)
    for b, s in enumerate(seed_lists):
        # the oracle takes the fanouts input-layer first and walks them reversed (FusedMapSampler.py:72)
        inputs, _, blocks = oc.sample_blocks(indptr, indices, np.asarray(s, dtype=np.int32), list(reversed(fanouts_sampling)),
                                             replace, rng_seed=31337, rng_ctr=800 + 8 * b)
        got_blocks = fb.blocks(b)
        assert np.array_equal(fb.input_nodes(b).cpu().numpy(), inputs), f"batch {b} node list"
        assert len(got_blocks) == L
        for (gptr, gsrc, n_src, n_dst), ref in zip(got_blocks, blocks):
            assert (n_src, n_dst) == (ref["n_src"], ref["n_dst"])
            assert np.array_equal(gptr.cpu().numpy(), ref["indptr"])
            assert np.array_equal(gsrc.cpu().numpy(), ref["src_local"])
    return fb


@pytest.mark.parametrize("replace", [False, True])
@pytest.mark.parametrize("n_teams", [1, 3])
def test_fused_matches_oracle(fastgl, graph, replace, n_teams):
    indptr, indices = graph
    rng = np.random.default_rng(17)
    seed_lists = [rng.choice(len(indptr) - 1, size=n, replace=False).astype(np.int32) for n in (256, 256, 100, 1, 256)]
    seed_lists[0][0] = 0
    run_fused_and_compare(fastgl, indptr, indices, seed_lists, [5, 10, 15], replace, n_teams)


def test_fused_with_a_capped_table_and_recovery_from_a_table_that_is_too_small(fastgl, graph):
    """A table capped at 4x the node count gives the same blocks; one that cannot hold the mini-batch is reported
    (no fault, the launch stops early), the asynchronous read-back shows the status, and the next launch with a
    large enough table is correct again."""
    indptr, indices = graph
    rng = np.random.default_rng(23)
    seed_lists = [rng.choice(len(indptr) - 1, size=256, replace=False).astype(np.int32) for _ in range(3)]
    fb = run_fused_and_compare(fastgl, indptr, indices, seed_lists, [5, 10, 15], False, 3, table_slots=1 << 16)
    assert int(fb.counts_host()[:, 3].max()) > 2048
    seeds = to_dev(np.stack(seed_lists))
    counts = to_dev(np.full(3, 256, dtype=np.int32))
    small = fastgl.sample_map_fused(to_dev(indptr, torch.int64), to_dev(indices), seeds, counts, [5, 10, 15], rng_seed=31337,
                                    rng_ctr=800, n_teams=3, table_slots=2048)
    small.start_readback()
    small.counts_host()
    assert small.device_status != 0
    with pytest.raises(RuntimeError, match="probe"):
        fastgl.check_status()
    run_fused_and_compare(fastgl, indptr, indices, seed_lists, [5, 10, 15], False, 3)


def test_fused_int32_indptr_single_batch_two_hops(fastgl, graph):
    indptr, indices = graph
    seeds = [np.arange(50, 1074, dtype=np.int32)]
    run_fused_and_compare(fastgl, indptr, indices, seeds, [10, 25], False, 0, ptr_dtype=torch.int32)


def test_fused_wide_fanout_uses_the_warp_per_seed_path(fastgl, graph):
    # fanouts above 32 take the warp-per-seed sampler inside the fused kernel; the hub (node 0) has 3000+ neighbours
    indptr, indices = graph
    seeds = [np.concatenate([[0], np.arange(500, 563)]).astype(np.int32), np.arange(900, 964, dtype=np.int32)]
    run_fused_and_compare(fastgl, indptr, indices, seeds, [40, 3], False, 2)
    run_fused_and_compare(fastgl, indptr, indices, seeds, [3, 64], True, 1)


def test_fused_frontier_saturates_small_graph(fastgl):
    # the frontier reaches every node: capacities are clamped by the node count
    indptr, indices = make_graph(600, 10, seed=2, hub=100)
    seeds = [np.arange(0, 128, dtype=np.int32), np.arange(300, 428, dtype=np.int32)]
    run_fused_and_compare(fastgl, indptr, indices, seeds, [5, 10, 15], False, 2)


def test_fused_empty_batch_list_and_empty_batch(fastgl, graph):
    indptr, indices = graph
    run_fused_and_compare(fastgl, indptr, indices, [np.zeros(0, dtype=np.int32), np.arange(10, dtype=np.int32)], [3, 3], False, 0)


def test_fused_arrival_order_invariants(fastgl, graph):
    indptr, indices = graph
    rng = np.random.default_rng(4)
    seeds = rng.choice(len(indptr) - 1, size=(3, 512), replace=False).astype(np.int32)
    counts = np.full(3, 512, dtype=np.int32)
    fan = [5, 10, 15]
    fb = fastgl.sample_map_fused(to_dev(indptr), to_dev(indices), to_dev(seeds), to_dev(counts), fan, replace=False,
                                 arrival_order=True, rng_seed=5, rng_ctr=0)
    fastgl.check_status()
    for b in range(3):
        nodes = fb.input_nodes(b).cpu().numpy()
        assert len(set(nodes.tolist())) == len(nodes)
        cur = seeds[b]
        for h, (gptr, gsrc, n_src, n_dst) in enumerate(reversed(fb.blocks(b))):
            rptr, rsrc, _ = oc.sample(indptr, indices, cur, fan[h], False, rng_seed=5, rng_ctr=8 * b + h)
            assert n_dst == len(cur) and np.array_equal(gptr.cpu().numpy(), rptr)
            assert np.array_equal(nodes[gsrc.cpu().numpy()], rsrc)      # every edge maps back to its global source
            assert np.array_equal(nodes[:n_dst], cur)
            cur = nodes[:n_src]


# ----------------------------------------------------------------------------------------------
# a4-a7
# ----------------------------------------------------------------------------------------------
def random_block(rng, n_dst, n_src, max_deg, zero_frac=0.1):
    deg = rng.integers(1, max_deg + 1, size=n_dst)
    deg[rng.random(n_dst) < zero_frac] = 0
    indptr = np.zeros(n_dst + 1, dtype=np.int32)
    indptr[1:] = np.cumsum(deg)
    src = rng.integers(0, n_src, size=int(indptr[-1])).astype(np.int32)
    return indptr, src


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("dim", [1, 6, 47, 100, 128, 130, 256, 260, 602, 1024])
def test_aggregate_forward_backward(fastgl, mode, dim):
    """Every forward kernel: rows staged through one 512-byte slot (100, 128), wider rows swept with several
    accumulators and a ragged last pass (130, 260, 602), 8-byte-aligned strides (6, 130, 602), odd widths (1, 47);
    in-degrees up to 40, i.e. beyond the 15 rows of a staged pass and beyond the 32 ids a warp keeps in registers."""
    rng = np.random.default_rng(dim * 3 + mode)
    n_dst, n_src = 700, 2500
    indptr, src = random_block(rng, n_dst, n_src, 40)
    x = rng.standard_normal((n_src, dim)).astype(np.float32)
    dy = rng.standard_normal((n_dst, dim)).astype(np.float32)
    sdeg = np.maximum(oc.cal_deg(src, n_src), 1)
    ddeg = np.maximum(np.diff(indptr), 1).astype(np.int32)
    out = fastgl.aggregate(mode, to_dev(indptr), to_dev(src), to_dev(x), n_dst, to_dev(sdeg), to_dev(ddeg))
    ref = oc.aggregate_fwd(mode, indptr, src, x, n_dst, sdeg, ddeg)
    assert rel_err(out.cpu().numpy(), ref) <= AGG_RTOL
    dx = fastgl.aggregate_backward(mode, to_dev(indptr), to_dev(src), to_dev(dy), n_src, to_dev(sdeg), to_dev(ddeg))
    refb = oc.aggregate_bwd(mode, indptr, src, dy, n_src, sdeg, ddeg)
    assert rel_err(dx.cpu().numpy(), refb) <= AGG_RTOL


@pytest.mark.parametrize("mode", [0, 2])
@pytest.mark.parametrize("with_map", [False, True])
@pytest.mark.parametrize("dim", [100, 602])
def test_aggregate_reports_an_out_of_range_id_and_matches_the_oracle_without_it(fastgl, mode, with_map, dim):
    """One edge carries a source id beyond the input rows (and one a negative id): the ids are never dereferenced,
    the status word reports them, and the result equals the oracle's on the block with those two edges removed."""
    rng = np.random.default_rng(99 + mode)
    n_dst, n_src, n_table = 300, 900, 5000
    indptr, src = random_block(rng, n_dst, n_src, 40, zero_frac=0.0)
    row_map = rng.permutation(n_table)[:n_src].astype(np.int32) if with_map else None
    table = rng.standard_normal((n_table if with_map else n_src, dim)).astype(np.float32)
    sdeg = np.maximum(oc.cal_deg(src, n_src), 1)
    ddeg = np.maximum(np.diff(indptr), 1).astype(np.int32)
    bad = src.copy()
    e_hi, e_lo = int(indptr[17]), int(indptr[170])              # the first edges of rows 17 and 170
    bad[e_hi] = n_src + 12345
    bad[e_lo] = -3
    if with_map:
        row_map_bad = row_map.copy()
        victim = int(bad[int(indptr[5])])                      # a third edge whose *mapped* row is beyond the table
        row_map_bad[victim] = n_table + 7
    out = fastgl.aggregate(mode, to_dev(indptr), to_dev(bad), to_dev(table), n_dst, to_dev(sdeg), to_dev(ddeg),
                           row_map=to_dev(row_map_bad) if with_map else None)
    with pytest.raises(RuntimeError, match="out of range"):
        fastgl.check_status(dev())
    fastgl.check_status(dev())                                  # cleared: the next check passes
    # the oracle on the same block without the bad edges, weights of the remaining edges unchanged
    x = table[row_map] if with_map else table
    w = np.ones(len(src), dtype=np.float64)
    if mode == 2:
        dst_of = np.repeat(np.arange(n_dst), np.diff(indptr))
        w = (1.0 / np.sqrt(ddeg[dst_of].astype(np.float32))).astype(np.float64) * (1.0 / np.sqrt(sdeg[src].astype(np.float32))).astype(np.float64)
    keep = np.ones(len(src), dtype=bool)
    keep[[e_hi, e_lo]] = False
    if with_map:
        keep &= src != victim
    ref = np.zeros((n_dst, dim), dtype=np.float64)
    dst_of = np.repeat(np.arange(n_dst), np.diff(indptr))
    np.add.at(ref, dst_of[keep], x[src[keep]].astype(np.float64) * w[keep, None])
    assert rel_err(out.cpu().numpy(), ref) <= AGG_RTOL
    # backward: the bad edges scatter nothing and are reported
    dy = rng.standard_normal((n_dst, dim)).astype(np.float32)
    dx = fastgl.aggregate_backward(mode, to_dev(indptr), to_dev(bad), to_dev(dy), n_src, to_dev(sdeg), to_dev(ddeg))
    with pytest.raises(RuntimeError, match="out of range"):
        fastgl.check_status(dev())
    refb = np.zeros((n_src, dim), dtype=np.float64)
    keep_b = np.ones(len(src), dtype=bool)
    keep_b[[e_hi, e_lo]] = False
    np.add.at(refb, src[keep_b], dy[dst_of[keep_b]].astype(np.float64) * w[keep_b, None])
    assert rel_err(dx.cpu().numpy(), refb) <= AGG_RTOL


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("dim", [47, 100, 256, 1024])
def test_backward_gather_over_the_transposed_block_is_exact_to_tolerance_and_reproducible(fastgl, mode, dim):
    """A power-law source side: one source with 12 000 in-block edges, a few dozen with hundreds, the rest with a
    handful, repeated edges included.  The gather equals the oracle (and the scatter) to the aggregation tolerance,
    gives the same bits twice, and folds the self gradient in."""
    rng = np.random.default_rng(1000 + 7 * dim + mode)
    n_dst, n_src = 40_000 if dim <= 256 else 14_000, 9000
    deg = rng.integers(0, 9, size=n_dst)
    indptr = np.zeros(n_dst + 1, dtype=np.int32)
    indptr[1:] = np.cumsum(deg)
    w = 1.0 / np.arange(1, n_src + 1) ** 1.1
    src = rng.choice(n_src, size=int(indptr[-1]), p=w / w.sum()).astype(np.int32)
    hub_rows = rng.choice(np.flatnonzero(deg > 0), size=min(12_000, int((deg > 0).sum())), replace=False)
    src[indptr[hub_rows]] = 7                                     # source 7 is in 12 000 rows (n_dst > 32768: two windows)
    dy = rng.standard_normal((n_dst, dim)).astype(np.float32)
    dself = rng.standard_normal((n_dst if n_dst <= n_src else n_src, dim)).astype(np.float32)
    sdeg = np.maximum(oc.cal_deg(src, n_src), 1)
    ddeg = np.maximum(deg, 1).astype(np.int32)
    d_ptr, d_src, d_dy, d_sdeg, d_ddeg = to_dev(indptr), to_dev(src), to_dev(dy), to_dev(sdeg), to_dev(ddeg)
    tb = fastgl.transpose_block(d_ptr, d_src, n_dst, n_src)
    fastgl.check_status(dev())
    assert int(tb.hubs[0]) >= 1 and 7 in tb.hubs[1: 1 + int(tb.hubs[0])].tolist()
    assert torch.equal(tb.t_indptr[1:].long(), torch.cumsum(torch.bincount(d_src.long(), minlength=n_src), 0))
    got = fastgl.aggregate_backward(mode, d_ptr, d_src, d_dy, n_src, d_sdeg, d_ddeg, transposed=tb)
    again = fastgl.aggregate_backward(mode, d_ptr, d_src, d_dy, n_src, d_sdeg, d_ddeg, transposed=tb)
    assert torch.equal(got, again)                                # bit-reproducible
    tb2 = fastgl.transpose_block(d_ptr, d_src, n_dst, n_src)     # another transposition (another fill order): same bits
    assert torch.equal(got, fastgl.aggregate_backward(mode, d_ptr, d_src, d_dy, n_src, d_sdeg, d_ddeg, transposed=tb2))
    ref = oc.aggregate_bwd(mode, indptr, src, dy, n_src, sdeg, ddeg)
    assert rel_err(got.cpu().numpy(), ref) <= AGG_RTOL
    scat = fastgl.aggregate_backward(mode, d_ptr, d_src, d_dy, n_src, d_sdeg, d_ddeg)
    assert rel_err(scat.cpu().numpy(), ref) <= AGG_RTOL
    if n_dst <= n_src:                                            # the self term (destinations are the first sources)
        with_self = fastgl.aggregate_backward(mode, d_ptr, d_src, d_dy, n_src, d_sdeg, d_ddeg, transposed=tb, d_self=to_dev(dself))
        want = ref.copy()
        want[:n_dst] += dself
        assert rel_err(with_self.cpu().numpy(), want) <= AGG_RTOL


def test_backward_gather_with_a_self_term_and_a_device_side_row_count(fastgl):
    rng = np.random.default_rng(77)
    n_real, n_pad, n_src, dim = 900, 1024, 5000, 128
    deg = rng.integers(0, 12, size=n_real)
    indptr = np.zeros(n_pad + 1, dtype=np.int32)
    indptr[1: n_real + 1] = np.cumsum(deg)
    indptr[n_real + 1:] = indptr[n_real]
    src = rng.integers(0, n_src, size=int(indptr[n_real]) + 64).astype(np.int32)   # stale entries beyond the real edges
    dcat = rng.standard_normal((n_pad, 2 * dim)).astype(np.float32)                # padded rows hold garbage
    d_ptr, d_src, d_cat = to_dev(indptr), to_dev(src), to_dev(dcat)
    n_dev = torch.tensor([n_real], dtype=torch.int32, device=dev())
    tb = fastgl.transpose_block(d_ptr, d_src, n_pad, n_src, n_dst_dev=n_dev)
    got = fastgl.aggregate_backward(fastgl.AGG_MEAN, d_ptr, d_src, d_cat[:, dim:], n_src, n_dst_dev=n_dev, d_self=d_cat[:, :dim],
                                    transposed=tb)
    ref = oc.aggregate_bwd(oc.MODE_MEAN, indptr[: n_real + 1], src[: indptr[n_real]], dcat[:n_real, dim:], n_src)
    ref[:n_real] += dcat[:n_real, :dim]
    assert rel_err(got.cpu().numpy(), ref) <= AGG_RTOL
    fastgl.check_status(dev())


def test_gather_rows_reports_an_out_of_range_id(fastgl):
    table = torch.randn((1000, 100), device=dev())
    ids = torch.tensor([5, 1000, 999, -1, 0], dtype=torch.int32, device=dev())
    got = fastgl.gather_rows(table, ids)
    with pytest.raises(RuntimeError, match="out of range"):
        fastgl.check_status(dev())
    assert torch.equal(got[[0, 2, 4]], table[[5, 999, 0]]) and not got[[1, 3]].any()


def test_window_overlap_kernel_matches_the_mask_product(fastgl):
    """|nodes_i & nodes_j| for the node lists of a window, against the dense-mask product Match-Reorder is defined by."""
    from fastgl_b200.scheduler import overlap_matrix
    rng = np.random.default_rng(12)
    n, W, stride = 200_000, 16, 40_000
    counts = rng.integers(1000, stride, size=W).astype(np.int32)
    counts[5] = 0
    nodes = rng.integers(0, n, size=(W, stride)).astype(np.int32)        # stale ids beyond every list
    lists = []
    for b in range(W):
        ids = rng.choice(n, size=counts[b], replace=False).astype(np.int32)
        nodes[b, : counts[b]] = ids
        lists.append(torch.from_numpy(ids).to(dev()))
    padded_counts = torch.zeros((W, 16), dtype=torch.int32, device=dev())  # one column of a wider array, as the sampler leaves it
    padded_counts[:, 3] = to_dev(counts)
    mask = torch.zeros(n, dtype=torch.int32, device=dev())
    got = fastgl.window_overlap(to_dev(nodes), padded_counts[:, 3], n, mask)
    want = overlap_matrix(lists, n)
    assert torch.equal(got.float(), want)
    assert not mask.any()                                                  # left clean for the next window
    assert torch.equal(fastgl.window_overlap(to_dev(nodes), padded_counts[:, 3], n, mask).float(), want)


def test_bounded_barrier_wait_runs_out_and_the_workspace_recovers(fastgl):
    """A team barrier that one arrival never reaches gives up after its spin limit, reports FGL_ERR_TIMEOUT through
    the status word (no fault, no hang), and the same workspace then runs the next barrier-using call correctly."""
    import ctypes
    from fastgl import _capi
    d = dev()
    ws = fastgl._ws(d)
    rc = _capi.lib().fgl_selftest_barrier_timeout(ws, 4, ctypes.c_int64(1000), ctypes.c_void_p(torch.cuda.current_stream(d).cuda_stream))
    assert rc == 0
    with pytest.raises(RuntimeError, match="wait gave up"):
        fastgl.check_status(d)
    fastgl.check_status(d)
    degs = torch.randint(0, 9, (1_000_003,), dtype=torch.int32, device=d)
    out = fastgl.exclusive_sum(degs)                            # two-level scan: uses the same barrier
    fastgl.check_status(d)
    assert torch.equal(out[1:].long(), torch.cumsum(degs.long(), 0))


@pytest.mark.parametrize("dim", [100, 128, 256, 602])
def test_aggregate_sampled_block_shapes_with_row_map(fastgl, dim):
    # in-degrees 0..15 (the sampled-block case) plus a few long rows, both zero-degree conventions
    rng = np.random.default_rng(dim)
    n_dst, n_src = 3000, 9000
    deg = rng.integers(0, 16, size=n_dst)
    deg[::97] = 40
    indptr = np.zeros(n_dst + 1, dtype=np.int32)
    indptr[1:] = np.cumsum(deg)
    src = rng.integers(0, n_src, size=int(indptr[-1])).astype(np.int32)
    table = rng.standard_normal((20000, dim)).astype(np.float32)
    row_map = rng.choice(20000, size=n_src, replace=False).astype(np.int32)
    for mode in (0, 1):
        for passthrough in (True, False):
            out = fastgl.aggregate(mode, to_dev(indptr), to_dev(src), to_dev(table), n_dst, row_map=to_dev(row_map),
                                   zero_deg_passthrough=passthrough)
            ref = oc.aggregate_fwd(mode, indptr, src, table, n_dst, zero_deg_passthrough=passthrough, row_map=row_map)
            assert rel_err(out.cpu().numpy(), ref) <= AGG_RTOL
    fastgl.check_status()


@pytest.mark.parametrize("dim", [100, 602, 1024])
def test_aggregate_window_matches_per_batch_aggregation(fastgl, graph, dim):
    indptr, indices = graph
    rng = np.random.default_rng(23)
    n = len(indptr) - 1
    feat = rng.standard_normal((n, dim)).astype(np.float32)
    seeds = rng.choice(n, size=(5, 200), replace=False).astype(np.int32)
    counts = np.array([200, 200, 7, 0, 200], dtype=np.int32)
    fan = [5, 10, 15]
    fb = fastgl.sample_map_fused(to_dev(indptr), to_dev(indices), to_dev(seeds), to_dev(counts), fan, rng_seed=1, rng_ctr=0)
    d_feat = to_dev(feat)
    hop = 2
    total = int(fb.counts_host()[:, hop].sum())
    for _ in range(1):
        out = torch.full((total, dim), 7.0, device=dev())
        self_out = torch.full((total, dim), 7.0, device=dev())
        timing = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        row_off = fastgl.aggregate_window(fastgl.AGG_MEAN, fb, hop, d_feat, out, self_out=self_out, timing=timing)
        assert row_off[-1] == total
        timing[1].synchronize()
        assert 0.0 < timing[0].elapsed_time(timing[1]) < 50.0    # the library recorded both events around its launch
        for b in range(5):
            (ptr, src, n_src, n_dst) = fb.blocks(b)[0]
            nodes = fb.input_nodes(b).cpu().numpy()
            ref = oc.aggregate_fwd(oc.MODE_MEAN, ptr.cpu().numpy(), src.cpu().numpy(), feat, n_dst, zero_deg_passthrough=False,
                                   row_map=nodes)
            got = out[row_off[b]: row_off[b + 1]].cpu().numpy()
            assert got.shape == ref.shape
            if n_dst:
                assert rel_err(got, ref) <= AGG_RTOL
                assert np.array_equal(self_out[row_off[b]: row_off[b + 1]].cpu().numpy(), feat[nodes[:n_dst]])
    fastgl.check_status()


@pytest.mark.parametrize("dim", [100, 602, 1024])
def test_gather_rows_dense_and_sharded(fastgl, dim):
    rng = np.random.default_rng(dim)
    n = 10_000
    table = rng.standard_normal((n, dim)).astype(np.float32)
    ids = rng.integers(0, n, size=7777).astype(np.int32)
    d_table = to_dev(table)
    got = fastgl.gather_rows(d_table, to_dev(ids))
    assert np.array_equal(got.cpu().numpy(), table[ids])               # a copy: bit-exact
    assert fastgl.gather_rows(d_table, torch.zeros(0, dtype=torch.int32, device=dev())).shape == (0, dim)
    # the same table cut into three row blocks (all on this GPU; on a multi-GPU box they would be peers' buffers)
    rps = 3400
    shards = [to_dev(np.ascontiguousarray(table[i * rps:(i + 1) * rps])) for i in range(3)]
    st = fastgl.ShardedTable(shards, rps, dim, n, dev())
    assert np.array_equal(fastgl.gather_rows(st, to_dev(ids)).cpu().numpy(), table[ids])


def test_aggregate_from_a_sharded_table_matches_the_dense_table(fastgl, graph):
    indptr, indices = graph
    rng = np.random.default_rng(31)
    n = len(indptr) - 1
    feat = rng.standard_normal((n, 128)).astype(np.float32)
    seeds = rng.choice(n, size=(2, 300), replace=False).astype(np.int32)
    fb = fastgl.sample_map_fused(to_dev(indptr), to_dev(indices), to_dev(seeds), to_dev(np.array([300, 300], dtype=np.int32)),
                                 [5, 10], rng_seed=2, rng_ctr=0)
    rps = (n + 3) // 4
    shards = [to_dev(np.ascontiguousarray(feat[i * rps:(i + 1) * rps])) for i in range(4)]
    st = fastgl.ShardedTable(shards, rps, 128, n, dev())
    d_feat = to_dev(feat)
    ptr, src, n_src, n_dst = fb.blocks(1)[0]
    nodes = fb.input_nodes(1)
    a = fastgl.aggregate(fastgl.AGG_MEAN, ptr, src, d_feat, n_dst, row_map=nodes, zero_deg_passthrough=False)
    b = fastgl.aggregate(fastgl.AGG_MEAN, ptr, src, st, n_dst, row_map=nodes, zero_deg_passthrough=False)
    assert torch.equal(a, b)
    total = int(fb.counts_host()[:, 1].sum())
    oa, ob = torch.empty((total, 128), device=dev()), torch.empty((total, 128), device=dev())
    sa, sb = torch.empty_like(oa), torch.empty_like(ob)
    fastgl.aggregate_window(fastgl.AGG_MEAN, fb, 1, d_feat, oa, self_out=sa)
    fastgl.aggregate_window(fastgl.AGG_MEAN, fb, 1, st, ob, self_out=sb)
    assert torch.equal(oa, ob) and torch.equal(sa, sb)


def test_aggregate_high_degree_rows_and_row_map(fastgl):
    rng = np.random.default_rng(9)
    n_dst, n_src, dim = 64, 30000, 100
    deg = np.array([20000, 0, 33, 1] * 16)
    indptr = np.zeros(n_dst + 1, dtype=np.int32)
    indptr[1:] = np.cumsum(deg)
    src = rng.integers(0, n_src, size=int(indptr[-1])).astype(np.int32)
    table = rng.standard_normal((50000, dim)).astype(np.float32)
    row_map = rng.choice(50000, size=n_src, replace=False).astype(np.int32)
    out = fastgl.aggregate(1, to_dev(indptr), to_dev(src), to_dev(table), n_dst, row_map=to_dev(row_map),
                           zero_deg_passthrough=False)
    ref = oc.aggregate_fwd(1, indptr, src, table, n_dst, zero_deg_passthrough=False, row_map=row_map)
    assert rel_err(out.cpu().numpy(), ref) <= AGG_RTOL
    assert not out[1].any()


def test_gcn_ops_match_oracle(fastgl):
    from oracle import oracle_np as on
    rng = np.random.default_rng(12)
    n_dst, n_src, din, dout = 300, 900, 100, 47
    indptr, src = random_block(rng, n_dst, n_src, 12)
    x = rng.standard_normal((n_src, din)).astype(np.float32)
    w = (rng.standard_normal((din, dout)) / 10).astype(np.float32)
    g = rng.standard_normal((n_dst, dout)).astype(np.float32)
    sdeg = np.maximum(oc.cal_deg(src, n_src), 1)
    ddeg = np.maximum(np.diff(indptr), 1).astype(np.int32)
    t = [to_dev(a) for a in (indptr, src, sdeg, ddeg, x, w, g)]
    out = fastgl.forward_gcn(t[0], t[1], t[2], t[3], t[4], t[5], 12, n_dst)[0]
    assert rel_err(out.cpu().numpy(), on.forward_gcn(indptr, src, sdeg, ddeg, x, w, n_dst)) <= 5e-5  # includes the tf32-free mm
    d_x, d_w = fastgl.backward_gcn(t[0], t[1], t[3], t[2], t[6], t[5], t[4])  # swapped degrees, GraphConv.py:37
    rx, rw = on.backward_gcn(indptr, src, ddeg, sdeg, g, w, x)
    assert rel_err(d_x.cpu().numpy(), rx) <= 5e-5 and rel_err(d_w.cpu().numpy(), rw) <= 5e-5


def test_gin_ops_match_oracle(fastgl):
    from oracle import oracle_np as on
    rng = np.random.default_rng(13)
    n_dst, n_src, din, dout = 300, 900, 128, 256
    indptr, src = random_block(rng, n_dst, n_src, 10)
    x = rng.standard_normal((n_src, din)).astype(np.float32)
    w = (rng.standard_normal((din, dout)) / 10).astype(np.float32)
    g = rng.standard_normal((n_dst, dout)).astype(np.float32)
    t = [to_dev(a) for a in (indptr, src, x, w, g)]
    out, tmp = fastgl.forwaed_gin(t[0], t[1], t[2], t[3], 10, n_dst)
    rout, rtmp = on.forward_gin(indptr, src, x, w, n_dst)
    assert rel_err(tmp.cpu().numpy(), rtmp) <= AGG_RTOL and rel_err(out.cpu().numpy(), rout) <= 5e-5
    d_x, d_w = fastgl.backward_gin(t[0], t[1], t[4], t[3], tmp, n_src)
    rx, rw = on.backward_gin(indptr, src, g, w, rtmp, n_src)
    assert rel_err(d_x.cpu().numpy(), rx) <= 5e-5 and rel_err(d_w.cpu().numpy(), rw) <= 5e-5


@pytest.mark.parametrize("dim,heads", [(64, 8), (256, 8), (47, 1), (24, 8), (602, 7)])
def test_gat_ops_match_oracle(fastgl, dim, heads):
    rng = np.random.default_rng(dim + heads)
    n_dst, n_src = 400, 1500
    indptr, src = random_block(rng, n_dst, n_src, 20)
    E = int(indptr[-1])
    x = rng.standard_normal((n_src, dim)).astype(np.float32)
    w = rng.random((E, heads)).astype(np.float32)
    g = rng.standard_normal((n_dst, dim)).astype(np.float32)
    t = [to_dev(a) for a in (indptr, w, src, x, g)]
    out = fastgl.forward_gat(t[0], t[1], t[2], t[3], 20, n_dst, heads)[0]
    assert rel_err(out.cpu().numpy(), oc.aggregate_edge_fwd(indptr, src, w, x, n_dst)) <= AGG_RTOL
    d_x = fastgl.backward_gat(t[0], t[1], t[2], t[4], n_src, heads)[0]
    assert rel_err(d_x.cpu().numpy(), oc.aggregate_edge_bwd(indptr, src, w, g, n_src)) <= AGG_RTOL
    # gradient of the coefficients (not in the reference): per edge and head, <dy[d], x[src]> over the head's columns
    d_w = fastgl.edge_weight_grad(t[0], t[2], t[3], t[4], heads).cpu().numpy()
    unit = dim // heads
    dst = np.repeat(np.arange(n_dst), np.diff(indptr))
    ref = (g[dst].astype(np.float64) * x[src].astype(np.float64)).reshape(E, heads, unit).sum(-1)
    assert rel_err(d_w, ref) <= AGG_RTOL


def test_golden_fixtures_on_gpu(fastgl):
    g = np.load(GOLDEN)
    indptr, indices, seeds = g["indptr"], g["indices"], g["seeds"]
    for name, replace in (("norep", False), ("rep", True)):
        src, dst, ptr, E = fastgl.sample_node_csr(to_dev(indices), to_dev(indptr), to_dev(seeds), 5, replace=replace,
                                                  rng_seed=12345, rng_ctr=3)
        assert np.array_equal(src.cpu().numpy(), g[f"{name}_src"]) and np.array_equal(ptr.cpu().numpy(), g[f"{name}_ptr"])
        src = src.contiguous().clone()
        dst = dst.contiguous().clone()
        out = fastgl.transfer_edge_id(src, dst, to_dev(seeds), len(seeds), len(seeds) + E, 5 * len(seeds), E)
        assert np.array_equal(out[0].cpu().numpy(), g[f"{name}_src_local"])
        assert np.array_equal(out[1].cpu().numpy(), g[f"{name}_dst_local"])
        assert np.array_equal(out[2].cpu().numpy(), g[f"{name}_unique"])
    x, dy = to_dev(g["x"]), to_dev(g["dy"])
    ptr0, src0 = to_dev(g["mh_ptr0"]), to_dev(g["mh_src0"])
    for mode, tag in ((0, "sum"), (1, "mean"), (2, "sym")):
        f = fastgl.aggregate(mode, ptr0, src0, x, ptr0.numel() - 1, to_dev(g["src_deg"]), to_dev(g["dst_deg"]))
        b = fastgl.aggregate_backward(mode, ptr0, src0, dy, x.size(0), to_dev(g["src_deg"]), to_dev(g["dst_deg"]))
        assert rel_err(f.cpu().numpy(), g[f"fwd_{tag}"]) <= AGG_RTOL and rel_err(b.cpu().numpy(), g[f"bwd_{tag}"]) <= AGG_RTOL

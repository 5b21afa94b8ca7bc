"""CPU tests of the oracle: Philox known answers, hand-derived cases from the reference kernels'
semantics, agreement of the C and numpy restatements, and the committed golden fixtures."""
import os

import numpy as np
import pytest

from conftest import make_graph
from oracle import oracle_c as oc
from oracle import oracle_np as on

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hotpath_small.npz")

# Philox4x32-10 known answers published with the generator (Random123 kat_vectors)
PHILOX_KAT = [
    ((0, 0, 0, 0), (0, 0), (0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8)),
    ((0xFFFFFFFF,) * 4, (0xFFFFFFFF,) * 2, (0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD)),
    ((0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344), (0xA4093822, 0x299F31D0),
     (0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1)),
]


@pytest.mark.parametrize("ctr,key,expect", PHILOX_KAT)
def test_philox_known_answers(ctr, key, expect):
    assert on.philox4x32_10(ctr, key) == expect
    assert oc.philox4x32_10(ctr, key) == expect


def test_sample_hand_case():
    # 4 nodes; in-neighbours: 0 <- {1,2,3}, 1 <- {0}, 2 <- {}, 3 <- {0,1}
    indptr = np.array([0, 3, 4, 4, 6], dtype=np.int64)
    indices = np.array([1, 2, 3, 0, 0, 1], dtype=np.int32)
    seeds = np.array([3, 2, 0], dtype=np.int32)
    for mod in (on, oc):
        # fanout >= every degree: whole lists in CSR order, grouped by seed (sample.cu:82-87)
        ptr, src, dst = mod.sample(indptr, indices, seeds, 3)
        assert ptr.tolist() == [0, 2, 2, 5]
        assert src.tolist() == [0, 1, 1, 2, 3]
        assert dst.tolist() == [3, 3, 0, 0, 0]
        # fanout 2 < deg(0) = 3: two picks out of {1,2,3}; the other seeds are unchanged
        ptr, src, dst = mod.sample(indptr, indices, seeds, 2, rng_seed=5, rng_ctr=1)
        assert ptr.tolist() == [0, 2, 2, 4]
        assert src[:2].tolist() == [0, 1] and set(src[2:].tolist()) <= {1, 2, 3} and src[2] != src[3]


def test_map_hand_case():
    # seeds keep ids 0..S-1; new sources are numbered in first-occurrence order (id_map.cu:259-383)
    seeds = np.array([7, 3, 9], dtype=np.int32)
    src = np.array([5, 3, 8, 5, 7, 2, 8], dtype=np.int32)
    dst = np.array([7, 7, 3, 3, 9, 9, 9], dtype=np.int32)
    for mod in (on, oc):
        sl, dl, uniq = mod.map_edges(src, dst, seeds)
        assert uniq.tolist() == [7, 3, 9, 5, 8, 2]
        assert sl.tolist() == [3, 1, 4, 3, 0, 5, 4]
        assert dl.tolist() == [0, 0, 1, 1, 2, 2, 2]


def test_csr_helpers_hand_case():
    ids = np.array([2, 0, 2, 2, 4], dtype=np.int32)
    for mod in (on, oc):
        deg = mod.cal_deg(ids, 6)
        assert deg.tolist() == [1, 0, 3, 0, 1, 0]
        assert mod.exclusive_sum(deg).tolist() == [0, 1, 1, 4, 4, 5, 5]
        assert mod.exclusive_sum(np.zeros(0, dtype=np.int32)).tolist() == [0]


def test_aggregate_hand_case():
    # rows: 0 <- {1, 2}, 1 <- {} (copies its own row), 2 <- {0}
    indptr = np.array([0, 2, 2, 3], dtype=np.int32)
    src = np.array([1, 2, 0], dtype=np.int32)
    x = np.array([[1, 2], [10, 20], [100, 200]], dtype=np.float32)
    src_deg = np.array([1, 1, 1], dtype=np.int32)
    dst_deg = np.array([2, 1, 1], dtype=np.int32)
    for mod in (on, oc):
        assert np.allclose(mod.aggregate_fwd(0, indptr, src, x, 3), [[110, 220], [10, 20], [1, 2]])
        assert np.allclose(mod.aggregate_fwd(1, indptr, src, x, 3), [[55, 110], [10, 20], [1, 2]])
        assert np.allclose(mod.aggregate_fwd(1, indptr, src, x, 3, zero_deg_passthrough=False)[1], [0, 0])
        sym = mod.aggregate_fwd(2, indptr, src, x, 3, src_deg, dst_deg)
        assert np.allclose(sym, [[110 / np.sqrt(2), 220 / np.sqrt(2)], [10, 20], [1, 2]], rtol=1e-6)
        dy = np.array([[1, 1], [5, 5], [2, 3]], dtype=np.float32)
        # the row without in-edges gives no gradient (aggregate_acc_kernel.cu:498-500)
        assert np.allclose(mod.aggregate_bwd(0, indptr, src, dy, 3), [[2, 3], [1, 1], [1, 1]])
        assert np.allclose(mod.aggregate_bwd(1, indptr, src, dy, 3), [[2, 3], [0.5, 0.5], [0.5, 0.5]])


@pytest.mark.parametrize("replace", [False, True])
@pytest.mark.parametrize("fanout", [1, 5, 16, 40])
def test_c_matches_numpy_sampling_and_map(small_graph, replace, fanout):
    indptr, indices = small_graph
    rng = np.random.default_rng(fanout)
    seeds = rng.choice(len(indptr) - 1, size=150, replace=False).astype(np.int32)
    seeds[0] = 0
    a = on.sample(indptr, indices, seeds, fanout, replace, rng_seed=77, rng_ctr=fanout)
    b = oc.sample(indptr, indices, seeds, fanout, replace, rng_seed=77, rng_ctr=fanout)
    for x, y in zip(a, b):
        assert np.array_equal(x, y)
    ma = on.map_edges(a[1], a[2], seeds)
    mb = oc.map_edges(b[1], b[2], seeds)
    for x, y in zip(ma, mb):
        assert np.array_equal(x, y)


def test_sampling_properties(small_graph):
    indptr, indices = small_graph
    n = len(indptr) - 1
    seeds = np.arange(n, dtype=np.int32)
    ptr, src, dst = oc.sample(indptr, indices, seeds, 10, False, rng_seed=1, rng_ctr=2)
    deg = np.diff(indptr)
    assert np.array_equal(np.diff(ptr), np.minimum(deg, 10))
    for s in range(n):
        got = src[ptr[s]:ptr[s + 1]]
        adj = indices[indptr[s]:indptr[s + 1]]
        if deg[s] <= 10:
            assert np.array_equal(got, adj)  # full-neighbour mode is bit-exact
        else:
            assert set(got.tolist()) <= set(adj.tolist())
    # full-neighbour mode for everyone: fanout >= max degree reproduces the CSR itself
    ptr, src, _ = oc.sample(indptr, indices, seeds, int(deg.max()), False)
    assert np.array_equal(ptr, indptr.astype(np.int32)) and np.array_equal(src, indices)


def test_without_replacement_picks_are_distinct_positions():
    # a hub whose neighbours are all different: picks must be distinct
    n = 500
    indptr = np.zeros(n + 1, dtype=np.int64)
    indptr[1:] = n - 1
    indices = np.arange(1, n, dtype=np.int32)
    seeds = np.zeros(64, dtype=np.int32)
    _, src, _ = oc.sample(indptr, indices, seeds, 25, False, rng_seed=3, rng_ctr=0)
    for s in range(64):
        assert len(set(src[s * 25:(s + 1) * 25].tolist())) == 25


@pytest.mark.parametrize("replace", [False, True])
def test_selection_frequency_chi_square(replace):
    # every neighbour of a hub is selected with probability fanout / deg
    deg, fanout, trials = 40, 8, 6000
    indptr = np.array([0, deg] + [deg] * deg, dtype=np.int64)
    indices = np.arange(1, deg + 1, dtype=np.int32)
    seeds = np.zeros(trials, dtype=np.int32)
    _, src, _ = oc.sample(indptr, indices, seeds, fanout, replace, rng_seed=2024, rng_ctr=9)
    counts = np.bincount(src, minlength=deg + 1)[1:]
    expected = trials * fanout / deg
    chi2 = float(((counts - expected) ** 2 / expected).sum())
    assert chi2 < 72.1  # chi-square(39) at p = 0.001


def test_sample_blocks_chain(small_graph):
    indptr, indices = small_graph
    seeds = np.arange(10, 74, dtype=np.int32)
    inputs_a, _, blocks_a = on.sample_blocks(indptr, indices, seeds, [5, 4, 3], rng_seed=8, rng_ctr=40)
    inputs_b, _, blocks_b = oc.sample_blocks(indptr, indices, seeds, [5, 4, 3], rng_seed=8, rng_ctr=40)
    assert np.array_equal(inputs_a, inputs_b)
    assert blocks_a[-1]["n_dst"] == 64 and blocks_a[0]["n_src"] == len(inputs_a)
    for x, y in zip(blocks_a, blocks_b):
        assert np.array_equal(x["indptr"], y["indptr"]) and np.array_equal(x["src_local"], y["src_local"])
    # blocks[i] was sampled with fanouts[i] (FusedMapSampler.py:72,107): in-degree bound per block
    for blk, f in zip(blocks_a, [5, 4, 3]):
        assert np.diff(blk["indptr"]).max() <= f
        assert blk["dst_local"].max() < blk["n_dst"]


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_c_matches_numpy_aggregation(mode):
    rng = np.random.default_rng(mode)
    n_dst, n_src, D = 40, 90, 7
    deg = rng.integers(0, 6, size=n_dst)
    indptr = np.zeros(n_dst + 1, dtype=np.int32)
    indptr[1:] = np.cumsum(deg)
    src = rng.integers(0, n_src, size=indptr[-1]).astype(np.int32)
    x = rng.standard_normal((n_src, D)).astype(np.float32)
    dy = rng.standard_normal((n_dst, D)).astype(np.float32)
    sdeg = np.maximum(on.cal_deg(src, n_src), 1)
    ddeg = np.maximum(deg, 1).astype(np.int32)
    row_map = rng.permutation(n_src).astype(np.int32)
    assert np.allclose(on.aggregate_fwd(mode, indptr, src, x, n_dst, sdeg, ddeg),
                       oc.aggregate_fwd(mode, indptr, src, x, n_dst, sdeg, ddeg), rtol=1e-6, atol=1e-6)
    assert np.allclose(on.aggregate_fwd(mode, indptr, src, x, n_dst, sdeg, ddeg, row_map=row_map),
                       oc.aggregate_fwd(mode, indptr, src, x, n_dst, sdeg, ddeg, row_map=row_map), rtol=1e-6, atol=1e-6)
    assert np.allclose(on.aggregate_bwd(mode, indptr, src, dy, n_src, sdeg, ddeg),
                       oc.aggregate_bwd(mode, indptr, src, dy, n_src, sdeg, ddeg), rtol=1e-6, atol=1e-6)


def test_edge_weighted_aggregation_hand_case_and_restatements_agree():
    # rows: 0 <- {1, 2}, 1 <- {} (copies its own row), 2 <- {0}; 2 heads over 4 columns
    indptr = np.array([0, 2, 2, 3], dtype=np.int32)
    src = np.array([1, 2, 0], dtype=np.int32)
    x = np.array([[1, 2, 3, 4], [10, 20, 30, 40], [100, 200, 300, 400]], dtype=np.float32)
    w = np.array([[0.5, 2.0], [0.25, 1.0], [3.0, -1.0]], dtype=np.float32)
    for mod in (on, oc):
        out = mod.aggregate_edge_fwd(indptr, src, w, x, 3)
        assert np.allclose(out, [[5 + 25, 10 + 50, 60 + 300, 80 + 400], [10, 20, 30, 40], [3, 6, -3, -4]])
        dy = np.ones((3, 4), dtype=np.float32)
        dx = mod.aggregate_edge_bwd(indptr, src, w, dy, 3)
        assert np.allclose(dx, [[3, 3, -1, -1], [0.5, 0.5, 2, 2], [0.25, 0.25, 1, 1]])
    rng = np.random.default_rng(8)
    n_dst, n_src, D, H = 50, 120, 24, 8
    deg = rng.integers(0, 7, size=n_dst)
    indptr = np.zeros(n_dst + 1, dtype=np.int32)
    indptr[1:] = np.cumsum(deg)
    src = rng.integers(0, n_src, size=indptr[-1]).astype(np.int32)
    x = rng.standard_normal((n_src, D)).astype(np.float32)
    w = rng.random((indptr[-1], H)).astype(np.float32)
    dy = rng.standard_normal((n_dst, D)).astype(np.float32)
    assert np.allclose(on.aggregate_edge_fwd(indptr, src, w, x, n_dst), oc.aggregate_edge_fwd(indptr, src, w, x, n_dst), rtol=1e-6, atol=1e-6)
    assert np.allclose(on.aggregate_edge_bwd(indptr, src, w, dy, n_src), oc.aggregate_edge_bwd(indptr, src, w, dy, n_src), rtol=1e-6, atol=1e-6)


def test_gcn_gin_ops_are_adjoint_consistent():
    # <forward(x), dy> == <x, backward(dy)> for the linear aggregation (rows with in-edges only)
    rng = np.random.default_rng(5)
    n_dst, n_src, D = 30, 70, 5
    deg = rng.integers(1, 5, size=n_dst)
    indptr = np.zeros(n_dst + 1, dtype=np.int32)
    indptr[1:] = np.cumsum(deg)
    src = rng.integers(0, n_src, size=indptr[-1]).astype(np.int32)
    x = rng.standard_normal((n_src, D))
    dy = rng.standard_normal((n_dst, D))
    sdeg = np.maximum(on.cal_deg(src, n_src), 1)
    ddeg = deg.astype(np.int32)
    for mode in (0, 1, 2):
        y = on.aggregate_fwd(mode, indptr, src, x, n_dst, sdeg, ddeg)
        dx = on.aggregate_bwd(mode, indptr, src, dy, n_src, sdeg, ddeg)
        assert np.isclose((y * dy).sum(), (x * dx).sum(), rtol=1e-9)
    w = rng.standard_normal((D, 3))
    out = on.forward_gcn(indptr, src, sdeg, ddeg, x, w, n_dst)
    g = rng.standard_normal(out.shape)
    d_x, d_w = on.backward_gcn(indptr, src, ddeg, sdeg, g, w, x)  # call-site order, GraphConv.py:37
    assert np.isclose((out * g).sum(), (x * d_x).sum(), rtol=1e-9)
    assert np.isclose((out * g).sum(), (w * d_w).sum(), rtol=1e-9)
    out, tmp = on.forward_gin(indptr, src, x, w, n_dst)
    d_x, d_w = on.backward_gin(indptr, src, g, w, tmp, n_src)
    assert np.isclose((out * g).sum(), (x * d_x).sum(), rtol=1e-9)
    assert np.isclose((out * g).sum(), (w * d_w).sum(), rtol=1e-9)


def test_golden_fixtures():
    g = np.load(GOLDEN)
    indptr, indices, seeds = g["indptr"], g["indices"], g["seeds"]
    for mod in (on, oc):
        for name, replace in (("norep", False), ("rep", True)):
            ptr, src, dst = mod.sample(indptr, indices, seeds, 5, replace=replace, rng_seed=12345, rng_ctr=3)
            assert np.array_equal(ptr, g[f"{name}_ptr"]) and np.array_equal(src, g[f"{name}_src"])
            assert np.array_equal(dst, g[f"{name}_dst"])
            sl, dl, uniq = mod.map_edges(src, dst, seeds)
            assert np.array_equal(sl, g[f"{name}_src_local"]) and np.array_equal(dl, g[f"{name}_dst_local"])
            assert np.array_equal(uniq, g[f"{name}_unique"])
        inputs, _, blocks = mod.sample_blocks(indptr, indices, seeds, [4, 3], rng_seed=99, rng_ctr=16)
        assert np.array_equal(inputs, g["mh_inputs"])
        for i, blk in enumerate(blocks):
            assert np.array_equal(blk["indptr"], g[f"mh_ptr{i}"]) and np.array_equal(blk["src_local"], g[f"mh_src{i}"])
        blk = blocks[0]
        for mode, tag in ((0, "sum"), (1, "mean"), (2, "sym")):
            f = mod.aggregate_fwd(mode, blk["indptr"], blk["src_local"], g["x"], blk["n_dst"], g["src_deg"], g["dst_deg"])
            b = mod.aggregate_bwd(mode, blk["indptr"], blk["src_local"], g["dy"], blk["n_src"], g["src_deg"], g["dst_deg"])
            assert np.allclose(f, g[f"fwd_{tag}"], rtol=1e-6, atol=1e-6)
            assert np.allclose(b, g[f"bwd_{tag}"], rtol=1e-6, atol=1e-6)

"""Fixtures written by the reference's own CUDA operators (``tests/golden/ref_hotpath.npz``, made on a B200 by
``tests/golden/make_ref_golden.py`` from ``oracle/_ref/fastgl_ref.so``) pin the CPU oracle -- and, on a GPU, this
repository's kernels -- to the reference itself, on inputs inside the reference's preconditions.

What is compared exactly and what only up to the permutation / rounding the reference itself exhibits is stated
per test.  Tolerances: integer and index results bit-exact; fp32 aggregation within 1e-5 of the largest magnitude
(5e-5 where a cuBLAS fp32 product is part of the op).
"""
import os

import numpy as np
import pytest
import torch

from oracle import oracle_c as oc
from oracle import oracle_np as onp

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_hotpath.npz")
AGG_RTOL, MM_RTOL = 1e-5, 5e-5


@pytest.fixture(scope="module")
def ref():
    return dict(np.load(GOLDEN))


def rel_err(got, want):
    return float(np.abs(np.asarray(got, dtype=np.float64) - np.asarray(want, dtype=np.float64)).max()
                 / max(1e-30, float(np.abs(want).max())))


def check_map_against_reference(seeds, src_global, uniq, src_local, dst_local, r_src_local, r_dst_local, r_unique):
    """The properties of ``transfer_edge_id`` that do not depend on the reference's atomic arrival order."""
    S = len(seeds)
    assert np.array_equal(r_unique[:S], seeds) and np.array_equal(uniq[:S], seeds)          # seeds first, in order
    assert np.array_equal(dst_local, r_dst_local)                                            # destination = seed position
    assert len(uniq) == len(r_unique) and set(uniq[S:].tolist()) == set(r_unique[S:].tolist())
    assert len(set(r_unique.tolist())) == len(r_unique)
    assert np.array_equal(r_unique[r_src_local], src_global)                                 # the reference's relabelling ...
    assert np.array_equal(uniq[src_local], src_global)                                       # ... and ours invert the same way
    # both number the new nodes S, S+1, ...: the reference in arrival order, ours in first-occurrence order
    assert sorted(set(r_src_local.tolist()) - set(range(S))) == sorted(set(src_local.tolist()) - set(range(S)))


# ----------------------------------------------------------------------------------------------------------------
# the CPU oracle against the reference's outputs
# ----------------------------------------------------------------------------------------------------------------
def test_oracle_sampling_full_neighbourhood_equals_the_reference(ref):
    ptr, src, dst = oc.sample(ref["graph_indptr"].astype(np.int64), ref["graph_indices"], ref["full_seeds"], int(ref["full_fanout"]))
    assert int(ref["full_edges_num"][0]) == len(src) == int(ptr[-1])
    assert np.array_equal(src, ref["full_src"]) and np.array_equal(dst, ref["full_dst"])   # exact: the CSR slices, in order
    ptr_np, src_np, dst_np = onp.sample(ref["graph_indptr"].astype(np.int64), ref["graph_indices"], ref["full_seeds"],
                                        int(ref["full_fanout"]))
    assert np.array_equal(src_np, ref["full_src"]) and np.array_equal(dst_np, ref["full_dst"])


@pytest.mark.parametrize("replace", [True, False])
def test_oracle_sampling_with_hubs_has_the_reference_s_shape(ref, replace):
    """Hubs: the reference draws with replacement from cuRAND, so only the row lengths, the destinations and the
    membership of the picks are comparable."""
    indptr, indices = ref["graph_indptr"].astype(np.int64), ref["graph_indices"]
    seeds, fanout = ref["hub_seeds"], int(ref["hub_fanout"])
    ptr, src, dst = oc.sample(indptr, indices, seeds, fanout, replace, rng_seed=1, rng_ctr=2)
    assert len(src) == int(ref["hub_edges_num"][0])
    assert np.array_equal(dst, ref["hub_dst"])                                              # same rows of the same lengths
    deg = np.diff(indptr)[seeds]
    assert np.array_equal(np.diff(ptr), np.minimum(deg, fanout))
    for i, s in enumerate(seeds):                                                            # the reference's picks are neighbours
        nbrs = set(indices[indptr[s]: indptr[s + 1]].tolist())
        assert set(ref["hub_src"][ptr[i]: ptr[i + 1]].tolist()) <= nbrs
        assert set(src[ptr[i]: ptr[i + 1]].tolist()) <= nbrs
        if deg[i] <= fanout:                                                                 # short rows: exact
            assert np.array_equal(src[ptr[i]: ptr[i + 1]], ref["hub_src"][ptr[i]: ptr[i + 1]])


def test_oracle_id_map_agrees_with_the_reference_up_to_its_arrival_order(ref):
    for seeds, sg, dg, rs, rd, ru in ((ref["full_seeds"], ref["map_src_global"], ref["map_dst_global"], ref["map_src_local"],
                                       ref["map_dst_local"], ref["map_unique"]),
                                      (ref["hub_seeds"], ref["hub_src"], ref["hub_dst"], ref["hub_map_src_local"],
                                       ref["hub_map_dst_local"], ref["hub_map_unique"])):
        for impl in (oc, onp):
            src_l, dst_l, uniq = impl.map_edges(sg.copy(), dg.copy(), seeds)
            check_map_against_reference(seeds, sg, uniq, src_l, dst_l, rs, rd, ru)


def test_oracle_csr_helpers_equal_the_reference(ref):
    assert np.array_equal(oc.cal_deg(ref["deg_ids"], 500), ref["deg_out"])
    assert np.array_equal(oc.exclusive_sum(ref["deg_out"]), ref["scan_out"])
    assert np.array_equal(onp.cal_deg(ref["deg_ids"], 500), ref["deg_out"])
    assert np.array_equal(onp.exclusive_sum(ref["deg_out"]), ref["scan_out"])


@pytest.mark.parametrize("tag", ["eye", "rnd"])
def test_oracle_gcn_and_gin_ops_match_the_reference(ref, tag):
    ptr, src, sdeg, ddeg = ref["blk_indptr"], ref["blk_src"], ref["blk_src_deg"], ref["blk_dst_deg"]
    x, w, dy = ref[f"{tag}_x"], ref[f"{tag}_w"], ref[f"{tag}_dy"]
    n_dst, n_src = len(ptr) - 1, x.shape[0]
    tol = AGG_RTOL if tag == "eye" else MM_RTOL
    assert rel_err(onp.forward_gcn(ptr, src, sdeg, ddeg, x, w, n_dst), ref[f"{tag}_gcn_fwd"]) <= tol
    dx, dw = onp.backward_gcn(ptr, src, ddeg, sdeg, dy, w, x)
    assert rel_err(dx, ref[f"{tag}_gcn_bwd_dx"]) <= tol and rel_err(dw, ref[f"{tag}_gcn_bwd_dw"]) <= MM_RTOL
    out, tmp = onp.forward_gin(ptr, src, x, w, n_dst)
    assert rel_err(tmp, ref[f"{tag}_gin_tmp"]) <= AGG_RTOL and rel_err(out, ref[f"{tag}_gin_fwd"]) <= tol
    dx, dw = onp.backward_gin(ptr, src, dy, w, ref[f"{tag}_gin_tmp"], n_src)
    assert rel_err(dx, ref[f"{tag}_gin_bwd_dx"]) <= tol and rel_err(dw, ref[f"{tag}_gin_bwd_dw"]) <= MM_RTOL
    # the C restatement of the aggregation itself (what the GPU parity tests compare with), identity weight: no GEMM
    if tag == "eye":
        assert rel_err(oc.aggregate_fwd(oc.MODE_SYMNORM, ptr, src, x, n_dst, sdeg, ddeg), ref["eye_gcn_fwd"]) <= AGG_RTOL
        assert rel_err(oc.aggregate_fwd(oc.MODE_SUM, ptr, src, x, n_dst), ref["eye_gin_tmp"]) <= AGG_RTOL
        assert rel_err(oc.aggregate_bwd(oc.MODE_SYMNORM, ptr, src, dy, n_src, sdeg, ddeg), ref["eye_gcn_bwd_dx"]) <= AGG_RTOL
        assert rel_err(oc.aggregate_bwd(oc.MODE_SUM, ptr, src, dy, n_src), ref["eye_gin_bwd_dx"]) <= AGG_RTOL


# ----------------------------------------------------------------------------------------------------------------
# this repository's CUDA kernels against the reference's outputs, through the drop-in ops
# ----------------------------------------------------------------------------------------------------------------
def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.gpu
def test_cuda_sampling_and_id_map_against_the_reference(ref):
    import fastgl
    indptr, indices = _dev(ref["graph_indptr"]), _dev(ref["graph_indices"])
    unused = torch.zeros(1, dtype=torch.int32, device="cuda")
    seeds, fanout = ref["full_seeds"], int(ref["full_fanout"])
    src, dst, n_e = fastgl.sample_node(indices, unused, indptr, _dev(seeds), len(seeds), fanout)
    assert int(n_e[0]) == int(ref["full_edges_num"][0])
    assert np.array_equal(src.cpu().numpy(), ref["full_src"]) and np.array_equal(dst.cpu().numpy(), ref["full_dst"])
    E = int(n_e[0])
    for arrival in (False, True):
        fastgl.set_sampling(arrival_order=arrival)
        try:
            s_l, d_l, uniq = fastgl.transfer_edge_id(_dev(ref["map_src_global"]), _dev(ref["map_dst_global"]), _dev(seeds), len(seeds),
                                                     len(seeds) + E, min(len(ref["graph_indptr"]) - 1, fanout * len(seeds)), E)
        finally:
            fastgl.set_sampling(arrival_order=False)
        check_map_against_reference(seeds, ref["map_src_global"], uniq.cpu().numpy(), s_l.cpu().numpy(), d_l.cpu().numpy(),
                                    ref["map_src_local"], ref["map_dst_local"], ref["map_unique"])
    # hubs, in the reference's own mode (with replacement): same rows, picks from the neighbourhood
    seeds2, fanout2 = ref["hub_seeds"], int(ref["hub_fanout"])
    fastgl.set_sampling(replace=True)
    try:
        src2, dst2, n2 = fastgl.sample_node(indices, unused, indptr, _dev(seeds2), len(seeds2), fanout2)
    finally:
        fastgl.set_sampling(replace=False)
    assert int(n2[0]) == int(ref["hub_edges_num"][0]) and np.array_equal(dst2.cpu().numpy(), ref["hub_dst"])
    E2 = int(n2[0])
    s_l, d_l, uniq = fastgl.transfer_edge_id(_dev(ref["hub_src"]), _dev(ref["hub_dst"]), _dev(seeds2), len(seeds2), len(seeds2) + E2,
                                             min(len(ref["graph_indptr"]) - 1, fanout2 * len(seeds2)), E2)
    check_map_against_reference(seeds2, ref["hub_src"], uniq.cpu().numpy(), s_l.cpu().numpy(), d_l.cpu().numpy(),
                                ref["hub_map_src_local"], ref["hub_map_dst_local"], ref["hub_map_unique"])
    fastgl.check_status()


@pytest.mark.gpu
def test_cuda_csr_helpers_against_the_reference(ref):
    import fastgl
    deg = fastgl.cal_deg(_dev(ref["deg_ids"]), 500)
    assert np.array_equal(deg.cpu().numpy(), ref["deg_out"])
    assert np.array_equal(fastgl.exclusive_sum(deg).cpu().numpy(), ref["scan_out"])


@pytest.mark.gpu
@pytest.mark.parametrize("tag", ["eye", "rnd"])
def test_cuda_gcn_and_gin_ops_against_the_reference(ref, tag):
    import fastgl
    ptr, src, sdeg, ddeg = (_dev(ref[k]) for k in ("blk_indptr", "blk_src", "blk_src_deg", "blk_dst_deg"))
    x, w, dy = _dev(ref[f"{tag}_x"]), _dev(ref[f"{tag}_w"]), _dev(ref[f"{tag}_dy"])
    n_dst, n_src, nn = len(ref["blk_indptr"]) - 1, x.size(0), int(ref["blk_neighbor_num"])
    tol = AGG_RTOL if tag == "eye" else MM_RTOL
    assert rel_err(fastgl.forward_gcn(ptr, src, sdeg, ddeg, x, w, nn, n_dst)[0].cpu().numpy(), ref[f"{tag}_gcn_fwd"]) <= tol
    dx, dw = fastgl.backward_gcn(ptr, src, ddeg, sdeg, dy, w, x)                            # GraphConv.py:37 argument order
    assert rel_err(dx.cpu().numpy(), ref[f"{tag}_gcn_bwd_dx"]) <= tol and rel_err(dw.cpu().numpy(), ref[f"{tag}_gcn_bwd_dw"]) <= MM_RTOL
    out, tmp = fastgl.forwaed_gin(ptr, src, x, w, nn, n_dst)
    assert rel_err(tmp.cpu().numpy(), ref[f"{tag}_gin_tmp"]) <= AGG_RTOL and rel_err(out.cpu().numpy(), ref[f"{tag}_gin_fwd"]) <= tol
    dx, dw = fastgl.backward_gin(ptr, src, dy, w, tmp, n_src)
    assert rel_err(dx.cpu().numpy(), ref[f"{tag}_gin_bwd_dx"]) <= tol and rel_err(dw.cpu().numpy(), ref[f"{tag}_gin_bwd_dw"]) <= MM_RTOL
    fastgl.check_status()

#!/usr/bin/env python
"""Writes fixtures made by the reference's own CUDA operators (built by ``oracle/build_ref.py`` into
``oracle/_ref/fastgl_ref.so``) on small seeded inputs, and optionally times those operators beside this repository's.

Runs on a machine with a GPU:

    python tests/golden/make_ref_golden.py --out tests/golden/ref_hotpath.npz [--timing ref_timing.json]

The resulting ``ref_hotpath.npz`` is committed under ``tests/golden/``; ``tests/test_ref_golden.py`` checks the CPU
oracle and the CUDA kernels against it.

Every input stays inside what the reference's kernels can take without reading or writing out of bounds (checked by
reading them): ids are non-negative and in range, seeds are distinct, the in-degree of a block never exceeds the
``neighbor_num`` that sizes the kernels' shared memory (aggregate_acc_kernel.cu:315), every key looked up in the
hashtable was inserted (id_map.cu:242-255), ``unique_num >= 2`` (``TableSize``, cuda_hashtable.cuh:27-30), at least one
new node per id-map call (id_map.cu:451 launches ``ceil(n_new / 128)`` blocks) and at least one seed per sampling call
(sample.cu:163).  The seed lists have 100 and 90 entries: the reference's degree kernel reads ``seed_nodes[n_seeds]``
(sample.cu:24-29), and 400 / 360 bytes leave that word inside the 512-byte block torch's allocator hands out.

What the fixtures pin:

* ``sample_node`` in full-neighbour mode (fanout >= every degree): outputs are deterministic -- exact;
* ``sample_node`` with hubs (degree > fanout): the reference picks with replacement from cuRAND seeded by the thread
  id, and threads 64..127 of each block race with threads 0..63 (sample.cu:52,82-95), so only the edge count, the row
  lengths and membership of the picks are properties of the reference;
* ``transfer_edge_id``: seeds first, destination-local ids and the set of new nodes are deterministic; the order of the
  new nodes is the reference's atomic arrival order (id_map.cu:317-320) and differs from run to run;
* ``cal_deg`` / ``exclusive_sum``: exact;
* ``forward_gcn`` / ``backward_gcn`` / ``forwaed_gin`` / ``backward_gin``: fp32 results (the backward scatters add in
  arbitrary order, so they are reproducible to rounding only), with an identity weight (the dense product is then
  exact) and with a random weight.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "fastgl-ae_b200"))


def small_graph(n_nodes=3000, avg_degree=10, hub=300, seed=4242):
    """Seeded power-law multigraph as a by-destination CSR with int32 offsets (the reference's index type)."""
    rng = np.random.default_rng(seed)
    m = n_nodes * avg_degree // 2
    w = 1.0 / np.arange(1, n_nodes + 1) ** 0.8
    w /= w.sum()
    src = rng.choice(n_nodes, size=m, p=w)
    dst = rng.integers(0, n_nodes, size=m)
    keep = src != dst
    src, dst = src[keep], dst[keep]
    others = rng.choice(np.arange(1, n_nodes), size=hub, replace=False)
    src = np.concatenate([src, others])
    dst = np.concatenate([dst, np.zeros_like(others)])
    s2, d2 = np.concatenate([src, dst]), np.concatenate([dst, src])
    order = np.argsort(d2, kind="stable")
    indices = s2[order].astype(np.int32)
    indptr = np.zeros(n_nodes + 1, dtype=np.int32)
    indptr[1:] = np.cumsum(np.bincount(d2, minlength=n_nodes))
    return indptr, indices


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def make_fixtures(ref) -> dict:
    out = {}
    indptr, indices = small_graph()
    n = len(indptr) - 1
    deg = np.diff(indptr)
    rng = np.random.default_rng(777)
    out["graph_indptr"], out["graph_indices"] = indptr, indices
    dst_edges_unused = torch.zeros(len(indices), dtype=torch.int32, device="cuda")

    # --- a1, full-neighbour mode: seeds whose degree is at most the fanout -----------------------------------
    fanout = 40
    pool = np.flatnonzero((deg <= fanout) & (deg > 0))
    seeds = rng.choice(pool, size=100, replace=False).astype(np.int32)
    seeds[7] = np.flatnonzero(deg == 0)[0] if (deg == 0).any() else seeds[7]      # one isolated seed if there is one
    assert len(set(seeds.tolist())) == 100
    r = ref.sample_node(dev(indices), dst_edges_unused, dev(indptr), dev(seeds), 100, fanout)
    torch.cuda.synchronize()
    out["full_seeds"], out["full_fanout"] = seeds, np.int32(fanout)
    out["full_src"], out["full_dst"], out["full_edges_num"] = (t.cpu().numpy() for t in r)

    # --- a2 on those edges ------------------------------------------------------------------------------------
    E = int(out["full_edges_num"][0])
    src_g, dst_g = out["full_src"].copy(), out["full_dst"].copy()
    unique_num = min(n, fanout * 100)
    m = ref.transfer_edge_id(dev(src_g), dev(dst_g), dev(seeds), 100, 100 + E, unique_num, E)
    torch.cuda.synchronize()
    out["map_src_global"], out["map_dst_global"] = src_g, dst_g
    out["map_src_local"], out["map_dst_local"], out["map_unique"] = (t.cpu().numpy() for t in m)

    # --- a1 with hubs: seeds include the hub (degree > fanout); with-replacement picks, racy -> properties only --
    fanout2 = 5
    seeds2 = np.concatenate([[0], rng.choice(np.arange(1, n), size=89, replace=False)]).astype(np.int32)
    r2 = ref.sample_node(dev(indices), dst_edges_unused, dev(indptr), dev(seeds2), 90, fanout2)
    torch.cuda.synchronize()
    out["hub_seeds"], out["hub_fanout"] = seeds2, np.int32(fanout2)
    out["hub_src"], out["hub_dst"], out["hub_edges_num"] = (t.cpu().numpy() for t in r2)
    E2 = int(out["hub_edges_num"][0])
    m2 = ref.transfer_edge_id(dev(out["hub_src"].copy()), dev(out["hub_dst"].copy()), dev(seeds2), 90, 90 + E2,
                              min(n, fanout2 * 90), E2)
    torch.cuda.synchronize()
    out["hub_map_src_local"], out["hub_map_dst_local"], out["hub_map_unique"] = (t.cpu().numpy() for t in m2)

    # --- a3 -----------------------------------------------------------------------------------------------------
    ids = rng.integers(0, 500, size=20_000).astype(np.int32)
    cd = ref.cal_deg(dev(ids), 500)
    es = ref.exclusive_sum(cd)
    torch.cuda.synchronize()
    out["deg_ids"], out["deg_out"], out["scan_out"] = ids, cd.cpu().numpy(), es.cpu().numpy()

    # --- a4-a7: one block, in-degree <= neighbor_num, some destination rows without edges --------------------------
    n_dst, n_src, neighbor_num = 200, 600, 10
    row_deg = rng.integers(1, neighbor_num + 1, size=n_dst)
    row_deg[rng.random(n_dst) < 0.1] = 0
    blk_ptr = np.zeros(n_dst + 1, dtype=np.int32)
    blk_ptr[1:] = np.cumsum(row_deg)
    blk_src = rng.integers(0, n_src, size=int(blk_ptr[-1])).astype(np.int32)
    src_deg = np.maximum(np.bincount(blk_src, minlength=n_src), 1).astype(np.int32)    # GraphConv.py:96-97
    dst_deg = np.maximum(row_deg, 1).astype(np.int32)
    out["blk_indptr"], out["blk_src"], out["blk_src_deg"], out["blk_dst_deg"] = blk_ptr, blk_src, src_deg, dst_deg
    out["blk_neighbor_num"] = np.int32(neighbor_num)
    for tag, d_in, d_out, identity in (("eye", 48, 48, True), ("rnd", 48, 32, False)):
        x = rng.standard_normal((n_src, d_in)).astype(np.float32)
        w = np.eye(d_in, dtype=np.float32) if identity else (rng.standard_normal((d_in, d_out)) * 0.2).astype(np.float32)
        dy = rng.standard_normal((n_dst, d_out)).astype(np.float32)
        out[f"{tag}_x"], out[f"{tag}_w"], out[f"{tag}_dy"] = x, w, dy
        fg = ref.forward_gcn(dev(blk_ptr), dev(blk_src), dev(src_deg), dev(dst_deg), dev(x), dev(w), neighbor_num, n_dst)
        # GraphConv.py:37 passes (dst degrees, src degrees) in this order
        bg = ref.backward_gcn(dev(blk_ptr), dev(blk_src), dev(dst_deg), dev(src_deg), dev(dy), dev(w), dev(x))
        fi = ref.forwaed_gin(dev(blk_ptr), dev(blk_src), dev(x), dev(w), neighbor_num, n_dst)
        bi = ref.backward_gin(dev(blk_ptr), dev(blk_src), dev(dy), dev(w), fi[1], n_src)
        torch.cuda.synchronize()
        out[f"{tag}_gcn_fwd"] = fg[0].cpu().numpy()
        out[f"{tag}_gcn_bwd_dx"], out[f"{tag}_gcn_bwd_dw"] = bg[0].cpu().numpy(), bg[1].cpu().numpy()
        out[f"{tag}_gin_fwd"], out[f"{tag}_gin_tmp"] = fi[0].cpu().numpy(), fi[1].cpu().numpy()
        out[f"{tag}_gin_bwd_dx"], out[f"{tag}_gin_bwd_dw"] = bi[0].cpu().numpy(), bi[1].cpu().numpy()
    return out


def timed(fn, reps=7):
    fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        fn()
        torch.cuda.synchronize()
        ts.append((time.perf_counter() - t0) * 1e3)
    return float(np.median(ts))


def timing(ref) -> dict:
    """One mini-batch of the single-GPU benchmark shape (1024 seeds, fanouts 5 / 10 / 15 in sampling order, 100-d rows)
    through the reference's per-hop ops and through this repository's, on the same seeded R-MAT graph (int32 offsets,
    which is all the reference takes).  Host-synchronous milliseconds, median of 7: the reference's ops synchronise
    inside (``.item()``), so wall time is the only clock both sides share."""
    import fastgl
    from fastgl_b200.graphgen import rmat_graph, synthetic_node_data
    d = torch.device("cuda", 0)
    indptr64, indices = rmat_graph(2_450_000, 50.6, seed=12345, device=d)
    indptr = indptr64.to(torch.int32)
    n = indptr.numel() - 1
    feat, _, train = synthetic_node_data(n, 100, 47, 0.08, seed=12345, device=d)
    def padded(t):
        """The same ids at the front of a longer buffer: the reference's degree kernel reads one entry past its seed
        list (sample.cu:24-29: thread ``sample_nodes`` loads ``seed_nodes[sample_nodes]`` before it checks its index),
        which must stay inside the allocation."""
        buf = torch.zeros(t.numel() + 32, dtype=torch.int32, device=t.device)
        buf[: t.numel()] = t
        return buf[: t.numel()]

    seeds = padded(train[:1024])
    dst_unused = torch.zeros(1, dtype=torch.int32, device=d)
    fanouts = [5, 10, 15]
    res = {}

    def ref_sample():
        cur, blocks = seeds, []
        for f in fanouts:
            s, t, e = ref.sample_node(indices, dst_unused, indptr, cur, cur.numel(), f)
            E = int(e[0])
            s, t, u = ref.transfer_edge_id(s.contiguous(), t.contiguous(), cur, cur.numel(), cur.numel() + E,
                                           min(n, f * cur.numel()), E)
            blocks.append((s, t, cur.numel(), u.numel()))
            cur = padded(u)
        return cur, blocks

    def ours_sample_per_op():
        cur = seeds
        for f in fanouts:
            s, t, ptr, E = fastgl.sample_node_csr(indices, indptr, cur, f, replace=True)
            s, t, u = fastgl.transfer_edge_id(s, t, cur, cur.numel(), cur.numel() + E, min(n, f * cur.numel()), E)
            cur = u
        return cur

    counts = torch.full((1,), 1024, dtype=torch.int32, device=d)

    def ours_sample_fused():
        fb = fastgl.sample_map_fused(indptr, indices, seeds.view(1, -1), counts, fanouts, replace=False, rng_ctr=1 << 30)
        fb.counts_host()
        return fb

    res["ref_sample_map_ms"] = timed(ref_sample)
    res["ours_sample_map_per_op_ms"] = timed(ours_sample_per_op)
    res["ours_sample_map_fused_ms"] = timed(ours_sample_fused)
    cur, blocks = ref_sample()
    src_l, dst_l, n_dst, n_src = blocks[-1]
    res["edges_last_hop"], res["n_dst_last_hop"], res["n_src_last_hop"] = int(src_l.numel()), n_dst, n_src
    deg = fastgl.cal_deg(dst_l.contiguous(), n_dst)
    ptr = fastgl.exclusive_sum(deg)
    x = feat[cur.long()].contiguous()
    w = torch.eye(100, device=d)
    res["ref_gin_fwd_ms"] = timed(lambda: ref.forwaed_gin(ptr, src_l, x, w, 15, n_dst))
    res["ours_gin_fwd_ms"] = timed(lambda: fastgl.forwaed_gin(ptr, src_l, x, w, 15, n_dst))
    dy = torch.randn((n_dst, 100), device=d)
    tmp = fastgl.forwaed_gin(ptr, src_l, x, w, 15, n_dst)[1]
    res["ref_gin_bwd_ms"] = timed(lambda: ref.backward_gin(ptr, src_l, dy, w, tmp, n_src))
    res["ours_gin_bwd_ms"] = timed(lambda: fastgl.backward_gin(ptr, src_l, dy, w, tmp, n_src))
    sdeg = fastgl.cal_deg(src_l.contiguous(), n_src).clamp(min=1)
    ddeg = deg.clamp(min=1)
    res["ref_gcn_fwd_ms"] = timed(lambda: ref.forward_gcn(ptr, src_l, sdeg, ddeg, x, w, 15, n_dst))
    res["ours_gcn_fwd_ms"] = timed(lambda: fastgl.forward_gcn(ptr, src_l, sdeg, ddeg, x, w, 15, n_dst))
    res["ref_gcn_bwd_ms"] = timed(lambda: ref.backward_gcn(ptr, src_l, ddeg, sdeg, dy, w, x))
    res["ours_gcn_bwd_ms"] = timed(lambda: fastgl.backward_gcn(ptr, src_l, ddeg, sdeg, dy, w, x))
    res["note"] = ("host-synchronous wall time of one mini-batch (1024 seeds, fanouts 5/10/15) per call chain; weight = identity "
                   "100x100 so the dense product is the same cuBLAS call on both sides")
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--timing", default=None)
    a = ap.parse_args()
    from oracle import build_ref
    ref = build_ref.load()
    if ref is None:
        raise SystemExit("oracle/_ref/fastgl_ref.so is missing: run oracle/build_ref.py where the reference sources are")
    fixtures = make_fixtures(ref)
    os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
    np.savez_compressed(a.out, **fixtures)
    print(f"wrote {a.out}: {len(fixtures)} arrays")
    if a.timing:
        t = timing(ref)
        with open(a.timing, "w") as f:
            json.dump(t, f, indent=1)
        print(json.dumps(t))


if __name__ == "__main__":
    main()

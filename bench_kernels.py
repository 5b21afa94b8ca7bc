"""Per-kernel timing of the hot path on blocks of the sizes a mini-batch really has (``bench.py --kernels``).

Every entry times one C-ABI entry point alone, with CUDA events on the launching stream, after warm-up, with a
buffer larger than L2 rewritten between timed launches, and divides its *algorithmic* bytes by the median
duration:

* sampling, id map, fused sample + map:  ``S*40 + sum_seeds min(32*ceil(4*deg/32), 32*k) + 4*E + 4*U`` per hop
  (a random 4-byte pick costs a 32-byte sector; hash-table traffic is not credited);
* aggregation forward:  ``4*D*(R_src + n_dst) + 4*E + 4*(n_dst + 1)`` with ``R_src`` the number of *distinct*
  source rows (re-reads served by L2 are not credited), plus ``4*R_src`` when a row map is read;
* aggregation backward: ``4*D*(n_dst + n_src) + 4*E + 4*(n_dst + 1)``;
* row gather: ``(8*D + 4) * n``.

The inputs are one sampled window of the chosen workload, so block shapes, degree skew and row re-use are those
of training.
"""
from __future__ import annotations

import statistics

import torch

import fastgl


def _fwd_kernel_name(dim: int) -> str:
    """The forward kernel fgl_agg_fwd picks for contiguous rows of ``dim`` floats in one dense table."""
    return "agg_fwd_staged_kernel" if dim % 4 == 0 and dim <= 128 else "agg_fwd_kernel"


def _timed(fn, reps: int, flush: torch.Tensor) -> float:
    """Median milliseconds of ``fn(i)`` over ``reps`` launches, L2 flushed before each."""
    for i in range(2):
        fn(i)
    times = []
    for i in range(reps):
        flush.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn(i)
        end.record()
        end.synchronize()
        times.append(start.elapsed_time(end))
    return statistics.median(times)


def _sampler_bytes(deg_all, nodes, n_seeds, n_edges, n_new, fanout) -> int:
    d = deg_all[nodes[:n_seeds].long()]
    k = torch.clamp(d, max=fanout)
    sectors = int(torch.minimum(32 * ((4 * d + 31) // 32), 32 * k).sum())
    return n_seeds * 40 + sectors + 4 * n_edges + 4 * n_new


def run(indptr, indices, feat, train, fanouts, batch: int, window: int, peak_gbs: float, reps: int = 9,
        dims=(100, 128, 256, 602, 1024)) -> list[dict]:
    """Time the kernels on one window of ``window`` mini-batches of ``batch`` training seeds."""
    dev = indices.device
    n_nodes = indptr.numel() - 1
    L = len(fanouts)
    fan_s = list(reversed(fanouts))
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)        # twice the 126 MB L2
    deg_all = (indptr[1:] - indptr[:-1]).long()
    gen = torch.Generator(device="cpu")
    gen.manual_seed(1)
    out: list[dict] = []

    def entry(name, shape, nbytes, ms, note=None):
        gbs = nbytes / (ms * 1e-3) / 1e9
        e = {"kernel": name, "shape": shape, "algorithmic_bytes": int(nbytes), "ms": ms, "gb_per_s": gbs,
             "frac_of_measured_hbm_peak": gbs / peak_gbs}
        if note:
            e["note"] = note
        out.append(e)

    def window_seeds(i):
        g = torch.Generator(device="cpu")
        g.manual_seed(100 + i)
        perm = torch.randperm(train.numel(), generator=g)[: window * batch].to(dev)
        return train[perm].to(torch.int32).view(window, batch).contiguous()

    counts = torch.full((window,), batch, dtype=torch.int32, device=dev)
    seeds_list = [window_seeds(i) for i in range(reps)]
    state = {"fb": None}

    # ---- fused sample + map over a window (all hops, all batches, one launch) --------------------------------
    def fused(i):
        state["fb"] = fastgl.sample_map_fused(indptr, indices, seeds_list[i % reps], counts, fan_s, replace=False,
                                              rng_seed=12345, rng_ctr=1000 * i, out=state["fb"])
    ms = _timed(fused, reps, flush)
    fastgl.check_status(dev)
    fb = state["fb"]
    c = fb.counts_list()
    nbytes = 0
    for b in range(window):
        for h in range(L):
            nbytes += _sampler_bytes(deg_all, fb.nodes[b], c[b][h], c[b][8 + h], c[b][h + 1] - c[b][h], fan_s[h])
    edges = sum(sum(c[b][8: 8 + L]) for b in range(window))
    entry("sample_map_kernel (fgl_sample_map_fused)", f"window {window} x {batch} seeds, fanouts {fan_s}, {edges} edges",
          nbytes, ms, note=f"{edges / (ms * 1e-3) / 1e6:.0f} M sampled edges/s")

    # what the trainer does from its second window on: tables capped at 2.5 slots per node of the largest mini-batch
    # (L2-resident), every mini-batch of the window in flight
    import math
    most = max(c[b][L] for b in range(window))
    cap_slots = 1 << max(12, math.ceil(math.log2(2.5 * most)))
    capped = {"fb": None}

    def fused_capped(i):
        capped["fb"] = fastgl.sample_map_fused(indptr, indices, seeds_list[i % reps], counts, fan_s, replace=False,
                                               rng_seed=12345, rng_ctr=1000 * i, n_teams=min(window, 16),
                                               table_slots=cap_slots, out=capped["fb"])
    ms_cap = _timed(fused_capped, reps, flush)
    fastgl.check_status(dev)
    entry("sample_map_kernel, tables sized from the data (fgl_sample_map_fused)",
          f"window {window} x {batch} seeds, {min(window, 16)} teams, {cap_slots} slots per table", nbytes, ms_cap,
          note=f"{edges / (ms_cap * 1e-3) / 1e6:.0f} M sampled edges/s; the default above uses 4 teams and worst-case tables")
    del capped

    # what the memory system sustains for the sampler's access pattern alone: isolated 4-byte reads in this graph's
    # adjacency array, then the same followed by a probe of as many table bytes as the launch above holds
    n_tables = min(window, 16)
    probe_table = torch.zeros(1 << max(12, math.ceil(math.log2(n_tables * cap_slots))), dtype=torch.int64, device=dev)
    acc = {}

    def probe_reads(i):
        acc["n"] = fastgl.probe_access_pattern(indices, None, iters=64)
    ms_p = _timed(probe_reads, reps, flush)
    entry("access probe: isolated 4-byte reads (fgl_probe_access_pattern)", f"{indices.numel() * 4 / 1e6:.0f} MB adjacency array, "
          f"{acc['n']} reads", 32 * acc["n"], ms_p,
          note=f"{acc['n'] / (ms_p * 1e-3) / 1e9:.1f} G reads/s; bytes = 32 per read, the sector the sampler's formula charges per pick")

    def probe_pairs(i):
        probe_table.zero_()
        acc["n"] = fastgl.probe_access_pattern(indices, probe_table, iters=64)
    t_zero = _timed(lambda i: probe_table.zero_(), reps, flush)
    ms_pp = max(_timed(probe_pairs, reps, flush) - t_zero, 1e-6)
    entry("access probe: read + dependent table probe (fgl_probe_access_pattern)", f"{indices.numel() * 4 / 1e6:.0f} MB adjacency array, "
          f"{probe_table.numel() * 8 / 1e6:.0f} MB of table, {acc['n']} pairs", 40 * acc["n"], ms_pp,
          note=f"{acc['n'] / (ms_pp * 1e-3) / 1e9:.1f} G pairs/s against the sampler's {edges / (ms_cap * 1e-3) / 1e9:.1f} G edges/s; "
               "bytes = 32 + 8 per pair; the time of zero-filling the table is subtracted")
    del probe_table

    # the reference's own numbering (atomic arrival order) skips the two ranking phases
    arr = {"fb": None}

    def fused_arrival(i):
        arr["fb"] = fastgl.sample_map_fused(indptr, indices, seeds_list[i % reps], counts, fan_s, replace=False,
                                            arrival_order=True, rng_seed=12345, rng_ctr=1000 * i, out=arr["fb"])
    ms_arr = _timed(fused_arrival, reps, flush)
    entry("sample_map_kernel, arrival-order ids (fgl_sample_map_fused)", f"window {window} x {batch} seeds, fanouts {fan_s}",
          nbytes, ms_arr, note="node numbering as nondeterministic as the reference's; not the default")
    del arr

    # ---- the op-by-op pair on the widest hop of one batch: fgl_sample, then fgl_map ---------------------------
    hop = L - 1
    b0 = 0
    n_dst0, n_src0, n_e0 = c[b0][hop], c[b0][hop + 1], c[b0][8 + hop]
    hop_seeds = fb.nodes[b0, :n_dst0].contiguous()
    res = {}

    def sample(i):
        res["s"] = fastgl.sample_node_csr(indices, indptr, hop_seeds, fan_s[hop], replace=False, rng_seed=12345, rng_ctr=i)
    ms = _timed(sample, reps, flush)
    entry("sample kernels (fgl_sample)", f"{n_dst0} seeds, fanout {fan_s[hop]}, {n_e0} edges",
          _sampler_bytes(deg_all, fb.nodes[b0], n_dst0, n_e0, 0, fan_s[hop]), ms,
          note="includes the read-back of the edge count the reference's signature needs")
    src_global = fb.nodes[b0].long()[fb.block_src[hop][b0, :n_e0].long()].to(torch.int32)
    ptr0 = fb.block_indptr[hop][b0, : n_dst0 + 1].long()
    dst_global = torch.repeat_interleave(hop_seeds, (ptr0[1:] - ptr0[:-1]))

    def id_map(i):
        s, d = src_global.clone(), dst_global.clone()
        res["m"] = fastgl.transfer_edge_id(s, d, hop_seeds, n_dst0, n_dst0 + n_e0, min(n_nodes, n_dst0 * (fan_s[hop] + 1)), n_e0)

    def clones(i):
        res["c"] = (src_global.clone(), dst_global.clone())
    ms_map = _timed(id_map, reps, flush) - _timed(clones, reps, flush)
    entry("map_kernel (fgl_map)", f"{n_dst0} seeds + {n_e0} edges -> {n_src0} nodes",
          4 * n_dst0 + 8 * n_e0 + 8 * n_e0 + 4 * n_src0, max(ms_map, 1e-3),
          note="reads both edge arrays, rewrites them in place, writes the node list; includes the count read-back")

    # ---- CSR helpers -------------------------------------------------------------------------------------------
    ids = fb.block_src[hop][b0, :n_e0].contiguous()
    ms = _timed(lambda i: fastgl.cal_deg(ids, n_src0), reps, flush)
    entry("cal_deg_kernel (fgl_cal_deg)", f"{n_e0} ids into {n_src0} bins", 4 * n_e0 + 4 * n_src0, ms, note="launch-bound size")
    degs = (ptr0[1:] - ptr0[:-1]).to(torch.int32)
    ms = _timed(lambda i: fastgl.exclusive_sum(degs), reps, flush)
    entry("exclusive_sum_kernel (fgl_exclusive_sum)", f"{n_dst0} values", 8 * n_dst0 + 4, ms, note="launch-bound size")

    # ---- aggregation forward: first layer straight from the feature table ------------------------------------
    D = feat.size(1)
    n_dst = [c[b][hop] for b in range(window)]
    n_edges = [c[b][8 + hop] for b in range(window)]
    alg = []
    for b in range(window):
        touched = torch.cat([fb.block_src[hop][b, : n_edges[b]], torch.arange(n_dst[b], dtype=torch.int32, device=dev)])
        r_all = int(torch.unique(touched).numel())
        alg.append(4 * D * r_all + 4 * r_all + 4 * n_edges[b] + 4 * (n_dst[b] + 1) + 2 * 4 * D * n_dst[b])
    total = sum(n_dst)
    buf = torch.empty((total, 2 * D), dtype=torch.float32, device=dev)
    ms = _timed(lambda i: fastgl.aggregate_window(fastgl.AGG_MEAN, fb, hop, feat, buf[:, D:], self_out=buf[:, :D]), reps, flush)
    entry(f"{_fwd_kernel_name(D)}, window mode (fgl_agg_fwd_window)", f"{window} blocks, {total} rows, {sum(n_edges)} edges, D={D}, "
          "row map + self rows", sum(alg), ms)
    outs = torch.empty((n_dst[0], D), dtype=torch.float32, device=dev)
    r_src = int(torch.unique(fb.block_src[hop][b0, :n_e0]).numel())
    ms = _timed(lambda i: fastgl.aggregate(fastgl.AGG_MEAN, fb.block_indptr[hop][b0], fb.block_src[hop][b0], feat, n_dst0,
                                           zero_deg_passthrough=False, row_map=fb.nodes[b0], out=outs), reps, flush)
    entry(f"{_fwd_kernel_name(D)}, one block (fgl_agg_fwd)", f"{n_dst0} rows, {n_e0} edges, D={D}, row map",
          4 * D * (r_src + n_dst0) + 4 * r_src + 4 * n_e0 + 4 * (n_dst0 + 1), ms)
    del buf, outs

    # ---- aggregation forward / backward on block-local rows of other widths (inner layers, other models) ------
    ptr_b = fb.block_indptr[hop][b0, : n_dst0 + 1].contiguous()
    src_b = fb.block_src[hop][b0, :n_e0].contiguous()
    src_deg = fastgl.cal_deg(src_b, n_src0).clamp(min=1)
    dst_deg = (ptr_b[1:] - ptr_b[:-1]).clamp(min=1).to(torch.int32)
    for dim in dims:
        x = torch.randn((n_src0, dim), device=dev)
        y = torch.empty((n_dst0, dim), device=dev)
        for mode, label in ((fastgl.AGG_MEAN, "mean"), (fastgl.AGG_SYMNORM, "sym-norm")):
            kw = dict(src_norm_degs=src_deg, dst_norm_degs=dst_deg) if mode == fastgl.AGG_SYMNORM else {}
            ms = _timed(lambda i: fastgl.aggregate(mode, ptr_b, src_b, x, n_dst0, out=y, **kw), reps, flush)
            extra = 4 * (n_src0 + n_dst0) if mode == fastgl.AGG_SYMNORM else 0
            entry(f"{_fwd_kernel_name(dim)} {label} (fgl_agg_fwd)", f"{n_dst0} rows, {n_e0} edges, {r_src} distinct sources, D={dim}",
                  4 * dim * (r_src + n_dst0) + 4 * n_e0 + 4 * (n_dst0 + 1) + extra, ms)
        dy = torch.randn((n_dst0, dim), device=dev)
        ms = _timed(lambda i: res.__setitem__("dx", fastgl.aggregate_backward(fastgl.AGG_MEAN, ptr_b, src_b, dy, n_src0)), reps, flush)
        entry("agg_bwd_kernel mean (fgl_agg_bwd)", f"{n_dst0} gradient rows scattered over {n_e0} edges into {n_src0} rows, D={dim}",
              4 * dim * (n_dst0 + n_src0) + 4 * n_e0 + 4 * (n_dst0 + 1), ms, note="includes zero-filling the result")
        tb = fastgl.transpose_block(ptr_b, src_b, n_dst0, n_src0)
        dxg = torch.empty((n_src0, dim), device=dev)
        ms = _timed(lambda i: fastgl.aggregate_backward(fastgl.AGG_MEAN, ptr_b, src_b, dy, n_src0, transposed=tb, out=dxg), reps, flush)
        entry("agg_bwd_gather_kernel mean (fgl_agg_bwd_gather)", f"{n_dst0} gradient rows gathered over {n_e0} edges into {n_src0} rows, "
              f"D={dim}", 4 * dim * (n_dst0 + n_src0) + 8 * n_e0 + 4 * (n_src0 + 1), ms,
              note="deterministic; no zero-fill; the transposition is timed separately")
        if dim == dims[0]:
            ms = _timed(lambda i: fastgl.transpose_block(ptr_b, src_b, n_dst0, n_src0, out=tb), reps, flush)
            entry("block transposition (fgl_block_transpose)", f"{n_e0} edges, {n_src0} sources", 12 * n_e0 + 12 * n_src0, ms,
                  note="histogram, scan, fill, hub list: once per block, whatever the row width")
        del x, y, dy, dxg, tb
        res.pop("dx", None)

    # ---- row gather -----------------------------------------------------------------------------------------
    rows = fb.nodes[b0, :n_src0].contiguous()
    g_out = torch.empty((n_src0, D), dtype=torch.float32, device=dev)
    ms = _timed(lambda i: fastgl.gather_rows(feat, rows, out=g_out), reps, flush)
    entry("gather_rows_kernel (fgl_gather_rows)", f"{n_src0} rows of D={D}", (8 * D + 4) * n_src0, ms)
    fastgl.check_status(dev)
    return out

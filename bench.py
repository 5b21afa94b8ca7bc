#!/usr/bin/env python
"""Benchmark of the FastGL per-mini-batch hot path on B200: sample -> Fused-Map -> 3-layer GraphSAGE-mean
forward / backward / Adam, on a seeded synthetic R-MAT graph with the shape of the single-GPU configuration
(2.45 M nodes, ~124 M directed edges, 100-d fp32 features, 47 classes, 8 % train seeds, fanout [15,10,5],
batch 1024 per GPU).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl fastgl|reference]

One "step" is one data-parallel training step: every rank samples, maps and trains one mini-batch of 1024
seeds (windows of ``--window`` mini-batches are sampled by one kernel launch inside the timed region).
Rank 0 prints one JSON line.  ``--impl reference`` times the CPU restatement of the same step (the reference
itself has no CPU code path and is CUDA-only for sm_80) on the host cores.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "fastgl-ae_b200"))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))   # the size-independent gates (tests/checks.py)

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

CONFIGS = {
    # name: nodes, avg directed degree, feature dim, classes, train fraction, fanouts (input layer first)
    "products-like": dict(n_nodes=2_450_000, avg_degree=50.6, feat_dim=100, n_classes=47, train_frac=0.08,
                          fanouts=[15, 10, 5], hidden=256, batch=1024),
    "small": dict(n_nodes=100_000, avg_degree=20.0, feat_dim=128, n_classes=10, train_frac=0.10,
                  fanouts=[15, 10, 5], hidden=256, batch=1024),
    # large-scale data-parallel run (papers100M-shaped): ~57 GB of features + ~14 GB of graph replicated per GPU
    "papers-like": dict(n_nodes=111_000_000, avg_degree=28.8, feat_dim=128, n_classes=172, train_frac=0.011,
                        fanouts=[15, 10, 5], hidden=256, batch=1024),
    # feature-sharded run (IGB-shaped): 1024-d rows block-partitioned over the ranks' HBM, read with peer loads
    "igb-like": dict(n_nodes=100_000_000, avg_degree=12.0, feat_dim=1024, n_classes=19, train_frac=0.01,
                     fanouts=[15, 10, 5], hidden=256, batch=1024, sharded=True),
    "igb-like-small": dict(n_nodes=8_000_000, avg_degree=12.0, feat_dim=1024, n_classes=19, train_frac=0.01,
                           fanouts=[15, 10, 5], hidden=256, batch=1024, sharded=True),
    # high-degree aggregation stress (Reddit-shaped): dense graph, 602-d rows (2408 B: 8-byte aligned only), GCN
    "reddit-like": dict(n_nodes=233_000, avg_degree=492.0, feat_dim=602, n_classes=41, train_frac=0.66,
                        fanouts=[25, 10], hidden=256, batch=1024, model="gcn", rmat=(0.45, 0.22, 0.22)),
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 50 ms while the timed region runs.  The sampler is started
    before the settle phase and waited for until its first sample is there, so that its start-up (NVML initialisation)
    does not fall into the timed region.  Only samples taken after ``mark()`` are reported."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,clocks.mem")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None
        self.skip = 0

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.gpu_index)],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        self.skip = 0

    def _lines(self):
        try:
            with open(self.path) as f:
                return f.readlines()
        except OSError:
            return []

    def wait_ready(self, timeout: float = 3.0):
        """Block until the first sample has been written (or the time is up)."""
        if self.proc is None:
            return
        t_end = time.time() + timeout
        while time.time() < t_end and not self._lines():
            time.sleep(0.02)

    def mark(self):
        """Samples written so far are not part of the report."""
        if self.proc is not None:
            self.skip = len(self._lines())

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mem, power, reasons = [], [], [], set()
        try:
            for line in self._lines()[self.skip:]:
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9 or not f[1].isdigit():
                    continue
                sm.append(int(f[1]))
                out["sm_max_mhz"] = int(f[2])
                if len(f) > 9 and f[9].isdigit():
                    mem.append(int(f[9]))
                try:
                    power.append(float(f[3]))
                except ValueError:
                    pass
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except OSError:
            pass
        if sm:
            out["sm_mhz"] = statistics.median(sm)
            out["sm_mhz_min"] = min(sm)
        if mem:
            out["mem_mhz_min"], out["mem_mhz_max"] = min(mem), max(mem)
        if power:
            out["power_w_median"], out["power_w_max"] = statistics.median(power), max(power)
        out["reasons"] = sorted(reasons)
        out["samples"] = len(sm)
        return out


def load_ncu_traffic(config: str, window: int):
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the two window-level kernels, from the
    tracked summary of an ncu capture of this workload: (aggregation, sampler, note).  The summary names the kernel
    sources it was captured with; if those have changed since, the figures are withheld."""
    path = os.path.join(ROOT, "profiles", f"dram_traffic_{config}.json")
    if not os.path.exists(path):
        return None, None, None
    with open(path) as f:
        prof = json.load(f)
    entry = prof.get("window", {}).get(str(window))
    if entry is None:
        return None, None, None
    csrc = os.path.join(ROOT, "fastgl-ae_b200", "csrc")
    stale = []
    for name, sha in prof.get("sources_sha16", {}).items():
        with open(os.path.join(csrc, name), "rb") as f:
            if hashlib.sha256(f.read()).hexdigest()[:16] != sha:
                stale.append(name)
    agg = None if "aggregate.cu" in stale else entry.get("agg_fwd_window")
    smp = None if "sample_map.cu" in stale else entry.get("sample_map")
    note = f"profile predates the current {', '.join(stale)}: figure withheld" if stale else None
    return agg, smp, note


def build_inputs(cfg, device, rank=0, world=1):
    from fastgl_b200.graphgen import rmat_graph, synthetic_node_data
    a, b, c = cfg.get("rmat", (0.57, 0.19, 0.19))
    indptr, indices = rmat_graph(cfg["n_nodes"], cfg["avg_degree"], seed=12345, device=device, a=a, b=b, c=c)
    if cfg.get("layout") == "degree":
        # the same graph with its nodes renumbered by descending degree; features, labels and training seeds are drawn
        # afterwards, in the new numbering (they are i.i.d. per node, so the workload is the same in distribution)
        from fastgl_b200.graphgen import relabel_by_degree
        indptr, indices, _, _ = relabel_by_degree(indptr, indices)
    if cfg.get("sharded") and world > 1:
        # every rank fills only its own row block; the blocks are then opened by all ranks over CUDA IPC
        from fastgl_b200.sharding import rows_per_shard, share_feature_shards
        _, labels, train = synthetic_node_data(cfg["n_nodes"], 1, cfg["n_classes"], cfg["train_frac"], seed=12345, device=device)
        rps = rows_per_shard(cfg["n_nodes"], world)
        gen = torch.Generator(device=device)
        gen.manual_seed(12345 + 31 * rank)
        shard = torch.randn((rps, cfg["feat_dim"]), generator=gen, device=device, dtype=torch.float32)
        feat = share_feature_shards(shard, cfg["n_nodes"])
    else:
        feat, labels, train = synthetic_node_data(cfg["n_nodes"], cfg["feat_dim"], cfg["n_classes"], cfg["train_frac"],
                                                  seed=12345, device=device)
    return indptr, indices, feat, labels, train


# ----------------------------------------------------------------------------------------------------------
# CPU restatement of one training step (oracle sampling / mapping / aggregation + torch CPU dense algebra)
# ----------------------------------------------------------------------------------------------------------
def make_cpu_stepper(cfg, indptr, indices, feat, labels, train):
    from oracle import oracle_c as oc
    import torch.nn.functional as F

    oc.set_threads(os.cpu_count() or 1)
    torch.set_num_threads(os.cpu_count() or 1)
    ip, ix = indptr.cpu().numpy(), indices.cpu().numpy()
    feat_c, labels_c, train_c = feat.cpu(), labels.cpu(), train.cpu().numpy()
    feat_np = feat_c.numpy()

    class MeanAgg(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x, blk, row_map):
            ctx.blk = blk
            ctx.n_src = x.shape[0]
            out = oc.aggregate_fwd(oc.MODE_MEAN, blk["indptr"], blk["src_local"], x.detach().numpy(), blk["n_dst"],
                                   zero_deg_passthrough=False, row_map=row_map)
            return torch.from_numpy(out)

        @staticmethod
        def backward(ctx, dy):
            if not ctx.needs_input_grad[0]:
                return None, None, None
            blk = ctx.blk
            dx = oc.aggregate_bwd(oc.MODE_MEAN, blk["indptr"], blk["src_local"], dy.contiguous().numpy(), ctx.n_src)
            return torch.from_numpy(dx), None, None

    torch.manual_seed(0)
    dims = [cfg["feat_dim"]] + [cfg["hidden"]] * (len(cfg["fanouts"]) - 1) + [cfg["n_classes"]]
    params = []
    for i in range(len(dims) - 1):
        params += [torch.nn.Parameter(torch.randn(dims[i], dims[i + 1]) * 0.05),
                   torch.nn.Parameter(torch.randn(dims[i], dims[i + 1]) * 0.05),
                   torch.nn.Parameter(torch.zeros(dims[i + 1]))]
    opt = torch.optim.Adam(params, lr=0.01, weight_decay=5e-4)
    rng = np.random.default_rng(12345)
    state = {"ctr": 0}

    def step():
        seeds = rng.choice(train_c, size=cfg["batch"], replace=False).astype(np.int32)
        inputs, _, blocks = oc.sample_blocks(ip, ix, seeds, cfg["fanouts"], False, rng_seed=12345, rng_ctr=state["ctr"])
        state["ctr"] += 8
        h = None
        for i, blk in enumerate(blocks):
            ws, wn, b = params[3 * i: 3 * i + 3]
            if i == 0:
                neigh = MeanAgg.apply(feat_c, blk, inputs)
                h_self = torch.from_numpy(feat_np[inputs[: blk["n_dst"]]])
            else:
                h = torch.relu(h)
                neigh = MeanAgg.apply(h, blk, None)
                h_self = h[: blk["n_dst"]]
            h = torch.addmm(b, h_self, ws) + neigh @ wn
        loss = F.cross_entropy(h, labels_c[torch.from_numpy(seeds.astype(np.int64))])
        opt.zero_grad()
        loss.backward()
        opt.step()
        return sum(len(blk["src_local"]) for blk in blocks), float(loss.detach())

    return step, oc.max_threads()


def time_cpu_steps(step, n_steps):
    edges = 0
    t0 = time.perf_counter()
    for _ in range(n_steps):
        e, _ = step()
        edges += e
    dt = time.perf_counter() - t0
    return edges, dt


# ----------------------------------------------------------------------------------------------------------
def run_gates(cfg, args, indptr, indices, feat, train, device):
    """Sample one window of the workload and check it (raises on a violated gate)."""
    import fastgl
    from checks import EdgeKeys, check_window, check_window_aggregation
    nb, batch = args.window, cfg["batch"]
    if train.numel() < nb * batch:
        nb = max(1, train.numel() // batch)
    seeds = train[: nb * batch].to(torch.int32).view(nb, batch).contiguous()
    counts = torch.full((nb,), batch, dtype=torch.int32, device=device)
    fan_s = list(reversed(cfg["fanouts"]))
    fb = fastgl.sample_map_fused(indptr, indices, seeds, counts, fan_s, replace=False, rng_seed=12345, rng_ctr=1 << 40)
    fastgl.check_status(device)
    keys = EdgeKeys(indptr, indices)
    seen = check_window(fb, indptr, indices, seeds, [batch] * nb, replace=False, edge_keys=keys)
    del keys
    out = {"window_checked": seen, "status": "ok"}
    if cfg.get("model") != "gcn" and torch.is_tensor(feat):
        hop, D = len(fan_s) - 1, feat.size(1)
        total = int(fb.counts_host()[:, hop].sum())
        buf = torch.empty((total, 2 * D), dtype=torch.float32, device=device)
        row_off = fastgl.aggregate_window(fastgl.AGG_MEAN, fb, hop, feat, buf[:, D:], self_out=buf[:, :D])
        out["window_aggregation_rel_err"] = check_window_aggregation(fb, hop, feat, buf, row_off)
        del buf
    del fb
    torch.cuda.empty_cache()
    return out


def run_sharded_leg(cfg, args, tr, indptr, rank, world, device, barrier, max_over_ranks):
    """The feature-sharded configuration's data path on the graph at hand: 1024-d fp32 rows block-partitioned over
    the ranks' HBM (CUDA IPC, plain 128-bit peer loads over NVLink, no collective), one window's first-layer mean
    aggregation straight through the sharded table.  Gate: the result equals, bit for bit, the same launch on a dense
    local copy of the table (itself assembled with the sharded row gather)."""
    import fastgl
    from fastgl_b200.sharding import rows_per_shard, share_feature_shards
    D = 1024
    n = indptr.numel() - 1
    if n * D * 4 > 24e9:
        return {"status": "skipped", "reason": f"a dense local copy of {n} x {D} floats (the gate) does not fit the leg's budget"}
    out = {"status": "failed"}
    st = full = fb = got = want = None
    failure = None
    try:   # set-up: a rank that cannot allocate or map says so; the ranks then skip the measurement together
        rps = rows_per_shard(n, world)
        gen = torch.Generator(device=device)
        gen.manual_seed(777 + 31 * rank)
        shard = torch.randn((rps, D), generator=gen, device=device, dtype=torch.float32)
    except RuntimeError as e:
        failure = str(e).splitlines()[0][:200]
        shard = torch.zeros((1, D), device=device)
    if max_over_ranks(0.0 if failure is None else 1.0) > 0:
        return {"status": "failed", "reason": failure or "another rank could not allocate its shard"}
    st = share_feature_shards(shard, n)
    try:
        full = fastgl.gather_rows(st, torch.arange(n, dtype=torch.int32, device=device))
        nb, batch = args.window, cfg["batch"]
        seeds = tr.my_seeds[: nb * batch]
        if seeds.numel() < nb * batch:
            seeds = tr.my_seeds.repeat(-(-nb * batch // tr.my_seeds.numel()))[: nb * batch]
        counts = torch.full((nb,), batch, dtype=torch.int32, device=device)
        fb = tr.sampler.sample_window(seeds.view(nb, batch).contiguous(), counts, reuse=False)
        hop = len(cfg["fanouts"]) - 1
        ch = fb.counts_host()
        total = int(ch[:, hop].sum())
        got = torch.empty((total, D), dtype=torch.float32, device=device)
        want = torch.empty((total, D), dtype=torch.float32, device=device)
        fastgl.aggregate_window(fastgl.AGG_MEAN, fb, hop, st, got)
        torch.cuda.synchronize()
    except RuntimeError as e:
        failure = str(e).splitlines()[0][:200]
    if max_over_ranks(0.0 if failure is None else 1.0) > 0:
        out = {"status": "failed", "reason": failure or "another rank failed during set-up"}
    else:
        times = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            e0.record()
            fastgl.aggregate_window(fastgl.AGG_MEAN, fb, hop, st, got)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        fastgl.aggregate_window(fastgl.AGG_MEAN, fb, hop, full, want)
        fastgl.check_status(device)
        equal = bool(torch.equal(got, want))
        remote_edges = edges = 0
        for b in range(nb):
            n_e = int(ch[b, 8 + hop])
            rows = fb.nodes[b].long()[fb.block_src[hop][b, :n_e].long()]
            remote_edges += int(((rows // rps) != rank).sum())
            edges += n_e
        my_ms = statistics.median(times)
        ms = max_over_ranks(my_ms)
        all_equal = max_over_ranks(0.0 if equal else 1.0) == 0.0
        # NVLink ingress of the busiest rank: its own remote bytes over its own launch time
        remote_gbs = max_over_ranks(remote_edges * D * 4 / (my_ms * 1e-3) / 1e9)
        out = {"status": "ok" if all_equal else "mismatch", "table": f"{n} rows x {D} fp32, {world} shards of {rps} rows",
               "window_rows": total, "window_edges": edges, "launch_ms": ms,
               "remote_edge_fraction_max": max_over_ranks(remote_edges / max(1, edges)),
               "remote_gb_per_s_per_gpu": remote_gbs, "nvlink_peak_gb_per_s": 900.0, "frac_of_nvlink": remote_gbs / 900.0,
               "equal_to_local_copy": all_equal,
               "note": "largest over the ranks of (a rank's remote row bytes / its median launch time); rows a window re-reads "
                       "are served by the reading GPU's L2, so the figure can exceed the link rate"}
    got = want = fb = None
    # nobody unmaps a shard while a peer may still read it
    torch.cuda.synchronize()
    barrier()
    st = full = None
    torch.cuda.ipc_collect()
    torch.cuda.empty_cache()
    barrier()
    return out


DENSE_MATMUL = {
    "fp32": "fp32: cuBLAS SIMT float32 kernels",
    "3xtf32": "3xtf32: operands split into two TF32 parts each, one TF32 tensor-core GEMM over [hi|lo|hi].[hi;hi;lo] with float32 "
              "accumulation; relative error 2e-6 (SIMT float32: 5e-7; single-pass TF32, the reference's own setting: 3e-4); "
              "models without the hand-written step (GCN) run float32",
    "tf32": "tf32: single-pass TF32",
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=192)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="fastgl", choices=["fastgl", "reference"])
    ap.add_argument("--config", default="products-like", choices=sorted(CONFIGS))
    ap.add_argument("--window", type=int, default=16, help="mini-batches sampled per kernel launch")
    ap.add_argument("--teams", type=int, default=0)
    ap.add_argument("--table-slots", type=int, default=-1,
                    help="cap of the sampler's per-team hashtable (0: worst-case size; default: learnt from the first window)")
    ap.add_argument("--reorder", action="store_true", help="Match-Reorder each window")
    ap.add_argument("--matmul", default="3xtf32", choices=["fp32", "3xtf32", "tf32"],
                    help="arithmetic of the dense-layer GEMMs that stay in cuBLAS: fp32 = SIMT float32 kernels; 3xtf32 = "
                         "error-compensated split into three TF32 tensor-core products, float32-level error; tf32 = "
                         "single-pass TF32, what the reference's pinned PyTorch 1.10.1 used by default on Ampere")
    ap.add_argument("--no-graph", action="store_true", help="launch the per-batch step op by op instead of a CUDA graph")
    ap.add_argument("--cpu-steps", type=int, default=150, help="mini-batches of the CPU baseline sample (about 10 s of CPU work)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sustained", action="store_true", help="skip the second measurement after seconds of load")
    ap.add_argument("--soak-seconds", type=float, default=3.0, help="load before the sustained measurement")
    ap.add_argument("--settle-seconds", type=float, default=0.7,
                    help="steps run untimed before the warm-up (at least two windows; 0 for profiler runs, where every launch is slow)")
    ap.add_argument("--no-gates", action="store_true", help="skip the untimed correctness gates (profiler runs)")
    ap.add_argument("--layout", default="generated", choices=["generated", "degree"],
                    help="node numbering of the synthetic graph: as generated, or renumbered by descending degree (the "
                         "reference's sort_degree ranking used as a table layout)")
    ap.add_argument("--repeats", type=int, default=7, help="how often the --steps region is timed (the median is reported)")
    ap.add_argument("--no-sharded-leg", action="store_true", help="N > 1: skip the row-sharded feature table leg")
    ap.add_argument("--grad-sync", default="auto", choices=["auto", "nccl", "oneshot"],
                    help="N > 1: gradient all-reduce by NCCL, or by this library's one-launch peer-store kernel")
    ap.add_argument("--kernels", action="store_true",
                    help="print a per-kernel table (time, algorithmic bytes, fraction of the HBM peak) instead of training")
    args = ap.parse_args()
    cfg = dict(CONFIGS[args.config], layout=args.layout)
    args.warmup = max(args.warmup, 3) if args.impl == "fastgl" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    model_name = "GCN" if cfg.get("model") == "gcn" else "GraphSAGE-mean"
    table_mb = cfg["n_nodes"] * cfg["feat_dim"] * 4 / 1e6
    adj_mb = cfg["n_nodes"] * cfg["avg_degree"] * 4 / 1e6
    config_json = {"workload": f"{args.config}: seeded R-MAT {cfg['n_nodes']} nodes x avg degree {cfg['avg_degree']} "
                               f"(symmetrised), {cfg['feat_dim']}-d fp32 features resident in HBM, {cfg['n_classes']} classes, "
                               f"{len(cfg['fanouts'])}-layer {model_name} hidden {cfg['hidden']}, fanout {cfg['fanouts']}, "
                               f"batch {cfg['batch']} per GPU",
                   "layout": args.layout, "window": args.window, "parallelism": f"dp{world}", "global_batch": cfg["batch"] * world,
                   "l2": f"inputs larger than L2: {table_mb:.0f} MB feature table + {adj_mb:.0f} MB adjacency are gathered at "
                         "random each step"}

    if args.impl == "reference":
        if rank != 0:
            return
        device = "cuda" if torch.cuda.is_available() else "cpu"
        indptr, indices, feat, labels, train = build_inputs(cfg, device)
        step, cores = make_cpu_stepper(cfg, indptr, indices, feat, labels, train)
        for _ in range(args.warmup):
            step()
        edges, dt = time_cpu_steps(step, args.steps)
        val = edges / dt
        line = {"impl": "reference", "metric": "sampled_edges_per_s", "value": val, "unit": "edges/s", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / max(1, args.steps),
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": config_json, "gpu_launches": 0,
                "cpu_baseline": {"value": val, "unit": "edges/s", "cores": cores, "kind": "port",
                                 "sample": f"{args.steps} mini-batches of {cfg['batch']} seeds: C oracle sampling + mapping + "
                                           "aggregation, torch CPU dense layers and Adam"},
                "e2e": {"value": val, "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the fastgl ops have no CPU path")
    import fastgl
    from fastgl_b200.layers import GCN, GraphSAGE
    from fastgl_b200.trainer import Trainer

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    torch.manual_seed(12345)
    torch.backends.cuda.matmul.allow_tf32 = args.matmul == "tf32"
    indptr, indices, feat, labels, train = build_inputs(cfg, device, rank, world)
    if cfg.get("model") == "gcn":
        model = GCN(cfg["feat_dim"], cfg["hidden"], cfg["n_classes"], len(cfg["fanouts"]), dropout=0.5).to(device)
    else:
        model = GraphSAGE(cfg["feat_dim"], cfg["hidden"], cfg["n_classes"], len(cfg["fanouts"]), dropout=0.5).to(device)
    if args.kernels:
        # per-kernel roofline table on blocks of this workload (one GPU; no training)
        import bench_kernels as kernel_bench
        if world > 1 or not torch.is_tensor(feat):
            raise SystemExit("--kernels runs on one GPU with a dense feature table")
        peak, peak_kind = load_peaks()
        table = kernel_bench.run(indptr, indices, feat, train, cfg["fanouts"], cfg["batch"], args.window, peak)
        print(json.dumps({"kernels": table, "peak_gb_per_s": peak, "peak_kind": peak_kind, "config": config_json}))
        return
    model.train()
    tr = Trainer(indptr, indices, feat, labels, train, model, cfg["fanouts"], batch_size=cfg["batch"], window=args.window,
                 reorder=args.reorder, rank=rank, world=world, n_teams=args.teams, cuda_graph=not args.no_graph,
                 table_slots=None if args.table_slots < 0 else args.table_slots, grad_sync=args.grad_sync,
                 matmul="3xtf32" if args.matmul == "3xtf32" else "fp32")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    # --- correctness gates on one window of this very workload (untimed): the size-independent properties of
    #     the sampled blocks and, for the SAGE first layer, the window aggregation against float64 torch algebra
    gates = None if args.no_gates else run_gates(cfg, args, indptr, indices, feat, train, device)

    # --- set-up (tables, workspace, graph capture), then a settle phase of at least two full windows whatever
    #     --warmup says (the sampler's tables, the allocator and NCCL reach their steady state), then the warm-up
    tr.prime()
    clocks = ClockSampler(local_rank)
    if rank == 0:
        clocks.start()
        clocks.wait_ready()
    barrier()
    # The loop needs a moment to reach the rate it then keeps: launched back to back, the window aggregation alone is
    # 3.5 % faster during its first 0.35 s than afterwards (SM and memory clocks at their maxima throughout), and the
    # training state moves too (dead ReLU units change what the step's kernels skip).  The settle phase therefore runs
    # steps for 0.7 s (--settle-seconds), and a second measurement after 3 s of load is reported beside the first.
    t_settle = time.time()
    settle_steps = 0
    while settle_steps < 2 * args.window or float(max_over_ranks(time.time() - t_settle)) < args.settle_seconds:
        tr.run_steps(2 * args.window)
        torch.cuda.synchronize()
        settle_steps += 2 * args.window
    tr.run_steps(args.warmup)
    fastgl.check_status(device)
    barrier()
    if rank == 0:
        clocks.mark()
    tr.time_layer0 = True
    tr.layer0_events.clear()
    tr.sample_events.clear()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed_region(**kw):
        """EXACTLY --steps steps between two device events, a barrier and a synchronize on both sides; returns
        (milliseconds: max over ranks, sampled edges: sum over ranks, losses)."""
        tr.sampled_edges = 0
        barrier()
        ev0.record()
        losses = tr.run_steps(args.steps, **kw)
        ev1.record()
        barrier()
        return max_over_ranks(ev0.elapsed_time(ev1)), sum_over_ranks(float(tr.sampled_edges)), losses

    def repeats_for(first_ms: float) -> int:
        """The --steps region is repeated at least seven times, and often enough for the clock sampler to see it."""
        r = max(args.repeats, math.ceil(300.0 / max(first_ms, 1e-3)))
        r = int(max_over_ranks(float(min(r, 101))))
        return r if r % 2 == 1 else r + 1

    # --- device-resident regions: value = median over the repeats ---------------------------------------------
    regions = [timed_region()]
    for _ in range(repeats_for(regions[0][0]) - 1):
        regions.append(timed_region())
        if len(tr.layer0_events) > 256:
            del tr.layer0_events[:-128], tr.sample_events[:-128]
    tr.time_layer0 = False
    fastgl.check_status(device)
    by_ms = sorted(regions, key=lambda r: r[0])
    ms, edges_all, _ = by_ms[len(by_ms) // 2]
    value = edges_all / (ms * 1e-3)

    # --- roofline of the dominant kernel: the window-level first-layer aggregation (mean of neighbours + self
    #     rows, straight from the feature table), one launch per window, timed by events on the launching stream
    D = cfg["feat_dim"]
    peak, peak_kind = load_peaks()
    full = [(s_.elapsed_time(e_), fb) for s_, e_, fb in tr.layer0_events if fb.n_batches == args.window]
    agg_ms = [t for t, _ in full]
    roofline = {"kernel": "first-layer aggregation over a window (agg_fwd_staged_kernel<MEAN, row_map> for rows of up to 128 floats, "
                          "agg_fwd_kernel beyond)", "bound": "hbm", "achieved": None,
                "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": None, "traffic": None}
    sample_roofline = None
    if agg_ms:
        fb = full[-1][1]  # the last full window is still in the buffers
        counts_h = fb.counts_host()
        hop = len(cfg["fanouts"]) - 1
        alg, sm_bytes = 0, 0
        deg_all = indptr[1:] - indptr[:-1]
        fan_s = list(reversed(cfg["fanouts"]))
        for b in range(fb.n_batches):
            n_dst, n_edges = int(counts_h[b, hop]), int(counts_h[b, 8 + hop])
            touched = torch.cat([fb.block_src[hop][b, :n_edges], torch.arange(n_dst, dtype=torch.int32, device=device)])
            # distinct rows are counted per mini-batch and summed over the window: a row that two mini-batches of
            # the window share is credited twice, although the second read may be served by L2
            r_all = int(torch.unique(touched).numel())
            # reads: every distinct feature row once + its id; edge ids and offsets; writes: self and mean rows
            alg += 4 * D * r_all + 4 * r_all + 4 * n_edges + 4 * (n_dst + 1) + 2 * 4 * D * n_dst
            nodes = fb.nodes[b].long()
            for h in range(len(fan_s)):  # sampler: S*40 + sum_seeds min(32*ceil(4*deg/32), 32*k) + 4E + 4U per hop
                S, E, U = int(counts_h[b, h]), int(counts_h[b, 8 + h]), int(counts_h[b, h + 1]) - int(counts_h[b, h])
                dg = deg_all[nodes[:S]]
                k = torch.clamp(dg, max=fan_s[h])
                sm_bytes += S * 40 + int(torch.minimum(32 * ((4 * dg + 31) // 32), 32 * k).sum()) + 4 * E + 4 * U
        med_ms = statistics.median(agg_ms)
        achieved = alg / (med_ms * 1e-3) / 1e9
        roofline.update({"achieved": achieved, "frac": achieved / peak, "algorithmic_bytes_per_launch": alg,
                         "launch_ms": med_ms, "launch_ms_min": min(agg_ms), "launch_ms_max": max(agg_ms),
                         "launches_timed": len(agg_ms)})
        default_run = args.teams == 0 and args.table_slots < 0 and not args.reorder and args.layout == "generated"
        agg_traffic, smp_traffic, traffic_note = load_ncu_traffic(args.config, args.window) if default_run else (None, None, None)
        roofline["traffic"] = agg_traffic
        if traffic_note:
            roofline["traffic_note"] = traffic_note
        smp = [s_.elapsed_time(e_) for s_, e_, nb in tr.sample_events if nb == args.window]
        if smp:
            smp_ms = statistics.median(smp)
            sample_roofline = {"kernel": "sample_map_kernel (3 hops x window)", "bound": "hbm",
                               "achieved": sm_bytes / (smp_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                               "frac": sm_bytes / (smp_ms * 1e-3) / 1e9 / peak, "algorithmic_bytes_per_launch": sm_bytes,
                               "launch_ms": smp_ms, "launch_ms_min": min(smp), "launch_ms_max": max(smp),
                               "launches_timed": len(smp), "traffic": smp_traffic,
                               "note": "event-timed on the launching stream, the events recorded directly around the launch"}

    # --- end to end: seeds come from pinned host memory every window, the loss goes back every step -------
    host_rows, host_counts = [], []
    for _ in range(args.steps):
        s_, c_ = tr._next_window_seeds(1)
        host_rows.append(s_.cpu())
        host_counts.append(c_)
    seeds_h = torch.cat(host_rows).pin_memory()
    counts_h = torch.cat(host_counts).pin_memory()
    e2e_regions = [timed_region(host_seeds=(seeds_h, counts_h), read_loss_each_step=True) for _ in range(len(regions))]
    e2e_by_ms = sorted(e2e_regions, key=lambda r: r[0])
    ms_e2e, e2e_edges, losses = e2e_by_ms[len(e2e_by_ms) // 2]
    # --- the same loop after seconds of load: a job of many epochs runs at this rate; reported beside the headline,
    #     not instead of it, and as a check that the two do not drift apart (a value-dependent kernel once made them
    #     differ by 10 %)
    sustained = None
    if not args.no_sustained:
        t_load = time.time()
        while float(max_over_ranks(time.time() - t_load)) < args.soak_seconds:
            tr.run_steps(4 * args.window)
            torch.cuda.synchronize()
        n_before = len(tr.layer0_events)
        tr.time_layer0 = True
        soaked = sorted((timed_region() for _ in range(5)), key=lambda r: r[0])
        tr.time_layer0 = False
        s_ms, s_edges, _ = soaked[len(soaked) // 2]
        s_agg = [s_.elapsed_time(e_) for s_, e_, fb_ in tr.layer0_events[n_before:] if fb_.n_batches == args.window]
        sustained = {"after_seconds_of_load": args.soak_seconds, "value": s_edges / (s_ms * 1e-3), "unit": "edges/s",
                     "ms_per_step": s_ms / args.steps,
                     "ms_per_step_repeats": [round(r[0] / args.steps, 4) for r in soaked],
                     "window_aggregation_launch_ms": statistics.median(s_agg) if s_agg else None}
    clock_info = clocks.stop() if rank == 0 else None
    fastgl.check_status(device)

    sharded_leg = None
    if world > 1 and not args.no_sharded_leg:
        sharded_leg = run_sharded_leg(cfg, args, tr, indptr, rank, world, device, barrier, max_over_ranks)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and cfg.get("model") != "gcn" and cfg["n_nodes"] <= 10_000_000:
        step, cores = make_cpu_stepper(cfg, indptr, indices, feat, labels, train)
        step()
        edges, dt = time_cpu_steps(step, args.cpu_steps)
        cpu_baseline = {"value": edges / dt, "unit": "edges/s", "cores": cores, "kind": "port",
                        "sample": f"{args.cpu_steps} mini-batches of {cfg['batch']} seeds (after 1 warm-up): C oracle sampling + "
                                  "mapping + aggregation, torch CPU dense layers and Adam", "ms_per_step": 1e3 * dt / args.cpu_steps}

    if rank == 0:
        steps_per_epoch = tr.steps_per_epoch()
        # kernels of this library: per window one fused sampling launch and one first-layer aggregation launch; per
        # step one staging launch and, inside the replayed step program, per inner layer one forward aggregation, one
        # self-gradient initialisation and one backward scatter, per hidden layer one bias/ReLU/dropout epilogue and
        # one backward of it, two launches for the output layer with its loss, and one Adam launch (5 L - 1).  The
        # op-by-op path (--no-graph) launches one forward and one backward aggregation per inner layer.
        n_windows = (args.steps + args.window - 1) // args.window
        n_layers = len(cfg["fanouts"])
        per_step = (5 * n_layers - 1) if tr.graphed is not None else 2 * (n_layers - 1)
        if tr.graphed is not None and args.matmul == "3xtf32":
            # operand splits (n_layers weights, n_layers layer inputs -- the first one while staging --, the output
            # layer's gradient) and n_layers folds of the weight-gradient blocks
            per_step += 3 * n_layers + 1
        launches = args.steps * per_step + 2 * n_windows
        epoch_s = steps_per_epoch * ms / args.steps * 1e-3
        line = {"metric": "sampled_edges_per_s", "value": value, "unit": "edges/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "tf32" if args.matmul == "tf32" else "f32", "data": "synthetic", "config": config_json,
                "repeats": len(regions), "ms_per_step_min": by_ms[0][0] / args.steps, "ms_per_step_max": by_ms[-1][0] / args.steps,
                "ms_per_step_repeats": [round(r[0] / args.steps, 4) for r in regions],
                "settle_steps": settle_steps,
                "per_gpu_value": value / world, "epoch_time_s": epoch_s,
                "epoch_time_kind": "measured" if args.steps >= steps_per_epoch else f"extrapolated from {args.steps} steps",
                "steps_per_epoch": steps_per_epoch, "final_loss": losses[-1] if losses else None,
                "dense_matmul": DENSE_MATMUL[args.matmul], "cuda_graph": not args.no_graph, "graph_fallback_steps": tr.graph_fallbacks,
                "gradient_sync": tr.grad_sync_kind(),
                "e2e": {"value": e2e_edges / (ms_e2e * 1e-3), "unit": "edges/s", "ms_per_step": ms_e2e / args.steps,
                        "ms_per_step_min": e2e_by_ms[0][0] / args.steps, "ms_per_step_max": e2e_by_ms[-1][0] / args.steps,
                        "repeats": len(e2e_regions),
                        "h2d_bytes_per_step": cfg["batch"] * 4 + 4, "d2h_bytes_per_step": 4 + 64},
                "gpu_launches": launches * world, "roofline": roofline, "roofline_sample_map": sample_roofline,
                "gates": gates, "clocks": clock_info}
        if sustained is not None:
            line["sustained"] = sustained
        if cpu_baseline is not None:
            line["cpu_baseline"] = cpu_baseline
        if sharded_leg is not None:
            line["sharded"] = sharded_leg
        print(json.dumps(line))
    if world > 1:
        # every rank's GPU work has drained; only then drop the mappings of the peers' memory, and only after every
        # rank has dropped them tear the allocations down
        torch.cuda.synchronize()
        dist.barrier()
        tr.release_peers()
        tr.feat = None
        del tr, feat
        import gc
        gc.collect()      # the trainer and its captured step refer to each other: without this the shard mappings live on
        torch.cuda.ipc_collect()
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

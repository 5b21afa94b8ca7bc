"""``fastgl`` -- drop-in replacement of the reference's PyTorch extension of the same name.

The reference binds 19 ops with pybind11 (cuda_operators/aggregate_acc.cpp:601-621); the ones its
Python callers use (FusedMapSampler.py:76,98; GraphConv.py:26,37,93-96,109,132,204,224) are re-exposed here
with the same names, positional arguments, dtypes, return lists and error behaviour:

    sample_node, transfer_edge_id, cal_deg, exclusive_sum,
    forward_gcn, backward_gcn, forwaed_gin (sic), backward_gin, forward_gat, backward_gat

Each op allocates its outputs with torch and calls the C ABI of ``libfastgl_b200.so``
(include/fastgl_b200.h) with raw device pointers and torch's current CUDA stream.  The dense weight
products stay in torch (cuBLAS), as the reference keeps them in ``torch::mm``.  There is no CPU path:
importing this module without the built library raises ImportError, and every op raises
RuntimeError for a tensor that is not CUDA or not contiguous (aggregate_acc.cpp:4-6).

Additive ops (not in the reference): ``sample_node_csr``, ``aggregate`` / ``aggregate_backward``
(sum | mean | symnorm, optional row map into a feature table), ``sample_map_fused`` (all hops of many
mini-batches in one persistent kernel), ``set_sampling`` / ``seed``.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

from . import _capi
from ._capi import (AGG_MEAN, AGG_SUM, AGG_SYMNORM, COUNTS_STRIDE, FLAG_MAP_ARRIVAL_ORDER,
                    FLAG_SAMPLE_REPLACE, FLAG_ZERO_DEG_PASSTHROUGH, MAX_HOPS, FusedArgs, lib)

__all__ = [
    "sample_node", "transfer_edge_id", "cal_deg", "exclusive_sum", "forward_gcn", "backward_gcn",
    "forwaed_gin", "backward_gin", "forward_gat", "backward_gat", "edge_weight_grad", "sample_node_csr", "aggregate", "aggregate_backward", "aggregate_window",
    "sample_map_fused", "fused_capacity", "stage_segments", "stage_segments_raw", "gather_rows", "ShardedTable", "set_sampling", "seed", "FusedBatch",
    "exclusive_sum_noalloc", "exclusive_sum_noalloc_status", "check_status", "status_str", "PeerSync", "allreduce_adam_", "window_overlap", "TransposedBlock", "transpose_block", "split_tf32", "split_tf32_raw", "fold_blocks", "probe_access_pattern",
    "AGG_SUM", "AGG_MEAN", "AGG_SYMNORM",
]

# status codes of include/fastgl_b200.h that callers branch on
ERR_CAPACITY, ERR_PROBE, ERR_BOUNDS, ERR_TIMEOUT = 4, 5, 6, 7

_state_lock = threading.Lock()
_workspaces: dict[int, ctypes.c_void_p] = {}
_config = {"replace": False, "arrival_order": False, "rng_seed": 12345, "rng_ctr": 0}


# ------------------------------------------------------------------------------------------------
# plumbing
# ------------------------------------------------------------------------------------------------
def _check_input(t: torch.Tensor, name: str) -> None:
    # CHECK_INPUT of the reference: CUDA and contiguous (aggregate_acc.cpp:4-6)
    if not isinstance(t, torch.Tensor):
        raise RuntimeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def _check_i32(t: torch.Tensor, name: str) -> None:
    _check_input(t, name)
    if t.dtype != torch.int32:
        raise RuntimeError(f"{name} must be int32 (got {t.dtype})")


def _check_f32(t: torch.Tensor, name: str) -> None:
    _check_input(t, name)
    if t.dtype != torch.float32:
        raise RuntimeError(f"{name} must be float32 (got {t.dtype})")


def _check_rows_f32(t: torch.Tensor, name: str) -> None:
    """A float32 CUDA matrix whose rows are contiguous (a column slice of a wider buffer is fine)."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda or t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1:
        raise RuntimeError(f"{name} must be a float32 CUDA matrix with unit column stride")


def _ws(device: torch.device) -> ctypes.c_void_p:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    with _state_lock:
        ws = _workspaces.get(idx)
        if ws is None:
            ws = ctypes.c_void_p()
            rc = lib().fgl_ws_create(ctypes.c_int(idx), ctypes.byref(ws))
            if rc != 0:
                raise RuntimeError(f"fgl_ws_create(device={idx}) failed: {_capi.status_str(rc)}")
            _workspaces[idx] = ws
    return ws


def _stream(device: torch.device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _time_next_launch(dev, timing) -> None:
    """Have the library record the pair of ``torch.cuda.Event`` directly around its next window-level launch."""
    for ev in timing:
        ev.record()         # torch creates the CUDA event at its first record; the library records it again
    rc = lib().fgl_ws_time_next_launch(_ws(dev), ctypes.c_void_p(timing[0].cuda_event), ctypes.c_void_p(timing[1].cuda_event))
    _raise(rc, "time_next_launch")


def _ptr(t) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None or t.numel() == 0 else t.data_ptr())


def _raise(rc: int, what: str, ws=None) -> None:
    if rc != 0:
        detail = ""
        if ws is not None:
            msg = lib().fgl_last_error(ws)
            detail = f" ({msg.decode()})" if msg else ""
        raise RuntimeError(f"{what} failed: {_capi.status_str(rc)}{detail}")


class _on_device:
    """Make ``device`` current for a library call that launches without a workspace."""

    def __init__(self, device: torch.device):
        self.device = device
        self.ctx = None

    def __enter__(self):
        if self.device.index is not None and self.device.index != torch.cuda.current_device():
            self.ctx = torch.cuda.device(self.device)
            self.ctx.__enter__()

    def __exit__(self, *exc):
        if self.ctx is not None:
            self.ctx.__exit__(*exc)


def set_sampling(replace: bool | None = None, arrival_order: bool | None = None) -> None:
    """Choose the sampler's behaviour for the drop-in ops.

    ``replace=True`` reproduces the reference kernel for hubs (independent picks, duplicates
    possible, sample.cu:88-94); the default draws a uniform k-subset.  ``arrival_order=True`` numbers
    new nodes in atomic arrival order (id_map.cu:317-320); the default is first-occurrence order.
    """
    if replace is not None:
        _config["replace"] = bool(replace)
    if arrival_order is not None:
        _config["arrival_order"] = bool(arrival_order)


def seed(rng_seed: int, rng_ctr: int = 0) -> None:
    """Key of the sampler's Philox generator and the counter the next ``sample_node`` call uses."""
    _config["rng_seed"] = int(rng_seed) & 0xFFFFFFFFFFFFFFFF
    _config["rng_ctr"] = int(rng_ctr) & 0xFFFFFFFFFFFFFFFF


def _next_ctr() -> int:
    with _state_lock:
        c = _config["rng_ctr"]
        _config["rng_ctr"] = (c + 1) & 0xFFFFFFFFFFFFFFFF
    return c


# ------------------------------------------------------------------------------------------------
# a1  sampling
# ------------------------------------------------------------------------------------------------
def sample_node_csr(src_edges, edge_ptr, seed_nodes, neighbor_num, replace=None, rng_seed=None, rng_ctr=None,
                    want_dst=True):
    """Sample and also return the block CSR offsets: (src_out, dst_out | None, block_indptr, n_edges)."""
    _check_i32(src_edges, "src_edges")
    _check_input(edge_ptr, "edge_ptr")
    _check_i32(seed_nodes, "seed_nodes")
    if edge_ptr.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("edge_ptr must be int32 or int64")
    dev = seed_nodes.device
    S = seed_nodes.numel()
    fanout = int(neighbor_num)
    out_src = torch.empty(max(1, S * fanout), dtype=torch.int32, device=dev)
    out_dst = torch.empty(max(1, S * fanout), dtype=torch.int32, device=dev) if want_dst else None
    out_ptr = torch.empty(S + 1, dtype=torch.int32, device=dev)
    flags = FLAG_SAMPLE_REPLACE if (_config["replace"] if replace is None else replace) else 0
    n_edges = ctypes.c_int64(0)
    ws = _ws(dev)
    rc = lib().fgl_sample(ws, _ptr(edge_ptr), ctypes.c_int(1 if edge_ptr.dtype == torch.int64 else 0), _ptr(src_edges),
                          ctypes.c_int64(edge_ptr.numel() - 1), _ptr(seed_nodes), ctypes.c_int32(S),
                          ctypes.c_int32(fanout), ctypes.c_int32(flags),
                          ctypes.c_uint64(_config["rng_seed"] if rng_seed is None else rng_seed),
                          ctypes.c_uint64(_next_ctr() if rng_ctr is None else rng_ctr), _ptr(out_ptr), _ptr(out_src),
                          _ptr(out_dst), ctypes.byref(n_edges), _stream(dev))
    _raise(rc, "sample_node", ws)
    E = int(n_edges.value)
    return out_src[:E], (out_dst[:E] if want_dst else None), out_ptr, E


def sample_node(src_edges, dst_edges, edge_ptr, seed_nodes, dst_nodes, neighbor_num):
    """aggregate_acc.cpp:491-512 -> sample_node_cuda (sample.cu:102-203).

    Returns ``[src_out, dst_out, edges_num]``: the global source id and the global seed id of every
    sampled edge, grouped by seed in seed order, and the edge count as an int32[1] CUDA tensor.
    ``dst_edges`` is accepted and ignored, like the reference (sample.cu:43 never reads it).
    """
    _check_input(dst_edges, "dst_edges")
    if int(dst_nodes) < seed_nodes.numel():
        raise RuntimeError("dst_nodes must cover seed_nodes")
    src_out, dst_out, _, E = sample_node_csr(src_edges, edge_ptr, seed_nodes, neighbor_num)
    edges_num = torch.tensor([E], dtype=torch.int32, device=seed_nodes.device)
    return [src_out, dst_out, edges_num]


# ------------------------------------------------------------------------------------------------
# a2  Fused-Map
# ------------------------------------------------------------------------------------------------
def transfer_edge_id(src_edges, dst_edges, dst_edges_unique, dst_nodes, total_items, unique_num, edge_nums):
    """aggregate_acc.cpp:467-489 -> transfer_edge_id_cuda (id_map.cu:386-493).

    Rewrites ``src_edges`` / ``dst_edges`` in place with block-local ids and returns
    ``[src_edges, dst_edges, unique_nodes]`` where ``unique_nodes`` = the seeds followed by every new
    source once (first-occurrence order unless ``set_sampling(arrival_order=True)``).
    """
    _check_i32(src_edges, "src_edges")
    _check_i32(dst_edges, "dst_edges")
    _check_i32(dst_edges_unique, "dst_edges_unique")
    dev = src_edges.device
    S = min(int(dst_nodes), dst_edges_unique.numel())
    E = int(edge_nums)
    if E > src_edges.numel() or E > dst_edges.numel():
        raise RuntimeError("edge_nums exceeds the edge arrays")
    cap = S + max(0, min(int(unique_num), E))
    unique = torch.empty(max(1, cap), dtype=torch.int32, device=dev)
    n_unique = ctypes.c_int64(0)
    flags = FLAG_MAP_ARRIVAL_ORDER if _config["arrival_order"] else 0
    ws = _ws(dev)
    rc = lib().fgl_map(ws, _ptr(src_edges), _ptr(dst_edges), _ptr(dst_edges_unique), ctypes.c_int32(S),
                       ctypes.c_int64(E), _ptr(unique), ctypes.c_int64(cap), ctypes.c_int32(flags),
                       ctypes.byref(n_unique), _stream(dev))
    _raise(rc, "transfer_edge_id", ws)
    return [src_edges, dst_edges, unique[: int(n_unique.value)]]


# ------------------------------------------------------------------------------------------------
# a3  block-CSR helpers
# ------------------------------------------------------------------------------------------------
def cal_deg(edges, nodes_num):
    """aggregate_acc.cpp:522-529 -> cal_deg_cuda (utilis.cu:60-79): histogram of an id array."""
    _check_i32(edges, "edges")
    dev = edges.device
    deg = torch.empty(int(nodes_num), dtype=torch.int32, device=dev)
    with _on_device(dev):
        rc = lib().fgl_cal_deg(_ptr(edges), ctypes.c_int64(edges.numel()), _ptr(deg), ctypes.c_int32(int(nodes_num)),
                               _stream(dev))
    _raise(rc, "cal_deg")
    return deg


def exclusive_sum(in_degs):
    """aggregate_acc.cpp:514-520 -> exclusive_sum_cuda (utilis.cu:17-41): int32[n+1] offsets."""
    _check_i32(in_degs, "in_degs")
    dev = in_degs.device
    out = torch.empty(in_degs.numel() + 1, dtype=torch.int32, device=dev)
    ws = _ws(dev)
    rc = lib().fgl_exclusive_sum(ws, _ptr(in_degs), ctypes.c_int64(in_degs.numel()), _ptr(out), _stream(dev))
    _raise(rc, "exclusive_sum", ws)
    return out


def exclusive_sum_noalloc(in_degs, out):
    """``exclusive_sum`` into a caller-provided ``out`` (int32[n+1]) through the entry point that allocates
    nothing on the device: for callers that run under a fixed memory budget or cannot afford an allocation's
    device synchronisation.  At most 2**27 entries; calls on different streams must not overlap."""
    _check_i32(in_degs, "in_degs")
    _check_i32(out, "out")
    if out.numel() < in_degs.numel() + 1:
        raise RuntimeError("out needs in_degs.numel() + 1 entries")
    dev = in_degs.device
    with _on_device(dev):
        rc = lib().fgl_exclusive_sum_noalloc(_ptr(in_degs), ctypes.c_int64(in_degs.numel()), _ptr(out), _stream(dev))
    _raise(rc, "exclusive_sum_noalloc")
    return out


def exclusive_sum_noalloc_status(device=None) -> int:
    """Status of the ``exclusive_sum_noalloc`` calls on ``device`` since the last call of this function: 0, or the
    code of the first failure (a scan whose bounded barrier gave up leaves its output incomplete).  Synchronises the
    current stream; reads and clears the status word without allocating device memory."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if not hasattr(exclusive_sum_noalloc_status, "_pinned"):
        exclusive_sum_noalloc_status._pinned = torch.zeros(1, dtype=torch.int32).pin_memory()
    host = exclusive_sum_noalloc_status._pinned
    with _on_device(dev):
        rc = lib().fgl_exclusive_sum_noalloc_status(ctypes.c_void_p(host.data_ptr()), _stream(dev))
    _raise(rc, "exclusive_sum_noalloc_status")
    torch.cuda.current_stream(dev).synchronize()
    return int(host[0])


# ------------------------------------------------------------------------------------------------
# feature tables
# ------------------------------------------------------------------------------------------------
class ShardedTable:
    """A float32 feature table whose rows are block-partitioned over several device buffers -- typically one
    per GPU of the box, every peer's buffer mapped into this process (symmetric memory or CUDA IPC).  Global
    row ``r`` is row ``r % rows_per_shard`` of shard ``r // rows_per_shard``.  The kernels read peers' rows
    with plain 128-bit loads over NVLink.

    ``shards``: a list of CUDA tensors [rows_per_shard, dim] (kept alive here) or of raw device pointers."""

    def __init__(self, shards, rows_per_shard: int, dim: int, n_rows: int, device, ld: int | None = None):
        self.keep = [s for s in shards if isinstance(s, torch.Tensor)]
        ptrs = [int(s.data_ptr()) if isinstance(s, torch.Tensor) else int(s) for s in shards]
        for t in self.keep:
            if t.dtype != torch.float32 or t.dim() != 2 or t.stride(1) != 1 or t.size(1) != dim:
                raise RuntimeError("shards must be float32 [rows, dim] with unit column stride")
        self.device = torch.device(device)
        self.ptrs = torch.tensor(ptrs, dtype=torch.int64).to(self.device)
        self.rows_per_shard = int(rows_per_shard)
        self.dim = int(dim)
        self.ld = int(ld if ld is not None else (self.keep[0].stride(0) if self.keep else dim))
        self.n_rows = int(n_rows)

    def size(self, i):
        return (self.n_rows, self.dim)[i]


def _table_args(input_feat):
    """(x pointer, shards pointer, rows_per_shard, n_rows, ld, dim, device) of a dense or sharded table."""
    if isinstance(input_feat, ShardedTable):
        return (ctypes.c_void_p(0), _ptr(input_feat.ptrs), input_feat.rows_per_shard, input_feat.n_rows, input_feat.ld,
                input_feat.dim, input_feat.device)
    _check_rows_f32(input_feat, "input_feat")
    return (_ptr(input_feat), ctypes.c_void_p(0), 0, input_feat.size(0), input_feat.stride(0), input_feat.size(1),
            input_feat.device)


def gather_rows(table, ids, out=None):
    """``out[i] = table[ids[i]]`` for a dense CUDA matrix or a ``ShardedTable``; ``ids`` int32."""
    _check_i32(ids, "ids")
    x, shards, rps, n_rows, ld, dim, dev = _table_args(table)
    if out is None:
        out = torch.empty((ids.numel(), dim), dtype=torch.float32, device=dev)
    else:
        _check_rows_f32(out, "out")
    with _on_device(dev):
        rc = lib().fgl_gather_rows(_ws(dev), x, shards, ctypes.c_int64(rps), ctypes.c_int64(n_rows), ctypes.c_int64(ld),
                                   ctypes.c_int32(dim), _ptr(ids), ctypes.c_int64(ids.numel()), _ptr(out),
                                   ctypes.c_int64(out.stride(0)), _stream(dev))
    _raise(rc, "gather_rows")
    return out


# ------------------------------------------------------------------------------------------------
# a4-a7  aggregation
# ------------------------------------------------------------------------------------------------
def aggregate(mode, edge_ptr, src_edges, input_feat, dst_nodes, src_norm_degs=None, dst_norm_degs=None,
              zero_deg_passthrough=True, row_map=None, out=None, n_dst_dev=None):
    """out[d] = sum over the row's edges of w * input_feat[row(src)], w by ``mode`` (AGG_SUM | AGG_MEAN |
    AGG_SYMNORM); ``row_map`` (int32) turns block-local ids into rows of ``input_feat``.  ``n_dst_dev`` (int32
    CUDA tensor, optional) holds the real row count on the device; ``dst_nodes`` is then the padded count the
    output is sized for (used to replay a captured CUDA graph on blocks of different sizes)."""
    _check_i32(edge_ptr, "edge_ptr")
    _check_i32(src_edges, "src_edges")
    if not isinstance(input_feat, ShardedTable):
        _check_f32(input_feat, "input_feat")
        if input_feat.dim() != 2:
            raise RuntimeError("input_feat must be 2-D")
    for t, n in ((src_norm_degs, "src_norm_degs"), (dst_norm_degs, "dst_norm_degs"), (row_map, "row_map")):
        if t is not None:
            _check_i32(t, n)
    n_dst = int(dst_nodes)
    if edge_ptr.numel() < n_dst + 1:
        raise RuntimeError("edge_ptr is shorter than dst_nodes + 1")
    x, shards, rps, n_rows, ld, dim, dev = _table_args(input_feat)
    if mode == AGG_SYMNORM:
        n_src = row_map.numel() if row_map is not None else (input_feat.size(0) if torch.is_tensor(input_feat) else None)
        if (src_norm_degs is None or dst_norm_degs is None or dst_norm_degs.numel() < n_dst
                or (n_src is not None and src_norm_degs.numel() < n_src)):
            raise RuntimeError("sym-norm needs src_norm_degs[n_src] and dst_norm_degs[n_dst]")
    if out is None:
        out = torch.empty((n_dst, dim), dtype=torch.float32, device=dev)
    else:
        _check_rows_f32(out, "out")
    with _on_device(dev):
        rc = lib().fgl_agg_fwd_sharded(_ws(dev), ctypes.c_int32(mode), _ptr(edge_ptr), _ptr(src_edges), _ptr(src_norm_degs),
                                       _ptr(dst_norm_degs), _ptr(row_map),
                                       ctypes.c_int64(row_map.numel() if row_map is not None else 0), x, shards,
                                       ctypes.c_int64(rps), ctypes.c_int64(n_rows), ctypes.c_int64(ld),
                                       ctypes.c_int32(dim), ctypes.c_int32(n_dst),
                                       ctypes.c_int32(FLAG_ZERO_DEG_PASSTHROUGH if zero_deg_passthrough else 0), _ptr(out),
                                       ctypes.c_int64(out.stride(0)), _ptr(n_dst_dev), _stream(dev))
    _raise(rc, "aggregate")
    return out


def aggregate_window(mode, fb, hop, input_feat, out, self_out=None, use_row_map=True, timing=None):
    """One layer's forward aggregation for every mini-batch of a window in one launch.

    ``fb`` is a ``FusedBatch``; ``hop`` the sampling hop whose block is aggregated (the input layer is hop
    ``len(fanouts) - 1``).  Batch ``b``'s rows go to ``out[row_off[b] : row_off[b] + n_dst_b]`` where
    ``row_off`` is the exclusive prefix sum of the batches' destination counts; returns ``row_off`` (a host
    list with the total appended).  With ``use_row_map`` the rows of ``input_feat`` are addressed through the
    window's global node ids (aggregation straight from the feature table); ``self_out`` also receives each
    destination's own input row.  ``timing``: a pair of ``torch.cuda.Event`` that the library records directly around the
    kernel launch, so that the interval holds the kernel and not the host's way to it."""
    x, shards, rps, n_rows, ld, dim, dev = _table_args(input_feat)
    _check_rows_f32(out, "out")
    if self_out is not None:
        _check_rows_f32(self_out, "self_out")
    counts = fb.counts_host()
    n_dst = counts[:, hop].tolist()
    row_off = [0]
    for n in n_dst:
        row_off.append(row_off[-1] + int(n))
    if out.size(0) < row_off[-1] or (self_out is not None and self_out.size(0) < row_off[-1]):
        raise RuntimeError("out is too small for the window's destination rows")
    off_dev = torch.tensor(row_off, dtype=torch.int64).to(dev, non_blocking=True)
    ptr, src = fb.block_indptr[hop], fb.block_src[hop]
    if row_off[-1] == 0:
        if timing is not None:
            timing[0].record()
            timing[1].record()
        return row_off
    with _on_device(dev):
        args = (_ws(dev), ctypes.c_int32(mode), ctypes.c_int32(fb.n_batches), _ptr(ptr), ctypes.c_int64(ptr.stride(0)), _ptr(src),
                ctypes.c_int64(src.stride(0)), _ptr(fb.nodes if use_row_map else None), ctypes.c_int64(fb.nodes.stride(0)),
                _ptr(off_dev), ctypes.c_int64(row_off[-1]), x, shards, ctypes.c_int64(rps), ctypes.c_int64(n_rows),
                ctypes.c_int64(ld), ctypes.c_int32(dim), ctypes.c_int32(0), _ptr(out),
                ctypes.c_int64(out.stride(0)), _ptr(self_out), ctypes.c_int64(self_out.stride(0) if self_out is not None else dim),
                _stream(dev))
        if timing is not None:      # a pair of torch.cuda.Event the library records directly around the kernel launch
            _time_next_launch(dev, timing)
        rc = lib().fgl_agg_fwd_window(*args)
    _raise(rc, "aggregate_window")
    return row_off


class TransposedBlock:
    """Per-source lists of the destination rows of a block (``fgl_block_transpose``): what the deterministic backward
    gather reads.  Built once per block with ``transpose_block``; the buffers can be reused for the next block of at
    most the same size (``transpose_block(..., out=tb)``)."""

    def __init__(self, n_src: int, edge_cap: int, device):
        self.n_src, self.edge_cap = int(n_src), int(edge_cap)
        i32 = dict(dtype=torch.int32, device=device)
        self.t_indptr = torch.zeros(self.n_src + 1, **i32)
        self.t_dst = torch.zeros(max(1, self.edge_cap), **i32)
        self.hubs = torch.zeros(self.n_src + 1, **i32)
        self.work = torch.zeros(max(1, 2 * self.n_src), **i32)


def transpose_block(edge_ptr, src_edges, dst_nodes, src_nodes, n_dst_dev=None, out: TransposedBlock | None = None):
    """Transpose a block CSR (destination rows -> per-source lists).  ``src_edges`` holds at least ``edge_ptr[dst_nodes]``
    entries; ``out`` reuses buffers sized for at least ``src_nodes`` sources and ``src_edges.numel()`` edges."""
    _check_i32(edge_ptr, "edge_ptr")
    _check_i32(src_edges, "src_edges")
    dev = edge_ptr.device
    n_src, n_dst = int(src_nodes), int(dst_nodes)
    if out is None:
        out = TransposedBlock(n_src, src_edges.numel(), dev)
    elif out.n_src < n_src or out.edge_cap < src_edges.numel():
        raise RuntimeError("the TransposedBlock is too small for this block")
    ws = _ws(dev)
    rc = lib().fgl_block_transpose(ws, _ptr(edge_ptr), _ptr(src_edges), ctypes.c_int32(n_dst), ctypes.c_int32(n_src),
                                   _ptr(out.t_indptr), _ptr(out.t_dst), ctypes.c_int64(out.edge_cap), _ptr(out.hubs),
                                   _ptr(out.work), _ptr(n_dst_dev), _stream(dev))
    _raise(rc, "transpose_block", ws)
    return out


def aggregate_backward(mode, edge_ptr, src_edges, d_out, src_nodes, src_norm_degs=None, dst_norm_degs=None,
                       n_dst_dev=None, d_self=None, out=None, transposed: TransposedBlock | None = None):
    """d_x[src] += w * d_out[d] over every edge; returns d_x float32[src_nodes, dim].  ``n_dst_dev`` as in
    ``aggregate``.  ``d_self`` (float32[n_dst, dim], rows may be a column slice) is the gradient of a self term:
    d_x starts from it in its first n_dst rows instead of from zero.  ``d_out`` may be a column slice too;
    ``out`` receives the result when given.  With ``transposed`` (``transpose_block`` of the same block) the result is
    gathered row by row in a fixed order -- bit-reproducible -- instead of scattered with atomic reductions."""
    _check_i32(edge_ptr, "edge_ptr")
    _check_i32(src_edges, "src_edges")
    _check_rows_f32(d_out, "d_input")
    for t, n in ((src_norm_degs, "src_norm_degs"), (dst_norm_degs, "dst_norm_degs")):
        if t is not None:
            _check_i32(t, n)
    dev = d_out.device
    n_dst, dim = d_out.size(0), d_out.size(1)
    if mode == AGG_SYMNORM and (src_norm_degs is None or dst_norm_degs is None or src_norm_degs.numel() < int(src_nodes)
                                or dst_norm_degs.numel() < n_dst):
        raise RuntimeError("sym-norm needs src_norm_degs[src_nodes] and dst_norm_degs[n_dst]")
    if edge_ptr.numel() < n_dst + 1:
        raise RuntimeError("edge_ptr is shorter than n_dst + 1")
    if out is None:
        d_x = torch.empty((int(src_nodes), dim), dtype=torch.float32, device=dev)
    else:
        _check_rows_f32(out, "out")
        if out.size(0) < int(src_nodes) or out.size(1) != dim:
            raise RuntimeError("out must be float32[src_nodes, dim]")
        d_x = out
    if transposed is not None:
        if d_self is not None:
            _check_rows_f32(d_self, "d_self")
            if d_self.size(0) != n_dst or d_self.size(1) != dim:
                raise RuntimeError("d_self must be float32[n_dst, dim]")
        ws = _ws(dev)
        rc = lib().fgl_agg_bwd_gather(ws, ctypes.c_int32(mode), _ptr(edge_ptr), _ptr(transposed.t_indptr), _ptr(transposed.t_dst),
                                      _ptr(transposed.hubs), _ptr(src_norm_degs), _ptr(dst_norm_degs), _ptr(d_out),
                                      ctypes.c_int64(d_out.stride(0)), _ptr(d_self),
                                      ctypes.c_int64(d_self.stride(0) if d_self is not None else dim), ctypes.c_int32(dim),
                                      ctypes.c_int32(n_dst), ctypes.c_int32(int(src_nodes)), _ptr(d_x),
                                      ctypes.c_int64(d_x.stride(0)), _ptr(n_dst_dev), _stream(dev))
        _raise(rc, "aggregate_backward (gather)", ws)
        return d_x
    with _on_device(dev):
        if d_self is None:
            rc = lib().fgl_agg_bwd(_ws(dev), ctypes.c_int32(mode), _ptr(edge_ptr), _ptr(src_edges), _ptr(src_norm_degs),
                                   _ptr(dst_norm_degs), _ptr(d_out), ctypes.c_int64(d_out.stride(0)), ctypes.c_int32(dim),
                                   ctypes.c_int32(n_dst), ctypes.c_int32(int(src_nodes)), _ptr(d_x),
                                   ctypes.c_int64(d_x.stride(0)), _ptr(n_dst_dev), _stream(dev))
        else:
            _check_rows_f32(d_self, "d_self")
            if d_self.size(0) != n_dst or d_self.size(1) != dim:
                raise RuntimeError("d_self must be float32[n_dst, dim]")
            rc = lib().fgl_agg_bwd_self(_ws(dev), ctypes.c_int32(mode), _ptr(edge_ptr), _ptr(src_edges), _ptr(src_norm_degs),
                                        _ptr(dst_norm_degs), _ptr(d_out), ctypes.c_int64(d_out.stride(0)), _ptr(d_self),
                                        ctypes.c_int64(d_self.stride(0)), ctypes.c_int32(dim), ctypes.c_int32(n_dst),
                                        ctypes.c_int32(int(src_nodes)), _ptr(d_x), ctypes.c_int64(d_x.stride(0)),
                                        _ptr(n_dst_dev), _stream(dev))
    _raise(rc, "aggregate_backward")
    return d_x


# ------------------------------------------------------------------------------------------------
# element-wise kernels of the training step (no counterpart among the reference's operators)
# ------------------------------------------------------------------------------------------------
def bias_relu_dropout_(y, bias=None, p_drop=0.0, relu=True, rng_seed=None, rng_ctr=0, rng_ctr_dev=None, copy_out=None):
    """In place: y = dropout(relu(y + bias)).  ``rng_ctr_dev`` (int32 CUDA tensor) is added to ``rng_ctr`` on the
    device, so a captured launch draws a new mask per replay.  ``copy_out`` (float32[k, dim], k <= rows, may be a
    column slice) also receives the first k result rows.  Returns ``y``."""
    _check_rows_f32(y, "y")
    if copy_out is not None:
        _check_rows_f32(copy_out, "copy_out")
        if copy_out.size(1) != y.size(1) or copy_out.size(0) > y.size(0):
            raise RuntimeError("copy_out must be float32[k <= rows, dim]")
    if bias is not None:
        _check_f32(bias, "bias")
        if bias.numel() != y.size(1):
            raise RuntimeError("bias must have one entry per column")
    dev = y.device
    with _on_device(dev):
        rc = lib().fgl_bias_relu_dropout(_ptr(y), ctypes.c_int64(y.stride(0)), ctypes.c_int64(y.size(0)), ctypes.c_int32(y.size(1)),
                                         _ptr(bias), ctypes.c_float(p_drop),
                                         ctypes.c_uint64(_config["rng_seed"] if rng_seed is None else rng_seed),
                                         ctypes.c_uint64(rng_ctr), _ptr(rng_ctr_dev), ctypes.c_int32(1 if relu else 0),
                                         _ptr(copy_out), ctypes.c_int64(copy_out.stride(0) if copy_out is not None else 0),
                                         ctypes.c_int64(copy_out.size(0) if copy_out is not None else 0), _stream(dev))
    _raise(rc, "bias_relu_dropout_")
    return y


def relu_dropout_backward_(dy, out=None, p_drop=0.0, dbias=None, masked=True, split3=None, block_stride=None):
    """In place over ``dy``: the gradient through dropout(relu(.)) given the forward output ``out`` (``masked``), and
    ``dbias += column sums`` of the result.  Returns ``dy``.  With ``split3`` (a float32 matrix of ``dy``'s rows) the
    result is written there instead, as ``[hi | lo | hi]`` TF32 parts ``block_stride`` (default: ``dy``'s width) columns
    apart, and ``dy`` is left as it was; returns ``split3``."""
    _check_rows_f32(dy, "dy")
    if masked:
        _check_rows_f32(out, "out")
        if out.shape != dy.shape:
            raise RuntimeError("out and dy must have the same shape")
    if dbias is not None:
        _check_f32(dbias, "dbias")
        if dbias.numel() != dy.size(1):
            raise RuntimeError("dbias must have one entry per column")
    dev = dy.device
    if split3 is not None:
        _check_rows_f32(split3, "split3")
        bs = dy.size(1) if block_stride is None else int(block_stride)
        if split3.size(0) != dy.size(0) or bs < dy.size(1) or split3.size(1) < 2 * bs + dy.size(1):
            raise RuntimeError("split3 must have dy's rows and room for three blocks block_stride columns apart")
        with _on_device(dev):
            rc = lib().fgl_relu_dropout_bwd_split(_ptr(dy), ctypes.c_int64(dy.stride(0)), _ptr(out if masked else None),
                                                  ctypes.c_int64(out.stride(0) if masked else dy.size(1)), ctypes.c_int64(dy.size(0)),
                                                  ctypes.c_int32(dy.size(1)), ctypes.c_float(p_drop), _ptr(dbias),
                                                  ctypes.c_int32(1 if masked else 0), _ptr(split3), ctypes.c_int64(split3.stride(0)),
                                                  ctypes.c_int64(bs), _stream(dev))
        _raise(rc, "relu_dropout_backward_")
        return split3
    with _on_device(dev):
        rc = lib().fgl_relu_dropout_bwd(_ptr(dy), ctypes.c_int64(dy.stride(0)), _ptr(out if masked else None),
                                        ctypes.c_int64(out.stride(0) if masked else dy.size(1)), ctypes.c_int64(dy.size(0)),
                                        ctypes.c_int32(dy.size(1)), ctypes.c_float(p_drop), _ptr(dbias),
                                        ctypes.c_int32(1 if masked else 0), _stream(dev))
    _raise(rc, "relu_dropout_backward_")
    return dy


def softmax_xent(logits, labels, label_ids=None, n_valid=None, loss=None, dlogits=None, row_loss=None):
    """Mean softmax cross-entropy over the first ``n_valid`` rows (an int, an int32 CUDA tensor read on the device, or
    all rows) and its gradient: returns (loss float32[1], dlogits).  ``row_loss`` (float32[n_rows]) is scratch.  Row r's label is ``labels[label_ids[r]]`` when
    ``label_ids`` (int32) is given, else ``labels[r]``; ``labels`` is int64."""
    _check_rows_f32(logits, "logits")
    _check_input(labels, "labels")
    if labels.dtype != torch.int64:
        raise RuntimeError("labels must be int64")
    if label_ids is not None:
        _check_i32(label_ids, "label_ids")
    dev = logits.device
    n_rows, n_classes = logits.size(0), logits.size(1)
    loss = torch.empty(1, dtype=torch.float32, device=dev) if loss is None else loss
    dlogits = torch.empty((n_rows, n_classes), dtype=torch.float32, device=dev) if dlogits is None else dlogits
    _check_rows_f32(dlogits, "dlogits")
    row_loss = torch.empty(max(n_rows, 1), dtype=torch.float32, device=dev) if row_loss is None else row_loss
    _check_f32(row_loss, "row_loss")
    if row_loss.numel() < n_rows:
        raise RuntimeError("row_loss must hold one float per row")
    n_valid_dev = n_valid if torch.is_tensor(n_valid) else None
    if n_valid_dev is not None:
        _check_i32(n_valid_dev, "n_valid")
    ws = _ws(dev)
    with _on_device(dev):
        rc = lib().fgl_softmax_xent(ws, _ptr(logits), ctypes.c_int64(logits.stride(0)), _ptr(labels), _ptr(label_ids),
                                    ctypes.c_int64(labels.numel()), ctypes.c_int32(n_rows), ctypes.c_int32(n_classes),
                                    _ptr(n_valid_dev), ctypes.c_int32(n_rows if n_valid is None or n_valid_dev is not None else int(n_valid)),
                                    _ptr(loss), _ptr(dlogits), ctypes.c_int64(dlogits.stride(0)), _ptr(row_loss), _stream(dev))
    _raise(rc, "softmax_xent", ws)
    return loss, dlogits


def linear_softmax_xent(x, weight, bias, labels, label_ids=None, n_valid=None, loss=None, dlogits=None, row_loss=None,
                        dbias=None, logits=None):
    """``softmax_xent(x @ weight + bias, ...)`` in one pass for at most 128 classes: returns (loss, dlogits); ``dbias``
    (float32[n_classes], zeroed by the caller) also receives the bias gradient and ``logits`` the logits."""
    _check_rows_f32(x, "x")
    _check_rows_f32(weight, "weight")
    if weight.size(0) != x.size(1) or weight.size(1) > 128:
        raise RuntimeError("weight must be float32[x.size(1), n_classes <= 128]")
    _check_input(labels, "labels")
    if labels.dtype != torch.int64:
        raise RuntimeError("labels must be int64")
    for t, n in ((bias, "bias"), (dbias, "dbias")):
        if t is not None:
            _check_f32(t, n)
            if t.numel() != weight.size(1):
                raise RuntimeError(f"{n} must have one entry per class")
    if label_ids is not None:
        _check_i32(label_ids, "label_ids")
    dev = x.device
    n_rows, k, n_classes = x.size(0), x.size(1), weight.size(1)
    loss = torch.empty(1, dtype=torch.float32, device=dev) if loss is None else loss
    dlogits = torch.empty((n_rows, n_classes), dtype=torch.float32, device=dev) if dlogits is None else dlogits
    _check_rows_f32(dlogits, "dlogits")
    row_loss = torch.empty(max(n_rows, 1), dtype=torch.float32, device=dev) if row_loss is None else row_loss
    _check_f32(row_loss, "row_loss")
    if logits is not None:
        _check_rows_f32(logits, "logits")
    if row_loss.numel() < n_rows or dlogits.size(0) < n_rows or (logits is not None and logits.size(0) < n_rows):
        raise RuntimeError("row_loss, dlogits and logits must hold one row per row of x")
    n_valid_dev = n_valid if torch.is_tensor(n_valid) else None
    if n_valid_dev is not None:
        _check_i32(n_valid_dev, "n_valid")
    ws = _ws(dev)
    with _on_device(dev):
        rc = lib().fgl_linear_softmax_xent(
            ws, _ptr(x), ctypes.c_int64(x.stride(0)), ctypes.c_int32(k), _ptr(weight), ctypes.c_int64(weight.stride(0)),
            _ptr(bias), _ptr(labels), _ptr(label_ids), ctypes.c_int64(labels.numel()), ctypes.c_int32(n_rows),
            ctypes.c_int32(n_classes), _ptr(n_valid_dev),
            ctypes.c_int32(n_rows if n_valid is None or n_valid_dev is not None else int(n_valid)), _ptr(loss), _ptr(dlogits),
            ctypes.c_int64(dlogits.stride(0)), _ptr(dbias), _ptr(logits),
            ctypes.c_int64(logits.stride(0) if logits is not None else n_classes), _ptr(row_loss), _stream(dev))
    _raise(rc, "linear_softmax_xent", ws)
    return loss, dlogits


def adam_step_(param, grad, exp_avg, exp_avg_sq, step_dev, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0):
    """One Adam step (torch.optim.Adam's arithmetic, L2 weight decay) over flat float32 buffers, in place.
    ``step_dev``: int32[2] CUDA tensor, zero before the first step; the launch itself advances ``step_dev[0]``."""
    for t, n in ((param, "param"), (grad, "grad"), (exp_avg, "exp_avg"), (exp_avg_sq, "exp_avg_sq")):
        _check_f32(t, n)
        if t.numel() != param.numel():
            raise RuntimeError("param, grad and the two moment buffers must have the same length")
    _check_i32(step_dev, "step_dev")
    if step_dev.numel() < 2:
        raise RuntimeError("step_dev must hold two int32 words")
    dev = param.device
    with _on_device(dev):
        rc = lib().fgl_adam_step(_ptr(param), _ptr(grad), _ptr(exp_avg), _ptr(exp_avg_sq), ctypes.c_int64(param.numel()),
                                 ctypes.c_float(lr), ctypes.c_float(betas[0]), ctypes.c_float(betas[1]), ctypes.c_float(eps),
                                 ctypes.c_float(weight_decay), _ptr(step_dev), _stream(dev))
    _raise(rc, "adam_step_")


def split_tf32(x, dst=None):
    """Error-compensated TF32 operands of a float32 matrix (``fgl_split_tf32``): ``hi`` = ``x`` rounded to TF32, ``lo`` =
    the remainder rounded to TF32.  ``dst``: list of ``(matrix, "hi" | "lo")``, every matrix of ``x``'s shape with unit
    column stride (a block of columns or rows of a wider matrix is fine); without it two new tensors ``(hi, lo)`` are
    returned.  With ``torch.backends.cuda.matmul.allow_tf32`` on, ``[A_hi | A_lo | A_hi] @ [B_hi ; B_hi ; B_lo]`` is the
    product ``A @ B`` to float32-level error on the tensor cores."""
    if x.dim() == 1:
        x = x.view(1, -1)
    _check_rows_f32(x, "x")
    ret = None
    if dst is None:
        ret = (torch.empty_like(x, memory_format=torch.contiguous_format), torch.empty_like(x, memory_format=torch.contiguous_format))
        dst = [(ret[0], "hi"), (ret[1], "lo")]
    if not 1 <= len(dst) <= 8:
        raise RuntimeError("split_tf32 takes 1 to 8 destinations")
    ptrs = (ctypes.c_void_p * len(dst))()
    lds = (ctypes.c_int64 * len(dst))()
    parts = (ctypes.c_int32 * len(dst))()
    for q, (t, part) in enumerate(dst):
        _check_rows_f32(t, f"dst[{q}]")
        if tuple(t.shape) != tuple(x.shape) or t.device != x.device:
            raise RuntimeError("every destination must have x's shape and device")
        if part not in ("hi", "lo"):
            raise RuntimeError("a destination takes the part 'hi' or 'lo'")
        ptrs[q], lds[q], parts[q] = t.data_ptr(), (t.stride(0) if t.size(0) > 1 else max(t.stride(0), t.size(1))), int(part == "lo")
    ldx = x.stride(0) if x.size(0) > 1 else max(x.stride(0), x.size(1))
    dev = x.device
    with _on_device(dev):
        rc = lib().fgl_split_tf32(_ptr(x), ctypes.c_int64(x.size(0)), ctypes.c_int64(x.size(1)), ctypes.c_int64(ldx),
                                  ctypes.c_int(len(dst)), ptrs, lds, parts, _stream(dev))
    _raise(rc, "split_tf32")
    return ret


def fold_blocks(part, n_a, n_b, rows, cols, block_stride, out):
    """``out[r, c] = sum_{s, a, b} part[s, a * rows + r, b * block_stride + c]`` (``fgl_fold_blocks``): ``part`` is a
    contiguous float32 tensor ``[slabs, n_a * rows, width]`` or ``[n_a * rows, width]``."""
    _check_f32(part, "part")
    _check_rows_f32(out, "out")
    if part.dim() == 2:
        part = part.unsqueeze(0)
    if part.dim() != 3 or part.size(1) != n_a * rows or tuple(out.shape) != (rows, cols):
        raise RuntimeError("part must be [slabs, n_a * rows, width] and out [rows, cols]")
    dev = part.device
    with _on_device(dev):
        rc = lib().fgl_fold_blocks(_ptr(part), ctypes.c_int32(part.size(0)), ctypes.c_int32(n_a), ctypes.c_int32(n_b),
                                   ctypes.c_int32(rows), ctypes.c_int32(cols), ctypes.c_int32(block_stride),
                                   ctypes.c_int64(part.size(2)), ctypes.c_int64(part.size(1) * part.size(2)), _ptr(out),
                                   ctypes.c_int64(out.stride(0)), _stream(dev))
    _raise(rc, "fold_blocks")
    return out


def probe_access_pattern(array, table=None, iters=64) -> int:
    """Enqueue the access-pattern probe (``fgl_probe_access_pattern``) on the current stream: isolated 4-byte reads of
    ``array`` (int32 CUDA tensor), each followed by a probe of ``table`` (int64 CUDA tensor, a power of two of zeroed
    slots) when one is given.  Returns the number of accesses the launch performs; time the stream around it."""
    _check_i32(array, "array")
    if table is not None:
        _check_input(table, "table")
        if table.dtype != torch.int64:
            raise RuntimeError("table must be int64")
    dev = array.device
    sink = torch.zeros(1, dtype=torch.int32, device=dev)
    n = ctypes.c_int64(0)
    with _on_device(dev):
        rc = lib().fgl_probe_access_pattern(_ptr(array), ctypes.c_int64(array.numel()), _ptr(table),
                                            ctypes.c_int64(0 if table is None else table.numel()), ctypes.c_int32(iters),
                                            _ptr(sink), ctypes.byref(n), _stream(dev))
    _raise(rc, "probe_access_pattern")
    return int(n.value)


def split_tf32_raw(src_ptr: int, rows: int, cols: int, ldx: int, dst, device) -> None:
    """``split_tf32`` on raw addresses: ``dst`` is a list of ``(address, leading dimension, is_lo)``.  For per-step
    staging, where building tensor views would cost more host time than the launch."""
    n = len(dst)
    ptrs = (ctypes.c_void_p * n)(*[d[0] for d in dst])
    lds = (ctypes.c_int64 * n)(*[d[1] for d in dst])
    parts = (ctypes.c_int32 * n)(*[int(bool(d[2])) for d in dst])
    with _on_device(device):
        rc = lib().fgl_split_tf32(ctypes.c_void_p(src_ptr), ctypes.c_int64(rows), ctypes.c_int64(cols), ctypes.c_int64(ldx),
                                  ctypes.c_int(n), ptrs, lds, parts, _stream(device))
    _raise(rc, "split_tf32_raw")


class PeerSync:
    """The peer-mapped buffers ``allreduce_adam_`` exchanges gradients through (struct fgl_peer_sync).

    ``recv[q]`` / ``flags[q]``: rank q's receive buffer (float32[2 * world * n_pad]) and flag array
    (int32[2 * world * n_chunks]) as CUDA tensors mapped into this process -- this rank's own allocations at index
    ``rank``, the peers' opened over CUDA IPC (``fastgl_b200.sharding.open_peer_tensors``).  All zero before the first
    step."""

    def __init__(self, rank: int, world: int, recv, flags, n: int):
        if world > _capi.MAX_PEERS:
            raise RuntimeError(f"at most {_capi.MAX_PEERS} ranks")
        self.rank, self.world, self.n = int(rank), int(world), int(n)
        self.n_chunks = int(lib().fgl_peer_sync_chunks(ctypes.c_int64(n)))
        self.n_pad = self.n_chunks * 2048
        self.keep = (list(recv), list(flags))
        for t in recv:
            if t.dtype != torch.float32 or t.numel() < 2 * world * self.n_pad:
                raise RuntimeError("receive buffers must be float32[2 * world * n_pad]")
        for t in flags:
            if t.dtype != torch.int32 or t.numel() < 2 * world * self.n_chunks:
                raise RuntimeError("flag arrays must be int32[2 * world * n_chunks]")
        self.c = _capi.PeerSync()
        self.c.rank, self.c.world, self.c.n_pad, self.c.n_chunks = self.rank, self.world, self.n_pad, self.n_chunks
        for q in range(world):
            self.c.recv[q] = recv[q].data_ptr()
            self.c.flags[q] = flags[q].data_ptr()

    @staticmethod
    def sizes(n: int, world: int):
        """(floats of a receive buffer, int32 words of a flag array) for a flat gradient of ``n`` elements."""
        chunks = int(lib().fgl_peer_sync_chunks(ctypes.c_int64(n)))
        return 2 * world * chunks * 2048, 2 * world * chunks


def allreduce_adam_(peers: PeerSync, param, grad, exp_avg, exp_avg_sq, step_dev, lr=1e-3, betas=(0.9, 0.999), eps=1e-8,
                    weight_decay=0.0, spin_limit=4_000_000):
    """Average ``grad`` over the ranks of ``peers`` and apply one Adam step, in one launch (see fgl_allreduce_adam).
    ``step_dev``: int32[3] CUDA tensor, zero before the first step.  The flat buffers hold a multiple of 4 floats."""
    for t, n in ((param, "param"), (grad, "grad"), (exp_avg, "exp_avg"), (exp_avg_sq, "exp_avg_sq")):
        _check_f32(t, n)
        if t.numel() != param.numel():
            raise RuntimeError("param, grad and the two moment buffers must have the same length")
    _check_i32(step_dev, "step_dev")
    if step_dev.numel() < 3 or param.numel() != peers.n:
        raise RuntimeError("step_dev must hold three int32 words and the buffers peers.n floats")
    dev = param.device
    ws = _ws(dev)
    with _on_device(dev):
        rc = lib().fgl_allreduce_adam(ws, ctypes.byref(peers.c), _ptr(param), _ptr(grad), _ptr(exp_avg), _ptr(exp_avg_sq),
                                      ctypes.c_int64(param.numel()), ctypes.c_float(lr), ctypes.c_float(betas[0]),
                                      ctypes.c_float(betas[1]), ctypes.c_float(eps), ctypes.c_float(weight_decay),
                                      _ptr(step_dev), ctypes.c_int64(spin_limit), _stream(dev))
    _raise(rc, "allreduce_adam_", ws)


def forward_gat(edge_ptr, edge_data, src_edges, input_feat, neighbor_num, dst_nodes, num_heads):
    """aggregate_acc.cpp:211-246 -> computation_aware_forward_gat_cuda (aggregate_acc_kernel.cu:789-885).

    ``edge_data`` float32[E, num_heads] holds one attention coefficient per edge and head; head ``h`` owns the
    columns ``[h * dim / num_heads, (h + 1) * dim / num_heads)`` of ``input_feat``.  Returns ``[out]`` with
    ``out[d] = sum_e edge_data[e, head] * input_feat[src[e]]``; a row without in-edges copies its own input row."""
    _check_i32(edge_ptr, "edge_ptr")
    _check_i32(src_edges, "src_edges")
    _check_f32(edge_data, "edge_data")
    _check_f32(input_feat, "input_feat")
    H, dim, n_dst = int(num_heads), input_feat.size(1), int(dst_nodes)
    if edge_data.dim() != 2 or edge_data.size(1) != H or dim % H != 0 or edge_data.size(0) < src_edges.numel():
        raise RuntimeError("edge_data must be [n_edges, num_heads] and num_heads must divide the feature width")
    dev = input_feat.device
    out = torch.empty((n_dst, dim), dtype=torch.float32, device=dev)
    with _on_device(dev):
        rc = lib().fgl_agg_edge_fwd(_ws(dev), _ptr(edge_ptr), _ptr(src_edges), _ptr(edge_data), ctypes.c_int32(H), _ptr(input_feat),
                                    ctypes.c_int32(input_feat.size(0)), ctypes.c_int64(input_feat.stride(0)),
                                    ctypes.c_int32(dim), ctypes.c_int32(n_dst),
                                    ctypes.c_int32(FLAG_ZERO_DEG_PASSTHROUGH), _ptr(out), ctypes.c_int64(dim), _stream(dev))
    _raise(rc, "forward_gat")
    return [out]


def backward_gat(edge_ptr, edge_data, src_edges, d_input, src_nodes, num_heads):
    """aggregate_acc.cpp:248-281 -> computation_aware_backward_gat_cuda (aggregate_acc_kernel.cu:887-979).

    Returns ``[d_x]`` with ``d_x[src[e]] += edge_data[e, head] * d_input[d]``; like the reference, no gradient
    is produced for ``edge_data`` (GraphConv.py:227)."""
    _check_i32(edge_ptr, "edge_ptr")
    _check_i32(src_edges, "src_edges")
    _check_f32(edge_data, "edge_data")
    _check_f32(d_input, "d_input")
    H, dim, n_dst = int(num_heads), d_input.size(1), d_input.size(0)
    if edge_data.dim() != 2 or edge_data.size(1) != H or dim % H != 0:
        raise RuntimeError("edge_data must be [n_edges, num_heads] and num_heads must divide the feature width")
    dev = d_input.device
    d_x = torch.empty((int(src_nodes), dim), dtype=torch.float32, device=dev)
    with _on_device(dev):
        rc = lib().fgl_agg_edge_bwd(_ws(dev), _ptr(edge_ptr), _ptr(src_edges), _ptr(edge_data), ctypes.c_int32(H), _ptr(d_input),
                                    ctypes.c_int64(d_input.stride(0)), ctypes.c_int32(dim), ctypes.c_int32(n_dst),
                                    ctypes.c_int32(int(src_nodes)), _ptr(d_x), ctypes.c_int64(dim), _stream(dev))
    _raise(rc, "backward_gat")
    return [d_x]


def edge_weight_grad(edge_ptr, src_edges, input_feat, d_out, num_heads):
    """Gradient of ``forward_gat`` with respect to ``edge_data`` (not computed by the reference):
    ``d_w[e, h] = <d_out[d, head h], input_feat[src[e], head h]>`` for every edge ``e`` of row ``d``."""
    _check_i32(edge_ptr, "edge_ptr")
    _check_i32(src_edges, "src_edges")
    _check_f32(input_feat, "input_feat")
    _check_f32(d_out, "d_out")
    H, dim, E = int(num_heads), d_out.size(1), src_edges.numel()
    dev = d_out.device
    d_w = torch.empty((E, H), dtype=torch.float32, device=dev)
    with _on_device(dev):
        rc = lib().fgl_agg_edge_wgrad(_ws(dev), _ptr(edge_ptr), _ptr(src_edges), ctypes.c_int32(H), _ptr(input_feat),
                                      ctypes.c_int32(input_feat.size(0)), ctypes.c_int64(input_feat.stride(0)), _ptr(d_out), ctypes.c_int64(d_out.stride(0)),
                                      ctypes.c_int32(dim), ctypes.c_int32(d_out.size(0)), ctypes.c_int64(E), _ptr(d_w),
                                      _stream(dev))
    _raise(rc, "edge_weight_grad")
    return d_w


def forward_gcn(edge_ptr, src_edges, src_norm_degs, dst_norm_degs, input_feat, weight, neighbor_num, dst_nodes):
    """aggregate_acc.cpp:133-160 -> computation_aware_forward_gcn_cuda (aggregate_acc_kernel.cu:223-331).

    ``tmp = input_feat @ weight`` then the sym-normalised neighbour sum; a row without in-edges returns
    ``tmp[row]``.  ``neighbor_num`` only sized the reference's shared memory and is not needed here."""
    _check_f32(weight, "weight")
    _check_f32(input_feat, "input_feat")
    tmp = torch.mm(input_feat, weight)
    return [aggregate(AGG_SYMNORM, edge_ptr, src_edges, tmp, dst_nodes, src_norm_degs, dst_norm_degs)]


def backward_gcn(edge_ptr, src_edges, src_norm_degs, dst_norm_degs, d_input, weight, input_feat):
    """aggregate_acc.cpp:349-376 -> computation_aware_backward_gcn_cuda (aggregate_acc_kernel.cu:430-517).

    The third argument is indexed by the destination row and the fourth by the edge's source -- the
    reference kernel reads them that way (:490,:508) and GraphConv.py:37 passes the degree tensors in
    that (swapped) order.  Returns ``[d_x, d_w]``."""
    _check_f32(weight, "weight")
    _check_f32(input_feat, "input_feat")
    d_out = aggregate_backward(AGG_SYMNORM, edge_ptr, src_edges, d_input, input_feat.size(0),
                               src_norm_degs=dst_norm_degs, dst_norm_degs=src_norm_degs)
    return [torch.mm(d_out, weight.t()), torch.mm(input_feat.t(), d_out)]


def forwaed_gin(edge_ptr, src_edges, input_feat, weight, neighbor_num, dst_nodes):
    """aggregate_acc.cpp:173-199 -> computation_aware_forward_gin_cuda (aggregate_acc_kernel.cu:333-427).

    The name keeps the reference's spelling.  Returns ``[tmp @ weight, tmp]`` with ``tmp`` the plain
    neighbour sum (a row without in-edges copies its own input row)."""
    _check_f32(weight, "weight")
    tmp = aggregate(AGG_SUM, edge_ptr, src_edges, input_feat, dst_nodes)
    return [torch.mm(tmp, weight), tmp]


def backward_gin(edge_ptr, src_edges, d_input, weight, input_feat, src_nodes):
    """aggregate_acc.cpp:387-409 -> computation_aware_backward_gin_cuda (aggregate_acc_kernel.cu:519-596).

    ``input_feat`` is the aggregated ``tmp`` saved by the forward pass (GraphConv.py:117).  Returns
    ``[d_x, d_w]``."""
    _check_f32(weight, "weight")
    _check_f32(input_feat, "input_feat")
    _check_f32(d_input, "d_input")
    d_tmp = torch.mm(d_input, weight.t())
    d_w = torch.mm(input_feat.t(), d_input)
    return [aggregate_backward(AGG_SUM, edge_ptr, src_edges, d_tmp, src_nodes), d_w]


# ------------------------------------------------------------------------------------------------
# fused multi-hop, multi-mini-batch sampling + mapping
# ------------------------------------------------------------------------------------------------
def fused_capacity(n_nodes: int, max_seeds: int, fanouts) -> list[int]:
    """cap_nodes[h] for h = 0 .. len(fanouts) (``fanouts`` in sampling order)."""
    L = len(fanouts)
    fan = (ctypes.c_int32 * L)(*[int(f) for f in fanouts])
    cap = (ctypes.c_int64 * (L + 1))()
    rc = lib().fgl_fused_capacity(ctypes.c_int64(n_nodes), ctypes.c_int32(max_seeds), ctypes.c_int32(L), fan, cap)
    _raise(rc, "fused_capacity")
    return [int(c) for c in cap]


class FusedBatch:
    """Device-resident result of ``sample_map_fused`` for ``n_batches`` mini-batches.

    ``counts[b, h]`` (h = 0 .. L) is the number of nodes after hop h (``counts[b, 0]`` = seeds),
    ``counts[b, 8 + h]`` the number of edges of hop h.  Hop h's block has ``counts[b, h]`` destination
    rows and ``counts[b, h + 1]`` source nodes; ``nodes[b, :counts[b, L]]`` are the global ids, seeds
    first, and the first ``counts[b, h]`` of them are the hop's destinations."""

    def __init__(self, fanouts, nodes, counts, block_indptr, block_src, arena):
        self.fanouts = list(fanouts)
        self.nodes = nodes
        self.counts = counts
        self.block_indptr = block_indptr
        self.block_src = block_src
        self._arena = arena
        self._counts_host = None
        self._counts_pinned = None
        self._status_pinned = None
        self._readback = None
        self.device_status = 0   # the workspace's status word as of the last asynchronous read-back (0 = no error)

    @property
    def n_batches(self) -> int:
        return self.nodes.size(0)

    def start_readback(self) -> None:
        """Enqueue the copy of the counts to pinned host memory on the current stream, without waiting: the next
        ``counts_host()`` waits for that copy only, not for work enqueued after it."""
        dev = self.counts.device
        if self._counts_pinned is None:
            self._counts_pinned = torch.empty(self.counts.shape, dtype=self.counts.dtype).pin_memory()
            self._status_pinned = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._counts_pinned.copy_(self.counts, non_blocking=True)
        ws = _ws(dev)
        _raise(lib().fgl_ws_status_peek(ws, ctypes.c_void_p(self._status_pinned.data_ptr()), _stream(dev)), "status_peek", ws)
        self._readback = torch.cuda.Event()
        self._readback.record(torch.cuda.current_stream(self.counts.device))

    def counts_host(self) -> torch.Tensor:
        if self._counts_host is None:
            if self._readback is not None:
                self._readback.synchronize()
                self._counts_host = self._counts_pinned.clone()
                self.device_status = int(self._status_pinned[0])
                self._readback = None
            else:
                self._counts_host = self.counts.cpu()
            self._counts_list = self._counts_host.tolist()
        return self._counts_host

    def counts_list(self):
        """The counts as nested Python lists (one read-back per window)."""
        self.counts_host()
        return self._counts_list

    def blocks(self, b: int):
        """Blocks of mini-batch ``b``, input layer first (the order FusedMapSampler.sample_blocks returns):
        a list of (indptr[n_dst+1], src_local[E], n_src, n_dst)."""
        c = self.counts_host()[b].tolist()
        L = len(self.fanouts)
        out = []
        for h in reversed(range(L)):
            n_dst, n_src, E = c[h], c[h + 1], c[8 + h]
            out.append((self.block_indptr[h][b, : n_dst + 1], self.block_src[h][b, :E], n_src, n_dst))
        return out

    def input_nodes(self, b: int) -> torch.Tensor:
        return self.nodes[b, : int(self.counts_host()[b, len(self.fanouts)])]


def sample_map_fused(edge_ptr, src_edges, seeds, seed_counts, fanouts, replace=None, arrival_order=None,
                     rng_seed=None, rng_ctr=None, n_teams=0, table_slots=0, out: FusedBatch | None = None,
                     timing=None) -> FusedBatch:
    """All hops of ``seeds.size(0)`` mini-batches in one persistent kernel launch.

    ``seeds`` int32[n_batches, seed_stride], ``seed_counts`` int32[n_batches]; ``fanouts`` in sampling
    order (the reference walks ``reversed(self.fanouts)``, FusedMapSampler.py:72).  Nothing is copied to
    the host; pass ``out`` (a previous result of the same geometry) to reuse its buffers.  ``timing``: a pair of
    ``torch.cuda.Event`` that the library records directly around the kernel launch (``fgl_ws_time_next_launch``)."""
    _check_i32(src_edges, "src_edges")
    _check_input(edge_ptr, "edge_ptr")
    _check_i32(seeds, "seeds")
    _check_i32(seed_counts, "seed_counts")
    if seeds.dim() != 2 or seed_counts.numel() != seeds.size(0):
        raise RuntimeError("seeds must be [n_batches, seed_stride] with one count per batch")
    if edge_ptr.dtype not in (torch.int32, torch.int64):
        raise RuntimeError("edge_ptr must be int32 or int64")
    L = len(fanouts)
    if not 1 <= L <= MAX_HOPS:
        raise RuntimeError(f"1..{MAX_HOPS} hops supported")
    dev = seeds.device
    nb, stride = seeds.size(0), seeds.size(1)
    n_nodes = edge_ptr.numel() - 1
    cap = fused_capacity(n_nodes, stride, fanouts)
    if out is None:
        sizes = [cap[L], COUNTS_STRIDE] + [cap[h] + 1 for h in range(L)] + [cap[h] * int(fanouts[h]) for h in range(L)]
        # 128-byte aligned rows, except the counts rows whose stride the ABI fixes
        sizes = [s if i == 1 else (s + 31) // 32 * 32 for i, s in enumerate(sizes)]
        arena = torch.empty(nb * sum(sizes), dtype=torch.int32, device=dev)
        views, off = [], 0
        for s in sizes:
            views.append(arena[off: off + nb * s].view(nb, s))
            off += nb * s
        out = FusedBatch(fanouts, views[0], views[1], views[2: 2 + L], views[2 + L: 2 + 2 * L], arena)
    out._counts_host = None
    out._readback = None
    a = FusedArgs()
    a.indptr = edge_ptr.data_ptr()
    a.indices = src_edges.data_ptr()
    a.n_nodes = n_nodes
    a.indptr_is_64 = 1 if edge_ptr.dtype == torch.int64 else 0
    a.n_batches = nb
    a.n_hops = L
    for h in range(L):
        a.fanout[h] = int(fanouts[h])
        a.block_indptr[h] = out.block_indptr[h].data_ptr()
        a.block_indptr_stride[h] = out.block_indptr[h].stride(0)
        a.block_src[h] = out.block_src[h].data_ptr()
        a.block_src_stride[h] = out.block_src[h].stride(0)
    use_replace = _config["replace"] if replace is None else replace
    use_arrival = _config["arrival_order"] if arrival_order is None else arrival_order
    a.flags = (FLAG_SAMPLE_REPLACE if use_replace else 0) | (FLAG_MAP_ARRIVAL_ORDER if use_arrival else 0)
    a.n_teams = int(n_teams)
    a.table_slots_hint = int(table_slots)
    a.rng_seed = _config["rng_seed"] if rng_seed is None else rng_seed
    a.rng_ctr = _next_ctr() if rng_ctr is None else rng_ctr
    a.seeds = seeds.data_ptr()
    a.seed_stride = seeds.stride(0)
    a.seed_counts = seed_counts.data_ptr()
    a.nodes = out.nodes.data_ptr()
    a.nodes_stride = out.nodes.stride(0)
    a.counts = out.counts.data_ptr()
    ws = _ws(dev)
    if timing is not None:
        with _on_device(dev):
            _time_next_launch(dev, timing)
    rc = lib().fgl_sample_map_fused(ws, ctypes.byref(a), _stream(dev))
    _raise(rc, "sample_map_fused", ws)
    return out


def window_overlap(nodes, counts, n_nodes, mask, out=None):
    """int32[W, W] pairwise overlap of the node lists ``nodes[b, :counts[b]]`` of a window (W <= 32), computed on the
    device without a read-back.  ``counts``: int32 CUDA tensor (any stride); ``mask``: int32[n_nodes] scratch, zero on
    entry and zero again afterwards."""
    _check_i32(nodes, "nodes")
    _check_i32(mask, "mask")
    if nodes.dim() != 2 or nodes.size(0) > 32 or counts.dtype != torch.int32 or counts.dim() != 1 or counts.numel() != nodes.size(0):
        raise RuntimeError("nodes must be int32[W <= 32, stride] with one int32 count per row")
    if mask.numel() < int(n_nodes):
        raise RuntimeError("mask must hold one word per node")
    dev = nodes.device
    W = nodes.size(0)
    if out is None:
        out = torch.empty((W, W), dtype=torch.int32, device=dev)
    with _on_device(dev):
        rc = lib().fgl_window_overlap(_ptr(nodes), ctypes.c_int64(nodes.stride(0)), ctypes.c_void_p(counts.data_ptr()),
                                      ctypes.c_int64(counts.stride(0)), ctypes.c_int32(W), ctypes.c_int64(int(n_nodes)), _ptr(mask),
                                      _ptr(out), _stream(dev))
    _raise(rc, "window_overlap")
    return out


def stage_segments(copies, words_dst=None, words=()):
    """``copies``: up to 8 ``(dst, src)`` pairs of CUDA tensors (``src.numel()`` elements of a 4-byte dtype are
    copied to the front of ``dst``); ``words`` (up to 8 ints) are written to the int32 tensor ``words_dst``.
    One kernel launch on the current stream."""
    n = len(copies)
    if n > _capi.MAX_SEGMENTS or len(words) > _capi.MAX_SEGMENTS:
        raise RuntimeError("at most 8 copies and 8 words per call")
    segs = (_capi.Segment * max(1, n))()
    dev = None
    for i, (dst, src) in enumerate(copies):
        if dst.element_size() != 4 or src.element_size() != 4 or not dst.is_cuda or not src.is_cuda:
            raise RuntimeError("stage_segments copies 4-byte CUDA tensors")
        if dst.numel() < src.numel() or not src.is_contiguous() or not dst.is_contiguous():
            raise RuntimeError("stage_segments needs contiguous tensors and a destination at least as large as the source")
        segs[i].dst, segs[i].src, segs[i].bytes = dst.data_ptr(), src.data_ptr(), src.numel() * 4
        dev = dst.device
    if words_dst is not None:
        _check_i32(words_dst, "words_dst")
        dev = words_dst.device
    vals = (ctypes.c_int32 * max(1, len(words)))(*[int(w) for w in words])
    with _on_device(dev):
        rc = lib().fgl_stage_segments(segs, ctypes.c_int32(n), _ptr(words_dst), vals, ctypes.c_int32(len(words)), _stream(dev))
    _raise(rc, "stage_segments")


def stage_segments_raw(segments, words_dst_ptr, words, device):
    """``stage_segments`` for callers that already hold raw addresses: ``segments`` is a list of
    ``(dst_ptr, src_ptr, n_bytes)`` (addresses and sizes multiples of 4), ``words`` go to ``words_dst_ptr``.  No
    tensor views are built, which matters when this runs once per training step."""
    n = len(segments)
    if n > _capi.MAX_SEGMENTS or len(words) > _capi.MAX_SEGMENTS:
        raise RuntimeError("at most 8 copies and 8 words per call")
    segs = (_capi.Segment * max(1, n))()
    for i, (d, s_, nbytes) in enumerate(segments):
        segs[i].dst, segs[i].src, segs[i].bytes = d, s_, nbytes
    vals = (ctypes.c_int32 * max(1, len(words)))(*words)
    with _on_device(device):
        rc = lib().fgl_stage_segments(segs, ctypes.c_int32(n), ctypes.c_void_p(words_dst_ptr), vals,
                                      ctypes.c_int32(len(words)), _stream(device))
    _raise(rc, "stage_segments")


def status_str(code: int) -> str:
    return _capi.status_str(code)


def check_status(device=None) -> None:
    """Synchronise and raise if a kernel of this device's workspace recorded an error."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    ws = _ws(dev)
    _raise(lib().fgl_ws_check(ws, _stream(dev)), "device status", ws)

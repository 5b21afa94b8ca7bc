"""Size-independent correctness gates for a sampled window, computed with plain torch on the window's own device.

They restate, without any second implementation of the sampler, what every result of the fused sample + id-map
path must satisfy (the contract of sample.cu:82-95 and id_map.cu:259-383 of the reference):

* the node list of a mini-batch starts with its seeds and holds no id twice;
* hop h's block has one CSR row per node known before the hop, and row d holds ``min(deg(d), fanout)`` edges;
* a row whose node has at most ``fanout`` neighbours is that node's adjacency slice, in order;
* every other edge is an edge of the graph, and (sampling without replacement) no graph edge is picked more
  often than it occurs in the graph;
* local source ids index the node list of the hop.

The gates run at any size (they are what the timing runs check before they report a number).
"""
from __future__ import annotations

import torch


class EdgeKeys:
    """Sorted ``dst * n_nodes + src`` keys of a by-destination CSR, for membership tests.  Built only for graphs
    whose key array fits comfortably (8 bytes per edge plus the sort's scratch)."""

    MAX_EDGES = 400_000_000

    def __init__(self, indptr: torch.Tensor, indices: torch.Tensor):
        self.n_nodes = indptr.numel() - 1
        self.keys = None
        if indices.numel() <= self.MAX_EDGES:
            deg = (indptr[1:] - indptr[:-1]).long()
            dst = torch.repeat_interleave(torch.arange(self.n_nodes, device=indptr.device), deg)
            self.keys = (dst * self.n_nodes + indices.long()).sort().values

    def multiplicity(self, keys: torch.Tensor) -> torch.Tensor:
        lo = torch.searchsorted(self.keys, keys)
        hi = torch.searchsorted(self.keys, keys, right=True)
        return hi - lo


def check_window(fb, indptr: torch.Tensor, indices: torch.Tensor, seeds: torch.Tensor, seed_counts,
                 replace: bool = False, edge_keys: EdgeKeys | None = None) -> dict:
    """Raise AssertionError on the first violated gate; return counters of what was checked.

    ``fb`` is a ``fastgl.FusedBatch``; ``seeds`` / ``seed_counts`` are what was passed to the sampler."""
    L = len(fb.fanouts)
    counts = fb.counts_list()
    deg_all = (indptr[1:] - indptr[:-1]).long()
    checked = {"batches": 0, "edges": 0, "rows": 0, "copied_rows": 0, "membership_edges": 0}
    for b in range(fb.n_batches):
        c = counts[b]
        n_seed = int(seed_counts[b])
        assert c[0] == n_seed, (b, c[0], n_seed)
        nodes = fb.nodes[b, : c[L]].long()
        assert torch.equal(nodes[:n_seed], seeds[b, :n_seed].long()), f"batch {b}: seeds are not first"
        assert bool((nodes >= 0).all()) and bool((nodes < deg_all.numel()).all())
        assert torch.unique(nodes).numel() == nodes.numel(), f"batch {b}: a node id occurs twice"
        for h in range(L):
            n_dst, n_src, n_edges = c[h], c[h + 1], c[8 + h]
            fanout = int(fb.fanouts[h])
            ptr = fb.block_indptr[h][b, : n_dst + 1].long()
            src = fb.block_src[h][b, :n_edges].long()
            assert int(ptr[0]) == 0 and int(ptr[-1]) == n_edges
            row_deg = ptr[1:] - ptr[:-1]
            full_deg = deg_all[nodes[:n_dst]]
            want = full_deg if fanout <= 0 else torch.clamp(full_deg, max=fanout)
            assert torch.equal(row_deg, want), f"batch {b} hop {h}: row lengths differ from min(deg, fanout)"
            if n_edges == 0:
                continue
            assert int(src.min()) >= 0 and int(src.max()) < n_src
            row = torch.repeat_interleave(torch.arange(n_dst, device=src.device), row_deg)
            dst_global = nodes[row]
            src_global = nodes[src]
            # rows copied whole: the adjacency slice itself, in order
            copied = (full_deg <= fanout)[row] if fanout > 0 else torch.ones_like(row, dtype=torch.bool)
            pos = indptr[dst_global].long() + (torch.arange(n_edges, device=src.device) - ptr[row])
            assert torch.equal(src_global[copied], indices[pos[copied]].long()), \
                f"batch {b} hop {h}: a short row is not the adjacency slice"
            checked["copied_rows"] += int((full_deg <= fanout).sum()) if fanout > 0 else n_dst
            picked = ~copied
            if edge_keys is not None and edge_keys.keys is not None and bool(picked.any()):
                keys = dst_global[picked] * edge_keys.n_nodes + src_global[picked]
                uniq, times = torch.unique(keys, return_counts=True)
                mult = edge_keys.multiplicity(uniq)
                assert bool((mult > 0).all()), f"batch {b} hop {h}: a sampled edge is not in the graph"
                if not replace:
                    assert bool((times <= mult).all()), f"batch {b} hop {h}: an edge was picked more often than it exists"
                checked["membership_edges"] += int(picked.sum())
            checked["edges"] += n_edges
            checked["rows"] += n_dst
        checked["batches"] += 1
    return checked


def check_window_aggregation(fb, hop: int, feat: torch.Tensor, buf: torch.Tensor, row_off, tol: float = 1e-5) -> float:
    """The window-level first-layer rows ``[self | mean of neighbours]`` against float64 torch algebra on the same
    device; returns the largest error relative to the largest reference magnitude (must be <= ``tol``)."""
    counts = fb.counts_list()
    D = feat.size(1)
    worst = 0.0
    for b in range(fb.n_batches):
        c = counts[b]
        n_dst, n_edges = c[hop], c[8 + hop]
        nodes = fb.nodes[b, : c[hop + 1]].long()
        ptr = fb.block_indptr[hop][b, : n_dst + 1].long()
        src = fb.block_src[hop][b, :n_edges].long()
        row_deg = ptr[1:] - ptr[:-1]
        row = torch.repeat_interleave(torch.arange(n_dst, device=src.device), row_deg)
        ref = torch.zeros((n_dst, D), dtype=torch.float64, device=feat.device)
        ref.index_add_(0, row, feat[nodes[src]].double())
        ref /= row_deg.clamp(min=1).double().unsqueeze(1)
        got = buf[row_off[b]: row_off[b] + n_dst]
        scale = float(ref.abs().max().clamp(min=1e-30))
        err = float((got[:, D:].double() - ref).abs().max()) / scale
        assert torch.equal(got[:, :D], feat[nodes[:n_dst]]), f"batch {b}: self rows differ"
        assert err <= tol, (b, err)
        worst = max(worst, err)
    return worst

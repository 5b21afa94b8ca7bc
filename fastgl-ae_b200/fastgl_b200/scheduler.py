"""Match-Reorder: order the mini-batches of a window so that consecutive batches share input nodes.

Same greedy chain as the reference (``match_reorder.reorder``, utilis.py:31-62): the match degree of batches
i < j is |nodes_i & nodes_j| / |nodes_j| (stored symmetrically), the chain starts at batch 0 and always moves
to the unvisited batch with the highest match degree to the current one.  The reference keeps one N-sized
boolean mask per step of the whole epoch on the GPU (utilis.py:27-28, train_fastgl.py:305-309); here the
window is bounded and the overlap matrix is one GEMM over the window's masks, chunked over the node range.
A visited batch can never be picked again (the reference zeroes its row and column, which lets an all-zero
row fall back to batch 0).
"""
from __future__ import annotations

import torch


def overlap_matrix(node_lists, n_nodes: int, chunk: int = 1 << 22) -> torch.Tensor:
    """float32[W, W] with entry (i, j) = |nodes_i & nodes_j|; node_lists are int32/int64 id tensors."""
    W = len(node_lists)
    dev = node_lists[0].device
    out = torch.zeros((W, W), dtype=torch.float32, device=dev)
    for lo in range(0, n_nodes, chunk):
        hi = min(n_nodes, lo + chunk)
        mask = torch.zeros((W, hi - lo), dtype=torch.float32, device=dev)
        for i, ids in enumerate(node_lists):
            ids = ids.long()
            sel = ids[(ids >= lo) & (ids < hi)] - lo
            mask[i, sel] = 1.0
        out += mask @ mask.t()
    return out


def greedy_order(overlap: torch.Tensor, sizes: torch.Tensor) -> list[int]:
    """Greedy chain over the match degrees (utilis.py:41-60)."""
    W = overlap.size(0)
    ov = overlap.cpu()
    sz = sizes.cpu().to(torch.float32).clamp(min=1)
    match = torch.zeros((W, W))
    for i in range(W):
        for j in range(i + 1, W):
            match[i, j] = match[j, i] = ov[i, j] / sz[j]
    order, last = [0], 0
    visited = torch.zeros(W, dtype=torch.bool)
    visited[0] = True
    for _ in range(1, W):
        row = match[last].clone()
        row[visited] = -1.0
        last = int(torch.argmax(row))
        visited[last] = True
        order.append(last)
    return order


class MatchReorder:
    """``reorder(node_lists)`` -> the order in which to train the window's batches."""

    def __init__(self, num_nodes: int):
        self.num_nodes = int(num_nodes)

    def reorder(self, node_lists) -> list[int]:
        if len(node_lists) <= 2:
            return list(range(len(node_lists)))
        sizes = torch.tensor([n.numel() for n in node_lists])
        return greedy_order(overlap_matrix(node_lists, self.num_nodes), sizes)

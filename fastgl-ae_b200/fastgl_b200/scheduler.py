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


def overlap_matrix_padded(nodes: torch.Tensor, counts: torch.Tensor, n_nodes: int, chunk: int = 1 << 22) -> torch.Tensor:
    """``overlap_matrix`` for the node lists as the fused sampler leaves them on the device: ``nodes`` int32[W, stride]
    of which only the first ``counts[b]`` entries of row ``b`` are ids (the rest is stale), ``counts`` an integer CUDA
    tensor.  Nothing is read back, so this can be enqueued right behind the sampler."""
    W, stride = nodes.shape
    dev = nodes.device
    valid = torch.arange(stride, device=dev)[None, :] < counts.to(torch.int64)[:, None]
    ids = torch.where(valid, nodes, torch.zeros_like(nodes)).long()
    rows = torch.arange(W, device=dev)[:, None].expand(W, stride)
    out = torch.zeros((W, W), dtype=torch.float32, device=dev)
    for lo in range(0, n_nodes, chunk):
        hi = min(n_nodes, lo + chunk)
        inside = valid & (ids >= lo) & (ids < hi)
        mask = torch.zeros((W, hi - lo), dtype=torch.float32, device=dev)
        # ids are distinct within a row, so every cell receives at most one 1 (entries outside add 0 to column 0)
        mask.index_put_((rows, torch.where(inside, ids - lo, torch.zeros_like(ids))), inside.to(torch.float32), accumulate=True)
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

    def enqueue(self, nodes: torch.Tensor, counts: torch.Tensor, key=0) -> None:
        """Enqueue the overlap computation of a freshly sampled window on the current stream and copy the result to
        pinned host memory, without waiting: whoever later waits for a read-back enqueued after this call (the
        window's counts) finds the matrix there.  ``key`` tells windows in flight apart."""
        if not hasattr(self, "_pinned"):
            self._pinned = {}
        W = nodes.size(0)
        buf = self._pinned.get((key, W))
        if buf is None:
            buf = self._pinned[(key, W)] = torch.zeros((W, W), dtype=torch.float32).pin_memory()
        if nodes.is_cuda and W <= 32:
            import fastgl
            if getattr(self, "_mask", None) is None or self._mask.device != nodes.device:
                self._mask = torch.zeros(self.num_nodes, dtype=torch.int32, device=nodes.device)
            ov = fastgl.window_overlap(nodes, counts, self.num_nodes, self._mask).to(torch.float32)
        else:
            ov = overlap_matrix_padded(nodes, counts, self.num_nodes)
        buf.copy_(ov, non_blocking=True)

    def order(self, sizes, key=0) -> list[int]:
        """The greedy chain for the window whose overlap ``enqueue(..., key)`` produced (its copy must have
        completed: wait for a later read-back of the same stream first).  ``sizes``: the node-list lengths."""
        W = len(sizes)
        if W <= 2:
            return list(range(W))
        return greedy_order(self._pinned[(key, W)], torch.as_tensor(sizes))

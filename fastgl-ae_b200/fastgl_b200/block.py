"""A message-flow block: the bipartite graph of one GNN layer of one mini-batch.

Stand-in for the DGL block that the reference builds with ``dgl.create_block`` (FusedMapSampler.py:102) and
that its layers query with ``num_dst_nodes()``, ``num_src_nodes()`` and ``edges()`` (GraphConv.py:92-98).
Here the block carries the CSR the sampler already produced (``indptr`` over destinations, ``src`` local
source ids), so a layer does not have to rebuild it from a COO list; the COO view is still available for
code written against the reference's block interface.
"""
from __future__ import annotations

import torch


class Block:
    __slots__ = ("indptr", "src", "n_src", "n_dst", "_dst", "n_dst_dev")

    def __init__(self, indptr: torch.Tensor, src: torch.Tensor, n_src: int, n_dst: int, dst: torch.Tensor | None = None,
                 n_dst_dev: torch.Tensor | None = None):
        self.indptr = indptr
        self.src = src
        self.n_src = int(n_src)
        self.n_dst = int(n_dst)
        self._dst = dst
        # Optional int32[1] CUDA tensor with the real destination count; n_dst / n_src are then padded sizes
        # (a block of fixed shape that a captured CUDA graph re-reads for every mini-batch).
        self.n_dst_dev = n_dst_dev

    def num_src_nodes(self) -> int:
        return self.n_src

    def num_dst_nodes(self) -> int:
        return self.n_dst

    def num_edges(self) -> int:
        return int(self.src.numel())

    def edges(self):
        """(src_local, dst_local), both int32, edges grouped by destination in destination order."""
        if self._dst is None:
            deg = (self.indptr[1: self.n_dst + 1] - self.indptr[: self.n_dst]).to(torch.int64)
            self._dst = torch.repeat_interleave(torch.arange(self.n_dst, dtype=torch.int32, device=self.src.device), deg,
                                                output_size=self.src.numel())
        return self.src, self._dst

    def int(self):
        return self

    def to(self, device):
        if self.src.device == torch.device(device):
            return self
        return Block(self.indptr.to(device), self.src.to(device), self.n_src, self.n_dst,
                     None if self._dst is None else self._dst.to(device))

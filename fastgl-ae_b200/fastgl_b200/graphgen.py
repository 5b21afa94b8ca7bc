"""Seeded synthetic graphs standing in for the datasets the reference trains on.

The reference loads Reddit / ogbn-products / ogbn-papers100M / IGB (train_fastgl.py:491-503) and turns the
edge list into a by-destination CSR (train_fastgl.py:219-230: sort by destination, cumulative in-degree).
Here the edge list comes from an R-MAT generator (Chakrabarti et al., 2004) with the same node / edge
counts; the CSR has int64 offsets (the reference's int32 overflows beyond 2^31 edges) and int32 sources.
"""
from __future__ import annotations

import math

import torch


def rmat_edges(n_nodes: int, n_edges: int, a: float = 0.57, b: float = 0.19, c: float = 0.19, seed: int = 12345,
               device="cpu", chunk: int = 1 << 25):
    """``n_edges`` directed R-MAT edges (src, dst) as int64 tensors; ids folded mod ``n_nodes``,
    self-loops dropped (so slightly fewer edges come back), duplicates kept."""
    scale = max(1, math.ceil(math.log2(max(2, n_nodes))))
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    srcs, dsts = [], []
    done = 0
    while done < n_edges:
        m = min(chunk, n_edges - done)
        src = torch.zeros(m, dtype=torch.int64, device=device)
        dst = torch.zeros(m, dtype=torch.int64, device=device)
        for _ in range(scale):
            u = torch.rand(m, generator=gen, device=device)
            src_bit = (u >= a + b)
            dst_bit = ((u >= a) & (u < a + b)) | (u >= a + b + c)
            src = (src << 1) | src_bit.to(torch.int64)
            dst = (dst << 1) | dst_bit.to(torch.int64)
        src %= n_nodes
        dst %= n_nodes
        keep = src != dst
        srcs.append(src[keep])
        dsts.append(dst[keep])
        done += m
    return torch.cat(srcs), torch.cat(dsts)


def build_csr(n_nodes: int, src: torch.Tensor, dst: torch.Tensor):
    """By-destination CSR: ``indptr`` int64[n_nodes+1], ``indices`` int32 = sources sorted by destination
    (stable, so equal destinations keep edge-list order), as train_fastgl.py:219-230 builds it."""
    order = torch.argsort(dst, stable=True)
    indices = src[order].to(torch.int32)
    deg = torch.bincount(dst, minlength=n_nodes)
    indptr = torch.zeros(n_nodes + 1, dtype=torch.int64, device=dst.device)
    torch.cumsum(deg, 0, out=indptr[1:])
    return indptr, indices


def rmat_graph(n_nodes: int, avg_degree: float, seed: int = 12345, device="cpu", a=0.57, b=0.19, c=0.19):
    """Symmetrised R-MAT graph with about ``n_nodes * avg_degree`` directed edges -> (indptr, indices)."""
    n_und = int(n_nodes * avg_degree / 2)
    src, dst = rmat_edges(n_nodes, n_und, a, b, c, seed, device)
    s2 = torch.cat([src, dst])
    d2 = torch.cat([dst, src])
    del src, dst
    return build_csr(n_nodes, s2, d2)


def synthetic_node_data(n_nodes: int, feat_dim: int, n_classes: int, train_frac: float, seed: int = 12345,
                        device="cpu"):
    """fp32 N(0,1) features, uniform labels and a random training subset (sorted ids, int32)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed + 1)
    feat = torch.randn((n_nodes, feat_dim), generator=gen, device=device, dtype=torch.float32)
    labels = torch.randint(0, n_classes, (n_nodes,), generator=gen, device=device, dtype=torch.int64)
    n_train = max(1, int(n_nodes * train_frac))
    train = torch.randperm(n_nodes, generator=gen, device=device)[:n_train].sort().values.to(torch.int32)
    return feat, labels, train

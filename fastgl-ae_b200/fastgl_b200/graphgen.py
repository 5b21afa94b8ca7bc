"""Seeded synthetic graphs standing in for the datasets the reference trains on.

The reference loads Reddit / ogbn-products / ogbn-papers100M / IGB (train_fastgl.py:491-503) and turns the
edge list into a by-destination CSR (train_fastgl.py:219-230: sort by destination, cumulative in-degree).
Here the edge list comes from an R-MAT generator (Chakrabarti et al., 2004) with the same node / edge
counts; the CSR has int64 offsets (the reference's int32 overflows beyond 2^31 edges) and int32 sources.
"""
from __future__ import annotations

import math

import torch


def _rmat_chunk(n_nodes: int, m: int, a: float, b: float, c: float, seed: int, device):
    """``m`` R-MAT (src, dst) pairs from their own generator; ids folded mod ``n_nodes``, self-loops dropped."""
    scale = max(1, math.ceil(math.log2(max(2, n_nodes))))
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
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
    return src[keep], dst[keep]


def rmat_edges(n_nodes: int, n_edges: int, a: float = 0.57, b: float = 0.19, c: float = 0.19, seed: int = 12345,
               device="cpu", chunk: int = 1 << 25):
    """``n_edges`` directed R-MAT edges (src, dst) as int64 tensors (slightly fewer come back: self-loops are
    dropped); duplicates kept.  Chunk ``i`` draws from a generator seeded ``seed * 1000003 + i``."""
    srcs, dsts = [], []
    for i, lo in enumerate(range(0, n_edges, chunk)):
        s, d = _rmat_chunk(n_nodes, min(chunk, n_edges - lo), a, b, c, seed * 1000003 + i, device)
        srcs.append(s)
        dsts.append(d)
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


def rmat_graph(n_nodes: int, avg_degree: float, seed: int = 12345, device="cpu", a=0.57, b=0.19, c=0.19,
               chunk: int = 1 << 25):
    """Symmetrised R-MAT graph with about ``n_nodes * avg_degree`` directed edges -> (indptr int64, indices int32).

    Built chunk by chunk in two passes over the same seeded chunks (count degrees, then place edges), so that
    graphs with billions of edges never need a global sort: per chunk the pairs and their reverses are sorted by
    destination and written behind a per-node cursor.  Within a node's list the order is chunk order, then
    forward edges before reverse edges, then generation order."""
    n_pairs = int(n_nodes * avg_degree / 2)
    chunks = [(i, min(chunk, n_pairs - lo)) for i, lo in enumerate(range(0, n_pairs, chunk))]
    deg = torch.zeros(n_nodes, dtype=torch.int64, device=device)
    for i, m in chunks:
        s, d = _rmat_chunk(n_nodes, m, a, b, c, seed * 1000003 + i, device)
        deg += torch.bincount(d, minlength=n_nodes) + torch.bincount(s, minlength=n_nodes)
    indptr = torch.zeros(n_nodes + 1, dtype=torch.int64, device=device)
    torch.cumsum(deg, 0, out=indptr[1:])
    del deg
    indices = torch.empty(int(indptr[-1]), dtype=torch.int32, device=device)
    cursor = torch.zeros(n_nodes, dtype=torch.int64, device=device)
    for i, m in chunks:
        s, d = _rmat_chunk(n_nodes, m, a, b, c, seed * 1000003 + i, device)
        d2 = torch.cat([d, s])
        s2 = torch.cat([s, d])
        del s, d
        key, order = torch.sort(d2, stable=True)
        src_sorted = s2[order].to(torch.int32)
        del d2, s2, order
        uniq, counts = torch.unique_consecutive(key, return_counts=True)
        run_start = torch.cumsum(counts, 0) - counts
        rank = torch.arange(key.numel(), device=device) - torch.repeat_interleave(run_start, counts, output_size=key.numel())
        indices[indptr[key] + cursor[key] + rank] = src_sorted
        cursor[uniq] += counts
        del key, src_sorted, uniq, counts, run_start, rank
    return indptr, indices


def relabel_by_degree(indptr: torch.Tensor, indices: torch.Tensor, chunk_edges: int = 1 << 27):
    """Renumber the nodes by descending in-degree (ties by old id): new node ``i`` is old node ``order[i]``.

    The reference ranks nodes by degree to choose what its GPU feature cache holds (``sort_degree``, utilis.py:86-89;
    ``pre_sample`` :64-74 ranks by sampling frequency for the same purpose).  With the whole table resident in HBM
    the same ranking becomes a layout: the rows that most sampled edges request are packed at the front of the table
    (a few megabytes that stay in L2 and in a handful of TLB entries), and so are their adjacency lists.
    Returns ``(indptr, indices, order, new_of_old)``; per-node arrays move with ``x[order]``, node ids with
    ``new_of_old[ids]``.  Adjacency lists keep their order."""
    n = indptr.numel() - 1
    dev = indptr.device
    deg = indptr[1:] - indptr[:-1]
    order = torch.argsort(deg, descending=True, stable=True)
    new_of_old = torch.empty(n, dtype=torch.int64, device=dev)
    new_of_old[order] = torch.arange(n, device=dev)
    new_deg = deg[order]
    new_indptr = torch.zeros(n + 1, dtype=indptr.dtype, device=dev)
    torch.cumsum(new_deg, 0, out=new_indptr[1:])
    old_start = indptr[:-1][order]
    new_indices = torch.empty_like(indices)
    map32 = new_of_old.to(indices.dtype)
    lo = 0
    bounds = new_indptr.cpu()
    while lo < n:   # node ranges of at most chunk_edges edges (a single node with more edges forms its own range)
        hi = int(torch.searchsorted(bounds, bounds[lo] + chunk_edges, right=True)) - 1
        hi = min(n, max(hi, lo + 1))
        e0, e1 = int(bounds[lo]), int(bounds[hi])
        if e1 > e0:
            shift = torch.repeat_interleave(old_start[lo:hi] - new_indptr[lo:hi], new_deg[lo:hi], output_size=e1 - e0)
            pos = torch.arange(e0, e1, device=dev) + shift
            new_indices[e0:e1] = map32[indices[pos].long()]
            del shift, pos
        lo = hi
    return new_indptr, new_indices, order, new_of_old


def synthetic_node_data(n_nodes: int, feat_dim: int, n_classes: int, train_frac: float, seed: int = 12345,
                        device="cpu"):
    """fp32 N(0,1) features, uniform labels and a random training subset (sorted ids, int32)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed + 1)
    feat = torch.empty((n_nodes, feat_dim), dtype=torch.float32, device=device)
    rows = max(1, (1 << 28) // max(1, feat_dim))          # fill in slabs of about 1 GiB
    for lo in range(0, n_nodes, rows):
        feat[lo: lo + rows].normal_(generator=gen)
    labels = torch.randint(0, n_classes, (n_nodes,), generator=gen, device=device, dtype=torch.int64)
    n_train = max(1, int(n_nodes * train_frac))
    train = torch.randperm(n_nodes, generator=gen, device=device)[:n_train].sort().values.to(torch.int32)
    return feat, labels, train

"""CPU oracle (numpy / plain Python) for the FastGL per-mini-batch hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import this
module; it is the checker that the CUDA kernels are compared against, and
the timed CPU baseline.  PARITY UNPINNED: the reference ships no tests,
golden vectors or CPU implementation, so this restatement is derived from
the reference's CUDA kernel sources alone (cited per function below) and is
cross-checked only against the independent C restatement in
``fgl_oracle.c`` and a handful of hand-derived cases.

Every function is a sequential restatement of what the reference kernels
compute when their threads are executed one after another in index order:

* ``sample``            cuda_operators/sample.cu:17-38 (counts), :82-95 (copy / random)
* ``map_edges``         cuda_operators/id_map.cu:179-255 (table), :259-383 (four passes)
* ``cal_deg``           cuda_operators/utilis.cu:43-79
* ``exclusive_sum``     cuda_operators/utilis.cu:17-41
* ``forward_gcn``       cuda_operators/aggregate_acc_kernel.cu:223-331
* ``backward_gcn``      cuda_operators/aggregate_acc_kernel.cu:430-517
* ``forward_gin``       cuda_operators/aggregate_acc_kernel.cu:333-427
* ``backward_gin``      cuda_operators/aggregate_acc_kernel.cu:519-596
* ``aggregate_edge_fwd / _bwd``  cuda_operators/aggregate_acc_kernel.cu:789-979 (GAT)

Where the reference leaves a result to thread arrival order (the order of
the non-seed unique nodes, id_map.cu:317-320) the oracle takes the order a
sequential execution gives: first occurrence in edge order.

Random numbers: the reference draws ``curand(&state) % deg`` from a cuRAND
Philox4_32_10 state seeded with the thread id (sample.cu:69-70,91).  The
library instead keys a Philox4x32-10 block on (user seed, call counter,
seed slot, pick slot); the oracle restates that keyed generator (the
published Philox algorithm of Salmon et al., SC'11) so that random-mode
picks can be compared element for element.
"""
from __future__ import annotations

import numpy as np

MASK32 = 0xFFFFFFFF
PHILOX_M0 = 0xD2511F53
PHILOX_M1 = 0xCD9E8D57
PHILOX_W0 = 0x9E3779B9
PHILOX_W1 = 0xBB67AE85

MODE_SUM = 0       # plain sum (the reference's GIN aggregation)
MODE_MEAN = 1      # sum / in-degree (GraphSAGE-mean; additive, not in the reference)
MODE_SYMNORM = 2   # sum * rsqrt(deg_dst) * rsqrt(deg_src) (the reference's GCN aggregation)


# --------------------------------------------------------------------------
# Philox4x32-10
# --------------------------------------------------------------------------
def philox4x32_10(ctr, key):
    """One Philox4x32-10 block.  ``ctr``: 4 uint32, ``key``: 2 uint32 -> 4 uint32."""
    c0, c1, c2, c3 = (int(x) & MASK32 for x in ctr)
    k0, k1 = (int(x) & MASK32 for x in key)
    for _ in range(10):
        p0 = PHILOX_M0 * c0
        p1 = PHILOX_M1 * c2
        hi0, lo0 = p0 >> 32, p0 & MASK32
        hi1, lo1 = p1 >> 32, p1 & MASK32
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & MASK32, lo1, (hi0 ^ c3 ^ k1) & MASK32, lo0
        k0 = (k0 + PHILOX_W0) & MASK32
        k1 = (k1 + PHILOX_W1) & MASK32
    return c0, c1, c2, c3


def draw(rng_seed: int, rng_ctr: int, seed_slot: int, pick_slot: int) -> int:
    """The 32-bit random word for pick ``pick_slot`` of seed position ``seed_slot``.

    key = (lo32(rng_seed), hi32(rng_seed)); counter = (pick_slot // 4, seed_slot,
    lo32(rng_ctr), hi32(rng_ctr)); output word ``pick_slot % 4`` of the block is used,
    so one block serves four picks.
    """
    key = (rng_seed & MASK32, (rng_seed >> 32) & MASK32)
    ctr = (pick_slot >> 2, seed_slot, rng_ctr & MASK32, (rng_ctr >> 32) & MASK32)
    return philox4x32_10(ctr, key)[pick_slot & 3]


def bounded(r: int, n: int) -> int:
    """Map a 32-bit word onto [0, n) by the high half of the 64-bit product."""
    return (r * n) >> 32


# --------------------------------------------------------------------------
# a1: neighbour sampling   (sample.cu:17-38, 82-95)
# --------------------------------------------------------------------------
def sample(indptr, indices, seeds, fanout, replace=False, rng_seed=0, rng_ctr=0):
    """Per-seed fanout sampling over a by-destination CSR.

    For seed ``s`` with degree ``deg``: ``k = min(deg, fanout)`` edges are
    emitted.  ``deg <= fanout`` copies the adjacency list in CSR order
    (sample.cu:82-87).  Otherwise ``k`` picks are drawn: with
    ``replace=True`` each pick is an independent uniform offset (the
    reference's behaviour, sample.cu:88-94); with ``replace=False`` the
    picks are a uniform k-subset chosen by Floyd's algorithm.

    Returns (block_indptr int32[S+1], src_global int32[E], dst_global int32[E]).
    """
    indptr = np.asarray(indptr)
    indices = np.asarray(indices)
    seeds = np.asarray(seeds)
    S = int(seeds.shape[0])
    out_ptr = np.zeros(S + 1, dtype=np.int32)
    src, dst = [], []
    for s in range(S):
        v = int(seeds[s])
        start = int(indptr[v])
        deg = int(indptr[v + 1]) - start
        k = min(deg, fanout)
        if deg <= fanout:
            picks = list(range(deg))
        elif replace:
            picks = [bounded(draw(rng_seed, rng_ctr, s, i), deg) for i in range(k)]
        else:
            picks = []
            for i in range(k):
                j = deg - k + i
                t = bounded(draw(rng_seed, rng_ctr, s, i), j + 1)
                picks.append(j if t in picks else t)
        for p in picks:
            src.append(int(indices[start + p]))
            dst.append(v)
        out_ptr[s + 1] = out_ptr[s] + k
    return out_ptr, np.asarray(src, dtype=np.int32), np.asarray(dst, dtype=np.int32)


# --------------------------------------------------------------------------
# a2: Fused-Map id mapping   (id_map.cu:259-383)
# --------------------------------------------------------------------------
def map_edges(src_global, dst_global, seeds):
    """Relabel sampled edges to block-local ids.

    Pass 1 (id_map.cu:259-287): seed ``i`` is inserted with local id ``i``
    (a repeated seed keeps the id of its last position, as a sequential
    run of ``atomicExch`` would leave it).  Pass 2 (:290-322): every edge
    source is inserted; a key that was not present gets the next local id
    ``S + rank`` in first-occurrence order.  Pass 3/4 (:325-383): both
    endpoint arrays are rewritten with the local ids.

    Returns (src_local int32[E], dst_local int32[E], unique int32[S+U]).
    """
    seeds = np.asarray(seeds)
    S = int(seeds.shape[0])
    table = {}
    unique = []
    for i in range(S):
        table[int(seeds[i])] = i
        unique.append(int(seeds[i]))
    for g in np.asarray(src_global).tolist():
        if g not in table:
            table[g] = len(unique)
            unique.append(g)
    src_local = np.asarray([table[g] for g in np.asarray(src_global).tolist()], dtype=np.int32)
    dst_local = np.asarray([table[g] for g in np.asarray(dst_global).tolist()], dtype=np.int32)
    return src_local, dst_local, np.asarray(unique, dtype=np.int32)


def sample_blocks(indptr, indices, seeds, fanouts, replace=False, rng_seed=0, rng_ctr=0):
    """The multi-hop loop of FusedMapSampler.sample_blocks (FusedMapSampler.py:63-109).

    Hops walk ``reversed(fanouts)``; the unique-node list of one hop is the
    seed list of the next; blocks are returned input-layer first.  Hop ``h``
    (0 = nearest the seeds) uses call counter ``rng_ctr + h``.

    Returns (input_nodes, output_nodes, blocks) with each block a dict
    {indptr, src_local, n_src, n_dst}.
    """
    seeds = np.asarray(seeds, dtype=np.int32)
    cur = seeds
    blocks = []
    for h, fanout in enumerate(reversed(list(fanouts))):
        ptr, src_g, dst_g = sample(indptr, indices, cur, fanout, replace, rng_seed, rng_ctr + h)
        src_l, dst_l, uniq = map_edges(src_g, dst_g, cur)
        blocks.insert(0, dict(indptr=ptr, src_local=src_l, dst_local=dst_l,
                              n_src=int(uniq.shape[0]), n_dst=int(cur.shape[0])))
        cur = uniq
    return cur, seeds, blocks


# --------------------------------------------------------------------------
# a3: block-CSR helpers   (utilis.cu:17-79)
# --------------------------------------------------------------------------
def cal_deg(ids, nodes_num):
    """Histogram of an id array (utilis.cu:43-58)."""
    return np.bincount(np.asarray(ids, dtype=np.int64), minlength=nodes_num).astype(np.int32)[:nodes_num]


def exclusive_sum(degs):
    """Exclusive scan with the total appended: int32[n+1] (utilis.cu:17-41)."""
    out = np.zeros(len(degs) + 1, dtype=np.int64)
    np.cumsum(np.asarray(degs, dtype=np.int64), out=out[1:])
    return out.astype(np.int32)


# --------------------------------------------------------------------------
# a4-a7: aggregation   (aggregate_acc_kernel.cu)
# --------------------------------------------------------------------------
def _edge_weight(mode, d, s, src_deg, dst_deg, indptr):
    if mode == MODE_SUM:
        return 1.0
    if mode == MODE_MEAN:
        return 1.0 / float(int(indptr[d + 1]) - int(indptr[d]))
    # fp32 1/sqrtf on each side, then an fp32 product (aggregate_acc_kernel.cu:300,321)
    a = np.float32(1.0) / np.sqrt(np.float32(dst_deg[d]))
    b = np.float32(1.0) / np.sqrt(np.float32(src_deg[s]))
    return float(np.float32(a * b))


def aggregate_fwd(mode, indptr, src, x, n_dst, src_deg=None, dst_deg=None,
                  zero_deg_passthrough=True, row_map=None):
    """out[d,:] = sum_e w(d, src[e]) * x[row(src[e]),:]; float64 accumulation.

    A destination without in-edges copies its own input row when
    ``zero_deg_passthrough`` (aggregate_acc_kernel.cu:307-308, :405-406),
    else stays zero.  ``row_map`` (optional) maps a block-local id to the
    row of ``x`` that holds it (aggregation straight from a feature table).
    """
    x = np.asarray(x)
    D = x.shape[1]
    out = np.zeros((n_dst, D), dtype=np.float64)
    row = (lambda i: int(row_map[i])) if row_map is not None else (lambda i: int(i))
    for d in range(n_dst):
        a, b = int(indptr[d]), int(indptr[d + 1])
        if a == b:
            if zero_deg_passthrough:
                out[d] = x[row(d)]
            continue
        for e in range(a, b):
            s = int(src[e])
            out[d] += _edge_weight(mode, d, s, src_deg, dst_deg, indptr) * x[row(s)].astype(np.float64)
    return out


def aggregate_bwd(mode, indptr, src, dy, n_src, src_deg=None, dst_deg=None):
    """dx[s,:] += w(d, s) * dy[d,:] for every edge (d, s); float64 accumulation.

    A destination without in-edges contributes nothing
    (aggregate_acc_kernel.cu:498-500, :580-582), although the forward pass
    copied its input row.
    """
    dy = np.asarray(dy)
    n_dst, D = dy.shape
    dx = np.zeros((n_src, D), dtype=np.float64)
    for d in range(n_dst):
        for e in range(int(indptr[d]), int(indptr[d + 1])):
            s = int(src[e])
            dx[s] += _edge_weight(mode, d, s, src_deg, dst_deg, indptr) * dy[d].astype(np.float64)
    return dx


def aggregate_edge_fwd(indptr, src, edge_w, x, n_dst, zero_deg_passthrough=True):
    """out[d, f] = sum_e edge_w[e, head(f)] * x[src[e], f], head(f) = f // (dim / heads)
    (aggregate_acc_kernel.cu:836-885; a row without in-edges copies its own input row, :870-872)."""
    x = np.asarray(x)
    edge_w = np.asarray(edge_w)
    D, H = x.shape[1], edge_w.shape[1]
    head = np.arange(D) // (D // H)
    out = np.zeros((n_dst, D), dtype=np.float64)
    for d in range(n_dst):
        a, b = int(indptr[d]), int(indptr[d + 1])
        if a == b:
            if zero_deg_passthrough:
                out[d] = x[d]
            continue
        for e in range(a, b):
            out[d] += edge_w[e, head].astype(np.float64) * x[int(src[e])].astype(np.float64)
    return out


def aggregate_edge_bwd(indptr, src, edge_w, dy, n_src):
    """dx[src[e], f] += edge_w[e, head(f)] * dy[d, f] (aggregate_acc_kernel.cu:925-979); no gradient to edge_w."""
    dy = np.asarray(dy)
    edge_w = np.asarray(edge_w)
    n_dst, D = dy.shape
    head = np.arange(D) // (D // edge_w.shape[1])
    dx = np.zeros((n_src, D), dtype=np.float64)
    for d in range(n_dst):
        for e in range(int(indptr[d]), int(indptr[d + 1])):
            dx[int(src[e])] += edge_w[e, head].astype(np.float64) * dy[d].astype(np.float64)
    return dx


def forward_gcn(edge_ptr, src_edges, src_norm_degs, dst_norm_degs, input_feat, weight, dst_nodes):
    """tmp = X W, then the sym-normalised sum (aggregate_acc_kernel.cu:237, 271-331)."""
    tmp = np.asarray(input_feat, dtype=np.float64) @ np.asarray(weight, dtype=np.float64)
    return aggregate_fwd(MODE_SYMNORM, edge_ptr, src_edges, tmp, dst_nodes, src_norm_degs, dst_norm_degs)


def backward_gcn(edge_ptr, src_edges, dst_deg_of_rows, src_deg_of_cols, d_input, weight, input_feat):
    """Scatter, then d_x = d_out W^T and d_w = X^T d_out (aggregate_acc_kernel.cu:430-517).

    Argument order follows the call site, GraphConv.py:37, which passes the
    destination degrees third and the source degrees fourth.
    """
    n_src = np.asarray(input_feat).shape[0]
    d_out = aggregate_bwd(MODE_SYMNORM, edge_ptr, src_edges, d_input, n_src, src_deg_of_cols, dst_deg_of_rows)
    w = np.asarray(weight, dtype=np.float64)
    return d_out @ w.T, np.asarray(input_feat, dtype=np.float64).T @ d_out


def forward_gin(edge_ptr, src_edges, input_feat, weight, dst_nodes):
    """tmp = plain neighbour sum, out = tmp W (aggregate_acc_kernel.cu:333-427)."""
    tmp = aggregate_fwd(MODE_SUM, edge_ptr, src_edges, input_feat, dst_nodes)
    return tmp @ np.asarray(weight, dtype=np.float64), tmp


def backward_gin(edge_ptr, src_edges, d_input, weight, saved_tmp, src_nodes):
    """d_tmp = d_in W^T, d_w = tmp^T d_in, scatter d_tmp (aggregate_acc_kernel.cu:519-596)."""
    d_in = np.asarray(d_input, dtype=np.float64)
    d_tmp = d_in @ np.asarray(weight, dtype=np.float64).T
    d_w = np.asarray(saved_tmp, dtype=np.float64).T @ d_in
    return aggregate_bwd(MODE_SUM, edge_ptr, src_edges, d_tmp, src_nodes), d_w

"""The hot path at the full sizes of the timed workloads, checked through size-independent gates (the CPU oracle
would need minutes there): seeds first, no repeated node, row lengths ``min(deg, fanout)``, short rows equal to the
adjacency slice, every sampled edge a graph edge picked at most as often as it exists, and the window-level
aggregation within 1e-5 of float64 torch algebra."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def products_like():
    from checks import EdgeKeys
    from fastgl_b200.graphgen import rmat_graph
    dev = torch.device("cuda", 0)
    indptr, indices = rmat_graph(2_450_000, 50.6, seed=12345, device=dev)
    keys = EdgeKeys(indptr, indices)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1)
    feat = torch.randn((2_450_000, 100), generator=gen, device=dev)
    return indptr, indices, keys, feat


@pytest.mark.parametrize("replace", [False, True])
def test_products_sized_window_passes_every_gate(products_like, replace):
    import fastgl
    from checks import check_window, check_window_aggregation
    indptr, indices, keys, feat = products_like
    dev = feat.device
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)
    nb, batch = 8, 1024
    seeds = torch.randperm(indptr.numel() - 1, generator=gen, device=dev)[: nb * batch].to(torch.int32).view(nb, batch)
    counts = torch.full((nb,), batch, dtype=torch.int32, device=dev)
    counts[-1] = 700                                            # a short last batch
    fanouts = [5, 10, 15]                                       # sampling order of the [15, 10, 5] model
    fb = fastgl.sample_map_fused(indptr, indices, seeds, counts, fanouts, replace=replace, rng_seed=12345, rng_ctr=0)
    fastgl.check_status()
    seen = check_window(fb, indptr, indices, seeds, counts.tolist(), replace=replace, edge_keys=keys)
    assert seen["batches"] == nb and seen["edges"] > 2_000_000 and seen["membership_edges"] > 500_000
    if not replace:
        hop = len(fanouts) - 1
        total = int(fb.counts_host()[:, hop].sum())
        D = feat.size(1)
        buf = torch.empty((total, 2 * D), dtype=torch.float32, device=dev)
        row_off = fastgl.aggregate_window(fastgl.AGG_MEAN, fb, hop, feat, buf[:, D:], self_out=buf[:, :D])
        assert check_window_aggregation(fb, hop, feat, buf, row_off) <= 1e-5


def test_sampling_is_reproducible_and_counter_dependent_at_full_size(products_like):
    import fastgl
    indptr, indices, _, feat = products_like
    dev = feat.device
    seeds = torch.arange(0, 2 * 1024 * 997, 997, dtype=torch.int32, device=dev).view(2, 1024)
    counts = torch.full((2,), 1024, dtype=torch.int32, device=dev)
    runs = [fastgl.sample_map_fused(indptr, indices, seeds, counts, [5, 10, 15], rng_seed=12345, rng_ctr=c) for c in (0, 0, 16)]
    a, b, c = runs
    assert torch.equal(a.counts, b.counts) and torch.equal(a.nodes[0, : int(a.counts[0, 3])], b.nodes[0, : int(b.counts[0, 3])])
    for h in range(3):
        n = int(a.counts[1, 8 + h])
        assert torch.equal(a.block_src[h][1, :n], b.block_src[h][1, :n])
    assert not torch.equal(a.counts, c.counts) or not torch.equal(a.nodes, c.nodes)


def test_dense_graph_wide_fanout_window_passes_every_gate():
    """The shapes of the 2-layer GCN workload: average degree ~490, fanouts [25, 10]."""
    import fastgl
    from checks import EdgeKeys, check_window
    from fastgl_b200.graphgen import rmat_graph
    dev = torch.device("cuda", 0)
    indptr, indices = rmat_graph(233_000, 490.0, seed=12345, device=dev)
    keys = EdgeKeys(indptr, indices)
    gen = torch.Generator(device=dev)
    gen.manual_seed(3)
    seeds = torch.randperm(233_000, generator=gen, device=dev)[: 4 * 1024].to(torch.int32).view(4, 1024)
    counts = torch.full((4,), 1024, dtype=torch.int32, device=dev)
    fb = fastgl.sample_map_fused(indptr, indices, seeds, counts, [10, 25], rng_seed=12345, rng_ctr=0)
    fastgl.check_status()
    seen = check_window(fb, indptr, indices, seeds, counts.tolist(), edge_keys=keys)
    assert seen["batches"] == 4 and seen["membership_edges"] > 100_000


def test_int64_offsets_beyond_two_to_the_31_edges():
    """A CSR with more than 2^31 edges, which the reference's int32 ``edge_ptr`` (train_fastgl.py:228-230) cannot
    address at all.  ``indices`` is filled on the GPU by a closed formula, so every sampled edge can be checked against
    the formula instead of a second copy: node v has 1016 in-edges if v is even and 8 if it is odd, edge e has source
    (e * 2654435761 + 12345) mod N.  Seeds are taken where the offsets are beyond 2^31."""
    import fastgl
    from checks import check_window
    dev = torch.device("cuda", 0)
    n = (1 << 22) + (1 << 16)
    v = torch.arange(n + 1, dtype=torch.int64, device=dev)
    indptr = (v // 2) * 1024 + (v % 2) * 1016
    n_edges = int(indptr[-1])
    assert n_edges == (1 << 31) + (1 << 25)                             # 2.18e9 edges, 8.7 GB of int32 sources
    indices = torch.empty(n_edges, dtype=torch.int32, device=dev)
    step = 1 << 27
    for lo in range(0, n_edges, step):
        e = torch.arange(lo, min(n_edges, lo + step), dtype=torch.int64, device=dev)
        indices[lo: lo + e.numel()] = ((e * 2654435761 + 12345) % n).to(torch.int32)
    del e

    def formula(positions):
        return ((positions * 2654435761 + 12345) % n).to(torch.int32)

    first_beyond = (1 << 22) + 16                                       # indptr[v] > 2^31 from here on
    assert int(indptr[first_beyond]) > (1 << 31)
    seeds = torch.arange(first_beyond, first_beyond + 4096, dtype=torch.int32, device=dev)
    fanout = 16
    src, dst, ptr, n_e = fastgl.sample_node_csr(indices, indptr, seeds, fanout, replace=False, rng_seed=5, rng_ctr=9)
    fastgl.check_status(dev)
    k = torch.where(seeds % 2 == 0, 16, 8)
    assert n_e == int(k.sum()) and torch.equal(ptr[1:].long(), torch.cumsum(k, 0))
    row = torch.repeat_interleave(torch.arange(4096, device=dev), k)
    assert torch.equal(dst, seeds[row])
    start = indptr[seeds.long()][row]
    within = torch.arange(n_e, device=dev) - ptr[:-1].long()[row]
    odd = (seeds[row] % 2 == 1)
    # full-neighbour rows (8 <= fanout): the adjacency slice itself, in order -- i.e. the formula at start + position
    assert torch.equal(src[odd], formula(start[odd] + within[odd]))
    # hubs (1016 > fanout): sixteen distinct positions of the slice; every pick is the formula at one of them
    even_rows = torch.nonzero(seeds % 2 == 0).flatten()
    slices = formula(indptr[seeds.long()[even_rows]][:, None] + torch.arange(1016, device=dev)[None, :])       # [2048, 1016]
    picks = src[~odd].view(-1, 16)
    hit = (picks[:, :, None] == slices[:, None, :])
    assert bool(hit.any(dim=2).all())
    pos = hit.float().argmax(dim=2)                                     # a position per pick (first match)
    # without replacement: sixteen different positions unless the formula repeats a value inside the slice
    distinct_values = torch.tensor([len(set(r.tolist())) for r in picks[:64].cpu()])
    assert bool((distinct_values >= 15).all())
    del hit, slices, pos
    # the fused path over the same seeds, two hops: every structural gate of a window holds on this CSR too
    seeds2 = seeds[:2048].view(2, 1024).contiguous()
    counts = torch.full((2,), 1024, dtype=torch.int32, device=dev)
    fb = fastgl.sample_map_fused(indptr, indices, seeds2, counts, [4, 16], replace=False, rng_seed=5, rng_ctr=64)
    fastgl.check_status(dev)
    seen = check_window(fb, indptr, indices, seeds2, [1024, 1024], replace=False, edge_keys=None)
    assert seen["batches"] == 2 and seen["edges"] > 2 * 1024 * 4

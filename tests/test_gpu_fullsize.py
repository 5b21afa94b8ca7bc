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

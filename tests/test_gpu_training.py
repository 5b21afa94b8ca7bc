"""GPU tests of the training loop around the kernels: the windowed sampler path equals the per-op path, the
loss of the CUDA path tracks a float64 CPU restatement of the same GraphSAGE-mean model built on the oracle,
and the CUDA-graph step reproduces the op-by-op step."""
import numpy as np
import pytest
import torch

from conftest import make_graph
from oracle import oracle_c as oc

pytestmark = pytest.mark.gpu


def setup_problem(n=6000, feat_dim=100, classes=7, seed=5):
    indptr, indices = make_graph(n, 14, seed=seed, hub=400)
    rng = np.random.default_rng(seed)
    feat = rng.standard_normal((n, feat_dim)).astype(np.float32)
    labels = rng.integers(0, classes, n)
    train = np.sort(rng.choice(n, size=n // 2, replace=False)).astype(np.int32)
    return indptr, indices, feat, labels, train


def make_trainer(problem, cuda_graph, window=4, window_layer0=True, hidden=32, batch=256, fanouts=(15, 10, 5), dropout=0.0):
    from fastgl_b200.layers import GraphSAGE
    from fastgl_b200.trainer import Trainer
    indptr, indices, feat, labels, train = problem
    dev = torch.device("cuda", 0)
    torch.manual_seed(3)
    model = GraphSAGE(feat.shape[1], hidden, 7, len(fanouts), dropout=dropout).to(dev)
    tr = Trainer(torch.from_numpy(indptr).to(dev), torch.from_numpy(indices).to(dev), torch.from_numpy(feat).to(dev),
                 torch.from_numpy(labels).to(dev), torch.from_numpy(train).to(dev), model, list(fanouts), batch_size=batch,
                 window=window, cuda_graph=cuda_graph, window_layer0=window_layer0)
    return tr


def test_sample_blocks_and_sample_window_give_identical_blocks():
    from fastgl_b200.sampler import FusedMapSampler
    indptr, indices, _, _, train = setup_problem()
    dev = torch.device("cuda", 0)
    a, b = FusedMapSampler([15, 10, 5], rng_seed=11), FusedMapSampler([15, 10, 5], rng_seed=11)
    for s in (a, b):
        s.edge_src, s.edge_ptr, s.nodes_num = torch.from_numpy(indices).to(dev), torch.from_numpy(indptr).to(dev), len(indptr) - 1
    seeds = torch.from_numpy(train[:768].reshape(3, 256)).to(dev)
    fb = a.sample_window(seeds, torch.full((3,), 256, dtype=torch.int32, device=dev))
    for i in range(3):
        inputs_w, blocks_w = a.window_blocks(fb, i)
        inputs_o, outputs_o, blocks_o = b.sample_blocks(None, seeds[i])
        assert torch.equal(inputs_w, inputs_o) and torch.equal(outputs_o, seeds[i])
        for bw, bo in zip(blocks_w, blocks_o):
            assert torch.equal(bw.indptr, bo.indptr) and torch.equal(bw.src, bo.src)
            assert (bw.n_src, bw.n_dst) == (bo.n_src, bo.n_dst)
            assert torch.equal(bw.edges()[1], bo.edges()[1])     # dst-local ids of transfer_edge_id == CSR rows


def test_loss_curve_tracks_the_cpu_restatement():
    problem = setup_problem()
    indptr, indices, feat, labels, train = problem
    tr = make_trainer(problem, cuda_graph=False)
    # float64 CPU model with the same initial weights, same seeds, same sampled blocks (via the oracle)
    params = [p.detach().double().cpu().clone().requires_grad_(True) for p in tr.model.parameters()]
    opt = torch.optim.Adam(params, lr=0.01, weight_decay=5e-4)
    gpu_losses = tr.run_steps(6, read_loss_each_step=True)
    from fastgl_b200.trainer import shard_seeds
    seeds_all = shard_seeds(torch.from_numpy(train), 0, 1, 12345).numpy()
    f64 = torch.from_numpy(feat).double()
    cpu_losses = []
    for step in range(6):
        seeds = seeds_all[step * 256:(step + 1) * 256]
        inputs, _, blocks = oc.sample_blocks(indptr, indices, seeds, [15, 10, 5], False, rng_seed=12345, rng_ctr=8 * step)
        h = f64[torch.from_numpy(inputs.astype(np.int64))]
        for i, blk in enumerate(blocks):
            w, bias = params[2 * i], params[2 * i + 1]
            deg = np.diff(blk["indptr"])
            dst = np.repeat(np.arange(blk["n_dst"]), deg)
            agg = torch.zeros((blk["n_dst"], h.shape[1]), dtype=torch.float64)
            agg.index_add_(0, torch.from_numpy(dst), h[torch.from_numpy(blk["src_local"].astype(np.int64))])
            agg = agg / torch.from_numpy(np.maximum(deg, 1)).double().unsqueeze(1)
            if i:
                pass
            h = torch.cat([h[: blk["n_dst"]], agg], 1) @ w + bias
            if i != len(blocks) - 1:
                h = torch.relu(h)
        loss = torch.nn.functional.cross_entropy(h, torch.from_numpy(labels[seeds.astype(np.int64)]))
        opt.zero_grad()
        loss.backward()
        opt.step()
        cpu_losses.append(float(loss.detach()))
    assert np.allclose(gpu_losses, cpu_losses, rtol=2e-3, atol=2e-3), (gpu_losses, cpu_losses)
    assert gpu_losses[-1] < gpu_losses[0]


@pytest.mark.parametrize("window_layer0", [True])
def test_cuda_graph_step_matches_the_op_by_op_step(window_layer0):
    problem = setup_problem(seed=9)
    eager = make_trainer(problem, cuda_graph=False, window_layer0=window_layer0)
    graphed = make_trainer(problem, cuda_graph=True, window_layer0=window_layer0)
    le = eager.run_steps(10, read_loss_each_step=True)
    lg = graphed.run_steps(10, read_loss_each_step=True)
    assert graphed.graphed is not None and graphed.graph_fallbacks <= 2
    assert np.allclose(le, lg, rtol=1e-4, atol=1e-4), (le, lg)
    for pe, pg in zip(eager.model.parameters(), graphed.model.parameters()):
        assert torch.allclose(pe, pg, rtol=1e-3, atol=5e-4)    # Adam turns rounding-level gradient differences into lr-sized ones
    assert eager.sampled_edges == graphed.sampled_edges


def test_cuda_graph_step_takes_the_short_last_batch_of_an_epoch():
    """3000 training seeds in batches of 256: the twelfth batch has 184 seeds and is replayed through the same
    graph (its missing rows are left out of the loss); the run continues into the next epoch's shuffle."""
    problem = setup_problem(seed=9)
    eager = make_trainer(problem, cuda_graph=False)
    graphed = make_trainer(problem, cuda_graph=True)
    assert eager.steps_per_epoch() == 12
    le = eager.run_steps(16, read_loss_each_step=True)
    lg = graphed.run_steps(16, read_loss_each_step=True)
    assert graphed.graph_fallbacks == 0 and graphed.epoch == 1
    assert np.allclose(le, lg, rtol=1e-4, atol=1e-4), (le, lg)
    for pe, pg in zip(eager.model.parameters(), graphed.model.parameters()):
        assert torch.allclose(pe, pg, rtol=1e-3, atol=5e-4)    # Adam turns rounding-level gradient differences into lr-sized ones
    assert eager.sampled_edges == graphed.sampled_edges


@pytest.mark.parametrize("fanouts,hidden", [((10, 5), 64), ((6, 5, 4, 3), 32)])
def test_step_program_with_other_depths(fanouts, hidden):
    problem = setup_problem(seed=11)
    eager = make_trainer(problem, cuda_graph=False, fanouts=fanouts, hidden=hidden)
    graphed = make_trainer(problem, cuda_graph=True, fanouts=fanouts, hidden=hidden)
    le = eager.run_steps(8, read_loss_each_step=True)
    lg = graphed.run_steps(8, read_loss_each_step=True)
    assert graphed.graphed is not None and graphed.graph_fallbacks <= 2
    assert np.allclose(le, lg, rtol=1e-4, atol=1e-4), (le, lg)
    for pe, pg in zip(eager.model.parameters(), graphed.model.parameters()):
        assert torch.allclose(pe, pg, rtol=1e-3, atol=5e-4)    # Adam turns rounding-level gradient differences into lr-sized ones


def test_step_program_trains_with_dropout():
    """With dropout the captured step draws a new mask on every replay (the loss of a repeated batch changes) and
    still learns."""
    problem = setup_problem(seed=13)
    tr = make_trainer(problem, cuda_graph=True, dropout=0.5, hidden=64)
    losses = tr.run_steps(60, read_loss_each_step=True)
    assert tr.graphed is not None and all(np.isfinite(losses))
    assert np.mean(losses[-10:]) < np.mean(losses[:10]) - 0.02
    g = tr.graphed
    torch.cuda.synchronize()
    before = [p.detach().clone() for p in tr.model.parameters()]
    a = float(g._forward_backward())
    g.sizes[g.L] += 1                                  # what staging the next step does to the dropout counter
    b = float(g._forward_backward())
    assert a != b
    for p, q in zip(tr.model.parameters(), before):    # forward_backward alone leaves the parameters alone
        assert torch.equal(p, q)


def test_trainer_recovers_from_a_hashtable_cap_that_is_too_small():
    """With a cap no window fits, the trainer notices at the window's read-back, drops the cap, samples the window
    again with the same counters and trains exactly as without a cap."""
    problem = setup_problem(seed=15)
    plain = make_trainer(problem, cuda_graph=True)
    capped = make_trainer(problem, cuda_graph=True)
    capped.table_slots, capped._auto_table = 1024, False
    lp = plain.run_steps(9, read_loss_each_step=True)
    lc = capped.run_steps(9, read_loss_each_step=True)
    assert capped.table_overflows == 1 and capped.table_slots == 0
    assert plain.table_slots > 0 and plain.table_overflows == 0          # learnt from the first window
    assert np.allclose(lp, lc, rtol=1e-5, atol=1e-6), (lp, lc)
    assert plain.sampled_edges == capped.sampled_edges


def test_prime_changes_nothing_but_the_set_up():
    problem = setup_problem(seed=17)
    plain = make_trainer(problem, cuda_graph=True)
    primed = make_trainer(problem, cuda_graph=True)
    before = [p.detach().clone() for p in primed.model.parameters()]
    primed.prime()
    assert primed.graphed is not None and primed.table_slots > 0 and primed.sampler.batch_counter == 0
    for p, q in zip(primed.model.parameters(), before):
        assert torch.equal(p, q)
    lp = plain.run_steps(9, read_loss_each_step=True)
    lq = primed.run_steps(9, read_loss_each_step=True)
    assert np.allclose(lp, lq, rtol=1e-5, atol=1e-6), (lp, lq)
    assert plain.sampled_edges == primed.sampled_edges


def test_gcn_layer_gives_the_same_result_in_either_order(monkeypatch):
    """A (x W) (the reference's order) and (A x) W, forward and backward, including destinations without in-edges
    (copied forward, skipped backward, as aggregate_acc_kernel.cu:307-308,:498-500) and the table-direct first layer."""
    import fastgl
    from fastgl_b200 import layers
    dev = torch.device("cuda", 0)
    rng = np.random.default_rng(21)
    n_dst, n_src, fin, fout = 500, 4000, 96, 40
    deg = rng.integers(0, 12, n_dst)
    deg[::7] = 0
    indptr = torch.from_numpy(np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)).to(dev)
    src = torch.from_numpy(rng.integers(0, n_src, int(deg.sum())).astype(np.int32)).to(dev)
    dst_deg = (indptr[1:] - indptr[:-1]).clamp(min=1)
    src_deg = fastgl.cal_deg(src, n_src).clamp(min=1)
    x0 = torch.randn((n_src, fin), device=dev)
    w0 = torch.randn((fin, fout), device=dev) / 8
    g = torch.randn((n_dst, fout), device=dev)
    results = []
    for first in (False, True):
        monkeypatch.setattr(layers, "gcn_aggregate_first", lambda *a, first=first: first)
        x, w = x0.clone().requires_grad_(True), w0.clone().requires_grad_(True)
        out = layers.MA_Function.apply(indptr, src, src_deg, dst_deg, n_dst, x, w, 12, None)
        out.backward(g)
        results.append((out.detach(), x.grad, w.grad))
    for a, b in zip(*results):
        assert float((a - b).abs().max()) <= 2e-5 * float(a.abs().max())
    # the whole feature table through global ids: same output and weight gradient, no input gradient
    n_nodes = 20_000
    ids = torch.from_numpy(rng.permutation(n_nodes)[:n_src].astype(np.int32)).to(dev)
    table = torch.randn((n_nodes, fin), device=dev)
    w = w0.clone().requires_grad_(True)
    out_t = layers.MA_Function.apply(indptr, src, src_deg, dst_deg, n_dst, table, w, 12, ids)
    out_t.backward(g)
    monkeypatch.setattr(layers, "gcn_aggregate_first", lambda *a: False)
    xg, w2 = table[ids.long()].clone(), w0.clone().requires_grad_(True)
    out_g = layers.MA_Function.apply(indptr, src, src_deg, dst_deg, n_dst, xg, w2, 12, None)
    out_g.backward(g)
    assert float((out_t - out_g).detach().abs().max()) <= 2e-5 * float(out_g.detach().abs().max())
    assert float((w.grad - w2.grad).abs().max()) <= 2e-5 * float(w2.grad.abs().max())


def test_gat_layer_matches_a_dense_torch_restatement():
    """GATConv on the CUDA ops against the same layer written with dense torch algebra (float64), including
    the gradient of the attention parameters that the reference drops."""
    from fastgl_b200.block import Block
    from fastgl_b200.layers import GATConv
    rng = np.random.default_rng(4)
    dev = torch.device("cuda", 0)
    n_dst, n_src, din, dout, heads = 60, 200, 32, 16, 4
    deg = rng.integers(1, 9, size=n_dst)
    indptr = np.zeros(n_dst + 1, dtype=np.int32)
    indptr[1:] = np.cumsum(deg)
    src = rng.integers(0, n_src, size=int(indptr[-1])).astype(np.int32)
    dst = np.repeat(np.arange(n_dst), deg)
    x = torch.from_numpy(rng.standard_normal((n_src, din)).astype(np.float32)).to(dev)
    blk = Block(torch.from_numpy(indptr).to(dev), torch.from_numpy(src).to(dev), n_src, n_dst)
    torch.manual_seed(1)
    layer = GATConv(din, dout, heads, attention_grad=True).to(dev)
    out = layer(blk, x, 8)
    target = torch.from_numpy(rng.standard_normal((n_dst, heads * dout)).astype(np.float32)).to(dev)
    (out * target).sum().backward()

    W = layer.fc.weight.detach().double().cpu().clone().requires_grad_(True)
    al = layer.attn_l.detach().double().cpu().clone().requires_grad_(True)
    ar = layer.attn_r.detach().double().cpu().clone().requires_grad_(True)
    f = (x.double().cpu() @ W.t()).view(-1, heads, dout)
    el, er = (f * al).sum(-1), (f[:n_dst] * ar).sum(-1)
    s_idx, d_idx = torch.from_numpy(src.astype(np.int64)), torch.from_numpy(dst)
    e = torch.nn.functional.leaky_relu(el[s_idx] + er[d_idx], 0.2)
    A = torch.full((n_dst, len(src), heads), float("-inf"), dtype=torch.float64)
    A[d_idx, torch.arange(len(src))] = e
    alpha = torch.softmax(A, dim=1)[d_idx, torch.arange(len(src))]                    # [E, H]
    ref = torch.zeros((n_dst, heads, dout), dtype=torch.float64).index_add_(0, d_idx, alpha[:, :, None] * f[s_idx])
    ref = ref.reshape(n_dst, heads * dout)
    (ref * target.double().cpu()).sum().backward()
    assert torch.allclose(out.double().cpu(), ref.detach(), rtol=1e-4, atol=1e-5)
    for got, want in ((layer.fc.weight.grad, W.grad), (layer.attn_l.grad, al.grad), (layer.attn_r.grad, ar.grad)):
        assert torch.allclose(got.double().cpu(), want, rtol=1e-3, atol=1e-4)


# ----------------------------------------------------------------------------------------------------------------
# the reference's own model stacks (GCN, GIN) through the trainer, against float64 models on oracle-sampled blocks
# ----------------------------------------------------------------------------------------------------------------
def _oracle_epoch_losses(problem, fanouts, batch, n_steps, params, forward):
    """Losses of ``n_steps`` Adam steps of a float64 CPU model on the blocks the oracle samples for the trainer's own
    seed order and Philox counters.  ``forward(blocks, inputs, f64_features, params)`` returns the logits."""
    from fastgl_b200.trainer import shard_seeds
    indptr, indices, feat, labels, train = problem
    opt = torch.optim.Adam(params, lr=0.01, weight_decay=5e-4)
    seeds_all = shard_seeds(torch.from_numpy(train), 0, 1, 12345).numpy()
    f64 = torch.from_numpy(feat).double()
    losses = []
    for step in range(n_steps):
        seeds = seeds_all[step * batch:(step + 1) * batch]
        inputs, _, blocks = oc.sample_blocks(indptr, indices, seeds, list(fanouts), False, rng_seed=12345, rng_ctr=8 * step)
        logits = forward(blocks, inputs, f64, params)
        loss = torch.nn.functional.cross_entropy(logits, torch.from_numpy(labels[seeds.astype(np.int64)]))
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    return losses


def _f64_block_sum(blk, h, weights=None):
    """sum over in-edges of (weights *) h[src]; rows without in-edges copy their own row (aggregate_acc_kernel.cu:307,405)."""
    deg = np.diff(blk["indptr"])
    dst = torch.from_numpy(np.repeat(np.arange(blk["n_dst"]), deg))
    src = torch.from_numpy(blk["src_local"].astype(np.int64))
    rows = h[src] if weights is None else h[src] * weights[:, None]
    out = torch.zeros((blk["n_dst"], h.shape[1]), dtype=torch.float64).index_add_(0, dst, rows)
    lonely = torch.from_numpy(deg == 0)
    return torch.where(lonely[:, None], h[: blk["n_dst"]], out)


def _gcn_forward(blocks, inputs, f64, params):
    h = f64[torch.from_numpy(inputs.astype(np.int64))]
    for blk, w in zip(blocks, params):
        deg = np.diff(blk["indptr"])
        ddeg = np.maximum(deg, 1).astype(np.float64)                                         # GraphConv.py:97
        sdeg = np.maximum(np.bincount(blk["src_local"], minlength=blk["n_src"]), 1).astype(np.float64)   # GraphConv.py:96
        dst = np.repeat(np.arange(blk["n_dst"]), deg)
        wgt = torch.from_numpy(1.0 / (np.sqrt(ddeg[dst]) * np.sqrt(sdeg[blk["src_local"]])))
        h = _f64_block_sum(blk, h @ w, wgt)                                                  # update, then aggregate
    return h


def _gin_forward(blocks, inputs, f64, params):
    h = f64[torch.from_numpy(inputs.astype(np.int64))]
    for blk, w in zip(blocks, params):
        h = _f64_block_sum(blk, h) @ w                                                       # aggregate, then update
    return h


@pytest.mark.parametrize("kind", ["gcn", "gcn-gathered", "gin"])
def test_gcn_and_gin_stacks_through_the_trainer_track_the_float64_model(kind):
    """The dense-graph configuration scaled down: 602-d rows, fanout [25, 10], two layers, batch 256.  The GCN first
    layer reads the feature table in place (``gcn``) or the gathered rows as the reference does (``gcn-gathered``)."""
    from fastgl_b200.layers import GCN, GIN
    from fastgl_b200.trainer import Trainer
    problem = setup_problem(n=5000, feat_dim=602, classes=7, seed=23)
    indptr, indices, feat, labels, train = problem
    dev = torch.device("cuda", 0)
    torch.manual_seed(5)
    model = (GIN if kind == "gin" else GCN)(602, 48, 7, 2, dropout=0.0).to(dev)
    tr = Trainer(torch.from_numpy(indptr).to(dev), torch.from_numpy(indices).to(dev), torch.from_numpy(feat).to(dev),
                 torch.from_numpy(labels).to(dev), torch.from_numpy(train).to(dev), model, [25, 10], batch_size=256, window=4,
                 table_direct=(kind == "gcn"))
    params = [p.detach().double().cpu().clone().requires_grad_(True) for p in model.parameters()]
    gpu = tr.run_steps(6, read_loss_each_step=True)
    import fastgl
    fastgl.check_status(dev)
    cpu = _oracle_epoch_losses(problem, (25, 10), 256, 6, params, _gin_forward if kind == "gin" else _gcn_forward)
    assert np.allclose(gpu, cpu, rtol=2e-3, atol=2e-3), (gpu, cpu)
    assert gpu[-1] < gpu[0]


def test_one_epoch_of_the_cpu_runnable_configuration_tracks_the_float64_model():
    """The smallest benchmark configuration at full size: seeded R-MAT graph, 100 k nodes of average degree 20, 128-d
    N(0,1) rows, 10 classes, 10 % training seeds, 3-layer GraphSAGE-mean (hidden 256), fanout [15, 10, 5], batch 1024:
    the ten mini-batches of one epoch (the last one short), through the windowed, graph-replayed trainer, against a
    float64 CPU model stepping on the blocks the oracle samples."""
    from fastgl_b200.graphgen import rmat_graph, synthetic_node_data
    from fastgl_b200.layers import GraphSAGE
    from fastgl_b200.trainer import Trainer
    dev = torch.device("cuda", 0)
    indptr, indices = rmat_graph(100_000, 20.0, seed=12345, device=dev)
    feat, labels, train = synthetic_node_data(100_000, 128, 10, 0.10, seed=12345, device=dev)
    torch.manual_seed(12345)
    model = GraphSAGE(128, 256, 10, 3, dropout=0.0).to(dev)
    tr = Trainer(indptr, indices, feat, labels, train, model, [15, 10, 5], batch_size=1024, window=8, cuda_graph=True)
    assert tr.steps_per_epoch() == 10
    params = [p.detach().double().cpu().clone().requires_grad_(True) for p in model.parameters()]
    tr.prime()
    gpu = tr.run_steps(10, read_loss_each_step=True)
    import fastgl
    fastgl.check_status(dev)
    assert tr.epoch == 0 and tr.graph_fallbacks <= 1
    problem = (indptr.cpu().numpy(), indices.cpu().numpy(), feat.cpu().numpy(), labels.cpu().numpy(), train.cpu().numpy())

    def sage_forward(blocks, inputs, f64, ps):
        h = f64[torch.from_numpy(inputs.astype(np.int64))]
        for i, blk in enumerate(blocks):
            w, bias = ps[2 * i], ps[2 * i + 1]
            deg = np.diff(blk["indptr"])
            dst = torch.from_numpy(np.repeat(np.arange(blk["n_dst"]), deg))
            agg = torch.zeros((blk["n_dst"], h.shape[1]), dtype=torch.float64)
            agg.index_add_(0, dst, h[torch.from_numpy(blk["src_local"].astype(np.int64))])
            agg = agg / torch.from_numpy(np.maximum(deg, 1)).double().unsqueeze(1)
            h = torch.cat([h[: blk["n_dst"]], agg], 1) @ w + bias
            if i != len(blocks) - 1:
                h = torch.relu(h)
        return h

    cpu = _oracle_epoch_losses(problem, (15, 10, 5), 1024, 10, params, sage_forward)
    assert np.allclose(gpu, cpu, rtol=2e-3, atol=2e-3), (gpu, cpu)
    assert gpu[-1] < gpu[0]


def test_a_label_out_of_range_stops_the_run_instead_of_being_resampled_away():
    """A bad label is recorded by the loss kernel (FGL_ERR_BOUNDS).  The trainer sees the status word with the next
    window's read-back; it must raise, not treat the code as a hashtable overflow, drop the cap and carry on."""
    import fastgl
    problem = setup_problem(seed=31)
    indptr, indices, feat, labels, train = problem
    labels = labels.copy()
    labels[train] = 7000                                  # every training label is out of range (7 classes)
    tr = make_trainer((indptr, indices, feat, labels, train), cuda_graph=True)
    with pytest.raises(RuntimeError, match="out of range"):
        tr.run_steps(12, read_loss_each_step=False)        # three windows of four: the second read-back sees the word
        fastgl.check_status(torch.device("cuda", 0))
    assert tr.table_overflows == 0


def test_match_reorder_trains_the_same_batches_in_another_order():
    """Match-Reorder (utilis.py:31-62) only permutes the mini-batches of a window: over whole windows the sampled
    edges are those of the plain order, and training still converges."""
    problem = setup_problem(seed=33)
    from fastgl_b200.layers import GraphSAGE
    from fastgl_b200.trainer import Trainer
    indptr, indices, feat, labels, train = problem
    dev = torch.device("cuda", 0)
    runs = []
    for reorder in (False, True):
        torch.manual_seed(3)
        model = GraphSAGE(feat.shape[1], 32, 7, 3, dropout=0.0).to(dev)
        tr = Trainer(torch.from_numpy(indptr).to(dev), torch.from_numpy(indices).to(dev), torch.from_numpy(feat).to(dev),
                     torch.from_numpy(labels).to(dev), torch.from_numpy(train).to(dev), model, [15, 10, 5], batch_size=256,
                     window=4, cuda_graph=True, reorder=reorder)
        losses = tr.run_steps(8, read_loss_each_step=True)
        runs.append((losses, tr.sampled_edges, tr))
    assert runs[0][1] == runs[1][1]
    assert sorted(runs[1][2].last_order) == [0, 1, 2, 3]
    assert all(np.isfinite(runs[1][0])) and runs[1][0][-1] < runs[1][0][0] + 0.1


def test_the_error_compensated_tf32_step_tracks_the_float32_step_and_the_float64_model():
    """``matmul="3xtf32"``: every dense product of the hand-written step is three TF32 tensor-core products of split
    operands.  On the CPU-runnable configuration at full size its losses must agree with the SIMT float32 step to
    1e-4 over ten steps (single-pass TF32 would be off by 1e-3 and more) and track the float64 trajectory as the
    float32 step does."""
    from fastgl_b200.graphgen import rmat_graph, synthetic_node_data
    from fastgl_b200.layers import GraphSAGE
    from fastgl_b200.trainer import Trainer
    import fastgl
    dev = torch.device("cuda", 0)
    indptr, indices = rmat_graph(100_000, 20.0, seed=12345, device=dev)
    feat, labels, train = synthetic_node_data(100_000, 128, 10, 0.10, seed=12345, device=dev)
    runs = {}
    for kind in ("fp32", "3xtf32"):
        torch.manual_seed(12345)
        model = GraphSAGE(128, 256, 10, 3, dropout=0.0).to(dev)
        tr = Trainer(indptr, indices, feat, labels, train, model, [15, 10, 5], batch_size=1024, window=8, cuda_graph=True,
                     matmul=kind)
        tr.prime()
        runs[kind] = (np.asarray(tr.run_steps(10, read_loss_each_step=True)),
                      torch.cat([p.detach().flatten() for p in model.parameters()]).double().cpu())
        fastgl.check_status(dev)
        assert tr.graph_fallbacks <= 1
        assert torch.backends.cuda.matmul.allow_tf32 is False      # the program restores the global setting
    (l32, p32), (l3x, p3x) = runs["fp32"], runs["3xtf32"]
    assert np.allclose(l3x, l32, rtol=1e-4, atol=1e-5), (l3x, l32)
    # Adam divides by the gradient's own magnitude, so a parameter whose gradient is at rounding level can move by the
    # learning rate in either direction: compare the bulk, not the worst entry
    diff = (p3x - p32).abs()
    # (the two runs also differ in the order of their scatter atomics, which alone moves the mean by a few 1e-6)
    assert float(diff.mean()) <= 5e-5 and float((diff > 1e-4).double().mean()) <= 3e-2, (float(diff.mean()), float(diff.max()))
    assert l3x[-1] < l3x[0]

"""The element-wise kernels of the training step (no counterpart among the reference's operators) against plain
PyTorch fp32/fp64 algebra, and the dropout mask against the oracle's Philox restatement."""
import numpy as np
import pytest
import torch

from oracle import oracle_np as onp

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def fastgl():
    import fastgl as f
    return f


@pytest.mark.parametrize("rows,dim", [(1, 4), (37, 47), (300, 256), (1025, 100)])
def test_bias_relu_without_dropout(fastgl, rows, dim):
    g = torch.Generator(device=DEV).manual_seed(rows)
    y = torch.randn((rows, dim), generator=g, device=DEV)
    b = torch.randn(dim, generator=g, device=DEV)
    want = torch.relu(y + b)
    got = fastgl.bias_relu_dropout_(y.clone(), b, 0.0, relu=True)
    assert torch.equal(got, want)
    assert torch.equal(fastgl.bias_relu_dropout_(y.clone(), b, 0.0, relu=False), y + b)
    k = max(1, rows // 3)
    side = torch.full((k, 2 * dim), 7.0, device=DEV)                          # the first k rows also go to a column slice
    got = fastgl.bias_relu_dropout_(y.clone(), b, 0.0, relu=True, copy_out=side[:, :dim])
    assert torch.equal(side[:, :dim], got[:k]) and float(side[:, dim:].min()) == 7.0
    wide = torch.randn((rows, 2 * dim + 4), generator=g, device=DEV)          # a column slice of a wider buffer
    view = wide[:, 4: 4 + dim]
    want = torch.relu(view + b)
    fastgl.bias_relu_dropout_(view, b, 0.0)
    assert torch.equal(wide[:, 4: 4 + dim], want)


@pytest.mark.parametrize("dim", [8, 47])
def test_dropout_mask_is_the_documented_philox_stream(fastgl, dim):
    rows, p, seed, ctr = 9, 0.3, 0x1234567890ABCDEF, 5
    y = torch.ones((rows, dim), device=DEV)
    step = torch.tensor([7], dtype=torch.int32, device=DEV)
    got = fastgl.bias_relu_dropout_(y, None, p, relu=False, rng_seed=seed, rng_ctr=ctr, rng_ctr_dev=step).cpu().numpy()
    thresh = int(float(np.float32(p)) * 4294967296.0)
    want = np.empty((rows, dim), dtype=np.float32)
    for e in range(rows * dim):
        word = onp.draw(seed, ctr + 7, 0, e)
        want.flat[e] = 0.0 if word < thresh else 1.0 / (1.0 - p)
    assert np.allclose(got, want, rtol=1e-6)


def test_dropout_rate_and_fresh_masks_per_step(fastgl):
    y = torch.ones((4096, 256), device=DEV)
    step = torch.zeros(1, dtype=torch.int32, device=DEV)
    a = fastgl.bias_relu_dropout_(y.clone(), None, 0.5, relu=False, rng_ctr_dev=step)
    step += 1
    b = fastgl.bias_relu_dropout_(y.clone(), None, 0.5, relu=False, rng_ctr_dev=step)
    kept = float((a > 0).float().mean())
    assert abs(kept - 0.5) < 0.005 and float(a.max()) == 2.0
    assert 0.45 < float(((a > 0) == (b > 0)).float().mean()) < 0.55          # independent masks


@pytest.mark.parametrize("rows,dim,p", [(1, 4, 0.0), (70, 47, 0.5), (5000, 256, 0.5), (129, 600, 0.2)])
def test_relu_dropout_backward_and_bias_gradient(fastgl, rows, dim, p):
    g = torch.Generator(device=DEV).manual_seed(dim)
    z = torch.randn((rows, dim), generator=g, device=DEV)
    b = torch.randn(dim, generator=g, device=DEV)
    out = fastgl.bias_relu_dropout_(z.clone(), b, p, relu=True, rng_ctr=3)
    dy = torch.randn((rows, dim), generator=g, device=DEV)
    want = torch.where(out > 0, dy / (1.0 - p), torch.zeros_like(dy))
    dbias = torch.zeros(dim, device=DEV)
    got = fastgl.relu_dropout_backward_(dy.clone(), out, p, dbias=dbias)
    assert torch.allclose(got, want, rtol=1e-6, atol=0)
    ref = want.double().sum(0)
    assert float((dbias.double() - ref).abs().max()) <= 1e-5 * max(1.0, float(ref.abs().max()))
    # unmasked: only the column sums
    dbias.zero_()
    same = fastgl.relu_dropout_backward_(dy.clone(), masked=False, dbias=dbias)
    assert torch.equal(same, dy)
    ref = dy.double().sum(0)
    assert float((dbias.double() - ref).abs().max()) <= 1e-5 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("rows,classes,n_valid", [(1024, 47, 1024), (1024, 47, 700), (33, 7, 33), (5, 172, 3), (64, 10, 0)])
def test_softmax_cross_entropy_and_gradient(fastgl, rows, classes, n_valid):
    g = torch.Generator(device=DEV).manual_seed(rows + classes)
    logits = (4 * torch.randn((rows, classes), generator=g, device=DEV)).requires_grad_(True)
    table = torch.randint(0, classes, (5000,), generator=g, device=DEV)
    ids = torch.randint(0, 5000, (rows,), generator=g, device=DEV).to(torch.int32)
    for n_arg in (n_valid, torch.tensor([n_valid], dtype=torch.int32, device=DEV)):
        loss, dlogits = fastgl.softmax_xent(logits.detach(), table, label_ids=ids, n_valid=n_arg)
        fastgl.check_status()
        if n_valid == 0:
            assert float(loss) == 0.0 and float(dlogits.abs().max()) == 0.0
            continue
        y = table[ids.long()]
        ref = torch.nn.functional.cross_entropy(logits[:n_valid].double(), y[:n_valid])
        (grad,) = torch.autograd.grad(ref, logits)
        assert abs(float(loss) - float(ref.detach())) <= 1e-5 * max(1.0, abs(float(ref.detach())))
        assert float((dlogits.double() - grad.double()).abs().max()) <= 1e-6
        assert float(dlogits[n_valid:].abs().max()) == 0.0 if n_valid < rows else True
    # labels given row by row
    y = table[ids.long()].contiguous()
    loss2, _ = fastgl.softmax_xent(logits.detach(), y, n_valid=n_valid)
    assert float(loss2) == float(loss)


@pytest.mark.parametrize("rows,k,classes,n_valid", [(1024, 512, 47, 1024), (1024, 512, 47, 700), (50, 37, 7, 50), (300, 128, 100, 299),
                                                    (64, 256, 128, 64), (9, 3, 33, 0)])
def test_output_layer_and_loss_in_one_pass(fastgl, rows, k, classes, n_valid):
    g = torch.Generator(device=DEV).manual_seed(rows + k)
    x = torch.randn((rows, k), generator=g, device=DEV)
    w = (torch.randn((k, classes), generator=g, device=DEV) / k ** 0.5).requires_grad_(True)
    b = torch.randn(classes, generator=g, device=DEV).requires_grad_(True)
    table = torch.randint(0, classes, (3000,), generator=g, device=DEV)
    ids = torch.randint(0, 3000, (rows,), generator=g, device=DEV).to(torch.int32)
    dbias = torch.zeros(classes, device=DEV)
    logits = torch.empty((rows, classes), device=DEV)
    loss, dlogits = fastgl.linear_softmax_xent(x, w.detach(), b.detach(), table, label_ids=ids,
                                               n_valid=torch.tensor([n_valid], dtype=torch.int32, device=DEV), dbias=dbias,
                                               logits=logits)
    fastgl.check_status()
    ref_logits = x.double() @ w.double() + b.double()
    assert float((logits.double() - ref_logits.detach()).abs().max()) <= 2e-5 * max(1.0, float(ref_logits.abs().max()))
    if n_valid == 0:
        assert float(loss) == 0.0 and float(dlogits.abs().max()) == 0.0 and float(dbias.abs().max()) == 0.0
        return
    y = table[ids.long()]
    ref = torch.nn.functional.cross_entropy(ref_logits[:n_valid], y[:n_valid])
    gw, gb = torch.autograd.grad(ref, (w, b))
    assert abs(float(loss) - float(ref.detach())) <= 1e-5 * max(1.0, abs(float(ref.detach())))
    assert float((dbias.double() - gb.double()).abs().max()) <= 1e-6
    got_gw = x.double().t() @ dlogits.double()                 # the weight gradient the step computes from dlogits
    assert float((got_gw - gw.double()).abs().max()) <= 1e-5 * max(1.0, float(gw.abs().max()))
    # the unfused pair gives the same numbers
    loss2, dl2 = fastgl.softmax_xent(logits, table, label_ids=ids, n_valid=n_valid)
    assert abs(float(loss2) - float(loss)) <= 1e-6 and float((dl2 - dlogits).abs().max()) <= 1e-7


def test_softmax_cross_entropy_reports_a_bad_label(fastgl):
    logits = torch.zeros((4, 3), device=DEV)
    labels = torch.tensor([0, 1, 7, 2], device=DEV)
    fastgl.softmax_xent(logits, labels)
    with pytest.raises(RuntimeError):
        fastgl.check_status()
    fastgl.check_status()                                                       # the status word was cleared


@pytest.mark.parametrize("n", [1, 7, 4096, 200_003])
def test_adam_step_matches_torch_adam(fastgl, n):
    g = torch.Generator(device=DEV).manual_seed(n)
    p0 = torch.randn(n, generator=g, device=DEV)
    ref = p0.clone().double().requires_grad_(True)
    opt = torch.optim.Adam([ref], lr=0.01, weight_decay=5e-4)
    p, m, v = p0.clone(), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    step = torch.zeros(2, dtype=torch.int32, device=DEV)
    for _ in range(5):
        grad = torch.randn(n, generator=g, device=DEV)
        ref.grad = grad.double()
        opt.step()
        fastgl.adam_step_(p, grad, m, v, step, lr=0.01, weight_decay=5e-4)
    assert step.tolist() == [5, 0]
    assert float((p.double() - ref.detach()).abs().max()) <= 2e-6


def test_aggregate_backward_starting_from_the_self_gradient(fastgl):
    rng = np.random.default_rng(5)
    n_dst, n_src, deg, dim = 700, 3000, 9, 256
    indptr = torch.arange(0, (n_dst + 1) * deg, deg, dtype=torch.int32, device=DEV)
    src = torch.from_numpy(rng.integers(0, n_src, n_dst * deg).astype(np.int32)).to(DEV)
    dcat = torch.randn((n_dst, 2 * dim), device=DEV)
    plain = fastgl.aggregate_backward(fastgl.AGG_MEAN, indptr, src, dcat[:, dim:].contiguous(), n_src)
    want = plain.clone()
    want[:n_dst] += dcat[:, :dim]
    out = torch.full((n_src, dim), 9.0, device=DEV)
    got = fastgl.aggregate_backward(fastgl.AGG_MEAN, indptr, src, dcat[:, dim:], n_src, d_self=dcat[:, :dim], out=out)
    assert got.data_ptr() == out.data_ptr()
    assert float((got - want).abs().max()) <= 1e-5 * float(want.abs().max())
    # odd width: scalar path
    d2 = torch.randn((n_dst, 2 * 47), device=DEV)
    plain = fastgl.aggregate_backward(fastgl.AGG_SUM, indptr, src, d2[:, 47:].contiguous(), n_src)
    plain[:n_dst] += d2[:, :47]
    got = fastgl.aggregate_backward(fastgl.AGG_SUM, indptr, src, d2[:, 47:], n_src, d_self=d2[:, :47])
    assert float((got - plain).abs().max()) <= 1e-5 * float(plain.abs().max())


def test_self_gradient_rows_beyond_the_device_side_row_count_are_ignored(fastgl):
    """Padded launch (real row count on the device): whatever the padded rows of dy_self hold, dx is zero there."""
    rng = np.random.default_rng(6)
    n_real, n_pad, n_src, deg, dim = 500, 768, 2048, 7, 128
    indptr = torch.zeros(n_pad + 1, dtype=torch.int32, device=DEV)
    indptr[: n_real + 1] = torch.arange(0, (n_real + 1) * deg, deg, dtype=torch.int32, device=DEV)
    src = torch.from_numpy(rng.integers(0, n_src, n_pad * deg).astype(np.int32)).to(DEV)
    dcat = torch.randn((n_pad, 2 * dim), device=DEV)            # the padded rows hold non-zero garbage
    n_dev = torch.tensor([n_real], dtype=torch.int32, device=DEV)
    got = fastgl.aggregate_backward(fastgl.AGG_MEAN, indptr, src, dcat[:, dim:], n_src, n_dst_dev=n_dev, d_self=dcat[:, :dim])
    want = fastgl.aggregate_backward(fastgl.AGG_MEAN, indptr[: n_real + 1].contiguous(), src[: n_real * deg].contiguous(),
                                     dcat[:n_real, dim:].contiguous(), n_src)
    want[:n_real] += dcat[:n_real, :dim]
    assert float((got - want).abs().max()) <= 1e-5 * float(want.abs().max())


def _flat_problem(n, seed):
    g = torch.Generator(device=DEV)
    g.manual_seed(seed)
    p = torch.randn(n, device=DEV, generator=g)
    return p, torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)


def test_allreduce_adam_with_one_rank_is_the_plain_adam_step(fastgl):
    n = 10_240 + 4
    p1, m1, v1 = _flat_problem(n, 1)
    p2, m2, v2 = p1.clone(), m1.clone(), v1.clone()
    s1, s2 = torch.zeros(2, dtype=torch.int32, device=DEV), torch.zeros(3, dtype=torch.int32, device=DEV)
    n_recv, n_flags = fastgl.PeerSync.sizes(n, 1)
    peers = fastgl.PeerSync(0, 1, [torch.zeros(n_recv, device=DEV)], [torch.zeros(n_flags, dtype=torch.int32, device=DEV)], n)
    for step in range(3):
        g = torch.randn(n, device=DEV)
        g2 = g.clone()
        fastgl.adam_step_(p1, g, m1, v1, s1, lr=0.01, weight_decay=5e-4)
        fastgl.allreduce_adam_(peers, p2, g2, m2, v2, s2, lr=0.01, weight_decay=5e-4)
        assert torch.equal(g2, g)                                   # the average over one rank
    assert torch.equal(p1, p2) and torch.equal(m1, m2) and torch.equal(v1, v2)
    assert s2.tolist() == [3, 0, 3]


def test_allreduce_adam_reduces_a_delivered_contribution_and_times_out_on_a_missing_one(fastgl):
    """Rank 0 of two, on one GPU: the second rank's contribution is placed in rank 0's receive buffer by hand and its
    flags are raised before the launch (no kernel waits for another kernel here), for two steps in a row (both
    halves of the double buffer).  Then a step whose flags nobody raises: the bounded wait gives up, the status word
    says so, and the parameters stay as they were."""
    n = 3 * 2048 + 8
    p, m, v = _flat_problem(n, 2)
    ref_p, ref_m, ref_v = p.clone(), m.clone(), v.clone()
    step, ref_step = torch.zeros(3, dtype=torch.int32, device=DEV), torch.zeros(2, dtype=torch.int32, device=DEV)
    n_recv, n_flags = fastgl.PeerSync.sizes(n, 2)
    mine_recv, mine_flags = torch.zeros(n_recv, device=DEV), torch.zeros(n_flags, dtype=torch.int32, device=DEV)
    peer_recv, peer_flags = torch.zeros(n_recv, device=DEV), torch.zeros(n_flags, dtype=torch.int32, device=DEV)
    peers = fastgl.PeerSync(0, 2, [mine_recv, peer_recv], [mine_flags, peer_flags], n)
    n_pad, n_chunks = peers.n_pad, peers.n_chunks
    for e in (1, 2):
        g0, g1 = torch.randn(n, device=DEV), torch.randn(n, device=DEV)
        parity = e & 1
        mine_recv.view(2, 2, n_pad)[parity, 1, :n] = g1             # what rank 1's launch would have pushed
        mine_flags.view(2, 2, n_chunks)[parity, 1, :] = e
        avg = (g0 + g1) * 0.5
        g = g0.clone()
        fastgl.allreduce_adam_(peers, p, g, m, v, step, lr=0.01, weight_decay=5e-4)
        fastgl.adam_step_(ref_p, avg.clone(), ref_m, ref_v, ref_step, lr=0.01, weight_decay=5e-4)
        fastgl.check_status(DEV)
        assert torch.equal(g, avg) and torch.equal(p, ref_p) and torch.equal(m, ref_m)
        # this rank's own push: its gradient and its flags arrived in the "peer's" buffers
        assert torch.equal(peer_recv.view(2, 2, n_pad)[parity, 0, :n], g0)
        assert bool((peer_flags.view(2, 2, n_chunks)[parity, 0] == e).all())
    before = p.clone()
    g = torch.randn(n, device=DEV)
    fastgl.allreduce_adam_(peers, p, g, m, v, step, lr=0.01, weight_decay=5e-4, spin_limit=2000)
    with pytest.raises(RuntimeError, match="wait gave up"):
        fastgl.check_status(DEV)
    assert torch.equal(p, before)
    fastgl.check_status(DEV)


def test_split_tf32_parts_and_the_three_product_sum_reach_float32_accuracy():
    """fgl_split_tf32: both parts are TF32-representable, they add up to x within 2^-21 |x|, and
    A_lo B_hi + A_hi B_lo + A_hi B_hi under TF32 GEMMs is as close to the float64 product as the SIMT float32 GEMM,
    while a single TF32 pass is an order of magnitude further away (so the test would notice a path that quietly
    stayed in float32, or one that dropped the correction terms)."""
    import fastgl
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(5)
    x = torch.randn(1_000_003, device=dev, generator=g) * torch.exp(4 * torch.randn(1_000_003, device=dev, generator=g))
    x = torch.cat([x, torch.tensor([0.0, -0.0, 1.0, -1.0, 3.4e38, 1e-30], device=dev)])[: 1_000_004].contiguous()
    hi, lo = fastgl.split_tf32(x)
    assert int((hi.view(torch.int32) & 0x1FFF).abs().max()) == 0
    assert int((lo.view(torch.int32) & 0x1FFF).abs().max()) == 0
    rest = (x.double() - hi.double() - lo.double()).abs()
    assert bool((rest <= x.double().abs() * 2.0 ** -21 + 1e-45).all())
    a = torch.randn(4096, 200, device=dev, generator=g)
    b = torch.randn(200, 256, device=dev, generator=g) * 0.1
    ref = a.double() @ b.double()
    scale = float(ref.abs().max())
    keep = torch.backends.cuda.matmul.allow_tf32
    try:
        torch.backends.cuda.matmul.allow_tf32 = False
        err_f32 = float(((a @ b).double() - ref).abs().max()) / scale
        torch.backends.cuda.matmul.allow_tf32 = True
        err_tf32 = float(((a @ b).double() - ref).abs().max()) / scale
        (ah, al), (bh, bl) = fastgl.split_tf32(a), fastgl.split_tf32(b)
        c = al @ bh
        c.addmm_(ah, bl)
        c.addmm_(ah, bh)
        err_3x = float((c.double() - ref).abs().max()) / scale
        # the same sum as one product over a three times longer inner dimension, the parts written in place by the kernel
        a3 = torch.empty(4096, 600, device=dev)
        b3 = torch.empty(600, 256, device=dev)
        fastgl.split_tf32(a, [(a3[:, :200], "hi"), (a3[:, 200:400], "lo"), (a3[:, 400:], "hi")])
        fastgl.split_tf32(b, [(b3[:200], "hi"), (b3[200:400], "hi"), (b3[400:], "lo")])
        assert torch.equal(a3[:, :200], ah) and torch.equal(a3[:, 200:400], al) and torch.equal(b3[400:], bl)
        err_cat = float(((a3 @ b3).double() - ref).abs().max()) / scale
    finally:
        torch.backends.cuda.matmul.allow_tf32 = keep
    assert err_3x <= 4 * max(err_f32, 1e-7), (err_3x, err_f32)
    # one long inner dimension accumulates in the tensor cores' float32 adders only (no SIMT adds between the three
    # products), which costs a few units in the last place: still two orders of magnitude below a single TF32 pass
    assert err_cat <= 5e-6, (err_cat, err_f32)
    assert err_tf32 >= 10 * err_cat, (err_tf32, err_cat)
    # odd widths take the scalar path
    y = torch.randn(37, 47, device=dev, generator=g)
    y3 = torch.zeros(37, 141, device=dev)
    fastgl.split_tf32(y, [(y3[:, :47], "hi"), (y3[:, 47:94], "lo"), (y3[:, 94:], "hi")])
    yh, yl = fastgl.split_tf32(y)
    assert torch.equal(y3[:, :47], yh) and torch.equal(y3[:, 47:94], yl) and torch.equal(y3[:, 94:], yh)


def test_fold_blocks_and_the_split_form_of_the_relu_backward():
    """fgl_fold_blocks against torch's sum over slabs and blocks; fgl_relu_dropout_bwd_split against the in-place
    backward followed by fgl_split_tf32 (same parts bit for bit, same bias gradient, dy untouched)."""
    import fastgl
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(9)
    part = torch.randn(3, 2 * 50, 2 * 48, device=dev, generator=g)
    out = torch.full((50, 47), 9.0, device=dev)
    fastgl.fold_blocks(part, 2, 2, 50, 47, 48, out)
    ref = part.view(3, 2, 50, 2, 48)[..., :47].double().sum(dim=(0, 1, 3))
    assert float((out.double() - ref).abs().max()) <= 1e-5
    one = torch.randn(2 * 50, 2 * 48, device=dev, generator=g)
    fastgl.fold_blocks(one, 2, 2, 50, 47, 48, out)
    assert float((out.double() - one.view(2, 50, 2, 48)[..., :47].double().sum(dim=(0, 2))).abs().max()) <= 1e-5

    for rows, dim, stride in ((1000, 256, 256), (37, 47, 48), (5000, 64, 64)):
        dy = torch.randn(rows, dim, device=dev, generator=g)
        fwd = torch.relu(torch.randn(rows, dim, device=dev, generator=g))
        keep = dy.clone()
        plain, db_plain = dy.clone(), torch.zeros(dim, device=dev)
        fastgl.relu_dropout_backward_(plain, out=fwd, p_drop=0.5, dbias=db_plain)
        hi, lo = fastgl.split_tf32(plain)
        s3, db = torch.zeros(rows, 3 * stride, device=dev), torch.zeros(dim, device=dev)
        got = fastgl.relu_dropout_backward_(dy, out=fwd, p_drop=0.5, dbias=db, split3=s3, block_stride=stride)
        assert got is s3 and torch.equal(dy, keep)
        assert torch.equal(s3[:, :dim], hi) and torch.equal(s3[:, stride: stride + dim], lo)
        assert torch.equal(s3[:, 2 * stride: 2 * stride + dim], hi)
        assert torch.allclose(db, db_plain, rtol=1e-4, atol=1e-3)      # other bands, another order of the column sums

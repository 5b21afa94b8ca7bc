"""The GraphSAGE-mean training step as an explicit sequence of launches over static buffers.

PyTorch's autograd runs the same step as ~70 kernels (bias epilogues, ReLU, dropout, concatenations, padded
slice gradients, gradient accumulations, a single-CTA loss, a 7-CTA optimizer).  Written out by hand the step is
per layer one GEMM, one fused bias/ReLU/dropout launch (which also stores the next layer's self rows) and one
aggregation forward;
one loss launch; and per layer two GEMMs, one scatter that starts from the self gradient, and one fused
ReLU/dropout backward that also produces the bias gradient.  The dense products stay with cuBLAS (torch.mm), as
in the reference (aggregate_acc_kernel.cu:237,368); everything else is a kernel of this library.

``matmul="3xtf32"`` evaluates every dense product on the tensor cores with float32-level error: both operands are
split into two TF32-representable parts (``fastgl.split_tf32``) and ``A B = A_hi B_hi + A_lo B_hi + A_hi B_lo`` is ONE
TF32 GEMM accumulating in float32 over a three times longer inner dimension, ``[A_hi | A_lo | A_hi] [B_hi ; B_hi ; B_lo]``
(three separate GEMMs cost more in launches than the SIMT float32 product they replace).  The weight gradient
``X^T dZ`` contracts over the rows, so it takes the 2 x 2 block product ``[X_hi | X_lo]^T [dZ_hi | dZ_lo]`` and adds the
four blocks.  (The reference's pinned PyTorch 1.10 ran these products in single-pass TF32.)  ``matmul="fp32"`` keeps
cuBLAS's SIMT float32 kernels.

The model is the one of ``layers.GraphSAGE``: layer i computes ``z_i = [h_i[:n_dst] | mean_N(h_i)] W_i + b_i`` and
``h_{i+1} = dropout(relu(z_i))``; the last z is the logits.  ``layers.GraphSAGE`` under autograd is the reference
the tests compare this program with.
"""
from __future__ import annotations

import torch

import fastgl


class SageStepProgram:
    def __init__(self, model, grads, labels, x0, seeds, sizes, blocks, pad_dst, step_word, rng_seed=12345, matmul="fp32",
                 overlap_weight_grads=True):
        """``x0``: float32[pad_dst[0], 2*in] rows [self | neighbour mean] of the input layer; ``blocks[i]`` (i >= 1) the
        padded block of layer i with its real row count in ``sizes[i]``; ``seeds``: int32 node ids of the output rows
        (their labels are ``labels[seeds]``); ``sizes[len(blocks) - 1]`` = number of valid output rows;
        ``step_word``: int32[1] view that differs from step to step (the dropout counter)."""
        self.layers = list(model.layers)
        self.L = len(self.layers)
        self.p_drop = float(model.dropout.p) if model.training else 0.0
        self.model = model
        self.grads = grads
        self.labels, self.x0, self.seeds, self.sizes, self.blocks = labels, x0, seeds, sizes, blocks
        self.pad_dst = list(pad_dst)
        self.step_word = step_word
        self.rng_seed = rng_seed
        dev = x0.device
        L = self.L
        outs = [layer.weight.size(1) for layer in self.layers]
        ins = [layer.input_dim for layer in self.layers]
        f32 = dict(dtype=torch.float32, device=dev)
        self.z = [torch.zeros((self.pad_dst[i], outs[i]), **f32) for i in range(L)]
        self.cat = [x0] + [torch.zeros((self.pad_dst[i], 2 * ins[i]), **f32) for i in range(1, L)]
        self.dcat = [None] + [torch.zeros((self.pad_dst[i], 2 * ins[i]), **f32) for i in range(1, L)]
        self.dh = [None] + [torch.zeros((self.pad_dst[i - 1], ins[i]), **f32) for i in range(1, L)]
        self.dlogits = torch.zeros((self.pad_dst[L - 1], outs[L - 1]), **f32)
        self.loss = torch.zeros(1, **f32)
        self.row_loss = torch.zeros(self.pad_dst[L - 1], **f32)
        # split-K of the tall weight-gradient products: S slabs of rows, folded by a [1 x S] product.  The output is
        # only a few 128 x 64 tiles, so S is what fills the 148 SMs.
        self.slabs, self.part, self.ones = [], [], []
        for i in range(L):
            n = self.pad_dst[i]
            s = next((s for s in (32, 16, 8) if n % s == 0 and n // s >= 256), 0)
            self.slabs.append(s)
            self.part.append(torch.zeros((s, 2 * ins[i], outs[i]), **f32) if s else None)
            self.ones.append(torch.ones((1, s), **f32) if s else None)
        if matmul not in ("fp32", "3xtf32"):
            raise ValueError("matmul must be 'fp32' or '3xtf32'")
        # The weight-gradient products feed nothing but the optimizer, so they run on a second stream beside the chain
        # input gradient -> scatter -> ReLU backward of the layer below (in a captured graph: a parallel branch).
        self.side = torch.cuda.Stream(device=dev)
        self.overlap = bool(overlap_weight_grads)      # measured: 2.5 % off the step
        self.split = matmul == "3xtf32"
        # set by a caller that fills x3[0] itself while it stages the mini-batch (then cat[0] is not read at all)
        self.x0_presplit = False
        if self.split:
            ks = [2 * d for d in ins]
            # block width of the output-side operands: a multiple of four floats, so that every block starts 16-byte
            # aligned and cuBLAS can use its vectorised tensor-core kernels (47 classes -> 48; the padding stays zero)
            self.mp = [(m + 3) // 4 * 4 for m in outs]
            # [X_hi | X_lo | X_hi] of every layer input, [dZ_hi | dZ_lo | dZ_hi] of every output gradient,
            # [W_hi ; W_hi ; W_lo] (forward) and [W_hi | W_hi | W_lo] (input gradient) of every weight
            self.x3 = [torch.zeros((self.pad_dst[i], 3 * ks[i]), **f32) for i in range(L)]
            self.g3 = [torch.zeros((self.pad_dst[i], 3 * self.mp[i]), **f32) for i in range(L)]
            self.wv3 = [torch.zeros((3 * ks[i], outs[i]), **f32) for i in range(L)]
            self.wc3 = [torch.zeros((ks[i], 3 * self.mp[i]), **f32) for i in range(L)]
            # the tensor cores need far fewer split-K slabs than the SIMT product to fill the GPU, and every slab is
            # 2k x 2m floats that the fold has to read back
            self.slabs = [next((s for s in (8, 4) if n % s == 0 and n // s >= 256), 0) for n in self.pad_dst]
            self.part = [torch.zeros((s, 2 * ks[i], 2 * self.mp[i]), **f32) if s else torch.zeros((2 * ks[i], 2 * self.mp[i]), **f32)
                         for i, s in enumerate(self.slabs)]

    # ---- operands of the error-compensated products ------------------------------------------------------------------
    @staticmethod
    def _split3(x, x3, width=None):
        """[hi | lo | hi] of ``x`` into ``x3``, whose three blocks are ``width`` (default: ``x``'s) columns apart."""
        c = x.size(1)
        w = c if width is None else width
        fastgl.split_tf32(x, [(x3[:, :c], "hi"), (x3[:, w: w + c], "lo"), (x3[:, 2 * w: 2 * w + c], "hi")])

    def _split_weight(self, i):
        w = self.layers[i].weight.data
        k, m = w.shape
        mp = self.mp[i]
        v, c = self.wv3[i], self.wc3[i]
        fastgl.split_tf32(w, [(v[:k], "hi"), (v[k: 2 * k], "hi"), (v[2 * k:], "lo"),
                              (c[:, :m], "hi"), (c[:, mp: mp + m], "hi"), (c[:, 2 * mp: 2 * mp + m], "lo")])

    def forward_backward(self) -> torch.Tensor:
        """Forward, loss and backward; the parameter gradients land in the flat gradient buffer.  Returns the loss
        (float32[1], a static buffer)."""
        if self.split:      # the TF32 setting is read when a product is enqueued (or captured), not when it runs
            keep = torch.backends.cuda.matmul.allow_tf32
            torch.backends.cuda.matmul.allow_tf32 = True
            try:
                return self._forward_backward()
            finally:
                torch.backends.cuda.matmul.allow_tf32 = keep
        return self._forward_backward()

    def _forward_backward(self) -> torch.Tensor:
        L, p = self.L, self.p_drop
        training = self.model.training
        self.grads.zero()
        split = self.split
        x_split = set()
        if split:
            for i in range(L):
                self._split_weight(i)
        last = self.layers[L - 1]
        fused_head = last.weight.size(1) <= 128        # output layer and loss in one launch
        for i, layer in enumerate(self.layers):
            if i == L - 1 and fused_head:
                break
            if split:
                if not (i == 0 and self.x0_presplit):
                    self._split3(self.cat[i], self.x3[i])
                x_split.add(i)
                torch.mm(self.x3[i], self.wv3[i], out=self.z[i])
            else:
                torch.mm(self.cat[i], layer.weight, out=self.z[i])
            if i < L - 1:
                blk = self.blocks[i + 1]
                d = self.layers[i + 1].input_dim
                nxt = self.cat[i + 1]
                fastgl.bias_relu_dropout_(self.z[i], layer.bias, p if training else 0.0, relu=True, rng_seed=self.rng_seed,
                                          rng_ctr=(i + 1) << 40, rng_ctr_dev=self.step_word, copy_out=nxt[:, :d])
                fastgl.aggregate(fastgl.AGG_MEAN, blk.indptr, blk.src, self.z[i], self.pad_dst[i + 1],
                                 zero_deg_passthrough=False, out=nxt[:, d:], n_dst_dev=blk.n_dst_dev)
            else:
                fastgl.bias_relu_dropout_(self.z[i], layer.bias, 0.0, relu=False)
        if fused_head:
            fastgl.linear_softmax_xent(self.cat[L - 1], last.weight, last.bias, self.labels, label_ids=self.seeds,
                                       n_valid=self.sizes[L - 1: L], loss=self.loss, dlogits=self.dlogits,
                                       row_loss=self.row_loss, dbias=last.bias.grad)
        else:
            fastgl.softmax_xent(self.z[L - 1], self.labels, label_ids=self.seeds, n_valid=self.sizes[L - 1: L], loss=self.loss,
                                dlogits=self.dlogits, row_loss=self.row_loss)
        dz = self.dlogits
        for i in reversed(range(L)):
            layer = self.layers[i]
            if i == L - 1 and not fused_head:
                fastgl.relu_dropout_backward_(dz, masked=False, dbias=layer.bias.grad)
            if split:
                if dz is not None:          # the output layer's gradient; the inner ones were written split already
                    self._split3(dz, self.g3[i], self.mp[i])
                if i not in x_split:
                    self._split3(self.cat[i], self.x3[i])
            if self.overlap:
                main = torch.cuda.current_stream()
                self.side.wait_stream(main)            # the operands of this layer's weight gradient are ready
                with torch.cuda.stream(self.side):
                    self._weight_grad(i, dz)
            else:
                self._weight_grad(i, dz)
            if i > 0:
                d = layer.input_dim
                blk = self.blocks[i]
                if split:
                    torch.mm(self.g3[i], self.wc3[i].t(), out=self.dcat[i])
                else:
                    torch.mm(dz, layer.weight.t(), out=self.dcat[i])
                fastgl.aggregate_backward(fastgl.AGG_MEAN, blk.indptr, blk.src, self.dcat[i][:, d:], self.pad_dst[i - 1],
                                          n_dst_dev=blk.n_dst_dev, d_self=self.dcat[i][:, :d], out=self.dh[i])
                if split:       # straight into the operand form of layer i - 1's two gradient products
                    fastgl.relu_dropout_backward_(self.dh[i], out=self.z[i - 1], p_drop=p if training else 0.0,
                                                  dbias=self.layers[i - 1].bias.grad, split3=self.g3[i - 1],
                                                  block_stride=self.mp[i - 1])
                    dz = None
                else:
                    dz = fastgl.relu_dropout_backward_(self.dh[i], out=self.z[i - 1], p_drop=p if training else 0.0,
                                                       dbias=self.layers[i - 1].bias.grad)
        if self.overlap:
            torch.cuda.current_stream().wait_stream(self.side)      # the optimizer step that follows needs every gradient
        return self.loss

    def _weight_grad(self, i: int, dz=None) -> None:
        x, gw = self.cat[i], self.layers[i].weight.grad
        s = self.slabs[i]
        n, k, m = x.size(0), x.size(1), gw.size(1)
        if self.split:
            # [X_hi | X_lo]^T [dZ_hi | dZ_lo]: four k x m blocks (the lo-lo block is below float32's rounding; adding it
            # costs nothing), folded together with the split-K slabs by one reduction -- not by a product with ones,
            # which would round the partial sums to TF32
            mp = self.mp[i]
            x2, g2 = self.x3[i][:, : 2 * k], self.g3[i][:, : 2 * mp]
            part = self.part[i]
            if s:
                torch.bmm(x2.unflatten(0, (s, n // s)).transpose(1, 2), g2.unflatten(0, (s, n // s)), out=part)
            else:
                torch.mm(x2.t(), g2, out=part)
            fastgl.fold_blocks(part, 2, 2, k, m, mp, gw)
            return
        if s:
            torch.bmm(x.view(s, n // s, k).transpose(1, 2), dz.view(s, n // s, m), out=self.part[i])
            torch.mm(self.ones[i], self.part[i].view(s, k * m), out=gw.view(1, k * m))
        else:
            torch.mm(x.t(), dz, out=gw)

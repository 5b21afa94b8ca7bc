"""GNN layers over the ``fastgl`` aggregation ops.

``MA_Function`` / ``MA_Function_GIN`` / ``MA_Function_GAT``, ``GCNConv`` / ``GINConv`` / ``GATConv`` and ``GCN`` /
``GIN`` / ``GAT`` keep the interface and the arithmetic of the reference's GraphConv.py (:19-40, :102-135, :196-228,
:42-99, :138-195, :231-312): update-then-aggregate for
GCN, aggregate-then-update for GIN, dropout between layers, no bias and no activation.  ``SAGEConv`` /
``GraphSAGE`` add the mean aggregator that the benchmark configurations name (the reference has none): 
``h' = h_dst W_self + mean_{s in N(d)} h_s W_neigh + b``, with the first layer aggregating straight from the
HBM-resident feature table through the block's global ids, so the gathered input matrix is never built.
"""
from __future__ import annotations

import math

import torch
from torch import nn

import fastgl


def block_csr(block):
    """(edge_ptr, src_edges) of a block.  A block from this package carries its CSR; for any other object
    with the reference's block interface the CSR is rebuilt the way GraphConv.py:92-94 does."""
    if hasattr(block, "indptr"):
        return block.indptr, block.src
    src, dst = block.edges()
    deg = fastgl.cal_deg(dst.int().contiguous(), block.num_dst_nodes())
    return fastgl.exclusive_sum(deg), src.int().contiguous()


def gcn_aggregate_first(n_src: int, n_dst: int, n_edges: int, in_dim: int, out_dim: int) -> bool:
    """Whether ``(A x) W`` is cheaper than ``A (x W)``.  Both give the layer's output (aggregation is linear); the
    reference always updates first (aggregate_acc_kernel.cu:237), which multiplies all ``n_src`` gathered rows by W
    although only ``n_dst`` output rows exist.  Cost model: fp32 GEMM at 40 TFLOP/s, aggregation at 3 TB/s of
    row traffic."""
    update_first = 2.0 * n_src * in_dim * out_dim / 40e12 + 4.0 * n_edges * out_dim / 3e12
    aggregate_first = 4.0 * n_edges * in_dim / 3e12 + 2.0 * n_dst * in_dim * out_dim / 40e12
    return aggregate_first < update_first


class MA_Function(torch.autograd.Function):
    """GraphConv.py:19-40, with the order of update and aggregation chosen by cost.

    Update-first is the reference's op pair (``forward_gcn`` / ``backward_gcn``).  Aggregate-first computes
    ``tmp = A x`` (sym-normalised, rows without in-edges copy their own input row, as the reference's forward does),
    ``out = tmp W``; backward ``d_w = tmp^T d``, ``d_x = A^T (d W^T)`` only if the input takes a gradient, where
    ``d`` is the incoming gradient with the rows of destinations without in-edges zeroed, because the reference's
    backward skips those rows (aggregate_acc_kernel.cu:498-500).  With ``row_map`` the input is the whole feature
    table addressed through the block's global ids (no gathered copy of the input rows exists)."""

    @staticmethod
    def forward(ctx, edge_ptr, src_edges, src_norm_degs, dst_norm_degs, dst_nodes, input_feat, weight, neighbor_num,
                row_map=None):
        n_src = src_norm_degs.numel()
        ctx.aggregate_first = row_map is not None or gcn_aggregate_first(n_src, dst_nodes, src_edges.numel(),
                                                                        weight.size(0), weight.size(1))
        if not ctx.aggregate_first:
            ctx.save_for_backward(edge_ptr, src_edges, src_norm_degs, dst_norm_degs, weight, input_feat)
            return fastgl.forward_gcn(edge_ptr, src_edges, src_norm_degs, dst_norm_degs, input_feat, weight, neighbor_num,
                                      dst_nodes)[0]
        tmp = fastgl.aggregate(fastgl.AGG_SYMNORM, edge_ptr, src_edges, input_feat, dst_nodes, src_norm_degs, dst_norm_degs,
                               zero_deg_passthrough=True, row_map=row_map)
        ctx.n_src = n_src
        ctx.mapped = row_map is not None
        ctx.save_for_backward(edge_ptr, src_edges, src_norm_degs, dst_norm_degs, weight, tmp)
        return torch.mm(tmp, weight)

    @staticmethod
    def backward(ctx, d_input):
        if not ctx.aggregate_first:
            edge_ptr, src_edges, src_norm_degs, dst_norm_degs, weight, input_feat = ctx.saved_tensors
            # destination degrees third, source degrees fourth: GraphConv.py:37
            d_x, d_w = fastgl.backward_gcn(edge_ptr, src_edges, dst_norm_degs, src_norm_degs, d_input.contiguous(), weight,
                                           input_feat)
            return None, None, None, None, None, d_x, d_w, None, None
        edge_ptr, src_edges, src_norm_degs, dst_norm_degs, weight, tmp = ctx.saved_tensors
        n_dst = tmp.size(0)
        has_edges = (edge_ptr[1: n_dst + 1] > edge_ptr[:n_dst]).unsqueeze(1)
        d = d_input * has_edges
        d_w = torch.mm(tmp.t(), d)
        d_x = None
        if ctx.needs_input_grad[5]:
            if ctx.mapped:
                raise RuntimeError("no gradient flows into a feature table that is aggregated through a row map")
            d_x = fastgl.aggregate_backward(fastgl.AGG_SYMNORM, edge_ptr, src_edges, torch.mm(d, weight.t()), ctx.n_src,
                                            src_norm_degs=src_norm_degs, dst_norm_degs=dst_norm_degs)
        return None, None, None, None, None, d_x, d_w, None, None


class MA_Function_GIN(torch.autograd.Function):
    """GraphConv.py:102-135."""

    @staticmethod
    def forward(ctx, edge_ptr, src_edges, dst_nodes, input_feat, weight, neighbor_num):
        out, tmp = fastgl.forwaed_gin(edge_ptr, src_edges, input_feat, weight, neighbor_num, dst_nodes)
        ctx.src_nodes = input_feat.size(0)
        ctx.save_for_backward(edge_ptr, src_edges, weight, tmp)
        return out

    @staticmethod
    def backward(ctx, d_input):
        edge_ptr, src_edges, weight, tmp = ctx.saved_tensors
        d_x, d_w = fastgl.backward_gin(edge_ptr, src_edges, d_input.contiguous(), weight, tmp, ctx.src_nodes)
        return None, None, None, d_x, d_w, None


class _Conv(nn.Module):
    def __init__(self, input_dim, output_dim):
        super().__init__()
        self.weights = nn.Parameter(torch.empty(input_dim, output_dim))
        self.reset_parameters()

    def reset_parameters(self):
        stdv = 1.0 / math.sqrt(self.weights.size(1))  # GraphConv.py:50-53
        with torch.no_grad():
            self.weights.uniform_(-stdv, stdv)


class GCNConv(_Conv):
    def forward(self, edge_ptr, src_edges, src_norm_degs, dst_norm_degs, dst_nodes, input_feat, neighbor_num, row_map=None):
        return MA_Function.apply(edge_ptr, src_edges, src_norm_degs, dst_norm_degs, dst_nodes, input_feat, self.weights,
                                 neighbor_num, row_map)


class GINConv(_Conv):
    def forward(self, edge_ptr, src_edges, dst_nodes, input_feat, neighbor_num):
        return MA_Function_GIN.apply(edge_ptr, src_edges, dst_nodes, input_feat, self.weights, neighbor_num)


class _Stack(nn.Module):
    conv = None

    def __init__(self, in_feats, n_hidden, n_classes, n_layers, activation=None, weight=True, dropout=0.5):
        super().__init__()
        dims = [in_feats] + [n_hidden] * (n_layers - 1) + [n_classes]
        self.layers = nn.ModuleList([self.conv(dims[i], dims[i + 1]) for i in range(n_layers)])
        self.dropout = nn.Dropout(p=dropout)


class GCN(_Stack):
    """GraphConv.py:63-99: a linear stack (the reference accepts ``activation`` and never applies it)."""
    conv = GCNConv

    def forward(self, blocks, features, neighbor_list=(5, 10, 15), input_nodes=None):
        """``features``: the gathered input rows float32[n_src_0, in] (train_fastgl.py:357,365), or, with
        ``input_nodes`` (int32 global ids of block 0's sources), the whole feature table, which the first layer then
        aggregates in place."""
        h = features
        for i, layer in enumerate(self.layers):
            if i != 0:
                h = self.dropout(h)
            block = blocks[i]
            n_dst = block.num_dst_nodes()
            edge_ptr, src_edges = block_csr(block)
            dst_norm_degs = (edge_ptr[1: n_dst + 1] - edge_ptr[:n_dst]).clamp(min=1)         # GraphConv.py:93,97
            src_norm_degs = fastgl.cal_deg(src_edges, block.num_src_nodes()).clamp(min=1)    # GraphConv.py:96
            h = layer(edge_ptr, src_edges, src_norm_degs, dst_norm_degs, n_dst, h, neighbor_list[i],
                      row_map=input_nodes if i == 0 else None)
        return h


class GIN(_Stack):
    """GraphConv.py:159-195."""
    conv = GINConv

    def forward(self, blocks, features, neighbor_list=(5, 10, 15)):
        h = features
        for i, layer in enumerate(self.layers):
            if i != 0:
                h = self.dropout(h)
            block = blocks[i]
            edge_ptr, src_edges = block_csr(block)
            h = layer(edge_ptr, src_edges, block.num_dst_nodes(), h, neighbor_list[i])
        return h


class MA_Function_GAT(torch.autograd.Function):
    """GraphConv.py:196-228.  ``attention_grad=False`` is the reference: no gradient reaches ``edge_data``
    (backward returns None for it, GraphConv.py:227); ``True`` adds the missing term."""

    @staticmethod
    def forward(ctx, edge_ptr, edge_data, src_edges, dst_edges, dst_nodes, input_feat, num_heads, neighbor_num,
                attention_grad=False):
        edge_data = edge_data.contiguous()
        out = fastgl.forward_gat(edge_ptr, edge_data, src_edges, input_feat, neighbor_num, dst_nodes, num_heads)[0]
        ctx.src_nodes, ctx.num_heads, ctx.attention_grad = input_feat.size(0), num_heads, attention_grad
        ctx.save_for_backward(edge_ptr, edge_data, src_edges, input_feat)
        return out

    @staticmethod
    def backward(ctx, d_input):
        edge_ptr, edge_data, src_edges, input_feat = ctx.saved_tensors
        d_input = d_input.contiguous()
        d_x = fastgl.backward_gat(edge_ptr, edge_data, src_edges, d_input, ctx.src_nodes, ctx.num_heads)[0]
        d_w = None
        if ctx.attention_grad and ctx.needs_input_grad[1]:
            d_w = fastgl.edge_weight_grad(edge_ptr, src_edges, input_feat, d_input, ctx.num_heads)
        return None, d_w, None, None, None, d_x, None, None, None


def edge_softmax(e: torch.Tensor, dst: torch.Tensor, n_dst: int) -> torch.Tensor:
    """Softmax of the edge scores ``e`` [E, H] over the in-edges of every destination (what the reference
    takes from ``dgl.nn.functional.edge_softmax``, GraphConv.py:268)."""
    idx = dst.long()
    top = torch.full((n_dst, e.size(1)), float("-inf"), dtype=e.dtype, device=e.device)
    top = top.scatter_reduce(0, idx[:, None].expand_as(e), e, "amax", include_self=True)
    ex = torch.exp(e - top[idx])
    denom = torch.zeros((n_dst, e.size(1)), dtype=e.dtype, device=e.device).index_add_(0, idx, ex)
    return ex / denom[idx]


class GATConv(nn.Module):
    """GraphConv.py:231-283: shared linear map, additive attention, edge softmax, weighted multi-head sum."""

    def __init__(self, input_dim, output_dim, num_heads, feat_drop=0.0, attn_drop=0.0, negative_slope=0.2,
                 attention_grad=False):
        super().__init__()
        self.out_feats, self.num_heads, self.attention_grad = output_dim, num_heads, attention_grad
        self.fc = nn.Linear(input_dim, output_dim * num_heads, bias=False)
        self.attn_l = nn.Parameter(torch.empty(1, num_heads, output_dim))
        self.attn_r = nn.Parameter(torch.empty(1, num_heads, output_dim))
        self.feat_drop, self.attn_drop = nn.Dropout(feat_drop), nn.Dropout(attn_drop)
        self.leaky_relu = nn.LeakyReLU(negative_slope)
        gain = nn.init.calculate_gain("relu")
        nn.init.xavier_normal_(self.fc.weight, gain=gain)
        nn.init.xavier_normal_(self.attn_l, gain=gain)
        nn.init.xavier_normal_(self.attn_r, gain=gain)

    def forward(self, block, input_feat, neighbor_num):
        n_dst = block.num_dst_nodes()
        feat_src = self.fc(input_feat).view(-1, self.num_heads, self.out_feats)
        el = (feat_src * self.attn_l).sum(dim=-1)
        er = (feat_src[:n_dst] * self.attn_r).sum(dim=-1)
        edge_ptr, src_edges = block_csr(block)
        dst_edges = block.edges()[1]
        e = self.leaky_relu(el[src_edges.long()] + er[dst_edges.long()])
        edge_data = self.attn_drop(edge_softmax(e, dst_edges, n_dst))
        flat = feat_src.reshape(-1, self.num_heads * self.out_feats)
        return MA_Function_GAT.apply(edge_ptr, edge_data, src_edges, dst_edges, n_dst, flat, self.num_heads, neighbor_num,
                                     self.attention_grad)


class GAT(nn.Module):
    """GraphConv.py:285-312: ``heads`` heads of ``n_hidden`` in the inner layers, one head of ``n_classes`` last."""

    def __init__(self, in_feats, n_hidden, n_classes, n_layers, activation=None, dropout=0.5, heads=8, attention_grad=False):
        super().__init__()
        self.layers = nn.ModuleList([GATConv(in_feats, n_hidden, heads, attention_grad=attention_grad)])
        for _ in range(1, n_layers - 1):
            self.layers.append(GATConv(n_hidden * heads, n_hidden, heads, feat_drop=dropout, attention_grad=attention_grad))
        self.layers.append(GATConv(n_hidden * heads, n_classes, 1, feat_drop=dropout, attention_grad=attention_grad))

    def forward(self, blocks, features, neighbor_list=(5, 10, 15)):
        h = features
        for i, layer in enumerate(self.layers):
            h = layer(blocks[i], h, neighbor_list[i])
        return h


class MeanAggregate(torch.autograd.Function):
    """mean over in-neighbours (rows without in-edges give zeros); optional row map into a feature table."""

    @staticmethod
    def forward(ctx, x, edge_ptr, src_edges, n_dst, row_map, n_dst_dev=None):
        ctx.save_for_backward(edge_ptr, src_edges)
        ctx.n_src = x.size(0)
        ctx.mapped = row_map is not None
        ctx.n_dst_dev = n_dst_dev
        return fastgl.aggregate(fastgl.AGG_MEAN, edge_ptr, src_edges, x, n_dst, zero_deg_passthrough=False, row_map=row_map,
                                n_dst_dev=n_dst_dev)

    @staticmethod
    def backward(ctx, d_out):
        d_x = None
        if ctx.needs_input_grad[0]:
            if ctx.mapped:
                raise RuntimeError("no gradient flows into a feature table that is aggregated through a row map")
            edge_ptr, src_edges = ctx.saved_tensors
            d_x = fastgl.aggregate_backward(fastgl.AGG_MEAN, edge_ptr, src_edges, d_out.contiguous(), ctx.n_src,
                                            n_dst_dev=ctx.n_dst_dev)
        return d_x, None, None, None, None, None


class _TallLinear(torch.autograd.Function):
    """x W + b for a tall x (tens of thousands of rows, a few hundred columns).

    The weight gradient x^T dy has a tiny output and a very long reduction; as one GEMM it runs on a handful
    of CTAs.  Here the rows are split into S slabs, a batched GEMM produces S partial products on S times as
    many CTAs, and the partials (and the per-slab column sums for the bias) are folded by a 1 x S GEMM."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        return torch.addmm(bias, x, weight)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.mm(dy, weight.t()) if ctx.needs_input_grad[0] else None
        n, k, m = x.size(0), x.size(1), dy.size(1)
        slabs = next((s for s in (16, 8) if n % s == 0 and n // s >= 512), 0)
        if slabs and x.is_contiguous():
            ones = dy.new_ones((1, slabs))
            part = torch.bmm(x.view(slabs, n // slabs, k).transpose(1, 2), dy.view(slabs, n // slabs, m))
            dw = torch.mm(ones, part.view(slabs, k * m)).view(k, m)
            col = torch.bmm(dy.new_ones((slabs, 1, n // slabs)), dy.view(slabs, n // slabs, m))
            db = torch.mm(ones, col.view(slabs, m)).view(m)
        else:
            dw = torch.mm(x.t(), dy)
            db = torch.mv(dy.t(), dy.new_ones(n))
        return dx, dw, db


class SAGEConv(nn.Module):
    """h' = [h_dst | mean_{s in N(d)} h_s] W + b, with W = [W_self; W_neigh] stacked so that the layer is one GEMM."""

    def __init__(self, input_dim, output_dim):
        super().__init__()
        self.input_dim = input_dim
        self.weight = nn.Parameter(torch.empty(2 * input_dim, output_dim))
        self.bias = nn.Parameter(torch.zeros(output_dim))
        bound = math.sqrt(2.0) * math.sqrt(6.0 / (input_dim + output_dim))
        with torch.no_grad():
            self.weight.uniform_(-bound, bound)

    def forward(self, block, h, row_map=None, timer=None, self_neigh=None):
        """``h``: float32[n_src, in] -- or, with ``row_map`` (the block's global ids), the whole feature table.
        ``self_neigh``: float32[n_dst, 2*in] already holding [h_dst | mean of neighbours] (the window-level
        aggregation of the first layer); then ``block`` and ``h`` are not touched.
        ``timer`` (a list) receives (start_event, end_event, block) around the aggregation kernel."""
        if self_neigh is not None:
            return _TallLinear.apply(self_neigh, self.weight, self.bias)
        n_dst = block.num_dst_nodes()
        edge_ptr, src_edges = block_csr(block)
        if timer is not None:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        h_neigh = MeanAggregate.apply(h, edge_ptr, src_edges, n_dst, row_map, getattr(block, "n_dst_dev", None))
        if timer is not None:
            end.record()
            timer.append((start, end, block))
        h_self = h[:n_dst] if row_map is None else torch.index_select(h, 0, row_map[:n_dst].long())
        return _TallLinear.apply(torch.cat([h_self, h_neigh], 1), self.weight, self.bias)


class GraphSAGE(nn.Module):
    """3-layer GraphSAGE-mean of the benchmark configurations: ReLU and dropout between layers."""

    def __init__(self, in_feats, n_hidden, n_classes, n_layers, dropout=0.5):
        super().__init__()
        dims = [in_feats] + [n_hidden] * (n_layers - 1) + [n_classes]
        self.layers = nn.ModuleList([SAGEConv(dims[i], dims[i + 1]) for i in range(n_layers)])
        self.dropout = nn.Dropout(p=dropout)
        self.layer0_timer = None  # set to a list to time the first layer's aggregation kernel

    def forward(self, blocks, features, input_nodes=None, layer0=None):
        """``features``: the gathered input rows float32[n_src_0, in]; or, with ``input_nodes`` (int32 global
        ids of block 0's sources), the full feature table, read in place by the first layer; or ``None`` when
        ``layer0`` = float32[n_dst_0, 2*in] already holds the first layer's [self | neighbour mean] rows."""
        h = features
        for i, layer in enumerate(self.layers):
            if i != 0:
                h = self.dropout(torch.relu(h))
            if i == 0 and layer0 is not None:
                h = layer(None, None, self_neigh=layer0)
            else:
                h = layer(blocks[i], h, row_map=input_nodes if i == 0 else None,
                          timer=self.layer0_timer if i == 0 else None)
        return h

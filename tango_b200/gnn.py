"""The evaluation models of the reference (QGraphConv / GCN from evaluation/test_gcn.py:40-175, QGATConv / GAT from
evaluation/test_gat.py:30-224, HGT from evaluation/test_HGT.py:27-67, the link-prediction GCN and its scorer from
evaluation/link_pred_gcn.py:113-165) re-hosted on the DGL-free `Graph`, built only from the quantized operators of
this package.  They are the callers of the hot path: the epoch benchmark and the end-to-end parity tests run them.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.autograd.function import Function, once_differentiable

from . import config, kernels
from .QLinear import QLinear, Qlinear_func, Qlinear_func_reduce
from .SDDMM import sddmm_u_add_v, sddmm_u_dot_v
from .SPMM import spmm_copy_u, spmm_u_mul_e


def _norm(deg: torch.Tensor, both: bool) -> torch.Tensor:
    d = deg.float().clamp(min=1)
    return torch.pow(d, -0.5) if both else 1.0 / d


def _has_zero_in_degree(graph) -> bool:
    """The reference's layers check this on every forward (evaluation/test_gcn.py:69-79), which costs a device
    synchronisation per call; the graph is immutable here, so the answer is computed once."""
    cache = graph.ndata.setdefault("_tango_norm", {})
    if "zero_in" not in cache:
        cache["zero_in"] = bool((graph.in_degrees() == 0).any())
    return cache["zero_in"]


def _cached_norm(graph, which: str) -> torch.Tensor:
    """deg^-1/2 (degrees clamped to >= 1) as a contiguous fp32 vector, computed once per graph."""
    cache = graph.ndata.setdefault("_tango_norm", {})
    if which not in cache:
        deg = graph.in_degrees() if which == "in" else graph.out_degrees()
        cache[which] = _norm(deg, True).contiguous()
    return cache[which]


class _gcn_conv_fused(Function):
    """One "multiply first" graph convolution (in_feats > out_feats, norm='both') as a single autograd node:

        out = act( (A . Q(Q(X * d_out^-1/2) W^T)) * d_in^-1/2 + b )

    Same arithmetic, operation for operation, as the unfused composition in QGraphConv.forward (bit-identical
    results), but the element-wise passes of the reference's layer (evaluation/test_gcn.py:86-94,123-137) are folded
    into the kernels next to them: the left norm into the absmax/quantize of X, the right norm + bias + ReLU into the
    aggregation's epilogue, and the right norm of the backward pass into the quantizer of the incoming gradient."""

    @staticmethod
    def forward(ctx, g, X, W, b, out_norm, in_norm, relu):
        from .kernels import alloc_int8, next_call
        mode_f, mode_q, seed = config.mode_for("gemm_fwd"), config.mode_for("quantize"), config.seed()
        call = next_call() if mode_f == kernels.ROUND_STOCHASTIC else 0
        if mode_f == kernels.ROUND_STOCHASTIC:
            next_call()
        X = X.contiguous()
        sX = kernels._get_scale(X, out_norm)
        sW = kernels._get_scale(W)
        Xq, Wq = alloc_int8(X.shape, X.device), alloc_int8(W.shape, X.device)
        H = torch.empty((X.shape[0], W.shape[0]), dtype=torch.float32, device=X.device)
        sH = torch.zeros(1, dtype=torch.float32, device=X.device)
        # X * d_out^-1/2 is quantized on load inside the GEMM kernel, which also writes Xq for the backward pass
        kernels._qgemm_forward(H, X, Xq, W.contiguous(), Wq, None, sH, sX, sW, mode_f, seed, call, out_norm)
        Hq, _ = kernels.quantize(H, sH, mode=mode_q, seed=seed)
        out = kernels.csr_SPMM(g, Hq, sH, False, in_norm, b, relu)
        ctx.g, ctx.relu, ctx.has_bias = g, relu, b is not None
        ctx.save_for_backward(Xq, sX, Wq, sW, out_norm, in_norm, out if relu else None)
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, d_out):
        Xq, sX, Wq, sW, out_norm, in_norm, out = ctx.saved_tensors
        mode_q, seed = config.mode_for("quantize"), config.seed()
        want_db = ctx.has_bias and ctx.needs_input_grad[3]
        call = kernels.next_call() if mode_q == kernels.ROUND_STOCHASTIC else 0
        if ctx.relu:
            # ReLU mask, bias gradient, right norm, absmax and quantisation in two passes over (d_out, out)
            dZq, sdZ, db = kernels.relu_grad_quantize(d_out, out, in_norm, want_db, mode_q, seed, call)
        else:
            g1 = d_out.contiguous()
            db = g1.sum(0) if want_db else None
            sdZ = kernels._get_scale(g1, in_norm)
            dZq = kernels.alloc_int8(g1.shape, g1.device)
            kernels._quantize_into(dZq, g1, sdZ, mode_q, seed, call, in_norm)
        dH = kernels.csr_SPMM(ctx.g, dZq, sdZ, True)
        dHq, sdH = kernels.quantize(dH, mode=mode_q, seed=seed)
        dX, dW = kernels.QGEMM_backward(dHq, Xq, Wq, sdH, sX, sW, ctx.needs_input_grad[1], ctx.needs_input_grad[2],
                                        dx_row_scale=out_norm)   # backward of the left norm, in the GEMM epilogue
        return None, dX, dW, db, None, None, None


class QGraphConv(nn.Module):
    """Graph convolution with int8 GEMM and int8 aggregation (evaluation/test_gcn.py:40-139).  As in the reference,
    the linear layer runs first when it shrinks the features (and hands its output scale to the aggregation), else
    the aggregation runs first."""

    def __init__(self, in_feats, out_feats, norm="both", weight=True, bias=True, activation=None,
                 allow_zero_in_degree=False, fused=True):
        super().__init__()
        self._fused = fused
        if norm not in ("none", "both", "right", "left"):
            raise ValueError(f'Invalid norm value "{norm}"')
        self._in_feats, self._out_feats, self._norm = in_feats, out_feats, norm
        self._allow_zero_in_degree = allow_zero_in_degree
        self.weight = nn.Parameter(torch.empty(out_feats, in_feats)) if weight else None
        self.bias = nn.Parameter(torch.empty(out_feats)) if bias else None
        self._activation = activation
        self.reset_parameters()

    def reset_parameters(self):
        if self.weight is not None:
            nn.init.xavier_uniform_(self.weight)
        if self.bias is not None:
            nn.init.zeros_(self.bias)

    def forward(self, graph, feat):
        if not self._allow_zero_in_degree and _has_zero_in_degree(graph):
            raise RuntimeError("There are 0-in-degree nodes in the graph; add self loops first")
        if (self._fused and self._norm == "both" and self.weight is not None and self._in_feats > self._out_feats
                and feat.dim() == 2):
            relu = self._activation in (F.relu, torch.relu)
            rst = _gcn_conv_fused.apply(graph, feat, self.weight, self.bias, _cached_norm(graph, "out"),
                                        _cached_norm(graph, "in"), relu)
            if self._activation is not None and not relu:
                rst = self._activation(rst)
            return rst
        feat_src = feat
        if self._norm in ("left", "both"):
            feat_src = feat_src * _norm(graph.out_degrees(), self._norm == "both").unsqueeze(1)
        if self._in_feats > self._out_feats:
            if self.weight is not None:
                feat_src, s = Qlinear_func_reduce.apply(feat_src, self.weight)
                rst = spmm_copy_u.apply(graph, feat_src, s)
            else:
                rst = spmm_copy_u.apply(graph, feat_src)
        else:
            rst = spmm_copy_u.apply(graph, feat_src)
            if self.weight is not None:
                rst = Qlinear_func.apply(rst, self.weight)
        if self._norm in ("right", "both"):
            rst = rst * _norm(graph.in_degrees(), self._norm == "both").unsqueeze(1)
        if self.bias is not None:
            rst = rst + self.bias
        if self._activation is not None:
            rst = self._activation(rst)
        return rst


class GCN(nn.Module):
    """Stack of QGraphConv layers (evaluation/test_gcn.py:143-175): in -> hidden (x n_layers) -> classes."""

    def __init__(self, g, in_feats, n_hidden, n_classes, n_layers, activation=F.relu, dropout=0.0, fused=True):
        super().__init__()
        self.g = g
        self.layers = nn.ModuleList()
        self.layers.append(QGraphConv(in_feats, n_hidden, activation=activation, fused=fused))
        for _ in range(n_layers - 1):
            self.layers.append(QGraphConv(n_hidden, n_hidden, activation=activation, fused=fused))
        self.layers.append(QGraphConv(n_hidden, n_classes, fused=fused))
        self.dropout = nn.Dropout(p=dropout)

    def forward(self, features):
        h = features
        for i, layer in enumerate(self.layers):
            if i != 0:
                h = self.dropout(h)
            h = layer(self.g, h)
        return h


# ---------------------------------------------------------------------------------------------------- GAT
class _edge_softmax_fn(Function):
    """Softmax of edge scores (times a constant factor) over the incoming edges of every destination, per head (the
    reference calls dgl.ops.edge_softmax, evaluation/test_gat.py:146, evaluation/test_HGT.py:60).  fp32, as in the
    reference; one team-per-row kernel per direction."""

    @staticmethod
    def forward(ctx, g, e, factor):
        a, sa = kernels.edge_softmax_fwd(g, e, factor, want_scale=True)
        ctx.save_for_backward(a)
        ctx.g, ctx.factor = g, factor
        ctx.mark_non_differentiable(sa)
        return a, sa

    @staticmethod
    @once_differentiable
    def backward(ctx, da, _dsa):
        (a,) = ctx.saved_tensors
        return None, kernels.edge_softmax_bwd(ctx.g, a, da, ctx.factor), None


def edge_softmax(g, e, factor: float = 1.0, return_scale: bool = False):
    """softmax over each destination's incoming edges of e * factor; with return_scale also max|a|/127, which the
    kernel produces on the way and the consuming spmm_u_mul_e would otherwise recompute."""
    a, sa = _edge_softmax_fn.apply(g, e, factor)
    return (a, sa) if return_scale else a


class _gat_attention_fused(Function):
    """Attention weights of a GAT layer in one pass per direction:

        a = edge_softmax(leaky_relu(Q(el)[src] + Q(er)[dst]))

    i.e. the reference's sddmm_u_add_v -> nn.LeakyReLU -> dgl.ops.edge_softmax chain (evaluation/test_gat.py:141-146)
    without materialising the logits: el / er are quantized to int8 exactly as sddmm_u_add_v does, one kernel walks
    every destination's incoming edges (max, sum, normalise), and the backward kernel produces the gradient of the
    logits, which then takes sddmm_u_add_v's backward route (int8 quantisation + incidence sums)."""

    @staticmethod
    def forward(ctx, g, el, er, slope):
        mode, seed = config.mode_for("quantize"), config.seed()
        n, h = el.shape[0], el.shape[1]
        elq, sl = kernels.quantize(el.reshape(n, h), mode=mode, seed=seed, align=1)
        erq, sr = kernels.quantize(er.reshape(n, h), mode=mode, seed=seed, align=1)
        a, sa = kernels.gat_edge_softmax(g, elq, erq, sl, sr, slope, want_scale=True)
        ctx.g, ctx.slope, ctx.shapes = g, slope, (el.shape, er.shape)
        ctx.save_for_backward(elq, erq, sl, sr, a)
        ctx.mark_non_differentiable(sa)
        return a.view(a.shape[0], h, 1), sa

    @staticmethod
    @once_differentiable
    def backward(ctx, da, _dsa):
        elq, erq, sl, sr, a = ctx.saved_tensors
        g = ctx.g
        dz, sdz = kernels.gat_edge_softmax_bwd(g, elq, erq, sl, sr, a, da, ctx.slope, want_scale=True)
        dzq, sdz = kernels.quantize(dz, sdz, mode=config.mode_for("quantize"), seed=config.seed(), align=1)
        d_el = kernels.incidence_SPMM(g, dzq, sdz, True).view(ctx.shapes[0]) if ctx.needs_input_grad[1] else None
        d_er = kernels.incidence_SPMM(g, dzq, sdz).view(ctx.shapes[1]) if ctx.needs_input_grad[2] else None
        return None, d_el, d_er, None


class _gat_aggregate_fused(Function):
    """Attention + aggregation of a GAT layer with no fp32 copy of the attention weights:

        out[v,h,:] = sum_e Q(a)[e,h] * Q(ft)[src(e),h,:],   a = edge_softmax(leaky_relu(Q(el)[src] + Q(er)[dst]))

    Same arithmetic, bit for bit, as _gat_attention_fused followed by spmm_u_mul_e (and hence the same int8 weights
    as the reference's sddmm_u_add_v -> LeakyReLU -> edge_softmax -> quantize chain, evaluation/test_gat.py:141-152,
    cuda/SPMM.py:38-47), but the weights exist only as the int8 tensor the aggregation reads: one pass keeps the
    softmax statistics of every destination (which already fix the int8 scale), a second writes the int8 weights,
    and the backward pass recomputes the weights from the statistics."""

    @staticmethod
    def forward(ctx, g, ft, el, er, slope):
        mode, seed = config.mode_for("quantize"), config.seed()
        n, h = el.shape[0], el.shape[1]
        elq, sl = kernels.quantize(el.reshape(n, h), mode=mode, seed=seed, align=1)
        erq, sr = kernels.quantize(er.reshape(n, h), mode=mode, seed=seed, align=1)
        m, inv, sa = kernels.gat_edge_softmax_stats(g, elq, erq, sl, sr, slope)
        sN = kernels.cuda_kernels.get_scale(ft)
        call = kernels.next_call() if mode == kernels.ROUND_STOCHASTIC else 0
        aq = kernels.gat_edge_softmax_quantized(g, elq, erq, sl, sr, m, inv, sa, slope, mode, seed, call)
        Nq, _ = kernels.quantize(ft, sN, mode=mode, seed=seed)
        out = kernels.spmm_u_mul_e_int8(g, Nq, aq, sN * sa)
        ctx.g, ctx.slope, ctx.shapes = g, slope, (el.shape, er.shape)
        ctx.save_for_backward(elq, erq, sl, sr, m, inv, sa, aq, Nq, sN)
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, d_out):
        elq, erq, sl, sr, m, inv, sa, aq, Nq, sN = ctx.saved_tensors
        g = ctx.g
        mode, seed = config.mode_for("quantize"), config.seed()
        dZq, sdZ = kernels.quantize(d_out, mode=mode, seed=seed)
        d_ft = kernels.spmm_u_mul_e_int8(g, dZq, aq, sdZ * sa, True) if ctx.needs_input_grad[1] else None
        d_el = d_er = None
        if ctx.needs_input_grad[2] or ctx.needs_input_grad[3]:
            da, _ = kernels.mySDDMM_int8(g, "dot", Nq, dZq, sN, sdZ, False)          # [E, H, 1] fp32
            dz, sdz = kernels.gat_edge_softmax_bwd_stats(g, elq, erq, sl, sr, m, inv, da, ctx.slope)
            dzq, sdz = kernels.quantize(dz, sdz, mode=mode, seed=seed, align=1)
            if ctx.needs_input_grad[2]:
                d_el = kernels.incidence_SPMM(g, dzq, sdz, True).view(ctx.shapes[0])
            if ctx.needs_input_grad[3]:
                d_er = kernels.incidence_SPMM(g, dzq, sdz).view(ctx.shapes[1])
        return None, d_ft, d_el, d_er, None


class QGATConv(nn.Module):
    """Graph attention layer on the quantized operators (evaluation/test_gat.py:30-169): QLinear projection,
    int8 u_add_v edge logits, LeakyReLU, edge softmax (fp32), int8 u_mul_e aggregation."""

    def __init__(self, in_feats, out_feats, num_heads, feat_drop=0.0, attn_drop=0.0, negative_slope=0.2,
                 residual=False, activation=None, allow_zero_in_degree=False, bias=True, fused=True):
        super().__init__()
        self._fused, self._slope = fused, negative_slope
        self._num_heads, self._in_feats, self._out_feats = num_heads, in_feats, out_feats
        self._allow_zero_in_degree = allow_zero_in_degree
        self.fc = QLinear(in_feats, out_feats * num_heads, bias=False)
        self.attn_l = nn.Parameter(torch.empty(1, num_heads, out_feats))
        self.attn_r = nn.Parameter(torch.empty(1, num_heads, out_feats))
        self.feat_drop = nn.Dropout(feat_drop)
        self.attn_drop = nn.Dropout(attn_drop)
        self.leaky_relu = nn.LeakyReLU(negative_slope)
        self.bias = nn.Parameter(torch.empty(num_heads * out_feats)) if bias else None
        if residual:
            self.res_fc = (QLinear(in_feats, num_heads * out_feats, bias=False)
                           if in_feats != out_feats * num_heads else nn.Identity())
        else:
            self.res_fc = None
        self.activation = activation
        self.reset_parameters()

    def reset_parameters(self):
        gain = nn.init.calculate_gain("relu")
        nn.init.xavier_normal_(self.fc.weight, gain=gain)
        nn.init.xavier_normal_(self.attn_l, gain=gain)
        nn.init.xavier_normal_(self.attn_r, gain=gain)
        if self.bias is not None:
            nn.init.constant_(self.bias, 0)
        if isinstance(self.res_fc, QLinear):
            nn.init.xavier_normal_(self.res_fc.weight, gain=gain)

    def forward(self, graph, feat, get_attention=False):
        if not self._allow_zero_in_degree and _has_zero_in_degree(graph):
            raise RuntimeError("There are 0-in-degree nodes in the graph.")
        prefix = feat.shape[:-1]
        h = self.feat_drop(feat).contiguous()
        ft = self.fc(h).view(*prefix, self._num_heads, self._out_feats)
        el = (ft * self.attn_l).sum(dim=-1).unsqueeze(-1)
        er = (ft * self.attn_r).sum(dim=-1).unsqueeze(-1)
        sa = None
        # fused="int8": the attention weights never exist in fp32 (needs no attention dropout and no caller that wants
        # the weights back); fused=True: one fused softmax pass writes them as fp32 [E, H]; fused=False: the
        # reference's operator-by-operator chain
        int8_path = (self._fused == "int8" and not get_attention
                     and not (self.training and self.attn_drop.p > 0))
        if int8_path:
            rst = _gat_aggregate_fused.apply(graph, ft, el, er, self._slope)
        else:
            if self._fused:
                a, sa = _gat_attention_fused.apply(graph, el, er, self._slope)
                if self.training and self.attn_drop.p > 0:
                    a, sa = self.attn_drop(a), None   # dropout rescales a: its absmax has to be taken again
            else:
                e = self.leaky_relu(sddmm_u_add_v.apply(graph, el, er))
                a = self.attn_drop(edge_softmax(graph, e))
            rst = spmm_u_mul_e.apply(graph, ft, a, sa)
        if self.res_fc is not None:
            rst = rst + self.res_fc(h).view(*prefix, -1, self._out_feats)
        if self.bias is not None:
            rst = rst + self.bias.view(*((1,) * len(prefix)), self._num_heads, self._out_feats)
        if self.activation:
            rst = self.activation(rst)
        return (rst, a) if get_attention else rst      # (get_attention never takes the int8 path, so `a` exists)


class GAT(nn.Module):
    """evaluation/test_gat.py:172-224."""

    def __init__(self, g, num_layers, in_dim, num_hidden, num_classes, heads, activation=F.elu, feat_drop=0.0,
                 attn_drop=0.0, negative_slope=0.2, residual=False, fused=True):
        super().__init__()
        self.g, self.num_layers = g, num_layers
        self.gat_layers = nn.ModuleList()
        if num_layers > 1:
            self.gat_layers.append(QGATConv(in_dim, num_hidden, heads[0], feat_drop, attn_drop, negative_slope,
                                            False, activation, fused=fused))
            for l in range(1, num_layers - 1):
                self.gat_layers.append(QGATConv(num_hidden * heads[l - 1], num_hidden, heads[l], feat_drop, attn_drop,
                                                negative_slope, residual, activation, fused=fused))
            self.gat_layers.append(QGATConv(num_hidden * heads[-2], num_classes, heads[-1], feat_drop, attn_drop,
                                            negative_slope, residual, None, fused=fused))
        else:
            self.gat_layers.append(QGATConv(in_dim, num_classes, heads[0], feat_drop, attn_drop, negative_slope,
                                            residual, None))

    def forward(self, inputs):
        h = inputs
        for l in range(self.num_layers - 1):
            h = self.gat_layers[l](self.g, h).flatten(1)
        return self.gat_layers[-1](self.g, h).mean(1)


# ---------------------------------------------------------------------------------------------------- HGT
class HGT(nn.Module):
    """Single-relation heterogeneous-graph-transformer layer of evaluation/test_HGT.py:27-67: six QLinear
    projections, int8 per-head dot-product scores (sddmm_u_dot_v), 1/sqrt(d_k), edge softmax over each destination's
    incoming edges (fp32, as in the reference), int8 attention-weighted aggregation (spmm_u_mul_e)."""

    def __init__(self, in_dim, out_dim, n_heads, dropout=0.2, use_norm=False):
        super().__init__()
        assert out_dim % n_heads == 0, "out_dim must be a multiple of n_heads"
        self.in_dim, self.out_dim, self.n_heads = in_dim, out_dim, n_heads
        self.d_k = out_dim // n_heads
        self.sqrt_dk = math.sqrt(self.d_k)
        self.q_linear = QLinear(in_dim, out_dim)
        self.k_linear = QLinear(in_dim, out_dim)
        self.v_linear = QLinear(in_dim, out_dim)
        self.msg_linear = QLinear(out_dim, out_dim)
        self.attn_linear = QLinear(out_dim, out_dim)
        self.a_linear = QLinear(out_dim, out_dim)
        self.norm = nn.LayerNorm(out_dim) if use_norm else nn.Identity()

    def forward(self, g, h):
        k = self.attn_linear(self.k_linear(h)).view(-1, self.n_heads, self.d_k)
        v = self.msg_linear(self.v_linear(h)).view(-1, self.n_heads, self.d_k)
        q = self.q_linear(h).view(-1, self.n_heads, self.d_k)
        t = sddmm_u_dot_v.apply(g, k, q)
        attn, s_attn = edge_softmax(g, t, 1.0 / self.sqrt_dk, True)   # the reference divides t by sqrt(d_k) first
        out = spmm_u_mul_e.apply(g, v, attn, s_attn).view(-1, self.out_dim)
        return self.a_linear(out)


# ---------------------------------------------------------------------------------------------------- link prediction
def construct_negative_graph(graph, k, generator=None):
    """k random destinations per source of every edge (evaluation/link_pred_gcn.py:160-165) as a `Graph` over the
    same nodes, preprocessed for the quantized operators."""
    from .graph import Graph
    from .util import graph_preprocess
    src, _ = graph.coo
    neg_src = src.long().repeat_interleave(k)
    neg_dst = torch.randint(0, graph.num_nodes(), (neg_src.numel(),), device=src.device, generator=generator)
    return graph_preprocess(Graph(neg_src, neg_dst, graph.num_nodes()))


class LinkPredGCN(nn.Module):
    """GCN encoder plus dot-product edge scorer (evaluation/link_pred_gcn.py:113-147): node embeddings from
    QGraphConv layers on the positive graph, then score[e] = <h[src(e)], h[dst(e)]> on int8 operands for the edges
    of the positive and of the negative graph.  Returns (pos_score [E+,1,1], neg_score [E-,1,1])."""

    def __init__(self, in_feats, n_hidden, n_classes, n_layers, activation=F.relu, dropout=0.0):
        super().__init__()
        self.layers = nn.ModuleList([QGraphConv(in_feats, n_hidden, activation=activation)])
        for _ in range(n_layers - 1):
            self.layers.append(QGraphConv(n_hidden, n_hidden, activation=activation))
        self.layers.append(QGraphConv(n_hidden, n_classes))
        self.dropout = nn.Dropout(p=dropout)

    def forward(self, features, pos_graph, neg_graph):
        h = features
        for i, layer in enumerate(self.layers):
            if i != 0:
                h = self.dropout(h)
            h = layer(pos_graph, h)
        h = h.unsqueeze(1)
        return sddmm_u_dot_v.apply(pos_graph, h, h), sddmm_u_dot_v.apply(neg_graph, h, h)


def link_pred_loss(pos_score, neg_score):
    """Binary cross-entropy on the logits, positives labelled 1 and negatives 0 (evaluation/link_pred_gcn.py:150-157)."""
    score = torch.cat([pos_score, neg_score])
    label = torch.cat([torch.ones_like(pos_score), torch.zeros_like(neg_score)])
    return F.binary_cross_entropy_with_logits(score, label)

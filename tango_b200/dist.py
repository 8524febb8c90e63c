"""1-D row-partitioned full-graph training over the GPUs of one node (one process per GPU, torch.distributed).

The reference is single-GPU only.  Here rank r owns a contiguous block of nodes: their feature rows, the CSC rows of
the adjacency (forward aggregation) and the CSR rows (backward aggregation), both with global column ids.  The only
data-path exchange is one all-gather per aggregation of the int8-quantized feature shard plus its fp32 scale; the
aggregation kernel then applies the scale of the shard each neighbour came from.  Weight gradients are summed with
an all-reduce after the backward pass.

Two transports carry that exchange: torch.distributed collectives (NCCL on GPUs, gloo on CPU), or -- on the GPUs of
one node, `transport="peer"` -- quantizer kernels that store into every GPU's gathered table over NVLink plus a
one-CTA rendezvous kernel for the barrier and the scale agreement (tango_b200.peer).
"""
from __future__ import annotations

import warnings
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F
from torch.autograd.function import Function, once_differentiable

from . import config
from .graph import HUB_BLOCK_MIN_DENSITY, Graph, HubBlock, RowPartition, balanced_bounds, uniform_bounds


HUB_BLOCK_MIN_EDGES = 4_000_000     # smaller graphs are launch-bound: the dense hub block would not pay for its launches


def all_gather_quantized(q_local: torch.Tensor, s_local: torch.Tensor, shard_rows: int, group=None,
                         gather_scales: bool = True):
    """Gathers every rank's int8 shard ([<= shard_rows, ld], same ld everywhere) and scale.

    Returns (q_all [world * shard_rows, ld], scales [world]); rank k's rows start at k * shard_rows.  Works on any
    backend (NCCL on GPUs, gloo on CPU)."""
    world = dist.get_world_size(group)
    ld = q_local.shape[1]
    q_all = torch.empty((world * shard_rows, ld), dtype=torch.int8, device=q_local.device)
    if q_local.shape[0] == shard_rows and q_local.is_contiguous():
        send = q_local
    else:
        send = torch.zeros((shard_rows, ld), dtype=torch.int8, device=q_local.device)
        send[:q_local.shape[0]] = q_local
    dist.all_gather_into_tensor(q_all, send, group=group)
    if not gather_scales:
        return q_all, s_local
    scales = torch.empty(world, dtype=torch.float32, device=s_local.device)
    dist.all_gather_into_tensor(scales, s_local.reshape(1).contiguous(), group=group)
    return q_all, scales


class DistGraph:
    """Rank-local view of a graph that every rank holds (or can rebuild from the same seed)."""

    def __init__(self, g: Graph, rank: int, world: int, balance: str = "dealt", scale_mode: str = "global",
                 transport: str = "nccl"):
        """balance='dealt': nodes sorted by in-degree + out-degree are dealt round-robin to the ranks (equal rows,
        nearly equal edges even on power-law graphs, no padding of the gathered buffer);
        balance='cyclic': node v lives on rank v % world;
        balance='nnz': contiguous blocks of equal cost (in-degree + out-degree + 300 per row for the dense per-row
        work); balance='rows': contiguous blocks of equal row counts.
        scale_mode='global': the ranks agree on one quantisation scale per aggregated tensor (all-reduce max of one
        float), which makes the result bit-identical to the single-GPU run; scale_mode='shard': every shard keeps its
        own scale and the aggregation kernel applies the scale of the shard a neighbour came from.
        transport='nccl': all-gather / all-reduce through torch.distributed; transport='peer' (global scale mode, one
        node, CUDA devices): the quantizers store straight into every GPU's gathered table over NVLink and the ranks
        meet in a one-CTA rendezvous kernel (tango_b200.peer) -- no library collective on the data path;
        transport='auto': 'peer' when it applies and its set-up succeeds on every rank, else 'nccl'."""
        assert scale_mode in ("global", "shard")
        assert transport in ("nccl", "peer", "auto")
        if transport == "auto":      # peer memory where it applies, NCCL otherwise (decided alike on all ranks)
            transport = "peer" if (scale_mode == "global" and world > 1 and g.device.type == "cuda") else "nccl"
            self._fallback = True
        else:
            self._fallback = False
        assert transport == "nccl" or scale_mode == "global", "the peer transport implements the global scale mode"
        self.peer = None
        n = g.num_nodes()
        self.rank, self.world, self.n_total, self.scale_mode = rank, world, n, scale_mode
        csc, csr = g.adj_csc, g.adj_csr
        assert balance in ("dealt", "cyclic", "nnz", "rows")
        layout = balance if balance in ("cyclic", "dealt") else "block"
        bounds, order = None, None
        if balance == "dealt":
            order = torch.argsort(g.in_degrees() + g.out_degrees(), descending=True, stable=True)
        if balance == "nnz":
            bounds = balanced_bounds(g.in_degrees() + g.out_degrees() + 300, world)
        elif balance == "rows":
            bounds = uniform_bounds(n, world)
        self.bounds = bounds
        self.fwd = RowPartition(csc[0], csc[1], None, n, rank, world, bounds, layout, order)
        self.bwd = RowPartition(csr[0], csr[1], None, n, rank, world, bounds, layout, order)
        self.shard_rows, self.n_local, self.local_ids = self.fwd.shard_rows, self.fwd.n_local, self.fwd.local_ids
        self.r0, self.r1 = self.fwd.r0, self.fwd.r1
        # dense hub block of this rank's rows (global scale mode: one scale, unsegmented rows): the rank's longest
        # rows x the most referenced rows of the gathered table, multiplied on the tensor cores
        self.hubs = {}
        side = config.hub_block()
        if scale_mode == "global" and side > 0 and g.device.type == "cuda" and g.num_edges() >= HUB_BLOCK_MIN_EDGES:
            for key, part in (("fwd", self.fwd), ("bwd", self.bwd)):
                # The region is an optimisation with a bit-identical result, decided per rank with no collective: a
                # rank that cannot build it, or whose region does not reproduce the gathered aggregation, goes
                # without (and says so) while the other ranks keep theirs.
                from . import kernels
                try:
                    hub = HubBlock(part.indptr_flat, part.indices, world * self.shard_rows, side, side,
                                   HUB_BLOCK_MIN_DENSITY)
                    if hub.ok and kernels.hub_self_check(hub, part.indptr_flat, part.indices, part.schedule_flat,
                                                         world * self.shard_rows):
                        self.hubs[key] = hub
                    elif hub.ok:
                        warnings.warn(f"rank {rank}: dense hub region of the {key} aggregation did not reproduce the "
                                      "gathered result; not used", RuntimeWarning)
                except (RuntimeError, AssertionError, IndexError, ValueError) as exc:
                    warnings.warn(f"rank {rank}: dense hub region of the {key} aggregation not built: {exc}",
                                  RuntimeWarning)
        self.in_norm = g.in_degrees()[self.local_ids].float().clamp(min=1).pow(-0.5).contiguous()
        self.out_norm = g.out_degrees()[self.local_ids].float().clamp(min=1).pow(-0.5).contiguous()
        if transport == "peer" and world > 1:
            from .peer import PeerTransport
            try:
                self.peer = PeerTransport(rank, world, self.in_norm.device)
            except RuntimeError:
                if not self._fallback:
                    raise
                self.peer = None     # the set-up fails on all ranks or on none, so all of them fall back to NCCL
        self.transport = "peer" if self.peer is not None else "nccl"

    def close(self) -> None:
        """Releases the peer-memory buffers of this partition (a collective; no kernel may be in flight)."""
        if self.peer is not None:
            self.peer.close()
            self.peer = None


def _padded_storage(q: torch.Tensor) -> torch.Tensor:
    """The [rows, ld] storage behind an int8 tensor returned by kernels.quantize."""
    ld = q.stride(0)
    return torch.as_strided(q, (q.shape[0], ld), (ld, 1))


class dist_spmm_copy_u(Function):
    """spmm_copy_u over a row partition: quantize the local shard, all-gather int8 shards + scales, aggregate the
    local rows.  Backward does the same on the transposed partition."""

    @staticmethod
    def forward(ctx, dg: DistGraph, x_local, scale_local=None):
        ctx.dg = dg
        return _aggregate(dg, dg.fwd, x_local, scale_local)

    @staticmethod
    @once_differentiable
    def backward(ctx, dz):
        dg = ctx.dg
        dn = _aggregate(dg, dg.bwd, dz.contiguous(), None) if ctx.needs_input_grad[1] else None
        return None, dn, None


def _aggregate(dg: DistGraph, part: RowPartition, x_local: torch.Tensor, scale_local: Optional[torch.Tensor],
               row_scale=None, bias=None, relu=False, in_row_scale=None):
    """Quantize the local rows (optionally times in_row_scale[r]) with the local scale, all-gather the int8 shards
    and scales, aggregate this rank's rows; row_scale / bias / relu go to the aggregation's epilogue."""
    from . import kernels as K
    mode, seed = config.mode_for("quantize"), config.seed()
    x_local = x_local.contiguous()
    if scale_local is None:
        scale_local = K._get_scale(x_local, in_row_scale)
    scale_local = _agree_on_scale(dg, scale_local)
    call = K.next_call() if mode == K.ROUND_STOCHASTIC else 0
    if dg.peer is not None:
        f = x_local.shape[1]
        table, ptrs, ld = _peer_table(dg, part, f)
        dg.peer.quantize_push(x_local, scale_local, ptrs, dg.rank * dg.shard_rows, ld, mode, seed, call, in_row_scale)
        dg.peer.barrier()
        return _spmm_gathered(dg, part, table, scale_local, f, row_scale, bias, relu)
    q = K.alloc_int8(x_local.shape, x_local.device)
    K._quantize_into(q, x_local, scale_local, mode, seed, call, in_row_scale)
    return _aggregate_quantized(dg, part, q, scale_local, x_local.shape[1], row_scale, bias, relu)


def _peer_table(dg: DistGraph, part: RowPartition, f: int):
    """(this rank's gathered int8 table for aggregations of width f over `part`, every rank's table address, ld)."""
    ld = (f + 15) // 16 * 16
    table, ptrs = dg.peer.table(("fwd" if part is dg.fwd else "bwd", ld), dg.world * dg.shard_rows, ld)
    return table, ptrs, ld


def _spmm_gathered(dg: DistGraph, part: RowPartition, q_all: torch.Tensor, scales: torch.Tensor, f: int,
                   row_scale=None, bias=None, relu=False):
    """Aggregates this rank's rows from the gathered int8 table (one scale, or one per shard in shard mode)."""
    from . import kernels as K
    out = torch.empty((dg.n_local, f), dtype=torch.float32, device=q_all.device)
    feats = q_all[:, :f] if q_all.shape[1] != f else q_all
    if dg.scale_mode == "global":
        hub = dg.hubs.get("fwd" if part is dg.fwd else "bwd")
        if hub is not None and q_all.shape[1] == (f + 15) // 16 * 16:
            K._csr_spmm(out, hub.indptr, hub.indices, feats, scales, hub.schedule, 1, row_scale, bias, relu)
        else:
            K._csr_spmm(out, part.indptr_flat, part.indices, feats, scales, part.schedule_flat, 1, row_scale, bias, relu)
    else:
        K._csr_spmm(out, part.indptr, part.indices, feats, scales, part.schedule, dg.world, row_scale, bias, relu)
    return out


def _agree_on_scale(dg: DistGraph, scale_local: torch.Tensor) -> torch.Tensor:
    """global scale mode: the largest local scale becomes everybody's scale (one-float all-reduce)."""
    if dg.scale_mode != "global":
        return scale_local
    if dg.peer is not None:
        return dg.peer.max_scalar(scale_local)
    s = scale_local.clone()
    dist.all_reduce(s, op=dist.ReduceOp.MAX)
    return s


def _aggregate_quantized(dg: DistGraph, part: RowPartition, q: torch.Tensor, scale_local: torch.Tensor, f: int,
                         row_scale=None, bias=None, relu=False):
    """All-gather the int8 shard `q` (and its scale in shard mode) and aggregate this rank's rows."""
    from . import kernels as K
    shared = dg.scale_mode == "global"
    q_all, scales = all_gather_quantized(_padded_storage(q), scale_local, dg.shard_rows, gather_scales=not shared)
    return _spmm_gathered(dg, part, q_all, scale_local if shared else scales, f, row_scale, bias, relu)


class _dist_gcn_conv_fused(Function):
    """The fused "multiply first" graph convolution of tango_b200.gnn on a row partition: left norm folded into the
    quantizer of the local features, int8 GEMM with output scale, all-gather of the int8 shard, aggregation with the
    right norm + bias + ReLU in its epilogue.  The backward pass mirrors it on the transposed partition."""

    @staticmethod
    def forward(ctx, dg, X, W, b, relu):
        from . import kernels as K
        mode_f, mode_q, seed = config.mode_for("gemm_fwd"), config.mode_for("quantize"), config.seed()
        call = K.next_call() if mode_f == K.ROUND_STOCHASTIC else 0
        if mode_f == K.ROUND_STOCHASTIC:
            K.next_call()
        X = X.contiguous()
        sX, sW = _agree_on_scale(dg, K._get_scale(X, dg.out_norm)), K._get_scale(W)
        Xq, Wq = K.alloc_int8(X.shape, X.device), K.alloc_int8(W.shape, X.device)
        H = torch.empty((X.shape[0], W.shape[0]), dtype=torch.float32, device=X.device)
        sH = torch.zeros(1, dtype=torch.float32, device=X.device)
        K._qgemm_forward(H, X, Xq, W.contiguous(), Wq, None, sH, sX, sW, mode_f, seed, call, dg.out_norm)
        out = _aggregate(dg, dg.fwd, H, sH, dg.in_norm, b, relu)
        ctx.dg, ctx.relu, ctx.has_bias = dg, relu, b is not None
        ctx.save_for_backward(Xq, sX, Wq, sW, out if relu else None)
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, d_out):
        from . import kernels as K
        dg = ctx.dg
        Xq, sX, Wq, sW, out = ctx.saved_tensors
        mode_q, seed = config.mode_for("quantize"), config.seed()
        want_db = ctx.has_bias and ctx.needs_input_grad[3]
        if ctx.relu:
            call = K.next_call() if mode_q == K.ROUND_STOCHASTIC else 0
            s_loc, db = K.relu_grad_stats(d_out, out, dg.in_norm, want_db)
            s_loc = _agree_on_scale(dg, s_loc)
            if dg.peer is not None:
                f = d_out.shape[1]
                table, ptrs, ld = _peer_table(dg, dg.bwd, f)
                dg.peer.relu_grad_quantize_push(d_out, out, s_loc, ptrs, dg.rank * dg.shard_rows, ld, mode_q, seed,
                                                call, dg.in_norm)
                dg.peer.barrier()
                dH = _spmm_gathered(dg, dg.bwd, table, s_loc, f)
            else:
                dZq = K.relu_grad_quant(d_out, out, dg.in_norm, s_loc, mode_q, seed, call)
                dH = _aggregate_quantized(dg, dg.bwd, dZq, s_loc, d_out.shape[1])
        else:
            g1 = d_out.contiguous()
            db = g1.sum(0) if want_db else None
            dH = _aggregate(dg, dg.bwd, g1, None, None, None, False, in_row_scale=dg.in_norm)
        sdH = _agree_on_scale(dg, K._get_scale(dH))
        dHq, _ = K.quantize(dH, sdH, mode=mode_q, seed=seed)
        dX, dW = K.QGEMM_backward(dHq, Xq, Wq, sdH, sX, sW, ctx.needs_input_grad[1], ctx.needs_input_grad[2],
                                  dx_row_scale=dg.out_norm)
        return None, dX, dW, db, None


class DistQGraphConv(nn.Module):
    """QGraphConv (norm='both') on a row partition."""

    def __init__(self, in_feats, out_feats, activation=None):
        super().__init__()
        self._in_feats, self._out_feats, self._activation = in_feats, out_feats, activation
        self.weight = nn.Parameter(torch.empty(out_feats, in_feats))
        self.bias = nn.Parameter(torch.zeros(out_feats))
        nn.init.xavier_uniform_(self.weight)

    def forward(self, dg: DistGraph, feat_local):
        from .QLinear import Qlinear_func
        if self._in_feats > self._out_feats:
            relu = self._activation in (F.relu, torch.relu)
            rst = _dist_gcn_conv_fused.apply(dg, feat_local, self.weight, self.bias, relu)
            return self._activation(rst) if (self._activation is not None and not relu) else rst
        h = feat_local * dg.out_norm.unsqueeze(1)
        rst = Qlinear_func.apply(dist_spmm_copy_u.apply(dg, h), self.weight)
        rst = rst * dg.in_norm.unsqueeze(1) + self.bias
        return self._activation(rst) if self._activation is not None else rst


class DistGCN(nn.Module):
    def __init__(self, dg: DistGraph, in_feats, n_hidden, n_classes, n_layers=1, activation=F.relu):
        super().__init__()
        self.dg = dg
        dims = [in_feats] + [n_hidden] * n_layers + [n_classes]
        self.layers = nn.ModuleList(
            DistQGraphConv(dims[i], dims[i + 1], activation if i < len(dims) - 2 else None) for i in range(len(dims) - 1))

    def forward(self, feat_local):
        h = feat_local
        for layer in self.layers:
            h = layer(self.dg, h)
        return h


def allreduce_grads(module: nn.Module, group=None, peer=None) -> None:
    """Sums the parameter gradients over the ranks (each rank holds the contribution of its rows).  With `peer` (a
    PeerTransport) the rank's rendezvous status word rides along in the same all-reduce, so that after the step every
    rank knows whether ANY rank gave up a wait (`peer.raise_if_expired()`); no extra collective, no synchronisation."""
    grads = [p.grad for p in module.parameters() if p.grad is not None]
    if not grads:
        return
    parts = [g.reshape(-1) for g in grads]
    if peer is not None:
        parts.append(peer.status_word().float().abs())
    flat = torch.cat(parts)
    dist.all_reduce(flat, group=group)
    off = 0
    for g in grads:
        g.copy_(flat[off:off + g.numel()].view_as(g))
        off += g.numel()
    if peer is not None:
        peer.group_status.add_(flat[off:off + 1])

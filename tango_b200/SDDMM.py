"""Quantized edge-score operators: the autograd surface of the reference's cuda/SDDMM.py, plus `sddmm_u_dot_v`,
which the reference's HGT and link-prediction scripts call (evaluation/test_HGT.py:58) but never define."""
from __future__ import annotations

from torch.autograd.function import Function, once_differentiable

from . import config
from .kernels import *  # noqa: F401,F403  (the reference's module re-exports its kernels the same way)
from .kernels import incidence_SPMM, mySDDMM_int8, quantize, spmm_u_mul_e_int8


def _q(t, scale=None, align=16):
    return quantize(t, scale, mode=config.mode_for("quantize"), seed=config.seed(), align=align)


class sddmm_u_add_v(Function):
    """e[k] = U[src(k)] + V[dst(k)] on int8 operands (cuda/SDDMM.py:10-32); the gradients are the sums of dZ over
    the out-edges (dU) and in-edges (dV) of each node."""

    @staticmethod
    def forward(ctx, g, U, V, scaleU_=None, scaleV_=None):
        narrow = 1 if U[0].numel() < 16 else 16
        Uq, sU = _q(U, scaleU_, narrow)
        Vq, sV = (Uq, sU) if U is V else _q(V, scaleV_, narrow)
        out, _ = mySDDMM_int8(g, "add", Uq, Vq, sU, sV, False)
        ctx.backward_cache = g
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, dZ):
        g = ctx.backward_cache
        dZq, sdZ = _q(dZ, None, 1 if dZ[0].numel() < 16 else 16)
        dU = incidence_SPMM(g, dZq, sdZ, True) if ctx.needs_input_grad[1] else None
        dV = incidence_SPMM(g, dZq, sdZ) if ctx.needs_input_grad[2] else None
        return None, dU, dV, None, None


class sddmm_u_dot_v(Function):
    """e[k,h] = <U[src(k),h,:], V[dst(k),h,:]> on int8 operands.  Backward: dU[u] = sum over out-edges of
    dZ[k] * V[dst(k)], dV[v] = sum over in-edges of dZ[k] * U[src(k)], both as int8 weighted SpMMs."""

    @staticmethod
    def forward(ctx, g, U, V):
        Uq, sU = _q(U)
        Vq, sV = (Uq, sU) if U is V else _q(V)
        out, _ = mySDDMM_int8(g, "dot", Uq, Vq, sU, sV, False)
        ctx.backward_cache = (g, Uq, sU, Vq, sV)
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, dZ):
        g, Uq, sU, Vq, sV = ctx.backward_cache
        dZq, sdZ = _q(dZ.reshape(dZ.shape[0], -1), None, 1)
        three_d = Uq.dim() == 3
        U3 = Uq if three_d else Uq.unsqueeze(1)
        V3 = Vq if three_d else Vq.unsqueeze(1)
        dU = dV = None
        if ctx.needs_input_grad[1]:
            dU = spmm_u_mul_e_int8(g, V3, dZq, sV * sdZ, True)
            dU = dU if three_d else dU.squeeze(1)
        if ctx.needs_input_grad[2]:
            dV = spmm_u_mul_e_int8(g, U3, dZq, sU * sdZ)
            dV = dV if three_d else dV.squeeze(1)
        return None, dU, dV

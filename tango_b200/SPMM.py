"""Quantized aggregation operators: the autograd surface of the reference's cuda/SPMM.py."""
from __future__ import annotations

from torch.autograd.function import Function, once_differentiable

from . import config
from .kernels import *  # noqa: F401,F403  (the reference's module re-exports its kernels the same way)
from .kernels import cuda_kernels, csr_SPMM, mySDDMM_int8, quantize, spmm_u_mul_e_int8


def _q(t, scale=None, align=16):
    return quantize(t, scale, mode=config.mode_for("quantize"), seed=config.seed(), align=align)


class spmm_copy_u(Function):
    """out[v] = sum of the int8-quantized features of v's in-neighbours (cuda/SPMM.py:8-24)."""

    @staticmethod
    def forward(ctx, g, N, scaleN=None):
        Nq, scaleN = _q(N, scaleN)
        ctx.backward_cache = g
        return csr_SPMM(g, Nq, scaleN)

    @staticmethod
    @once_differentiable
    def backward(ctx, dZ):
        g = ctx.backward_cache
        dN = None
        if ctx.needs_input_grad[1]:
            dZq, sdZ = _q(dZ)
            dN = csr_SPMM(g, dZq, sdZ, True)
        return None, dN, None


def _need_reduce_last_dim(ufeat, efeat):
    """True when the edge feature broadcasts over the node feature's last dim, so dE is a per-head dot product
    (cuda/SPMM.py:26-34)."""
    if ufeat is None or efeat is None:
        return False
    us, es = ufeat.shape, efeat.shape
    return us[1:-1] == es[1:-1] and es[-1] == 1 and us[-1] > 1


class spmm_u_mul_e(Function):
    """out[v,h,:] = sum_e E[e,h] * N[src(e),h,:] with both operands int8 (cuda/SPMM.py:36-62).

    `compat_dn_scale=True` reproduces the reference's backward, which scales dN with the forward product
    s(N)*s(E) (cuda/SPMM.py:52,56) instead of s(dZ)*s(E); the default uses the consistent scale."""

    compat_dn_scale = False

    @staticmethod
    def forward(ctx, g, N, E, scaleE_=None):
        sN = cuda_kernels.get_scale(N)
        sE = cuda_kernels.get_scale(E) if scaleE_ is None else scaleE_     # producer already knows max|E|/127
        Eq, _ = _q(E.reshape(E.shape[0], -1), sE, 1)          # [E, H] int8, edge-id order (no transposed copy)
        Nq, _ = _q(N, sN)
        scale = sN * sE
        out = spmm_u_mul_e_int8(g, Nq, Eq, scale)
        ctx.backward_cache = (g, Nq, sN, Eq, sE, scale, _need_reduce_last_dim(N, E), E.shape)
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, dZ):
        g, Nq, sN, Eq, sE, scale, reduce_last, eshape = ctx.backward_cache
        dZq, sdZ = _q(dZ)
        dN = dE = None
        if ctx.needs_input_grad[1]:
            s = scale if spmm_u_mul_e.compat_dn_scale else sdZ * sE
            dN = spmm_u_mul_e_int8(g, dZq, Eq, s, True)
        if ctx.needs_input_grad[2]:
            op = "dot" if reduce_last else "mul"
            dE, _ = mySDDMM_int8(g, op, Nq, dZq, sN, sdZ, False)
            dE = dE.reshape(eshape)
        return None, dN, dE, None

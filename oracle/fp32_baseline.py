"""The reference's fp32 formulation of the same operators, restated in plain PyTorch CPU ops.

TEST / BENCHMARK INFRASTRUCTURE ONLY (the timed CPU baseline and an fp32 cross-check); never imported by the product.

The reference's evaluation scripts compare the quantized operators with DGL's fp32 ones
(dgl.ops.u_mul_e_sum / copy_e_sum / u_add_v / u_dot_v / edge_softmax, GraphConv, GATConv, nn.Linear:
evaluation/SPMM_broadcast.py:24, evaluation/test_incidence.py:28, evaluation/SDDMM_test.py:24-28,
evaluation/linear_test.py:14, evaluation/test_gcn.py:155, evaluation/test_gat.py:191).  DGL cannot be installed
here, so the same formulas (evaluation/test_gcn.py:86-137, evaluation/test_gat.py:134-165) are written with
torch.sparse CSR products, gathers and index_add_.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def csr_matrix(indptr, indices, n_cols, values=None):
    indptr = indptr.to(torch.int64).cpu()
    indices = indices.to(torch.int64).cpu()
    if values is None:
        values = torch.ones(indices.numel(), dtype=torch.float32)
    return torch.sparse_csr_tensor(indptr, indices, values, size=(indptr.numel() - 1, n_cols))


class _SpMM(torch.autograd.Function):
    """out = A @ x with A fixed; backward uses the transposed matrix given explicitly (CSR of the reverse graph)."""

    @staticmethod
    def forward(ctx, a, a_t, x):
        ctx.a_t = a_t
        return a @ x

    @staticmethod
    def backward(ctx, g):
        return None, None, ctx.a_t @ g


def spmm_copy_u(a, a_t, x):
    return _SpMM.apply(a, a_t, x)


def sddmm_dot(src, dst, u, v):
    return (u[src.long()] * v[dst.long()]).sum(-1)


def sddmm_add(src, dst, u, v):
    return u[src.long()] + v[dst.long()]


def incidence_sum(node_of_edge, e, n_nodes):
    out = torch.zeros((n_nodes,) + e.shape[1:], dtype=e.dtype)
    return out.index_add_(0, node_of_edge.long(), e)


def edge_softmax(dst, e, n_nodes):
    dst = dst.long()
    e2 = e.reshape(e.shape[0], -1)
    idx = dst.unsqueeze(1).expand_as(e2)
    m = torch.full((n_nodes, e2.shape[1]), float("-inf")).scatter_reduce(0, idx, e2, "amax")
    ex = torch.exp(e2 - m[dst])
    s = torch.zeros((n_nodes, e2.shape[1])).index_add_(0, dst, ex)
    return (ex / s[dst]).reshape(e.shape)


class GCNfp32(torch.nn.Module):
    """2-layer (or deeper) GraphConv stack with norm='both' in fp32 (evaluation/test_gcn.py:86-137 without the
    quantized operators).  `a` = CSC-as-CSR adjacency (rows = destinations), `a_t` = its transpose."""

    def __init__(self, a, a_t, out_deg, in_deg, weights, biases):
        super().__init__()
        self.a, self.a_t = a, a_t
        self.on = out_deg.float().clamp(min=1).pow(-0.5).unsqueeze(1).cpu()
        self.inn = in_deg.float().clamp(min=1).pow(-0.5).unsqueeze(1).cpu()
        self.weights = torch.nn.ParameterList([torch.nn.Parameter(w.detach().cpu().clone()) for w in weights])
        self.biases = torch.nn.ParameterList([torch.nn.Parameter(b.detach().cpu().clone()) for b in biases])

    def forward(self, x):
        h = x
        n = len(self.weights)
        for i, (w, b) in enumerate(zip(self.weights, self.biases)):
            h = h * self.on
            if w.shape[1] > w.shape[0]:
                h = spmm_copy_u(self.a, self.a_t, F.linear(h, w))
            else:
                h = F.linear(spmm_copy_u(self.a, self.a_t, h), w)
            h = h * self.inn + b
            if i < n - 1:
                h = torch.relu(h)
        return h

"""Single-head SpMM / SDDMM (reference: operators/spmm.py, src/sddmm/sddmm.cu).

The reference's ``csrspmm`` cannot be imported (its sources src/spmm/spmm.cpp and
spmm_kernel.cu are absent, operators/spmm.py:13-33 falls back to ``None``) and its
backward returns a bound method (:66).  This module implements the documented
semantics: ``out = A @ x`` with optional edge weights, ``grad_x = A^T @ grad_out``,
``grad_w[e] = <grad_out[row(e)], x[col(e)]>``.
"""
from __future__ import annotations

import torch

from .. import _capi as capi
from .csr2csc import csr2csc
from .mhspmm import mhsddmm_forward, mhspmm_forward

I32, F32 = torch.int32, torch.float32


def csr_spmm(rowptr, colind, edge_weight, x, perm=None):
    att = None if edge_weight is None else edge_weight.reshape(-1, 1)
    return mhspmm_forward(rowptr, colind, att, x.unsqueeze(1), perm=perm).squeeze(1)


def csr_sddmm(rowptr, colind, d1, d2):
    """out[e] = <d1[row(e)], d2[colind[e]]> — sddmm.csr_sddmm (src/sddmm/sddmm.cpp:29-44)."""
    return mhsddmm_forward(rowptr, colind, d1.unsqueeze(1).contiguous(),
                           d2.unsqueeze(1).contiguous()).squeeze(1)


def coo_sddmm(rowind, colind, d1, d2):
    """out[e] = <d1[rowind[e]], d2[colind[e]]> — sddmm.coo_sddmm (src/sddmm/sddmm.cpp:12-27)."""
    dev = d1.device
    capi.require(d1, F32, "D1", 2)
    capi.require(d2, F32, "D2", 2, dev)
    capi.require(rowind, I32, "rowind", 1, dev)
    capi.require(colind, I32, "colind", 1, dev)
    nnz = colind.numel()
    out = torch.empty(nnz, dtype=F32, device=dev)
    with torch.cuda.device(dev):
        capi.call("gnn_sddmm_coo", capi.ptr(rowind), capi.ptr(colind), nnz, capi.ptr(d1),
                  capi.ptr(d2), d1.shape[1], capi.ptr(out), capi.stream_ptr(dev))
    return out


class SPMMFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rowptr, colind, feat, edge_weight_csr=None, sym=False):
        feat = feat.contiguous()
        if edge_weight_csr is not None:
            edge_weight_csr = edge_weight_csr.contiguous()
        out = csr_spmm(rowptr, colind, edge_weight_csr, feat)
        ctx.save_for_backward(rowptr, colind, feat, edge_weight_csr)
        ctx.sym = sym
        return out

    @staticmethod
    def backward(ctx, grad_out):
        rowptr, colind, feat, w = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        if ctx.sym:
            grad_feat = csr_spmm(rowptr, colind, w, grad_out)
        else:
            colptr, rowind, permute = csr2csc(rowptr, colind, n_cols=feat.shape[0])
            grad_feat = csr_spmm(colptr, rowind, w, grad_out, perm=permute if w is not None else None)
        grad_w = None
        if w is not None and ctx.needs_input_grad[3]:
            grad_w = csr_sddmm(rowptr, colind, grad_out, feat).reshape(w.shape)
        return None, None, grad_feat, grad_w, None


def csrspmm(rowptr, colind, x, csr_data, sym=False, actnn=False):
    if actnn:
        raise NotImplementedError(
            "the actnn activation-compression path needs the third-party `actnn` package, "
            "which the reference imports optionally (operators/spmm.py:69-72)")
    return SPMMFunction.apply(rowptr, colind, x, csr_data, sym)

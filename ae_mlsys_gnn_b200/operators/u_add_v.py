"""u_add_v on a CSR graph (reference: operators/u_add_v.py)."""
from __future__ import annotations

import torch

from .. import _capi as capi

I32, F32 = torch.int32, torch.float32


def u_add_v_forward(row_ptr, col_ind, row_val, col_val):
    """out[e,f] = row_val[row(e),f] + col_val[col_ind[e],f] — u_add_v.u_add_v_forward
    (src/u_add_v/u_add_v.cu:30-41)."""
    dev = row_val.device
    capi.require(row_val, F32, "row_val", 2)
    capi.require(col_val, F32, "col_val", 2, dev)
    capi.require(row_ptr, I32, "row_ptr", 1, dev)
    capi.require(col_ind, I32, "col_ind", 1, dev)
    F = row_val.shape[1]
    nnz = col_ind.numel()
    out = torch.empty((nnz, F), dtype=F32, device=dev)
    with torch.cuda.device(dev):
        capi.call("gnn_u_add_v_fwd", capi.ptr(row_ptr), capi.ptr(col_ind), row_ptr.numel() - 1, nnz,
                  capi.ptr(row_val), capi.ptr(col_val), F, capi.ptr(out), capi.stream_ptr(dev))
    return out


def u_add_v_backward(row_ptr, col_ind, grad_out, n_cols=None):
    """(grad_row, grad_col): row sums and column sums of the (E,F) gradient —
    u_add_v.u_add_v_backward (u_add_v.cu:80-90), with grad_col zero-initialised."""
    dev = grad_out.device
    capi.require(grad_out, F32, "grad_out", 2)
    n_rows = row_ptr.numel() - 1
    n_cols = n_rows if n_cols is None else int(n_cols)
    nnz, F = grad_out.shape
    grad_row = torch.empty((n_rows, F), dtype=F32, device=dev)
    grad_col = torch.empty((n_cols, F), dtype=F32, device=dev)
    with torch.cuda.device(dev):
        capi.call("gnn_u_add_v_bwd", capi.ptr(row_ptr), capi.ptr(col_ind), n_rows, n_cols, nnz,
                  capi.ptr(grad_out), F, capi.ptr(grad_row), capi.ptr(grad_col),
                  capi.stream_ptr(dev))
    return grad_row, grad_col


class u_add_v_Function(torch.autograd.Function):
    @staticmethod
    def forward(ctx, row_ptr, col_ind, row_val, col_val):
        row_val, col_val = row_val.contiguous(), col_val.contiguous()
        result = u_add_v_forward(row_ptr, col_ind, row_val, col_val)
        ctx.save_for_backward(row_ptr, col_ind)
        ctx.n_cols = col_val.shape[0]
        return result

    @staticmethod
    def backward(ctx, grad_out):
        row_ptr, col_ind = ctx.saved_tensors
        grad_row, grad_col = u_add_v_backward(row_ptr, col_ind, grad_out.contiguous(), ctx.n_cols)
        return None, None, grad_row, grad_col


def u_add_v_op(row_ptr, col_ind, row_val, col_val):
    return u_add_v_Function.apply(row_ptr, col_ind, row_val, col_val)

"""CSR edge softmax (reference: operators/edge_softmax.py)."""
from __future__ import annotations

import torch

from .. import _capi as capi

I32, F32 = torch.int32, torch.float32


def edge_softmax_forward(rowptr, h):
    """Softmax of the (E,H) values over every CSR row — edge_softmax.edge_softmax
    (src/edge_softmax/edge_softmax.cu:100-113)."""
    dev = h.device
    capi.require(h, F32, "h", 2)
    capi.require(rowptr, I32, "rowptr", 1, dev)
    E, H = h.shape
    out = torch.empty_like(h)
    with torch.cuda.device(dev):
        capi.call("gnn_edge_softmax_fwd", capi.ptr(rowptr), rowptr.numel() - 1, E, capi.ptr(h), H,
                  capi.ptr(out), capi.stream_ptr(dev))
    return out


def edge_softmax_backward(rowptr, out, grad_out):
    """grad_in = out * (grad_out - sum_row(out * grad_out)) —
    edge_softmax.edge_softmax_backward (edge_softmax.cu:115-128)."""
    dev = out.device
    capi.require(out, F32, "out", 2)
    capi.require(grad_out, F32, "grad_out", 2, dev)
    E, H = out.shape
    grad = torch.empty_like(out)
    with torch.cuda.device(dev):
        capi.call("gnn_edge_softmax_bwd", capi.ptr(rowptr), rowptr.numel() - 1, E, capi.ptr(out),
                  capi.ptr(grad_out), H, capi.ptr(grad), capi.stream_ptr(dev))
    return grad


class EdgeSoftmaxFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rowptr, h):
        out = edge_softmax_forward(rowptr, h.contiguous())
        ctx.save_for_backward(rowptr, out)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        rowptr, out = ctx.saved_tensors
        return None, edge_softmax_backward(rowptr, out, grad_out.contiguous())


def csr_edge_softmax(rowptr, h):
    return EdgeSoftmaxFunction.apply(rowptr, h)

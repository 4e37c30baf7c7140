"""Fused EdgeConv max aggregation (reference: operators/fused_edgeconv.py)."""
from __future__ import annotations

import torch

from .. import _capi as capi

I32, F32 = torch.int32, torch.float32


def edgeconv_forward(k, src_ind, h_src, h_dst, slope=None):
    """(out, max_idx) — fused_edgeconv.edgeconv_forward
    (src/fused_edgeconv/fused_edgeconv.cu:148-173).  ``max_idx`` is int32.  With ``slope``
    the stored output is LeakyReLU(slope) of the maximum (gnn_edgeconv_fwd_act)."""
    dev = h_src.device
    capi.require(h_src, F32, "h_src", 2)
    capi.require(h_dst, F32, "h_dst", 2, dev)
    capi.require(src_ind, I32, "src_ind", 1, dev)
    n, F = h_dst.shape
    k = int(k)
    if h_src.shape[1] != F:
        raise ValueError("h_src and h_dst must have the same feature width")
    if src_ind.numel() != n * k:
        raise ValueError(f"src_ind must hold n*k = {n * k} ids, got {src_ind.numel()}")
    out = torch.empty((n, F), dtype=F32, device=dev)
    max_idx = torch.empty((n, F), dtype=I32, device=dev)
    with torch.cuda.device(dev):
        if slope is None:
            capi.call("gnn_edgeconv_fwd", k, capi.ptr(src_ind), capi.ptr(h_src), capi.ptr(h_dst), n, F,
                      capi.ptr(out), capi.ptr(max_idx), capi.stream_ptr(dev))
        else:
            capi.call("gnn_edgeconv_fwd_act", k, capi.ptr(src_ind), capi.ptr(h_src), capi.ptr(h_dst), n, F,
                      float(slope), capi.ptr(out), capi.ptr(max_idx), capi.stream_ptr(dev))
    return out, max_idx


def edgeconv_backward(grad_out, max_idx, n_src=None):
    """grad_src — fused_edgeconv.edgeconv_backward (fused_edgeconv.cu:189-200)."""
    dev = grad_out.device
    capi.require(grad_out, F32, "grad_out", 2)
    capi.require(max_idx, I32, "max_idx", 2, dev)
    n, F = grad_out.shape
    n_src = n if n_src is None else int(n_src)
    grad_src = torch.empty((n_src, F), dtype=F32, device=dev)
    with torch.cuda.device(dev):
        capi.call("gnn_edgeconv_bwd", capi.ptr(grad_out), capi.ptr(max_idx), n, n_src, F,
                  capi.ptr(grad_src), capi.stream_ptr(dev))
    return grad_src


def edgeconv_backward_act(grad_out, out, slope, max_idx, n_src=None):
    """(grad_src, grad_dst) of the activated forward: grad_dst = grad_out * LeakyReLU'(out),
    grad_src its scatter to the arg-max rows (gnn_edgeconv_bwd_act)."""
    dev = grad_out.device
    capi.require(grad_out, F32, "grad_out", 2)
    capi.require(out, F32, "out", 2, dev)
    capi.require(max_idx, I32, "max_idx", 2, dev)
    n, F = grad_out.shape
    n_src = n if n_src is None else int(n_src)
    grad_src = torch.empty((n_src, F), dtype=F32, device=dev)
    grad_dst = torch.empty((n, F), dtype=F32, device=dev)
    with torch.cuda.device(dev):
        capi.call("gnn_edgeconv_bwd_act", capi.ptr(grad_out), capi.ptr(out), float(slope), capi.ptr(max_idx),
                  n, n_src, F, capi.ptr(grad_src), capi.ptr(grad_dst), capi.stream_ptr(dev))
    return grad_src, grad_dst


class FusedEdgeConvFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, k, src_ind, h_src, h_dst):
        h_src = h_src.contiguous()
        h_dst = h_dst.contiguous()
        out, max_idx = edgeconv_forward(k, src_ind, h_src, h_dst)
        ctx.save_for_backward(max_idx)
        ctx.n_src = h_src.shape[0]
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (max_idx,) = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        grad_src = edgeconv_backward(grad_out, max_idx, ctx.n_src)
        return None, None, grad_src, grad_out


class FusedEdgeConvLeakyFunction(torch.autograd.Function):
    """EdgeConv max aggregation followed by LeakyReLU(slope) as one node of the graph."""

    @staticmethod
    def forward(ctx, k, src_ind, h_src, h_dst, slope):
        h_src = h_src.contiguous()
        h_dst = h_dst.contiguous()
        out, max_idx = edgeconv_forward(k, src_ind, h_src, h_dst, slope)
        ctx.save_for_backward(max_idx, out)
        ctx.n_src = h_src.shape[0]
        ctx.slope = float(slope)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        max_idx, out = ctx.saved_tensors
        grad_src, grad_dst = edgeconv_backward_act(grad_out.contiguous(), out, ctx.slope, max_idx, ctx.n_src)
        return None, None, grad_src, grad_dst, None


def fused_edgeconv_op(k, src_ind, h_src, h_dst, negative_slope=None):
    """``negative_slope`` (None, as in the reference, or a positive float): LeakyReLU applied
    to the aggregated output inside the same kernels."""
    if negative_slope is None:
        return FusedEdgeConvFunction.apply(k, src_ind, h_src, h_dst)
    return FusedEdgeConvLeakyFunction.apply(k, src_ind, h_src, h_dst, float(negative_slope))

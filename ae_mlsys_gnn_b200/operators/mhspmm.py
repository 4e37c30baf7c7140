"""Multi-head SpMM / SDDMM / edge-value transpose (reference: operators/mhspmm.py)."""
from __future__ import annotations

import torch

from .. import _capi as capi

I32, F32 = torch.int32, torch.float32


def mhspmm_forward(ptr, idx, att, feat, perm=None):
    """out[s,h,:] = sum_e att[pe,h] * feat[idx[e],h,:] — mhspmm.mhspmm
    (src/spmm/mhspmm.cu:44-66).  ``att`` may be None (unit weights)."""
    dev = feat.device
    capi.require(feat, F32, "feat", 3)
    capi.require(ptr, I32, "ptr", 1, dev)
    capi.require(idx, I32, "idx", 1, dev)
    _, H, F = feat.shape
    nnz = idx.numel()
    if att is not None:
        capi.require(att, F32, "attention", 2, dev)
        if att.shape != (nnz, H):
            raise ValueError(f"attention must be ({nnz},{H}), got {tuple(att.shape)}")
    if perm is not None:
        capi.require(perm, I32, "permute", 1, dev)
    n_seg = ptr.numel() - 1
    out = torch.empty((n_seg, H, F), dtype=F32, device=dev)
    nbytes = capi.workspace_bytes("gnn_mhspmm_workspace_bytes", nnz, H, F)
    ws = capi.workspace(dev, nbytes)
    with torch.cuda.device(dev):
        capi.call("gnn_mhspmm", capi.ptr(ptr), capi.ptr(idx), n_seg, nnz, capi.ptr(att),
                  capi.ptr(perm), capi.ptr(feat), H, F, capi.ptr(out), capi.ptr(ws), ws.numel(),
                  capi.stream_ptr(dev))
    return out


def mhsddmm_forward(ptr, idx, a, b):
    """out[e,h] = <a[seg(e),h,:], b[idx[e],h,:]> — mhsddmm.mhsddmm
    (src/sddmm/mhsddmm.cu:83-99)."""
    dev = a.device
    capi.require(a, F32, "a", 3)
    capi.require(b, F32, "b", 3, dev)
    capi.require(ptr, I32, "ptr", 1, dev)
    capi.require(idx, I32, "idx", 1, dev)
    _, H, F = a.shape
    nnz = idx.numel()
    out = torch.empty((nnz, H), dtype=F32, device=dev)
    with torch.cuda.device(dev):
        capi.call("gnn_mhsddmm", capi.ptr(ptr), capi.ptr(idx), ptr.numel() - 1, nnz, capi.ptr(a),
                  capi.ptr(b), H, F, capi.ptr(out), capi.stream_ptr(dev))
    return out


def mhtranspose_forward(permute, vals):
    """out[i,:] = vals[permute[i],:] — mhtranspose.mhtranspose
    (src/csr2csc/mhtranspose.cu:28-47)."""
    dev = vals.device
    capi.require(vals, F32, "vals", 2)
    capi.require(permute, I32, "permute", 1, dev)
    E, H = vals.shape
    out = torch.empty_like(vals)
    with torch.cuda.device(dev):
        capi.call("gnn_mhtranspose", capi.ptr(permute), capi.ptr(vals), E, H, capi.ptr(out),
                  capi.stream_ptr(dev))
    return out


class MHSPMMFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rowptr, colind, colptr, rowind, permute, feat, attention):
        feat = feat.contiguous()
        attention = attention.contiguous()
        out = mhspmm_forward(rowptr, colind, attention, feat)
        ctx.save_for_backward(rowptr, colind, colptr, rowind, permute, feat, attention)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        rowptr, colind, colptr, rowind, permute, feat, attention = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        # attention is read through permute inside the kernel; no E x H transpose is written
        grad_feat = mhspmm_forward(colptr, rowind, attention, grad_out, perm=permute)
        grad_att = mhsddmm_forward(rowptr, colind, grad_out, feat)
        return None, None, None, None, None, grad_feat, grad_att


def csrmhspmm(rowptr, colind, colptr, rowind, permute, feat, attention):
    return MHSPMMFunction.apply(rowptr, colind, colptr, rowind, permute, feat, attention)

"""Fused GMMConv operators (reference: operators/fused_gmmconv.py)."""
from __future__ import annotations

import torch

from .. import _capi as capi
from .mhspmm import mhsddmm_forward, mhspmm_forward, mhtranspose_forward

I32, F32 = torch.int32, torch.float32


def gmmconv(ptr, idx, node_feat, pseudo, mu, sigma, perm=None):
    """out[s,k,:] = sum_e gauss(pseudo[pe], mu[k], sigma[k]) * node_feat[idx[e],k,:] —
    gmm.gmmconv (src/fused_gmmconv/gmmconv.cu:201-219).  ``sigma`` is the inverse
    sigma parameter.  With ``perm`` the pseudo-coordinates of edge e are
    ``pseudo[perm[e]]`` (used for the pass over the transposed graph)."""
    dev = node_feat.device
    capi.require(node_feat, F32, "node_feat", 3)
    capi.require(pseudo, F32, "pseudo", 2, dev)
    capi.require(mu, F32, "mu", 2, dev)
    capi.require(sigma, F32, "sigma", 2, dev)
    capi.require(ptr, I32, "ptr", 1, dev)
    capi.require(idx, I32, "idx", 1, dev)
    _, K, F = node_feat.shape
    D = pseudo.shape[1]
    nnz = idx.numel()
    if pseudo.shape[0] != nnz or mu.shape != (K, D) or sigma.shape != (K, D):
        raise ValueError("pseudo must be (E,D); mu and sigma must be (K,D)")
    if perm is not None:
        capi.require(perm, I32, "permute", 1, dev)
    n_seg = ptr.numel() - 1
    out = torch.empty((n_seg, K, F), dtype=F32, device=dev)
    nbytes = capi.workspace_bytes("gnn_gmm_fwd_workspace_bytes", nnz, K, F)
    ws = capi.workspace(dev, nbytes)
    with torch.cuda.device(dev):
        capi.call("gnn_gmm_fwd", capi.ptr(ptr), capi.ptr(idx), n_seg, nnz, capi.ptr(node_feat),
                  capi.ptr(pseudo), capi.ptr(perm), capi.ptr(mu), capi.ptr(sigma), K, D, F,
                  capi.ptr(out), capi.ptr(ws), ws.numel(), capi.stream_ptr(dev))
    return out


def gaussian(pseudo, mu, sigma):
    """(E,K) Gaussian weights — gmm.Gaussian (gmmconv.cu:186-199)."""
    dev = pseudo.device
    capi.require(pseudo, F32, "pseudo", 2)
    capi.require(mu, F32, "mu", 2, dev)
    capi.require(sigma, F32, "sigma", 2, dev)
    E, D = pseudo.shape
    K = mu.shape[0]
    out = torch.empty((E, K), dtype=F32, device=dev)
    with torch.cuda.device(dev):
        capi.call("gnn_gaussian_fwd", capi.ptr(pseudo), capi.ptr(mu), capi.ptr(sigma), E, K, D,
                  capi.ptr(out), capi.stream_ptr(dev))
    return out


def gaussian_bp(pseudo, mu, sigma, grad_w):
    """(grad_pseudo, grad_mu, grad_sigma) — the analytic gradient of ``gaussian``; the
    reference's gmm.GaussianBp (gmmconv.cu:154-184) does not compute it correctly."""
    dev = pseudo.device
    capi.require(grad_w, F32, "grad_w", 2, dev)
    E, D = pseudo.shape
    K = mu.shape[0]
    gp = torch.empty_like(pseudo)
    gm = torch.empty_like(mu)
    gs = torch.empty_like(sigma)
    nbytes = capi.workspace_bytes("gnn_gaussian_bwd_workspace_bytes", E, K, D)
    ws = capi.workspace(dev, nbytes)
    with torch.cuda.device(dev):
        capi.call("gnn_gaussian_bwd", capi.ptr(pseudo), capi.ptr(mu), capi.ptr(sigma),
                  capi.ptr(grad_w), E, K, D, capi.ptr(gp), capi.ptr(gm), capi.ptr(gs),
                  capi.ptr(ws), ws.numel(), capi.stream_ptr(dev))
    return gp, gm, gs


class GmmFuseFunction(torch.autograd.Function):
    """operators/fused_gmmconv.py:43-58."""

    @staticmethod
    def forward(ctx, rowptr, colind, colptr, rowind, permute, node_feat, pseudo, mu, sigma):
        node_feat, pseudo = node_feat.contiguous(), pseudo.contiguous()
        mu, sigma = mu.contiguous(), sigma.contiguous()
        out = gmmconv(rowptr, colind, node_feat, pseudo, mu, sigma)
        ctx.save_for_backward(rowptr, colind, colptr, rowind, permute, node_feat, pseudo, mu, sigma)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        rowptr, colind, colptr, rowind, permute, node_feat, pseudo, mu, sigma = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        gaussian_grad = mhsddmm_forward(rowptr, colind, grad_out, node_feat)
        node_feat_grad = gmmconv(colptr, rowind, grad_out, pseudo, mu, sigma, perm=permute)
        pseudo_out, mu_out, sigma_out = gaussian_bp(pseudo, mu, sigma, gaussian_grad)
        return None, None, None, None, None, node_feat_grad, pseudo_out, mu_out, sigma_out


class GmmFuseEbFunction(GmmFuseFunction):
    """Edge-balanced variant of the reference (operators/fused_gmmconv.py:64-79).  The
    kernel behind GmmFuseFunction is already edge-balanced, so this is the same op."""


class GmmStashFunction(torch.autograd.Function):
    """operators/fused_gmmconv.py:103-118: keeps the (E,K) Gaussian weights."""

    @staticmethod
    def forward(ctx, rowptr, colind, colptr, rowind, permute, node_feat, pseudo, mu, sigma):
        node_feat, pseudo = node_feat.contiguous(), pseudo.contiguous()
        mu, sigma = mu.contiguous(), sigma.contiguous()
        gauss = gaussian(pseudo, mu, sigma)
        out = mhspmm_forward(rowptr, colind, gauss, node_feat)
        ctx.save_for_backward(rowptr, colind, colptr, rowind, permute, gauss, node_feat, pseudo,
                              mu, sigma)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (rowptr, colind, colptr, rowind, permute, gauss, node_feat, pseudo, mu,
         sigma) = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        gaussian_grad = mhsddmm_forward(rowptr, colind, grad_out, node_feat)
        node_feat_grad = mhspmm_forward(colptr, rowind, gauss, grad_out, perm=permute)
        pseudo_out, mu_out, sigma_out = gaussian_bp(pseudo, mu, sigma, gaussian_grad)
        return None, None, None, None, None, node_feat_grad, pseudo_out, mu_out, sigma_out


class GaussianFunction(torch.autograd.Function):
    """operators/fused_gmmconv.py:85-98."""

    @staticmethod
    def forward(ctx, pseudo, mu, sigma):
        pseudo, mu, sigma = pseudo.contiguous(), mu.contiguous(), sigma.contiguous()
        out = gaussian(pseudo, mu, sigma)
        ctx.save_for_backward(pseudo, mu, sigma)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        pseudo, mu, sigma = ctx.saved_tensors
        return gaussian_bp(pseudo, mu, sigma, grad_out.contiguous())


class KernelSumFunction(torch.autograd.Function):
    """out = x.sum(1) (+ residual) (+ bias) in one pass (gnn_gmm_sum_fwd); the backward of x is
    one broadcast store (gnn_gmm_sum_bwd)."""

    @staticmethod
    def forward(ctx, x, residual, bias):
        x = x.contiguous()
        capi.require(x, F32, "x", 3)
        dev = x.device
        n, K, F = x.shape
        if residual is not None:
            residual = residual.contiguous()
            capi.require(residual, F32, "residual", 2, dev)
            if residual.shape != (n, F):
                raise ValueError("residual must be (n, F)")
        if bias is not None:
            bias = bias.contiguous()
            capi.require(bias, F32, "bias", 1, dev)
            if bias.shape != (F,):
                raise ValueError("bias must be (F,)")
        out = torch.empty((n, F), dtype=F32, device=dev)
        with torch.cuda.device(dev):
            capi.call("gnn_gmm_sum_fwd", capi.ptr(x), capi.ptr(residual), capi.ptr(bias), n, K, F,
                      capi.ptr(out), capi.stream_ptr(dev))
        ctx.shape = (n, K, F)
        ctx.has = (residual is not None, bias is not None)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        grad_out = grad_out.contiguous()
        n, K, F = ctx.shape
        grad_x = None
        if ctx.needs_input_grad[0]:
            grad_x = torch.empty((n, K, F), dtype=F32, device=grad_out.device)
            with torch.cuda.device(grad_out.device):
                capi.call("gnn_gmm_sum_bwd", capi.ptr(grad_out), n, K, F, capi.ptr(grad_x),
                          capi.stream_ptr(grad_out.device))
        grad_res = grad_out if ctx.has[0] and ctx.needs_input_grad[1] else None
        grad_bias = grad_out.sum(0) if ctx.has[1] and ctx.needs_input_grad[2] else None
        return grad_x, grad_res, grad_bias


def kernel_sum(x, residual=None, bias=None):
    """(n,K,F) -> (n,F): the sum over the K mixture kernels plus the optional residual and bias."""
    return KernelSumFunction.apply(x, residual, bias)


def GmmConvFuse(rowptr, colind, colptr, rowind, permute, node_feat, pseudo, mu, sigma):
    return GmmFuseFunction.apply(rowptr, colind, colptr, rowind, permute, node_feat, pseudo, mu, sigma)


def GmmConvFuseEb(rowptr, colind, colptr, rowind, permute, node_feat, pseudo, mu, sigma):
    return GmmFuseEbFunction.apply(rowptr, colind, colptr, rowind, permute, node_feat, pseudo, mu, sigma)


def GmmConvStash(rowptr, colind, colptr, rowind, permute, node_feat, pseudo, mu, sigma):
    return GmmStashFunction.apply(rowptr, colind, colptr, rowind, permute, node_feat, pseudo, mu, sigma)


def GaussianCp(pseudo, mu, sigma):
    return GaussianFunction.apply(pseudo, mu, sigma)


__all__ = ["kernel_sum", "GmmConvFuse", "GmmConvFuseEb", "GmmConvStash", "GaussianCp", "gmmconv", "gaussian",
           "gaussian_bp", "mhtranspose_forward"]

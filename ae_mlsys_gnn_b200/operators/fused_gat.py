"""Fused GAT operators (reference: operators/fused_gat.py).

``fused_gat_op`` is the recompute flavour the reference's ``GATConv`` uses
(operators/fused_gat.py:30-31, 52-71); ``fused_gat_stash_op`` and
``fused_gat_fusescatter`` keep the reference signatures (:27-28, :33-34) and, like
the reference variants, hold the E x H activated logits and attention values
between forward and backward.  All three produce the same values.
"""
from __future__ import annotations

import torch

from .. import _capi as capi

I32, F32 = torch.int32, torch.float32


def _rows(n_rows, pad_to, tail_shape, dev):
    """Uninitialised (rows, *tail_shape) fp32 tensor with rows = max(n_rows, pad_to); rows
    past n_rows (padding of a partitioned tensor) are zeroed, the kernels fill the rest."""
    rows = n_rows if pad_to is None else max(n_rows, int(pad_to))
    t = torch.empty((rows,) + tuple(tail_shape), dtype=F32, device=dev)
    if rows > n_rows:
        t[n_rows:].zero_()
    return t


def _check_graph(row_ptr, col_ind, dev, what="row_ptr/col_ind"):
    capi.require(row_ptr, I32, f"{what}[0]", 1, dev)
    capi.require(col_ind, I32, f"{what}[1]", 1, dev)


def gat_forward_part(attn_row, attn_col, row_ptr, col_ind, negative_slope, in_feat, out, edge_max,
                     edge_sum, accumulate, finalize):
    """gat_forward over one column block of the graph, into caller-provided ``out`` /
    ``edge_max`` / ``edge_sum`` that carry the running state between blocks (first block:
    accumulate=False; last block: finalize=True)."""
    dev = in_feat.device
    n_rows = row_ptr.numel() - 1
    H, F = in_feat.shape[1], in_feat.shape[2]
    nnz = col_ind.numel()
    for name, t in (("attn_row", attn_row), ("attn_col", attn_col), ("edge_max", edge_max),
                    ("edge_sum", edge_sum)):
        capi.require(t, F32, name, 2, dev)
    capi.require(in_feat, F32, "in_feat", 3, dev)
    capi.require(out, F32, "out", 3, dev)
    if out.shape[0] < n_rows or edge_max.shape[0] < n_rows or attn_row.shape[0] < n_rows:
        raise ValueError("out / edge_max / attn_row need at least one row per CSR row")
    nbytes = capi.workspace_bytes("gnn_gat_fwd_workspace_bytes", nnz, H, F)
    ws = capi.workspace(dev, nbytes)
    with torch.cuda.device(dev):
        capi.call("gnn_gat_fwd_part", capi.ptr(row_ptr), capi.ptr(col_ind), n_rows, nnz,
                  capi.ptr(attn_row), capi.ptr(attn_col), capi.ptr(in_feat), H, F,
                  float(negative_slope), capi.ptr(out), capi.ptr(edge_max), capi.ptr(edge_sum),
                  int(bool(accumulate)), int(bool(finalize)), capi.ptr(ws), ws.numel(),
                  capi.stream_ptr(dev))


def gat_backward_col_part(negative_slope, col_ptr, row_ind, in_feat, attn_col, rowpack, grad_out,
                          grad_feat, grad_attn_col, accumulate):
    """Column pass over one row block of the graph, into caller-provided ``grad_feat`` /
    ``grad_attn_col`` (accumulate=False on the first block)."""
    dev = in_feat.device
    n_cols = col_ptr.numel() - 1
    H, F = in_feat.shape[1], in_feat.shape[2]
    nnz = row_ind.numel()
    nbytes = capi.workspace_bytes("gnn_gat_bwd_col_workspace_bytes", nnz, H, F)
    ws = capi.workspace(dev, nbytes)
    with torch.cuda.device(dev):
        capi.call("gnn_gat_bwd_col_part", capi.ptr(col_ptr), capi.ptr(row_ind), n_cols, nnz,
                  capi.ptr(in_feat), capi.ptr(attn_col), capi.ptr(rowpack), capi.ptr(grad_out),
                  H, F, float(negative_slope), capi.ptr(grad_feat), capi.ptr(grad_attn_col),
                  int(bool(accumulate)), capi.ptr(ws), ws.numel(), capi.stream_ptr(dev))


def gat_forward(attn_row, attn_col, row_ptr, col_ind, negative_slope, in_feat, pad_to=None):
    """(out, edge_max, edge_sum) — fused_gat_SM.gat_forward
    (src/fused_gat/fused_gat_SM.cu:536-558).  ``attn_row`` and the outputs have one
    row per CSR row; ``attn_col`` / ``in_feat`` are indexed by ``col_ind``."""
    dev = in_feat.device
    capi.require(in_feat, F32, "in_feat", 3)
    n_rows = row_ptr.numel() - 1
    H, F = in_feat.shape[1], in_feat.shape[2]
    capi.require(attn_row, F32, "attn_row", 2, dev)
    capi.require(attn_col, F32, "attn_col", 2, dev)
    _check_graph(row_ptr, col_ind, dev)
    if attn_row.shape != (n_rows, H):
        raise ValueError(f"attn_row must be ({n_rows},{H}), got {tuple(attn_row.shape)}")
    if attn_col.shape != (in_feat.shape[0], H):
        raise ValueError("attn_col must have one row per in_feat row and H columns")
    nnz = col_ind.numel()
    out = _rows(n_rows, pad_to, (H, F), dev)
    edge_max = torch.empty((n_rows, H), dtype=F32, device=dev)
    edge_sum = torch.empty((n_rows, H), dtype=F32, device=dev)
    nbytes = capi.workspace_bytes("gnn_gat_fwd_workspace_bytes", nnz, H, F)
    ws = capi.workspace(dev, nbytes)
    with torch.cuda.device(dev):
        capi.call("gnn_gat_fwd", capi.ptr(row_ptr), capi.ptr(col_ind), n_rows, nnz,
                  capi.ptr(attn_row), capi.ptr(attn_col), capi.ptr(in_feat), H, F,
                  float(negative_slope), capi.ptr(out), capi.ptr(edge_max), capi.ptr(edge_sum),
                  capi.ptr(ws), ws.numel(), capi.stream_ptr(dev))
    return out, edge_max, edge_sum


def gat_forward_act(attn_row, attn_col, row_ptr, col_ind, negative_slope, in_feat, alpha=1.0, out=None,
                    act=None):
    """(out, elu(out), edge_max, edge_sum): ``gat_forward`` with the ELU a model applies to the layer
    output stored by the same kernel.  ``out`` / ``act`` may be given (n_rows, H, F) buffers."""
    dev = in_feat.device
    capi.require(in_feat, F32, "in_feat", 3)
    n_rows = row_ptr.numel() - 1
    H, F = in_feat.shape[1], in_feat.shape[2]
    capi.require(attn_row, F32, "attn_row", 2, dev)
    capi.require(attn_col, F32, "attn_col", 2, dev)
    _check_graph(row_ptr, col_ind, dev)
    if attn_row.shape[0] < n_rows or attn_row.shape[1] != H:
        raise ValueError(f"attn_row must be (>= {n_rows}, {H}), got {tuple(attn_row.shape)}")
    nnz = col_ind.numel()
    out = torch.empty((n_rows, H, F), dtype=F32, device=dev) if out is None else capi.require(out, F32, "out", 3, dev)
    act = torch.empty((n_rows, H, F), dtype=F32, device=dev) if act is None else capi.require(act, F32, "act", 3, dev)
    edge_max = torch.empty((n_rows, H), dtype=F32, device=dev)
    edge_sum = torch.empty((n_rows, H), dtype=F32, device=dev)
    nbytes = capi.workspace_bytes("gnn_gat_fwd_workspace_bytes", nnz, H, F)
    ws = capi.workspace(dev, nbytes)
    with torch.cuda.device(dev):
        capi.call("gnn_gat_fwd_act", capi.ptr(row_ptr), capi.ptr(col_ind), n_rows, nnz,
                  capi.ptr(attn_row), capi.ptr(attn_col), capi.ptr(in_feat), H, F,
                  float(negative_slope), float(alpha), capi.ptr(out), capi.ptr(act), capi.ptr(edge_max),
                  capi.ptr(edge_sum), capi.ptr(ws), ws.numel(), capi.stream_ptr(dev))
    return out, act, edge_max, edge_sum


def to_bf16(x: torch.Tensor) -> torch.Tensor:
    """fp32 CUDA tensor -> bfloat16 copy (round to nearest even); the element count must be a multiple of 8."""
    capi.require(x, F32, "x")
    out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        capi.call("gnn_to_bf16", capi.ptr(x), x.numel(), capi.ptr(out), capi.stream_ptr(x.device))
    return out


def gat_forward_bf16(attn_row, attn_col, row_ptr, col_ind, negative_slope, in_feat_bf16):
    """``gat_forward`` with the gathered rows stored as bfloat16 (opt-in: half the gather traffic,
    fp32 arithmetic and outputs; equals ``gat_forward`` on the rounded features)."""
    dev = in_feat_bf16.device
    capi.require(in_feat_bf16, torch.bfloat16, "in_feat_bf16", 3)
    n_rows = row_ptr.numel() - 1
    H, F = in_feat_bf16.shape[1], in_feat_bf16.shape[2]
    capi.require(attn_row, F32, "attn_row", 2, dev)
    capi.require(attn_col, F32, "attn_col", 2, dev)
    _check_graph(row_ptr, col_ind, dev)
    nnz = col_ind.numel()
    out = torch.empty((n_rows, H, F), dtype=F32, device=dev)
    edge_max = torch.empty((n_rows, H), dtype=F32, device=dev)
    edge_sum = torch.empty((n_rows, H), dtype=F32, device=dev)
    nbytes = capi.workspace_bytes("gnn_gat_fwd_workspace_bytes", nnz, H, F)
    ws = capi.workspace(dev, nbytes)
    with torch.cuda.device(dev):
        capi.call("gnn_gat_fwd_bf16", capi.ptr(row_ptr), capi.ptr(col_ind), n_rows, nnz,
                  capi.ptr(attn_row), capi.ptr(attn_col), capi.ptr(in_feat_bf16), H, F,
                  float(negative_slope), capi.ptr(out), capi.ptr(edge_max), capi.ptr(edge_sum),
                  capi.ptr(ws), ws.numel(), capi.stream_ptr(dev))
    return out, edge_max, edge_sum


def gat_backward(negative_slope, row_ptr, col_ind, col_ptr, row_ind, edge_max, edge_sum,
                 in_feat, attn_row, attn_col, grad_out):
    """(grad_feat, grad_attn_row, grad_attn_col) — fused_gat_SM.gat_backward
    (src/fused_gat/fused_gat_SM.cu:865-893) for a square graph."""
    dev = in_feat.device
    capi.require(in_feat, F32, "in_feat", 3)
    capi.require(grad_out, F32, "grad_out", 3, dev)
    n, H, F = in_feat.shape
    _check_graph(row_ptr, col_ind, dev)
    _check_graph(col_ptr, row_ind, dev, "col_ptr/row_ind")
    for name, t in (("edge_max", edge_max), ("edge_sum", edge_sum), ("attn_row", attn_row),
                    ("attn_col", attn_col)):
        capi.require(t, F32, name, 2, dev)
    if row_ptr.numel() - 1 != n or col_ptr.numel() - 1 != n:
        raise ValueError("gat_backward expects a square graph with one row per in_feat row")
    if not fused_backward_supported(H, F):
        return _gat_backward_per_head(negative_slope, row_ptr, col_ind, col_ptr, row_ind, edge_max, edge_sum,
                                      in_feat, attn_row, attn_col, grad_out)
    # the two passes of gnn_gat_bwd, called one after the other so that each can be timed
    grad_attn_row, rowpack = gat_backward_row(negative_slope, row_ptr, col_ind, edge_max, edge_sum,
                                              in_feat, attn_row, attn_col, grad_out)
    grad_feat, grad_attn_col = gat_backward_col(negative_slope, col_ptr, row_ind, in_feat, attn_col,
                                                rowpack, grad_out)
    return grad_feat, grad_attn_row, grad_attn_col


def fused_backward_supported(H, F):
    """Shapes the backward kernels take in one launch: at most 8 heads whose rows fit one tile
    (512 floats with 16-byte aligned rows, 256 otherwise)."""
    return H <= 8 and H * F <= (512 if F % 4 == 0 else 256)


def _gat_backward_per_head(negative_slope, row_ptr, col_ind, col_ptr, row_ind, edge_max, edge_sum, in_feat,
                           attn_row, attn_col, grad_out):
    """The backward for more than 8 heads or rows wider than a tile: the heads are independent, so
    each is run as a one-head problem on contiguous copies (the forward does the same inside
    gnn_gat_fwd with strided launches).  A single head wider than a tile is refused."""
    n, H, F = in_feat.shape
    if not fused_backward_supported(1, F):
        raise ValueError(f"fused GAT backward: per-head width {F} exceeds the largest tile "
                         "(512 floats, 256 when F is not a multiple of 4)")
    grad_feat = torch.empty_like(in_feat)
    grad_attn_row = torch.empty_like(attn_row)
    grad_attn_col = torch.empty_like(attn_col)
    for h in range(H):
        one = [t[:, h:h + 1].contiguous() for t in (edge_max, edge_sum, in_feat, attn_row, attn_col, grad_out)]
        gf, gar, gac = gat_backward(negative_slope, row_ptr, col_ind, col_ptr, row_ind, *one)
        grad_feat[:, h:h + 1] = gf
        grad_attn_row[:, h:h + 1] = gar
        grad_attn_col[:, h:h + 1] = gac
    return grad_feat, grad_attn_row, grad_attn_col


def gat_backward_single_call(negative_slope, row_ptr, col_ind, col_ptr, row_ind, edge_max, edge_sum,
                             in_feat, attn_row, attn_col, grad_out):
    """Same result as ``gat_backward`` through the single entry point gnn_gat_bwd (both
    passes and the per-row pack inside one caller-provided workspace)."""
    dev = in_feat.device
    n, H, F = in_feat.shape
    nnz = col_ind.numel()
    grad_feat = torch.empty_like(in_feat)
    grad_attn_row = torch.empty((n, H), dtype=F32, device=dev)
    grad_attn_col = torch.empty((n, H), dtype=F32, device=dev)
    nbytes = capi.workspace_bytes("gnn_gat_bwd_workspace_bytes", n, nnz, H, F)
    ws = capi.workspace(dev, nbytes)
    with torch.cuda.device(dev):
        capi.call("gnn_gat_bwd", capi.ptr(row_ptr), capi.ptr(col_ind), capi.ptr(col_ptr),
                  capi.ptr(row_ind), n, nnz, capi.ptr(edge_max), capi.ptr(edge_sum),
                  capi.ptr(in_feat), capi.ptr(attn_row), capi.ptr(attn_col), capi.ptr(grad_out),
                  H, F, float(negative_slope), capi.ptr(grad_feat), capi.ptr(grad_attn_row),
                  capi.ptr(grad_attn_col), capi.ptr(ws), ws.numel(), capi.stream_ptr(dev))
    return grad_feat, grad_attn_row, grad_attn_col


def gat_backward_row(negative_slope, row_ptr, col_ind, edge_max, edge_sum, in_feat, attn_row,
                     attn_col, grad_out, pad_to=None):
    """Row pass of the backward on a CSR row block: (grad_attn_row, rowpack)."""
    dev = in_feat.device
    n_rows = row_ptr.numel() - 1
    H, F = in_feat.shape[1], in_feat.shape[2]
    nnz = col_ind.numel()
    capi.require(grad_out, F32, "grad_out", 3, dev)
    grad_attn_row = torch.empty((n_rows, H), dtype=F32, device=dev)
    rowpack = _rows(n_rows, pad_to, (4, H), dev)
    nbytes = capi.workspace_bytes("gnn_gat_bwd_row_workspace_bytes", nnz, H, F)
    ws = capi.workspace(dev, nbytes)
    with torch.cuda.device(dev):
        capi.call("gnn_gat_bwd_row", capi.ptr(row_ptr), capi.ptr(col_ind), n_rows, nnz,
                  capi.ptr(edge_max), capi.ptr(edge_sum), capi.ptr(in_feat), capi.ptr(attn_row),
                  capi.ptr(attn_col), capi.ptr(grad_out), H, F, float(negative_slope),
                  capi.ptr(grad_attn_row), capi.ptr(rowpack), capi.ptr(ws), ws.numel(),
                  capi.stream_ptr(dev))
    return grad_attn_row, rowpack


def gat_backward_col(negative_slope, col_ptr, row_ind, in_feat, attn_col, rowpack, grad_out,
                     pad_to=None):
    """Column pass of the backward on a CSC column block: (grad_feat, grad_attn_col).
    ``in_feat`` / ``attn_col`` have one row per CSC column; ``rowpack`` / ``grad_out``
    are indexed by ``row_ind``."""
    dev = in_feat.device
    n_cols = col_ptr.numel() - 1
    H, F = in_feat.shape[1], in_feat.shape[2]
    nnz = row_ind.numel()
    grad_feat = _rows(n_cols, pad_to, (H, F), dev)
    grad_attn_col = torch.empty((n_cols, H), dtype=F32, device=dev)
    nbytes = capi.workspace_bytes("gnn_gat_bwd_col_workspace_bytes", nnz, H, F)
    ws = capi.workspace(dev, nbytes)
    with torch.cuda.device(dev):
        capi.call("gnn_gat_bwd_col", capi.ptr(col_ptr), capi.ptr(row_ind), n_cols, nnz,
                  capi.ptr(in_feat), capi.ptr(attn_col), capi.ptr(rowpack), capi.ptr(grad_out),
                  H, F, float(negative_slope), capi.ptr(grad_feat), capi.ptr(grad_attn_col),
                  capi.ptr(ws), ws.numel(), capi.stream_ptr(dev))
    return grad_feat, grad_attn_col


def gat_backward_pack(out, grad_out, attn_row, edge_max, edge_sum, pad_to=None, rowpack=None):
    """rowpack (n, 4, H) = {attn_row, edge_max, 1/edge_sum, S} with S = <grad_out, out> per
    head: the per-row record of the column pass, from the forward output instead of a pass
    over the edges.  ``rowpack``: an existing (>= n, 4, H) buffer to write into."""
    dev = out.device
    capi.require(out, F32, "out", 3)
    capi.require(grad_out, F32, "grad_out", 3, dev)
    n, H, F = edge_max.shape[0], out.shape[1], out.shape[2]
    for name, t in (("attn_row", attn_row), ("edge_max", edge_max), ("edge_sum", edge_sum)):
        capi.require(t, F32, name, 2, dev)
    if out.shape[0] < n or grad_out.shape[0] < n or attn_row.shape[0] < n:
        raise ValueError("out / grad_out / attn_row need at least one row per edge_max row")
    if rowpack is None:
        rowpack = _rows(n, pad_to, (4, H), dev)
    else:
        capi.require(rowpack, F32, "rowpack", 3, dev)
    with torch.cuda.device(dev):
        capi.call("gnn_gat_bwd_pack", n, capi.ptr(out), capi.ptr(grad_out), capi.ptr(attn_row),
                  capi.ptr(edge_max), capi.ptr(edge_sum), H, F, capi.ptr(rowpack), capi.stream_ptr(dev))
    return rowpack


def gat_backward_pack_elu(out, grad_act, attn_row, edge_max, edge_sum, alpha=1.0, grad_pre=None, rowpack=None):
    """(grad_pre, rowpack) for a layer output that went through ELU: ``grad_act`` is the gradient
    with respect to elu(out); grad_pre = grad_act * elu'(out) is what the column pass takes.
    ``grad_pre`` / ``rowpack``: existing (>= n, H, F) / (>= n, 4, H) buffers to write into."""
    dev = out.device
    capi.require(out, F32, "out", 3)
    capi.require(grad_act, F32, "grad_act", 3, dev)
    n, H, F = edge_max.shape[0], out.shape[1], out.shape[2]
    for name, t in (("attn_row", attn_row), ("edge_max", edge_max), ("edge_sum", edge_sum)):
        capi.require(t, F32, name, 2, dev)
    if out.shape[0] < n or grad_act.shape[0] < n or attn_row.shape[0] < n:
        raise ValueError("out / grad_act / attn_row need at least one row per edge_max row")
    grad_pre = (torch.empty((n, H, F), dtype=F32, device=dev) if grad_pre is None
                else capi.require(grad_pre, F32, "grad_pre", 3, dev))
    rowpack = (torch.empty((n, 4, H), dtype=F32, device=dev) if rowpack is None
               else capi.require(rowpack, F32, "rowpack", 3, dev))
    with torch.cuda.device(dev):
        capi.call("gnn_gat_bwd_pack_elu", n, capi.ptr(out), capi.ptr(grad_act), capi.ptr(attn_row),
                  capi.ptr(edge_max), capi.ptr(edge_sum), H, F, float(alpha), capi.ptr(grad_pre),
                  capi.ptr(rowpack), capi.stream_ptr(dev))
    return grad_pre, rowpack


def gat_backward_col_edges(negative_slope, col_ptr, row_ind, in_feat, attn_col, rowpack, grad_out,
                           pad_to=None):
    """``gat_backward_col`` that also returns edge_grad (E, H): the gradient of every edge
    logit, in the position order of this CSC."""
    dev = in_feat.device
    n_cols = col_ptr.numel() - 1
    H, F = in_feat.shape[1], in_feat.shape[2]
    nnz = row_ind.numel()
    grad_feat = _rows(n_cols, pad_to, (H, F), dev)
    grad_attn_col = torch.empty((n_cols, H), dtype=F32, device=dev)
    edge_grad = torch.empty((nnz, H), dtype=F32, device=dev)
    nbytes = capi.workspace_bytes("gnn_gat_bwd_col_workspace_bytes", nnz, H, F)
    ws = capi.workspace(dev, nbytes)
    with torch.cuda.device(dev):
        capi.call("gnn_gat_bwd_col_edges", capi.ptr(col_ptr), capi.ptr(row_ind), n_cols, nnz,
                  capi.ptr(in_feat), capi.ptr(attn_col), capi.ptr(rowpack), capi.ptr(grad_out),
                  H, F, float(negative_slope), capi.ptr(grad_feat), capi.ptr(grad_attn_col),
                  capi.ptr(edge_grad), 0, capi.ptr(ws), ws.numel(), capi.stream_ptr(dev))
    return grad_feat, grad_attn_col, edge_grad


def gat_backward_col_edges_part(negative_slope, col_ptr, row_ind, in_feat, attn_col, rowpack, grad_out,
                                grad_feat, grad_attn_col, accumulate):
    """``gat_backward_col_part`` that also returns edge_grad (E, H) of this block."""
    dev = in_feat.device
    n_cols = col_ptr.numel() - 1
    H, F = in_feat.shape[1], in_feat.shape[2]
    nnz = row_ind.numel()
    edge_grad = torch.empty((nnz, H), dtype=F32, device=dev)
    nbytes = capi.workspace_bytes("gnn_gat_bwd_col_workspace_bytes", nnz, H, F)
    ws = capi.workspace(dev, nbytes)
    with torch.cuda.device(dev):
        capi.call("gnn_gat_bwd_col_edges", capi.ptr(col_ptr), capi.ptr(row_ind), n_cols, nnz,
                  capi.ptr(in_feat), capi.ptr(attn_col), capi.ptr(rowpack), capi.ptr(grad_out),
                  H, F, float(negative_slope), capi.ptr(grad_feat), capi.ptr(grad_attn_col),
                  capi.ptr(edge_grad), int(bool(accumulate)), capi.ptr(ws), ws.numel(),
                  capi.stream_ptr(dev))
    return edge_grad


def gat_backward_row_sum(row_ptr, csr_pos, edge_grad):
    """grad_attn_row (n_rows, H): sum of edge_grad over each row's edges; ``csr_pos`` gives,
    for every CSR edge, its row in ``edge_grad``."""
    dev = edge_grad.device
    capi.require(edge_grad, F32, "edge_grad", 2)
    capi.require(row_ptr, I32, "row_ptr", 1, dev)
    capi.require(csr_pos, I32, "csr_pos", 1, dev)
    n_rows = row_ptr.numel() - 1
    nnz, H = csr_pos.numel(), edge_grad.shape[1]
    out = torch.empty((n_rows, H), dtype=F32, device=dev)
    nbytes = capi.workspace_bytes("gnn_gat_bwd_row_sum_workspace_bytes", nnz, H)
    ws = capi.workspace(dev, nbytes)
    with torch.cuda.device(dev):
        capi.call("gnn_gat_bwd_row_sum", capi.ptr(row_ptr), capi.ptr(csr_pos), n_rows, nnz,
                  capi.ptr(edge_grad), H, capi.ptr(out), capi.ptr(ws), ws.numel(), capi.stream_ptr(dev))
    return out


def invert_permutation(perm):
    capi.require(perm, I32, "perm", 1)
    inv = torch.empty_like(perm)
    with torch.cuda.device(perm.device):
        capi.call("gnn_invert_permutation", capi.ptr(perm), perm.numel(), capi.ptr(inv),
                  capi.stream_ptr(perm.device))
    return inv


# The one-gather backward needs, for every CSR edge, its position in the CSC: a property of
# the graph, computed on first use and kept while the graph's index tensors are alive
# (a few entries; the tensors are referenced so that their addresses stay theirs).
one_gather_backward = True
_CSR_POS: "dict[tuple, tuple]" = {}
_CSR_POS_MAX = 4


_CSC_PERM: "dict[tuple, tuple]" = {}


def _graph_key(row_ptr, col_ind, col_ptr, row_ind):
    return ((row_ptr.data_ptr(), col_ind.data_ptr(), col_ptr.data_ptr(), row_ind.data_ptr(),
             col_ind.numel(), row_ptr.numel(), str(row_ptr.device)),
            (row_ptr._version, col_ind._version, col_ptr._version, row_ind._version))


def note_csr2csc(row_ptr, col_ind, col_ptr, row_ind, permute):
    """Called by operators.csr2csc for every CSC it builds: the permutation it returns is
    the one ``csr_positions`` would otherwise have to rebuild for that graph."""
    key, vers = _graph_key(row_ptr, col_ind, col_ptr, row_ind)
    if len(_CSC_PERM) >= _CSR_POS_MAX:
        _CSC_PERM.pop(next(iter(_CSC_PERM)))
    _CSC_PERM[key] = (vers, permute, (row_ptr, col_ind, col_ptr, row_ind))


def csr_positions(row_ptr, col_ind, col_ptr, row_ind):
    """int32 (E,) position of every CSR edge in the CSC (col_ptr, row_ind), or None when that
    CSC is not the one csr2csc builds from the CSR (then the two-pass backward applies).
    A permutation handed in by the caller is not trusted: the map is rebuilt and checked."""
    key, vers = _graph_key(row_ptr, col_ind, col_ptr, row_ind)
    hit = _CSR_POS.get(key)
    if hit is not None and hit[0] == vers:
        return hit[1]
    from .csr2csc import csr2csc

    pos = None
    known = _CSC_PERM.pop(key, None)
    if known is not None and known[0] == vers and known[1]._version == 0:
        pos = invert_permutation(known[1])  # this very CSC came out of csr2csc
    elif row_ptr.numel() == col_ptr.numel():
        cp, ri, permute = csr2csc(row_ptr, col_ind)
        if torch.equal(cp, col_ptr) and torch.equal(ri, row_ind):
            pos = invert_permutation(permute)
    if len(_CSR_POS) >= _CSR_POS_MAX:
        _CSR_POS.pop(next(iter(_CSR_POS)))
    _CSR_POS[key] = (vers, pos, (row_ptr, col_ind, col_ptr, row_ind))
    return pos


def gat_backward_with_output(negative_slope, row_ptr, col_ind, col_ptr, row_ind, csr_pos, edge_max,
                             edge_sum, in_feat, attn_row, attn_col, out, grad_out):
    """(grad_feat, grad_attn_row, grad_attn_col), the values of ``gat_backward``, with one
    gather pass: needs the forward output ``out`` and ``csr_pos`` (see ``csr_positions``)."""
    rowpack = gat_backward_pack(out, grad_out, attn_row, edge_max, edge_sum)
    grad_feat, grad_attn_col, edge_grad = gat_backward_col_edges(negative_slope, col_ptr, row_ind, in_feat,
                                                                 attn_col, rowpack, grad_out)
    grad_attn_row = gat_backward_row_sum(row_ptr, csr_pos, edge_grad)
    return grad_feat, grad_attn_row, grad_attn_col


def _backward(negative_slope, row_ptr, col_ind, col_ptr, row_ind, edge_max, edge_sum, in_feat,
              attn_row, attn_col, out, grad_out, activation=None):
    """Backward of the autograd nodes: one gather pass when the graph allows, else two.
    ``activation`` = "elu": ``grad_out`` is the gradient with respect to elu(out)."""
    if one_gather_backward and fused_backward_supported(in_feat.shape[1], in_feat.shape[2]):
        pos = csr_positions(row_ptr, col_ind, col_ptr, row_ind)
        if pos is not None:
            if activation == "elu":  # the elu backward rides on the per-row pack
                grad_pre, rowpack = gat_backward_pack_elu(out, grad_out, attn_row, edge_max, edge_sum)
                grad_feat, grad_attn_col, edge_grad = gat_backward_col_edges(
                    negative_slope, col_ptr, row_ind, in_feat, attn_col, rowpack, grad_pre)
                return grad_feat, gat_backward_row_sum(row_ptr, pos, edge_grad), grad_attn_col
            return gat_backward_with_output(negative_slope, row_ptr, col_ind, col_ptr, row_ind, pos,
                                            edge_max, edge_sum, in_feat, attn_row, attn_col, out, grad_out)
    if activation == "elu":
        grad_out = grad_out * torch.where(out > 0, torch.ones_like(out), torch.exp(out))
    return gat_backward(negative_slope, row_ptr, col_ind, col_ptr, row_ind, edge_max, edge_sum,
                        in_feat, attn_row, attn_col, grad_out)


def gat_edge_alpha(attn_row, attn_col, row_ptr, col_ind, edge_max, edge_sum, negative_slope):
    """(edge_relu_csr, edge_softmax_csr), each (E, H)."""
    dev = attn_row.device
    n_rows, H = attn_row.shape
    nnz = col_ind.numel()
    edge_relu = torch.empty((nnz, H), dtype=F32, device=dev)
    edge_alpha = torch.empty((nnz, H), dtype=F32, device=dev)
    with torch.cuda.device(dev):
        capi.call("gnn_gat_edge_alpha", capi.ptr(row_ptr), capi.ptr(col_ind), n_rows, nnz,
                  capi.ptr(attn_row), capi.ptr(attn_col), capi.ptr(edge_max), capi.ptr(edge_sum),
                  H, float(negative_slope), capi.ptr(edge_relu), capi.ptr(edge_alpha),
                  capi.stream_ptr(dev))
    return edge_relu, edge_alpha


def gat_scores_forward(h, attn_l, attn_r):
    """(attn_row, attn_col), each (N,H): the two score reductions of
    layers/gatconv_layer.py:52-53 in one pass over ``h`` (N,H,F)."""
    dev = h.device
    capi.require(h, F32, "h", 3)
    n, H, F = h.shape
    al = capi.require(attn_l.reshape(H, F), F32, "attn_l", 2, dev)
    ar = capi.require(attn_r.reshape(H, F), F32, "attn_r", 2, dev)
    attn_row = torch.empty((n, H), dtype=F32, device=dev)
    attn_col = torch.empty((n, H), dtype=F32, device=dev)
    with torch.cuda.device(dev):
        capi.call("gnn_gat_scores_fwd", capi.ptr(h), capi.ptr(al), capi.ptr(ar), n, H, F,
                  capi.ptr(attn_row), capi.ptr(attn_col), capi.stream_ptr(dev))
    return attn_row, attn_col


def gat_scores_backward(h, attn_l, attn_r, grad_attn_row, grad_attn_col, grad_feat):
    """Adds the score gradients into ``grad_feat`` IN PLACE and returns
    (grad_attn_l, grad_attn_r), each (H,F)."""
    dev = h.device
    n, H, F = h.shape
    al, ar = attn_l.reshape(H, F), attn_r.reshape(H, F)
    capi.require(grad_feat, F32, "grad_feat", 3, dev)
    capi.require(grad_attn_row, F32, "grad_attn_row", 2, dev)
    capi.require(grad_attn_col, F32, "grad_attn_col", 2, dev)
    gl = torch.empty((H, F), dtype=F32, device=dev)
    gr = torch.empty((H, F), dtype=F32, device=dev)
    nbytes = capi.workspace_bytes("gnn_gat_scores_bwd_workspace_bytes", n, H, F)
    ws = capi.workspace(dev, nbytes)
    with torch.cuda.device(dev):
        capi.call("gnn_gat_scores_bwd", capi.ptr(h), capi.ptr(al), capi.ptr(ar),
                  capi.ptr(grad_attn_row), capi.ptr(grad_attn_col), n, H, F, capi.ptr(grad_feat),
                  capi.ptr(gl), capi.ptr(gr), capi.ptr(ws), ws.numel(), capi.stream_ptr(dev))
    return gl, gr


def fused_scores_supported(H, F):
    """Shapes the one-pass score kernels cover (same limit as the fused backward)."""
    return fused_backward_supported(H, F)


class FusedGATLayerFunction(torch.autograd.Function):
    """Scores + fused_gat_op as one autograd node: h (N,H,F), attn_l / attn_r (1,H,F) ->
    out (N,H,F).  Same mathematics as GATConv.forward after the projection
    (layers/gatconv_layer.py:52-55), but the per-node scores and their gradients never
    go through framework elementwise kernels, and grad_h is accumulated in place."""

    @staticmethod
    def forward(ctx, h, attn_l, attn_r, row_ptr, col_ind, col_ptr, row_ind, negative_slope,
                activation=None):
        if activation not in (None, "elu"):
            raise ValueError("activation must be None or 'elu'")
        h = h.contiguous()
        attn_l, attn_r = attn_l.contiguous(), attn_r.contiguous()
        attn_row, attn_col = gat_scores_forward(h, attn_l, attn_r)
        # with an activation the node returns elu(out), stored by the forward kernel itself, and
        # keeps out: its backward folds the activation's derivative into the per-row pack
        act = None
        if activation == "elu":
            out, act, edge_max, edge_sum = gat_forward_act(attn_row, attn_col, row_ptr, col_ind, negative_slope, h)
        else:
            out, edge_max, edge_sum = gat_forward(attn_row, attn_col, row_ptr, col_ind, negative_slope, h)
        ctx.save_for_backward(row_ptr, col_ind, col_ptr, row_ind, edge_max, edge_sum, h, attn_row,
                              attn_col, attn_l, attn_r, out)
        ctx.negative_slope = negative_slope
        ctx.activation = activation
        return out if act is None else act

    @staticmethod
    def backward(ctx, grad_out):
        (row_ptr, col_ind, col_ptr, row_ind, edge_max, edge_sum, h, attn_row, attn_col, attn_l,
         attn_r, out) = ctx.saved_tensors
        grad_feat, gar, gac = _backward(ctx.negative_slope, row_ptr, col_ind, col_ptr, row_ind,
                                        edge_max, edge_sum, h, attn_row, attn_col, out,
                                        grad_out.contiguous(), ctx.activation)
        gl, gr = gat_scores_backward(h, attn_l, attn_r, gar, gac, grad_feat)
        return grad_feat, gl.view_as(attn_l), gr.view_as(attn_r), None, None, None, None, None, None


class FusedGATProjectedLayerFunction(torch.autograd.Function):
    """The whole GATConv layer as one autograd node: feat (N, in), W (in, H*F), attn_l / attn_r
    (1, H, F) -> out (N, H, F).  The projection runs on the tensor-core GEMM whose epilogue also
    forms attn_row / attn_col (no pass over h for the scores); the rest is FusedGATLayerFunction.
    Backward: the fused GAT backward and the score gradients give grad_h; grad_feat = grad_h W^T and
    grad_W = feat^T grad_h are the same GEMM kernel."""

    @staticmethod
    def forward(ctx, feat, W, attn_l, attn_r, row_ptr, col_ind, col_ptr, row_ind, negative_slope,
                activation=None):
        from . import dense

        if activation not in (None, "elu"):
            raise ValueError("activation must be None or 'elu'")
        H, F = attn_l.shape[1], attn_l.shape[2]
        feat, W = feat.contiguous(), W.contiguous()
        attn_l, attn_r = attn_l.contiguous(), attn_r.contiguous()
        # One head whose width is not a multiple of 4 floats (the 47- / 41- / 7-wide output layers): the
        # weights get zero columns up to the next multiple, so the projected rows, the aggregated rows and
        # their gradients have a 16-byte pitch and the sparse kernels move them with 128-bit accesses; the
        # extra columns are zero everywhere (a zero weight column, a zero gradient column) and are cut off
        # at the node's boundary.  It also makes the input gradient's GEMM a K % 4 == 0 product.
        pad = (-F) % 4 if H == 1 else 0
        Fp = F + pad
        Wp, alp, arp = W, attn_l.view(H, F), attn_r.view(H, F)
        if pad:
            Wp = torch.nn.functional.pad(W, (0, pad))
            alp = torch.nn.functional.pad(alp, (0, pad))
            arp = torch.nn.functional.pad(arp, (0, pad))
        h2, attn_row, attn_col = dense.gemm_any_k(feat, Wp, False, scores=(alp, arp))
        h = h2.view(-1, H, Fp)
        act = None
        if activation == "elu":
            out, act, edge_max, edge_sum = gat_forward_act(attn_row, attn_col, row_ptr, col_ind, negative_slope, h)
        else:
            out, edge_max, edge_sum = gat_forward(attn_row, attn_col, row_ptr, col_ind, negative_slope, h)
        ctx.save_for_backward(row_ptr, col_ind, col_ptr, row_ind, edge_max, edge_sum, h, attn_row,
                              attn_col, alp, arp, out, feat, Wp)
        ctx.negative_slope = negative_slope
        ctx.activation = activation
        ctx.width = (F, pad)
        res = out if act is None else act
        return res[:, :, :F] if pad else res

    @staticmethod
    def backward(ctx, grad_out):
        from . import dense

        (row_ptr, col_ind, col_ptr, row_ind, edge_max, edge_sum, h, attn_row, attn_col, alp,
         arp, out, feat, Wp) = ctx.saved_tensors
        F, pad = ctx.width
        grad_out = torch.nn.functional.pad(grad_out, (0, pad)) if pad else grad_out.contiguous()
        grad_h, gar, gac = _backward(ctx.negative_slope, row_ptr, col_ind, col_ptr, row_ind,
                                     edge_max, edge_sum, h, attn_row, attn_col, out,
                                     grad_out, ctx.activation)
        H = h.shape[1]
        gl, gr = gat_scores_backward(h, alp.view(1, H, -1), arp.view(1, H, -1), gar, gac, grad_h)
        g2 = grad_h.view(grad_h.shape[0], -1)
        grad_feat = grad_w = None
        if ctx.needs_input_grad[0]:
            grad_feat = dense.gemm_any_k(g2, Wp, True)      # g (N, HF) @ W^T: W is (in, HF) = "N x K" of this product
        if ctx.needs_input_grad[1]:
            if feat.shape[0] >= dense.TN_MIN_ROWS and feat.data_ptr() % 16 == 0 and g2.data_ptr() % 16 == 0:
                grad_w = dense.gemm_tn(feat, g2)
            else:
                dense._note_fallback()
                grad_w = feat.t() @ g2
            if pad:
                grad_w = grad_w[:, :F].contiguous()
        gl, gr = gl.reshape(1, H, -1), gr.reshape(1, H, -1)
        if pad:
            gl, gr = gl[:, :, :F].contiguous(), gr[:, :, :F].contiguous()
        return (grad_feat, grad_w, gl, gr, None, None, None, None, None, None)


def projected_layer_supported(feat, W, H, F):
    """Whether FusedGATProjectedLayerFunction applies: the tensor-core GEMM takes the product and
    its epilogue can form the scores for H heads of width F."""
    from . import dense

    return (feat.dim() == 2 and fused_scores_supported(H, F) and dense.scores_supported(H, F)
            and dense.supported(feat.shape[0], W.shape[1], W.shape[0], feat))


def fused_gat_layer_op(h, attn_l, attn_r, row_ptr, col_ind, col_ptr, row_ind, negative_slope,
                       activation=None):
    return FusedGATLayerFunction.apply(h, attn_l, attn_r, row_ptr, col_ind, col_ptr, row_ind,
                                       negative_slope, activation)


class FusedGATFunction_SM(torch.autograd.Function):
    """Recompute flavour (operators/fused_gat.py:52-71): only edge_max / edge_sum (N x H)
    are kept; the backward recomputes the attention values."""

    @staticmethod
    def forward(ctx, attn_row, attn_col, row_ptr, col_ind, col_ptr, row_ind, negative_slope,
                in_feat):
        attn_row = attn_row.contiguous()
        attn_col = attn_col.contiguous()
        in_feat = in_feat.contiguous()
        out, edge_max, edge_sum = gat_forward(attn_row, attn_col, row_ptr, col_ind,
                                              negative_slope, in_feat)
        ctx.save_for_backward(row_ptr, col_ind, col_ptr, row_ind, edge_max, edge_sum, in_feat,
                              attn_row, attn_col, out)
        ctx.negative_slope = negative_slope
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (row_ptr, col_ind, col_ptr, row_ind, edge_max, edge_sum, in_feat, attn_row,
         attn_col, out) = ctx.saved_tensors
        grad_feat, grad_attn_row, grad_attn_col = _backward(
            ctx.negative_slope, row_ptr, col_ind, col_ptr, row_ind, edge_max, edge_sum, in_feat,
            attn_row, attn_col, out, grad_out.contiguous())
        return grad_attn_row, grad_attn_col, None, None, None, None, None, grad_feat


class FusedGATFunction_stash(torch.autograd.Function):
    """Stash flavour (operators/fused_gat.py:73-87): additionally materialises
    edge_relu_csr and edge_softmax_csr (E x H) in the forward and keeps them."""

    @staticmethod
    def forward(ctx, attn_row, attn_col, row_ptr, col_ind, col_ptr, row_ind, negative_slope,
                in_feat, permute):
        attn_row = attn_row.contiguous()
        attn_col = attn_col.contiguous()
        in_feat = in_feat.contiguous()
        out, edge_max, edge_sum = gat_forward(attn_row, attn_col, row_ptr, col_ind,
                                              negative_slope, in_feat)
        edge_relu, edge_alpha = gat_edge_alpha(attn_row, attn_col, row_ptr, col_ind, edge_max,
                                               edge_sum, negative_slope)
        ctx.save_for_backward(row_ptr, col_ind, col_ptr, row_ind, permute, edge_alpha, edge_relu,
                              edge_max, edge_sum, in_feat, attn_row, attn_col, out)
        ctx.negative_slope = negative_slope
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (row_ptr, col_ind, col_ptr, row_ind, _permute, _edge_alpha, _edge_relu, edge_max,
         edge_sum, in_feat, attn_row, attn_col, out) = ctx.saved_tensors
        grad_feat, grad_attn_row, grad_attn_col = _backward(
            ctx.negative_slope, row_ptr, col_ind, col_ptr, row_ind, edge_max, edge_sum, in_feat,
            attn_row, attn_col, out, grad_out.contiguous())
        return grad_attn_row, grad_attn_col, None, None, None, None, None, grad_feat, None


class FusedGATFunction(FusedGATFunction_stash):
    """"fusescatter" flavour (operators/fused_gat.py:36-50); same values and the same
    kept tensors as the stash flavour."""


def fused_gat_op(attn_row, attn_col, row_ptr, col_ind, col_ptr, row_ind, negative_slope, in_feat,
                 save_memory=True):
    return FusedGATFunction_SM.apply(attn_row, attn_col, row_ptr, col_ind, col_ptr, row_ind,
                                     negative_slope, in_feat)


def fused_gat_stash_op(attn_row, attn_col, row_ptr, col_ind, col_ptr, row_ind, negative_slope,
                       in_feat, permute):
    return FusedGATFunction_stash.apply(attn_row, attn_col, row_ptr, col_ind, col_ptr, row_ind,
                                        negative_slope, in_feat, permute)


def fused_gat_fusescatter(attn_row, attn_col, row_ptr, col_ind, col_ptr, row_ind, negative_slope,
                          in_feat, permute):
    return FusedGATFunction.apply(attn_row, attn_col, row_ptr, col_ind, col_ptr, row_ind,
                                  negative_slope, in_feat, permute)

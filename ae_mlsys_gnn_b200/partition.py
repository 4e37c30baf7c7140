"""Destination-row-block partitioning of one graph over the GPUs of a node, and the
GAT layer / model that run on such a partition.

The reference is single-GPU; nothing here has a counterpart in it.  Design:

* Rows (destination nodes) are cut into P contiguous blocks with about nnz/P edges
  each (a row is never split).  Rank g owns block g: the CSR rows of the block (for
  the forward and the backward row pass) and the CSC columns of the block (for the
  backward column pass, which produces gradients of the sources the rank owns).
* Every per-node tensor of a rank has ``max_n`` rows (the largest block, so that
  all ranks contribute equally sized pieces to an all-gather); rows past the
  rank's own count are zero padding.  Gathered tensors therefore have P*max_n rows,
  and the column ids of the local CSR / row ids of the local CSC are remapped once
  into that padded index space.
* Per layer the only exchanges are: all-gather of the projected features h and of
  attn_col (forward); all-gather of grad_out and of the per-row pack
  {attn_row, max, 1/sum, S} (backward).  No reduction of feature gradients is
  needed because the column pass sums over all destinations of an owned source.
  Weight gradients are all-reduced after the backward (they are tiny).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from .layers.gatconv_layer import _GATBase
from .operators import dense


def edge_balanced_bounds(row_ptr: torch.Tensor, world: int) -> list[int]:
    """Block boundaries b[0..world] with b[g] the first row whose start is at or after
    g*nnz/world; every block then holds about nnz/world edges (hub rows stay whole)."""
    rp = row_ptr.long()
    n = rp.numel() - 1
    nnz = int(rp[-1].item())
    targets = torch.tensor([(g * nnz) // world for g in range(1, world)], dtype=torch.long,
                           device=rp.device)
    cuts = torch.searchsorted(rp[:-1].contiguous(), targets).tolist() if world > 1 else []
    bounds = [0] + [min(max(int(c), 0), n) for c in cuts] + [n]
    for g in range(1, len(bounds)):  # keep the boundaries monotone
        bounds[g] = max(bounds[g], bounds[g - 1])
    return bounds


@dataclass
class RowBlockPartition:
    rank: int
    world: int
    bounds: list[int]          # global row boundaries, world+1 entries
    max_n: int                 # rows of every per-rank tensor (largest block)
    row_ptr: torch.Tensor      # local CSR, int32 [n_local+1]
    col_ind: torch.Tensor      # int32, ids in the padded gathered space
    col_ptr: torch.Tensor      # local CSC of the owned sources, int32 [n_local+1]
    row_ind: torch.Tensor      # int32, ids in the padded gathered space

    @property
    def n_local(self) -> int:
        return self.bounds[self.rank + 1] - self.bounds[self.rank]

    @property
    def n_global(self) -> int:
        return self.bounds[-1]

    def pad_rows(self, x_local: torch.Tensor) -> torch.Tensor:
        """Local rows followed by zero rows up to max_n."""
        out = x_local.new_zeros((self.max_n,) + tuple(x_local.shape[1:]))
        out[: x_local.shape[0]] = x_local
        return out

    def local_slice(self, x_global: torch.Tensor) -> torch.Tensor:
        return x_global[self.bounds[self.rank]: self.bounds[self.rank + 1]]


def _to_padded_ids(ids: torch.Tensor, bounds: list[int], max_n: int) -> torch.Tensor:
    b = torch.tensor(bounds, dtype=torch.long, device=ids.device)
    v = ids.long()
    owner = torch.bucketize(v, b[1:-1], right=True)
    return (owner * max_n + (v - b[owner])).to(torch.int32)


def build_partition(row_ptr, col_ind, col_ptr, row_ind, rank: int, world: int,
                    bounds: list[int] | None = None) -> RowBlockPartition:
    """Cuts the global CSR (row_ptr, col_ind) and CSC (col_ptr, row_ind) of a square
    graph into rank `rank`'s blocks."""
    bounds = edge_balanced_bounds(row_ptr, world) if bounds is None else bounds
    max_n = max(bounds[g + 1] - bounds[g] for g in range(world))
    lo, hi = bounds[rank], bounds[rank + 1]

    def cut(ptr, idx):
        p = ptr[lo: hi + 1].long()
        e0, e1 = int(p[0].item()), int(p[-1].item())
        return (p - e0).to(torch.int32).contiguous(), _to_padded_ids(idx[e0:e1], bounds, max_n).contiguous()

    rp, ci = cut(row_ptr, col_ind)
    cp, ri = cut(col_ptr, row_ind)
    return RowBlockPartition(rank, world, bounds, max_n, rp, ci, cp, ri)


def all_gather_rows(x: torch.Tensor, world: int, group=None, async_op: bool = False):
    """All-gather of equally sized row blocks: (max_n, ...) -> (world*max_n, ...)."""
    if world == 1:
        return (x, None) if async_op else x
    out = x.new_empty((world * x.shape[0],) + tuple(x.shape[1:]))
    work = dist.all_gather_into_tensor(out, x.contiguous(), group=group, async_op=async_op)
    return (out, work) if async_op else out


class _CudaKernels:
    """The product kernels (C ABI).  Tests on CPU substitute an oracle-backed object
    with the same methods to exercise the exchange logic under gloo."""

    @staticmethod
    def scores_forward(h, attn_l, attn_r):
        from .operators.fused_gat import gat_scores_forward

        return gat_scores_forward(h, attn_l, attn_r)

    @staticmethod
    def scores_backward(h, attn_l, attn_r, grad_attn_row, grad_attn_col, grad_feat):
        from .operators.fused_gat import gat_scores_backward

        return gat_scores_backward(h, attn_l, attn_r, grad_attn_row, grad_attn_col, grad_feat)

    @staticmethod
    def forward(attn_row, attn_col_full, row_ptr, col_ind, slope, h_full, pad_to=None):
        from .operators.fused_gat import gat_forward

        return gat_forward(attn_row, attn_col_full, row_ptr, col_ind, slope, h_full, pad_to=pad_to)

    @staticmethod
    def backward_row(slope, row_ptr, col_ind, edge_max, edge_sum, h_full, attn_row, attn_col_full,
                     grad_out, pad_to=None):
        from .operators.fused_gat import gat_backward_row

        return gat_backward_row(slope, row_ptr, col_ind, edge_max, edge_sum, h_full, attn_row,
                                attn_col_full, grad_out, pad_to=pad_to)

    @staticmethod
    def backward_col(slope, col_ptr, row_ind, h_local, attn_col_local, rowpack_full, gout_full,
                     pad_to=None):
        from .operators.fused_gat import gat_backward_col

        return gat_backward_col(slope, col_ptr, row_ind, h_local, attn_col_local, rowpack_full,
                                gout_full, pad_to=pad_to)


class PartitionedGATFunction(torch.autograd.Function):
    """Scores + fused GAT aggregation on a row-block partition, one autograd node.
    ``h`` and the output have max_n rows (the rank's rows, then zero padding)."""

    @staticmethod
    def forward(ctx, h, attn_l, attn_r, part: RowBlockPartition, slope, kernels, group):
        n, P = part.n_local, part.world
        h, attn_l, attn_r = h.contiguous(), attn_l.contiguous(), attn_r.contiguous()
        # start moving h while the scores are computed from the local copy
        h_full, work = all_gather_rows(h, P, group, async_op=True)
        attn_row, attn_col = kernels.scores_forward(h, attn_l, attn_r)
        ac_full = all_gather_rows(attn_col, P, group)
        if work is not None:
            work.wait()
        out, edge_max, edge_sum = kernels.forward(attn_row[:n], ac_full, part.row_ptr, part.col_ind,
                                                  slope, h_full, pad_to=part.max_n)
        ctx.save_for_backward(attn_row, attn_col, h, h_full, ac_full, edge_max, edge_sum, attn_l,
                              attn_r)
        ctx.part, ctx.slope, ctx.kernels, ctx.group = part, slope, kernels, group
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (attn_row, attn_col, h, h_full, ac_full, edge_max, edge_sum, attn_l,
         attn_r) = ctx.saved_tensors
        part, slope, kernels, group = ctx.part, ctx.slope, ctx.kernels, ctx.group
        n, P = part.n_local, part.world
        grad_out = grad_out.contiguous()
        # the gather of grad_out does not depend on the row pass: run them together
        gout_full, work = all_gather_rows(grad_out, P, group, async_op=True)
        gar_l, rowpack = kernels.backward_row(slope, part.row_ptr, part.col_ind, edge_max, edge_sum,
                                              h_full, attn_row[:n], ac_full, grad_out[:n],
                                              pad_to=part.max_n)
        rp_full = all_gather_rows(rowpack, P, group)
        if work is not None:
            work.wait()
        gh, gac_l = kernels.backward_col(slope, part.col_ptr, part.row_ind, h[:n], attn_col[:n],
                                         rp_full, gout_full, pad_to=part.max_n)
        gl, gr = kernels.scores_backward(h[:n], attn_l, attn_r, gar_l, gac_l, gh[:n])
        return gh, gl.view_as(attn_l), gr.view_as(attn_r), None, None, None, None


class PartitionedGATConv(_GATBase):
    """GATConv (same parameters, same state_dict) on a RowBlockPartition."""

    def __init__(self, in_feats, out_feats, num_heads, negative_slope=0.2, kernels=_CudaKernels,
                 group=None):
        super().__init__(in_feats, out_feats, num_heads, negative_slope)
        self.kernels = kernels
        self.group = group

    def forward(self, part: RowBlockPartition, feat):
        h = dense.project(feat, self.W).view(-1, self.num_heads, self.out_feats)
        return PartitionedGATFunction.apply(h, self.attn_l, self.attn_r, part, self.negative_slope,
                                            self.kernels, self.group)


class PartitionedGAT(nn.Module):
    """models.GAT on a partition: identical parameters; inputs/outputs hold the rank's
    max_n (padded) rows."""

    def __init__(self, in_dim, hidden, heads, num_classes, out_heads=1, negative_slope=0.2,
                 activation="elu", kernels=_CudaKernels, group=None):
        super().__init__()
        if isinstance(hidden, int):
            hidden = [hidden] * len(heads)
        dims_in = [in_dim] + [h * f for h, f in zip(heads, hidden)]
        self.gat_layers = nn.ModuleList(
            [PartitionedGATConv(dims_in[i], hidden[i], heads[i], negative_slope, kernels, group)
             for i in range(len(heads))])
        self.gat_layers.append(
            PartitionedGATConv(dims_in[-1], num_classes, out_heads, negative_slope, kernels, group))
        self.activation = activation
        self.group = group

    def forward(self, part: RowBlockPartition, inputs):
        h = inputs
        for layer in self.gat_layers[:-1]:
            h = layer(part, h).flatten(1)
            if self.activation == "elu":
                h = F.elu(h)
        return self.gat_layers[-1](part, h).mean(1)

    def loss(self, part: RowBlockPartition, logits, labels_local):
        """Cross-entropy averaged over ALL nodes of the graph (sum over the owned rows
        divided by the global node count), so that summing gradients over ranks gives
        the single-GPU gradient."""
        n = part.n_local
        return F.cross_entropy(logits[:n], labels_local, reduction="sum") / part.n_global

    def all_reduce_grads(self, world: int):
        if world == 1:
            return
        grads = [p.grad for p in self.parameters() if p.grad is not None]
        flat = torch.cat([g.reshape(-1) for g in grads])
        dist.all_reduce(flat, group=self.group)
        off = 0
        for g in grads:
            g.copy_(flat[off: off + g.numel()].view_as(g))
            off += g.numel()

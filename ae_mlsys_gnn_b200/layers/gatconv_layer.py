"""GAT layers (reference: layers/gatconv_layer.py:10-159)."""
from __future__ import annotations

import torch
from torch import nn

from ..operators import dense
from ..operators.fused_gat import (FusedGATProjectedLayerFunction, fused_gat_fusescatter, fused_gat_layer_op,
                                   fused_gat_op, fused_gat_stash_op, fused_scores_supported,
                                   projected_layer_supported)


class _GATBase(nn.Module):
    """Parameters and initialisation shared by the three variants: ``W`` (in, H*F),
    ``attn_l`` / ``attn_r`` (1, H, F), xavier-normal with the ReLU gain
    (layers/gatconv_layer.py:22-45)."""

    def __init__(self, in_feats, out_feats, num_heads, negative_slope=0.2):
        super().__init__()
        self.in_feats = in_feats
        self.out_feats = out_feats
        self.num_heads = num_heads
        self.W = nn.Parameter(torch.empty(in_feats, out_feats * num_heads))
        self.attn_l = nn.Parameter(torch.zeros(1, num_heads, out_feats))
        self.attn_r = nn.Parameter(torch.zeros(1, num_heads, out_feats))
        self.negative_slope = negative_slope
        self.reset_parameters()

    def reset_parameters(self):
        gain = nn.init.calculate_gain("relu")
        nn.init.xavier_normal_(self.W, gain=gain)
        nn.init.xavier_normal_(self.attn_l, gain=gain)
        nn.init.xavier_normal_(self.attn_r, gain=gain)

    def project(self, feat):
        """h = feat @ W viewed (N,H,F); attn_row multiplies the destination (CSR row),
        attn_col the source (layers/gatconv_layer.py:50-53)."""
        h = dense.project(feat, self.W).view(-1, self.num_heads, self.out_feats)
        attn_row = (self.attn_l * h).sum(dim=-1)
        attn_col = (self.attn_r * h).sum(dim=-1)
        return h, attn_row, attn_col


class GATConv(_GATBase):
    """``fuse_scores`` (default on) computes attn_row / attn_col and their gradients with
    the one-pass score kernels inside the same autograd node as the fused op; off, the
    layer is composed exactly like the reference's (framework ops + fused_gat_op).

    ``activation`` (None, as in the reference layer, or "elu"): applied to the layer's output;
    inside the fused node its backward costs no pass of its own."""

    fuse_scores = True

    def __init__(self, in_feats, out_feats, num_heads, negative_slope=0.2, activation=None):
        super().__init__(in_feats, out_feats, num_heads, negative_slope)
        if activation not in (None, "elu"):
            raise ValueError("activation must be None or 'elu'")
        self.activation = activation

    def forward(self, row_ptr, col_ind, col_ptr, row_ind, feat, save_memory=True):
        if self.fuse_scores and projected_layer_supported(feat, self.W, self.num_heads, self.out_feats):
            # projection, scores (in the GEMM's epilogue) and the fused op as one node
            return FusedGATProjectedLayerFunction.apply(feat, self.W, self.attn_l, self.attn_r, row_ptr, col_ind,
                                                        col_ptr, row_ind, self.negative_slope, self.activation)
        if self.fuse_scores and fused_scores_supported(self.num_heads, self.out_feats):
            h = dense.project(feat, self.W).view(-1, self.num_heads, self.out_feats)
            return fused_gat_layer_op(h, self.attn_l, self.attn_r, row_ptr, col_ind, col_ptr,
                                      row_ind, self.negative_slope, self.activation)
        h, attn_row, attn_col = self.project(feat)
        out = fused_gat_op(attn_row, attn_col, row_ptr, col_ind, col_ptr, row_ind,
                           self.negative_slope, h, save_memory)
        return torch.nn.functional.elu(out) if self.activation == "elu" else out


class GATConv_stash(_GATBase):
    def forward(self, row_ptr, col_ind, col_ptr, row_ind, feat, permute):
        h, attn_row, attn_col = self.project(feat)
        return fused_gat_stash_op(attn_row, attn_col, row_ptr, col_ind, col_ptr, row_ind,
                                  self.negative_slope, h, permute)


class GATConv_fusescatter(_GATBase):
    def forward(self, row_ptr, col_ind, col_ptr, row_ind, feat, permute):
        h, attn_row, attn_col = self.project(feat)
        return fused_gat_fusescatter(attn_row, attn_col, row_ptr, col_ind, col_ptr, row_ind,
                                     self.negative_slope, h, permute)

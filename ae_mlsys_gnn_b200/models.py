"""The three models the reference's training scripts build from the fused layers,
used by bench.py and the tests.  They are harness code, not operators.

GAT    script/train/train_gatconv_our.py:14-53
DGCNN  script/train/train_edgeconv_our.py:14-73 (head reduced to global max-pool +
       one linear layer, and the kNN graph built once on the input coordinates, as
       the benchmark configuration states)
MoNet  script/train/train_gmmconv_our.py:22-68
"""
from __future__ import annotations

import torch
from torch import nn

from .layers import EdgeConv, GATConv, GMMConv


class GAT(nn.Module):
    """Stack of GATConv layers; heads are concatenated between layers and averaged
    at the output.  ``activation`` (None or "elu") is applied between layers: the
    reference model stores an activation but never applies it
    (train_gatconv_our.py:47-53); the benchmark configurations apply ELU."""

    def __init__(self, in_dim, hidden, heads, num_classes, out_heads=1, negative_slope=0.2,
                 activation="elu"):
        super().__init__()
        if isinstance(hidden, int):
            hidden = [hidden] * len(heads)
        dims_in = [in_dim] + [h * f for h, f in zip(heads, hidden)]
        # the hidden layers apply the activation themselves (elementwise, so before or after
        # the head concatenation is the same thing)
        self.gat_layers = nn.ModuleList(
            [GATConv(dims_in[i], hidden[i], heads[i], negative_slope, activation)
             for i in range(len(heads))])
        self.gat_layers.append(GATConv(dims_in[-1], num_classes, out_heads, negative_slope))
        self.activation = activation

    def forward(self, row_ptr, col_ind, col_ptr, row_ind, inputs, save_memory=True):
        h = inputs
        for layer in self.gat_layers[:-1]:
            h = layer(row_ptr, col_ind, col_ptr, row_ind, h, save_memory).flatten(1)
        out = self.gat_layers[-1](row_ptr, col_ind, col_ptr, row_ind, h, save_memory)
        # the mean over one output head is the head itself: a view, not a pass over N x F
        return out.squeeze(1) if out.shape[1] == 1 else out.mean(1)


class DGCNN(nn.Module):
    """EdgeConv stack on a fixed kNN graph: widths e.g. (64, 64, 128, 256), LeakyReLU(0.2)
    after every layer, global max-pool per cloud, one linear classifier."""

    def __init__(self, k, feature_dims, output_classes, input_dims=3):
        super().__init__()
        self.k = k
        dims = [input_dims] + list(feature_dims)
        # LeakyReLU(0.2) follows every layer; it runs inside the aggregation kernels
        self.conv = nn.ModuleList([EdgeConv(dims[i], dims[i + 1], negative_slope=0.2)
                                   for i in range(len(feature_dims))])
        self.proj_output = nn.Linear(dims[-1], output_classes)

    def forward(self, x, src_ind):
        batch, n_points, _ = x.shape
        h = x.reshape(batch * n_points, -1)
        for conv in self.conv:
            h = conv(self.k, src_ind, h)
        h = h.view(batch, n_points, -1).max(dim=1).values
        return self.proj_output(h)


class MoNet(nn.Module):
    """GMMConv stack; every layer maps the 2-d degree pseudo-coordinates through its
    own Linear + tanh (train_gmmconv_our.py:43-68)."""

    def __init__(self, in_feats, n_hidden, out_feats, n_layers, dim, n_kernels, dropout=0.0):
        super().__init__()
        dims = [in_feats] + [n_hidden] * (n_layers - 1) + [out_feats]
        self.layers = nn.ModuleList(
            [GMMConv(dims[i], dims[i + 1], dim, n_kernels) for i in range(n_layers)])
        self.pseudo_proj = nn.ModuleList(
            [nn.Sequential(nn.Linear(2, dim), nn.Tanh()) for _ in range(n_layers)])
        self.dropout = nn.Dropout(dropout)

    def forward(self, rowptr, colind, colptr, rowind, permute, feat, pseudo):
        h = feat
        for i, layer in enumerate(self.layers):
            if i != 0:
                h = self.dropout(h)
            h = layer(rowptr, colind, colptr, rowind, permute, h, self.pseudo_proj[i](pseudo))
        return h

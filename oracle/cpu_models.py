"""CPU (PyTorch, fp32, all host threads) models built from the oracle's DGL-style
layer restatements.  TEST / BASELINE INFRASTRUCTURE ONLY: bench.py times these as the
"reference's CPU path" (DGL's GATConv / EdgeConv / GMMConv on CPU; DGL itself is not
installable offline, so its message-passing formulation is restated with
index_select + index_add / scatter_reduce, layers/gatconv_layer.py:196-213,
layers/edgeconv_layer.py:102-108, layers/gmmconv_layer.py:130-149).  The tests use the same
models in float64 (``dtype=torch.float64`` and ``.double()``) as the checker of the GPU
models' logits, loss and parameter gradients."""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from . import ops as ref


class CpuGAT(nn.Module):
    def __init__(self, in_dim, hidden, heads, num_classes, out_heads=1, negative_slope=0.2,
                 activation="elu", dtype=torch.float32):
        super().__init__()
        self.dtype = dtype
        if isinstance(hidden, int):
            hidden = [hidden] * len(heads)
        dims_in = [in_dim] + [h * f for h, f in zip(heads, hidden)]
        shapes = [(dims_in[i], heads[i], hidden[i]) for i in range(len(heads))]
        shapes.append((dims_in[-1], out_heads, num_classes))
        gain = nn.init.calculate_gain("relu")
        self.W, self.al, self.ar = nn.ParameterList(), nn.ParameterList(), nn.ParameterList()
        for din, H, Fo in shapes:
            self.W.append(nn.Parameter(nn.init.xavier_normal_(torch.empty(din, H * Fo), gain=gain)))
            self.al.append(nn.Parameter(nn.init.xavier_normal_(torch.empty(1, H, Fo), gain=gain)))
            self.ar.append(nn.Parameter(nn.init.xavier_normal_(torch.empty(1, H, Fo), gain=gain)))
        self.slope, self.activation = negative_slope, activation

    def forward(self, row_ptr, col_ind, x):
        h = x
        last = len(self.W) - 1
        for i in range(len(self.W)):
            h = ref.gat_layer_dgl(row_ptr, col_ind, h, self.W[i], self.al[i], self.ar[i], self.slope,
                                  dtype=self.dtype)
            if i < last:
                h = h.flatten(1)
                if self.activation == "elu":
                    h = F.elu(h)
        return h.mean(1)


class CpuDGCNN(nn.Module):
    def __init__(self, k, feature_dims, output_classes, input_dims=3, dtype=torch.float32):
        super().__init__()
        self.k, self.dtype = k, dtype
        dims = [input_dims] + list(feature_dims)
        self.theta = nn.ModuleList([nn.Linear(dims[i], dims[i + 1], bias=False) for i in range(len(feature_dims))])
        self.phi = nn.ModuleList([nn.Linear(dims[i], dims[i + 1], bias=False) for i in range(len(feature_dims))])
        self.proj_output = nn.Linear(dims[-1], output_classes)

    def forward(self, x, src_ind):
        batch, n_points, _ = x.shape
        h = x.reshape(batch * n_points, -1).to(self.dtype)
        for t, p in zip(self.theta, self.phi):
            h = F.leaky_relu(ref.edgeconv_layer_dgl(self.k, src_ind, h, t.weight, p.weight,
                                                    dtype=self.dtype), 0.2)
        return self.proj_output(h.view(batch, n_points, -1).max(dim=1).values)


class CpuMoNet(nn.Module):
    def __init__(self, in_feats, n_hidden, out_feats, n_layers, dim, n_kernels, dtype=torch.float32):
        super().__init__()
        self.dtype = dtype
        dims = [in_feats] + [n_hidden] * (n_layers - 1) + [out_feats]
        self.K = n_kernels
        self.fc = nn.ModuleList([nn.Linear(dims[i], n_kernels * dims[i + 1], bias=False) for i in range(n_layers)])
        self.mu = nn.ParameterList([nn.Parameter(torch.randn(n_kernels, dim) * 0.1) for _ in range(n_layers)])
        self.inv_sigma = nn.ParameterList([nn.Parameter(torch.ones(n_kernels, dim)) for _ in range(n_layers)])
        self.bias = nn.ParameterList([nn.Parameter(torch.zeros(dims[i + 1])) for i in range(n_layers)])
        self.pseudo_proj = nn.ModuleList([nn.Sequential(nn.Linear(2, dim), nn.Tanh()) for _ in range(n_layers)])

    def forward(self, row_ptr, col_ind, feat, pseudo):
        h, pseudo = feat.to(self.dtype), pseudo.to(self.dtype)
        for i in range(len(self.fc)):
            nf = self.fc[i](h).view(h.shape[0], self.K, -1)
            h = ref.gmm_forward(row_ptr, col_ind, nf, self.pseudo_proj[i](pseudo), self.mu[i],
                                self.inv_sigma[i], dtype=self.dtype).sum(1) + self.bias[i]
        return h

"""EdgeConv layer (reference: layers/edgeconv_layer.py:6-43)."""
from __future__ import annotations

from torch import nn

from ..operators import dense
from ..operators.fused_edgeconv import fused_edgeconv_op


class EdgeConv(nn.Module):
    """out_i = max_j theta(x_j - x_i) + phi(x_i), computed as
    max_j (h_dst[i] + h_src[j]) with h_src = theta(x), h_dst = phi(x) - theta(x)."""

    def __init__(self, in_feat, out_feat, batch_norm=False, allow_zero_in_degree=False, negative_slope=None):
        super().__init__()
        self.batch_norm = batch_norm
        # None as in the reference layer; a positive float applies LeakyReLU to the output
        # inside the aggregation kernels (what the DGCNN model does after every layer).
        self.negative_slope = negative_slope
        self._allow_zero_in_degree = allow_zero_in_degree
        self.theta = nn.Linear(in_feat, out_feat, bias=False)
        self.phi = nn.Linear(in_feat, out_feat, bias=False)
        if batch_norm:
            self.bn = nn.BatchNorm1d(out_feat)

    def set_allow_zero_in_degree(self, set_value):
        self._allow_zero_in_degree = set_value

    def forward(self, k, src_ind, feat):
        h_theta = dense.linear(feat, self.theta.weight)
        h_phi = dense.linear(feat, self.phi.weight)
        return fused_edgeconv_op(k, src_ind, h_theta, h_phi - h_theta, self.negative_slope)

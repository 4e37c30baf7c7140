"""k-nearest-neighbour graph of point clouds: the graph EdgeConv aggregates over.

The reference builds it with DGL's ``KNNGraph(k)`` in front of every EdgeConv layer
(script/train/train_edgeconv_our.py:20,52).  ``knn_graph`` returns the source ids in the
layout ``fused_edgeconv_op`` reads: the k sources of node i at [i*k, (i+1)*k), ids global over
the batch of clouds.
"""
from __future__ import annotations

import torch

from .. import _capi as capi


def knn_graph(points: torch.Tensor, k: int) -> torch.Tensor:
    """points (B, P, C) float32 on a GPU -> int32 (B*P*k,).  Neighbours of a point are the k points
    of the same cloud with the smallest squared Euclidean distance (float64, coordinates summed in
    ascending order), ordered by (distance, index): the point itself comes first."""
    capi.require(points, torch.float32, "points", 3)
    B, P, Cn = points.shape
    if k > P:
        raise ValueError(f"k = {k} exceeds the {P} points of a cloud")
    out = torch.empty(B * P * k, dtype=torch.int32, device=points.device)
    with torch.cuda.device(points.device):
        capi.call("gnn_knn_graph", capi.ptr(points), B, P, Cn, int(k), capi.ptr(out), capi.stream_ptr(points.device))
    return out

"""Shared helpers of the test-suite: crafted graphs and tolerance checks."""
from __future__ import annotations

import numpy as np
import torch

from ae_mlsys_gnn_b200.graphs import Graph, csr_from_edges

# fp32 outputs and gradients: rel 1e-4 / abs 1e-5 against the oracle
RTOL, ATOL = 1e-4, 1e-5


def assert_close(actual: torch.Tensor, expected: torch.Tensor, what: str, rtol=RTOL, atol=ATOL,
                 scale_atol=False):
    """|actual - expected| <= atol + rtol * |expected| element-wise.  With
    ``scale_atol`` the absolute term is multiplied by max|expected| — for sums of many
    terms whose cancellation makes individual elements arbitrarily small."""
    a = actual.detach().cpu().double()
    e = expected.detach().cpu().double()
    assert a.shape == e.shape, f"{what}: shape {tuple(a.shape)} vs {tuple(e.shape)}"
    at = atol * (max(1.0, e.abs().max().item()) if scale_atol and e.numel() else 1.0)
    err = (a - e).abs()
    tol = at + rtol * e.abs()
    bad = err > tol
    if bad.any():
        i = torch.nonzero(bad)[0].tolist()
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{a.numel()} elements out of tolerance; first at {i}: "
            f"got {a[tuple(i)].item():.9g}, expected {e[tuple(i)].item():.9g}; "
            f"max abs err {err.max().item():.3g}")


def graph_from_degrees(degs, n_cols=None, seed=0) -> Graph:
    """CSR whose row r has exactly degs[r] distinct random sources (ascending)."""
    rng = np.random.default_rng(seed)
    n = len(degs)
    n_cols = n if n_cols is None else n_cols
    cols = []
    for d in degs:
        d = int(d)
        assert d <= n_cols
        cols.append(np.sort(rng.choice(n_cols, size=d, replace=False)) if d else np.empty(0, np.int64))
    row_ptr = np.zeros(n + 1, dtype=np.int64)
    row_ptr[1:] = np.cumsum([len(c) for c in cols])
    col = np.concatenate(cols) if cols else np.empty(0, np.int64)
    return Graph(n, torch.from_numpy(row_ptr.astype(np.int32)), torch.from_numpy(col.astype(np.int32)))


def crafted_graphs():
    """Small graphs that hit the edge cases of the segment traversal: empty rows,
    degree 1, 31/32/33, rows longer than one chunk, a hub, trailing empty rows."""
    out = {}
    out["tiny"] = graph_from_degrees([1, 2, 0, 3], seed=1)
    out["empty_rows"] = graph_from_degrees([0, 0, 5, 0, 1, 0, 0], seed=2)
    out["deg_31_32_33"] = graph_from_degrees([31, 32, 33, 1, 64, 65], n_cols=80, seed=3)
    out["hub"] = graph_from_degrees([3] * 40 + [700] + [2] * 40 + [0, 0], n_cols=900, seed=4)
    out["long_rows"] = graph_from_degrees([150, 0, 97, 260, 1, 33], n_cols=300, seed=5)
    rng = np.random.default_rng(6)
    out["random_200"] = graph_from_degrees(rng.integers(0, 40, size=200), n_cols=200, seed=6)
    out["no_edges"] = graph_from_degrees([0, 0, 0], seed=7)
    return out


def power_law_graph(n, mean_deg, seed=0) -> Graph:
    from ae_mlsys_gnn_b200.graphs import chung_lu_graph

    return chung_lu_graph(n, mean_deg, max_deg=min(n - 1, mean_deg * 20), seed=seed)

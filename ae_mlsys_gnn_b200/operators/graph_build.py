"""Graph construction on the GPU: what the reference's scripts do on the host with DGL and
SciPy before the first kernel runs (script/train/train_gatconv_our.py:82-95,
train_gmmconv_our.py:80-93), plus the bookkeeping of the row-block partition.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _capi as capi

I32 = torch.int32


def coo_to_csr(dst: torch.Tensor, src: torch.Tensor, n_nodes: int, self_loops: bool = True):
    """(row_ptr, col_ind) of the in-edge CSR (row = destination, column = source) of the edge list:
    sorted by (dst, src), duplicates removed; with ``self_loops`` existing self-loops are dropped
    and exactly one per node is added (DGL's remove_self_loop + add_self_loop).  int32 CUDA
    tensors in, int32 out.  One host read of the edge count."""
    capi.require(dst, I32, "dst", 1)
    capi.require(src, I32, "src", 1, dst.device)
    dev = dst.device
    m = dst.numel()
    if src.numel() != m:
        raise ValueError("dst and src must have the same length")
    cap = m + (n_nodes if self_loops else 0)
    row_ptr = torch.empty(n_nodes + 1, dtype=I32, device=dev)
    col_buf = torch.empty(max(cap, 1), dtype=I32, device=dev)
    nnz = torch.zeros(1, dtype=torch.int64, device=dev)
    nbytes = capi.workspace_bytes("gnn_coo_to_csr_workspace_bytes", m, n_nodes)
    ws = capi.workspace(dev, nbytes)
    with torch.cuda.device(dev):
        capi.call("gnn_coo_to_csr", capi.ptr(dst), capi.ptr(src), m, n_nodes, int(bool(self_loops)),
                  capi.ptr(row_ptr), capi.ptr(col_buf), capi.ptr(nnz), capi.ptr(ws), ws.numel(), capi.stream_ptr(dev))
    return row_ptr, col_buf[: int(nnz.item())].clone()


def edge_balanced_bounds(row_ptr: torch.Tensor, parts: int) -> list:
    """Row-block boundaries b[0..parts]: b[g] is the first row whose first edge is at or after
    g * nnz / parts, so every block holds about nnz / parts edges and no row is cut."""
    capi.require(row_ptr, I32, "row_ptr", 1)
    dev = row_ptr.device
    out = torch.empty(parts + 1, dtype=I32, device=dev)
    with torch.cuda.device(dev):
        capi.call("gnn_edge_balanced_bounds", capi.ptr(row_ptr), row_ptr.numel() - 1, int(parts), capi.ptr(out),
                  capi.stream_ptr(dev))
    b = out.tolist()
    for g in range(1, len(b)):  # keep the boundaries monotone
        b[g] = max(b[g], b[g - 1])
    return b


def halo_needs(ptr: torch.Tensor, idx: torch.Tensor, bounds: list):
    """For the segment array (ptr, idx) of a square graph cut into row blocks at ``bounds``:
    ``positions`` (uint32 as int32 tensor, world * n + 1 entries), the exclusive scan of the flags
    "block q references id v outside itself" laid out [q][v]; and ``needs`` (int32), the
    concatenation over q of the sorted ids block q needs."""
    capi.require(ptr, I32, "ptr", 1)
    capi.require(idx, I32, "idx", 1, ptr.device)
    dev = ptr.device
    n, world = ptr.numel() - 1, len(bounds) - 1
    positions = torch.empty(world * n + 1, dtype=I32, device=dev)
    bd = torch.tensor(bounds, dtype=I32, device=dev)
    nbytes = capi.workspace_bytes("gnn_halo_needs_workspace_bytes", n, world)
    ws = capi.workspace(dev, nbytes)
    with torch.cuda.device(dev):
        capi.call("gnn_halo_needs", capi.ptr(ptr), capi.ptr(idx), n, idx.numel(), capi.ptr(bd), world,
                  capi.ptr(positions), capi.ptr(ws), ws.numel(), capi.stream_ptr(dev))
        total = int(positions[-1].item())
        needs = torch.empty(max(total, 1), dtype=I32, device=dev)
        capi.call("gnn_compact_flagged", capi.ptr(positions), world * n, n, capi.ptr(needs), capi.stream_ptr(dev))
    return positions, needs[:total]


def halo_remap(idx_block: torch.Tensor, lo: int, hi: int, positions: torch.Tensor, rank: int, n: int) -> torch.Tensor:
    """Ids of one block's edges in the [own rows | halo rows] index space of rank ``rank``."""
    capi.require(idx_block, I32, "idx_block", 1)
    dev = idx_block.device
    ext = torch.empty_like(idx_block)
    base = positions[rank * n:]
    with torch.cuda.device(dev):
        capi.call("gnn_halo_remap", capi.ptr(idx_block), idx_block.numel(), int(lo), int(hi), capi.ptr(base),
                  capi.ptr(ext), capi.stream_ptr(dev))
    return ext

"""CSR -> CSC transpose on the GPU (reference: operators/csr2csc.py).

``csr2csc`` returns ``(col_ptr, row_ind, permute)`` as int32, bit-identical to
``scipy.sparse.csr_matrix((arange(E), col_ind, row_ptr)).tocsc()``, which is what the
reference's training scripts compute on the host
(script/train/train_gatconv_our.py:107-121).  ``sparsetrans`` keeps the reference
signature (operators/csr2csc.py:14-16): it returns the edge values in CSC order.
"""
from __future__ import annotations

import torch

from .. import _capi as capi

I32 = torch.int32


def csr2csc(rowptr, colind, n_cols=None):
    dev = rowptr.device
    capi.require(rowptr, I32, "rowptr", 1)
    capi.require(colind, I32, "colind", 1, dev)
    n_rows = rowptr.numel() - 1
    if n_rows < 0:
        raise ValueError("rowptr must have at least one element")
    n_cols = n_rows if n_cols is None else int(n_cols)
    nnz = colind.numel()
    col_ptr = torch.empty(n_cols + 1, dtype=I32, device=dev)
    row_ind = torch.empty(nnz, dtype=I32, device=dev)
    permute = torch.empty(nnz, dtype=I32, device=dev)
    nbytes = capi.workspace_bytes("gnn_csr2csc_workspace_bytes", nnz)
    ws = capi.workspace(dev, nbytes)
    with torch.cuda.device(dev):
        capi.call("gnn_csr2csc", capi.ptr(rowptr), capi.ptr(colind), n_rows, n_cols, nnz,
                  capi.ptr(col_ptr), capi.ptr(row_ind), capi.ptr(permute), capi.ptr(ws),
                  ws.numel(), capi.stream_ptr(dev))
    if n_cols == n_rows:
        from .fused_gat import note_csr2csc

        note_csr2csc(rowptr, colind, col_ptr, row_ind, permute)
    return col_ptr, row_ind, permute


def sparsetrans(rowptr, colind, numlist):
    """Edge values ``numlist`` (E,) or (E, H) reordered from CSR to CSC order."""
    _, _, permute = csr2csc(rowptr, colind)
    return numlist[permute.long()]

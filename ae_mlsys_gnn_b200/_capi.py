"""ctypes binding of libgnn_b200.so (C ABI declared in include/gnn_b200.h).

The library is built ahead of time by ``ae_mlsys_gnn_b200.build``; there is no
fallback: if it cannot be loaded, importing an operator raises.  PyTorch is used
only to own device memory and streams — tensors cross the boundary as raw
pointers plus sizes.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import build as _build

_I64 = C.c_int64
_INT = C.c_int
_F32 = C.c_float
_PTR = C.c_void_p
_SZ = C.c_size_t
_SZP = C.POINTER(C.c_size_t)

# name -> argument types (return type is int unless listed in _RESTYPES)
PROTOTYPES = {
    "gnn_abi_version": [],
    "gnn_last_error_string": [],
    "gnn_debug_set_chunk": [_INT],
    "gnn_csr2csc_workspace_bytes": [_I64, _SZP],
    "gnn_csr2csc": [_PTR, _PTR, _I64, _I64, _I64, _PTR, _PTR, _PTR, _PTR, _SZ, _PTR],
    "gnn_gat_fwd_workspace_bytes": [_I64, _INT, _INT, _SZP],
    "gnn_gat_fwd": [_PTR, _PTR, _I64, _I64, _PTR, _PTR, _PTR, _INT, _INT, _F32,
                    _PTR, _PTR, _PTR, _PTR, _SZ, _PTR],
    "gnn_gat_fwd_act": [_PTR, _PTR, _I64, _I64, _PTR, _PTR, _PTR, _INT, _INT, _F32, _F32,
                        _PTR, _PTR, _PTR, _PTR, _PTR, _SZ, _PTR],
    "gnn_to_bf16": [_PTR, _I64, _PTR, _PTR],
    "gnn_gat_fwd_bf16": [_PTR, _PTR, _I64, _I64, _PTR, _PTR, _PTR, _INT, _INT, _F32,
                         _PTR, _PTR, _PTR, _PTR, _SZ, _PTR],
    "gnn_gat_fwd_part": [_PTR, _PTR, _I64, _I64, _PTR, _PTR, _PTR, _INT, _INT, _F32,
                         _PTR, _PTR, _PTR, _INT, _INT, _PTR, _SZ, _PTR],
    "gnn_gat_bwd_col_part": [_PTR, _PTR, _I64, _I64, _PTR, _PTR, _PTR, _PTR, _INT, _INT, _F32,
                             _PTR, _PTR, _INT, _PTR, _SZ, _PTR],
    "gnn_gat_bwd_col_edges": [_PTR, _PTR, _I64, _I64, _PTR, _PTR, _PTR, _PTR, _INT, _INT, _F32,
                              _PTR, _PTR, _PTR, _INT, _PTR, _SZ, _PTR],
    "gnn_gat_bwd_pack": [_I64, _PTR, _PTR, _PTR, _PTR, _PTR, _INT, _INT, _PTR, _PTR],
    "gnn_gat_bwd_pack_elu": [_I64, _PTR, _PTR, _PTR, _PTR, _PTR, _INT, _INT, _F32, _PTR, _PTR, _PTR],
    "gnn_gat_bwd_row_sum_workspace_bytes": [_I64, _INT, _SZP],
    "gnn_gat_bwd_row_sum": [_PTR, _PTR, _I64, _I64, _PTR, _INT, _PTR, _PTR, _SZ, _PTR],
    "gnn_invert_permutation": [_PTR, _I64, _PTR, _PTR],
    "gnn_gat_fwd_static_scratch": [_PTR, _PTR, _I64, _I64, _PTR, _PTR, _PTR, _INT, _INT, _F32,
                                   _PTR, _PTR, _PTR, _PTR],
    "gnn_gat_bwd_workspace_bytes": [_I64, _I64, _INT, _INT, _SZP],
    "gnn_gat_bwd": [_PTR, _PTR, _PTR, _PTR, _I64, _I64, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR,
                    _INT, _INT, _F32, _PTR, _PTR, _PTR, _PTR, _SZ, _PTR],
    "gnn_gat_bwd_row_workspace_bytes": [_I64, _INT, _INT, _SZP],
    "gnn_gat_bwd_row": [_PTR, _PTR, _I64, _I64, _PTR, _PTR, _PTR, _PTR, _PTR, _PTR,
                        _INT, _INT, _F32, _PTR, _PTR, _PTR, _SZ, _PTR],
    "gnn_gat_bwd_col_workspace_bytes": [_I64, _INT, _INT, _SZP],
    "gnn_gat_bwd_col": [_PTR, _PTR, _I64, _I64, _PTR, _PTR, _PTR, _PTR, _INT, _INT, _F32,
                        _PTR, _PTR, _PTR, _SZ, _PTR],
    "gnn_gat_scores_fwd": [_PTR, _PTR, _PTR, _I64, _INT, _INT, _PTR, _PTR, _PTR],
    "gnn_gat_scores_bwd_workspace_bytes": [_I64, _INT, _INT, _SZP],
    "gnn_gat_scores_bwd": [_PTR, _PTR, _PTR, _PTR, _PTR, _I64, _INT, _INT, _PTR, _PTR, _PTR,
                           _PTR, _SZ, _PTR],
    "gnn_gat_edge_alpha": [_PTR, _PTR, _I64, _I64, _PTR, _PTR, _PTR, _PTR, _INT, _F32,
                           _PTR, _PTR, _PTR],
    "gnn_edgeconv_fwd": [_INT, _PTR, _PTR, _PTR, _I64, _INT, _PTR, _PTR, _PTR],
    "gnn_edgeconv_bwd": [_PTR, _PTR, _I64, _I64, _INT, _PTR, _PTR],
    "gnn_gmm_sum_fwd": [_PTR, _PTR, _PTR, _I64, _INT, _INT, _PTR, _PTR],
    "gnn_gmm_sum_bwd": [_PTR, _I64, _INT, _INT, _PTR, _PTR],
    "gnn_edgeconv_fwd_act": [_INT, _PTR, _PTR, _PTR, _I64, _INT, _F32, _PTR, _PTR, _PTR],
    "gnn_edgeconv_bwd_act": [_PTR, _PTR, _F32, _PTR, _I64, _I64, _INT, _PTR, _PTR, _PTR],
    "gnn_gmm_fwd_workspace_bytes": [_I64, _INT, _INT, _SZP],
    "gnn_gmm_fwd": [_PTR, _PTR, _I64, _I64, _PTR, _PTR, _PTR, _PTR, _PTR, _INT, _INT, _INT,
                    _PTR, _PTR, _SZ, _PTR],
    "gnn_gaussian_fwd": [_PTR, _PTR, _PTR, _I64, _INT, _INT, _PTR, _PTR],
    "gnn_gaussian_bwd_workspace_bytes": [_I64, _INT, _INT, _SZP],
    "gnn_gaussian_bwd": [_PTR, _PTR, _PTR, _PTR, _I64, _INT, _INT, _PTR, _PTR, _PTR,
                         _PTR, _SZ, _PTR],
    "gnn_gemm_tf32x3_supported": [_I64, _I64, _I64],
    "gnn_gemm_tf32x3_workspace_bytes": [_I64, _I64, _I64, _SZP],
    "gnn_gemm_tf32x3": [_PTR, _PTR, _INT, _PTR, _I64, _I64, _I64, _PTR, _SZ, _PTR, _PTR],
    "gnn_gemm_tf32x3_scores_supported": [_INT, _INT],
    "gnn_gemm_tf32x3_scores": [_PTR, _PTR, _INT, _PTR, _I64, _I64, _I64, _PTR, _PTR, _INT, _INT, _PTR, _PTR,
                               _PTR, _SZ, _PTR, _PTR],
    "gnn_gemm_tf32x3_tn_workspace_bytes": [_I64, _I64, _I64, _SZP],
    "gnn_gemm_tf32x3_tn": [_PTR, _PTR, _PTR, _I64, _I64, _I64, _PTR, _SZ, _PTR, _PTR],
    "gnn_mhspmm_workspace_bytes": [_I64, _INT, _INT, _SZP],
    "gnn_mhspmm": [_PTR, _PTR, _I64, _I64, _PTR, _PTR, _PTR, _INT, _INT, _PTR, _PTR, _SZ, _PTR],
    "gnn_mhsddmm": [_PTR, _PTR, _I64, _I64, _PTR, _PTR, _INT, _INT, _PTR, _PTR],
    "gnn_sddmm_coo": [_PTR, _PTR, _I64, _PTR, _PTR, _INT, _PTR, _PTR],
    "gnn_mhtranspose": [_PTR, _PTR, _I64, _INT, _PTR, _PTR],
    "gnn_u_add_v_fwd": [_PTR, _PTR, _I64, _I64, _PTR, _PTR, _INT, _PTR, _PTR],
    "gnn_u_add_v_bwd": [_PTR, _PTR, _I64, _I64, _I64, _PTR, _INT, _PTR, _PTR, _PTR],
    "gnn_edge_softmax_fwd": [_PTR, _I64, _I64, _PTR, _INT, _PTR, _PTR],
    "gnn_edge_softmax_bwd": [_PTR, _I64, _I64, _PTR, _PTR, _INT, _PTR, _PTR],
    "gnn_coo_to_csr_workspace_bytes": [_I64, _I64, _SZP],
    "gnn_coo_to_csr": [_PTR, _PTR, _I64, _I64, _INT, _PTR, _PTR, _PTR, _PTR, _SZ, _PTR],
    "gnn_edge_balanced_bounds": [_PTR, _I64, _INT, _PTR, _PTR],
    "gnn_halo_needs_workspace_bytes": [_I64, _INT, _SZP],
    "gnn_halo_needs": [_PTR, _PTR, _I64, _I64, _PTR, _INT, _PTR, _PTR, _SZ, _PTR],
    "gnn_compact_flagged": [_PTR, _I64, _I64, _PTR, _PTR],
    "gnn_halo_remap": [_PTR, _I64, _INT, _INT, _PTR, _PTR, _PTR],
    "gnn_knn_graph": [_PTR, _I64, _I64, _INT, _INT, _PTR, _PTR],
    "gnn_peer_alloc": [_SZ, C.POINTER(C.c_void_p), _PTR],
    "gnn_peer_free": [_PTR],
    "gnn_peer_open": [_PTR, C.POINTER(C.c_void_p)],
    "gnn_peer_close": [_PTR],
    "gnn_halo_push": [_PTR, _I64, _PTR, _PTR, _PTR, _INT, _PTR, _I64, _PTR],
    "gnn_halo_push_ranges": [_PTR, _I64, _PTR, _PTR, _PTR, _PTR, _INT, _PTR, _I64, _PTR],
}
_RESTYPES = {"gnn_last_error_string": C.c_char_p}

_lib = None


class GnnError(RuntimeError):
    """A negative return code from libgnn_b200.so."""


def library_path() -> str:
    return _build.LIB


def lib() -> C.CDLL:
    """Loads (building first if the sources are newer) and returns the library."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB
    if os.environ.get("GNN_B200_NO_BUILD", "0") != "1" and _build.needs_build():
        path = _build.build()
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: run `python -m ae_mlsys_gnn_b200.build` (nvcc, sm_100a). "
            "There is no CPU or PyTorch fallback for these operators.")
    handle = C.CDLL(path)
    for name, args in PROTOTYPES.items():
        fn = getattr(handle, name)  # AttributeError if the symbol is not exported
        fn.argtypes = args
        fn.restype = _RESTYPES.get(name, C.c_int)
    if handle.gnn_abi_version() != 1:
        raise ImportError("libgnn_b200.so ABI version mismatch; rebuild the library")
    _lib = handle
    return _lib


def last_error() -> str:
    msg = lib().gnn_last_error_string()
    return msg.decode() if msg else ""


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise GnnError(f"{what} failed with code {rc}: {last_error()}")


# Kernels launched by one call of each entry point (main kernels, merge kernels,
# memsets excluded); bench.py uses it to count its own launches.
KERNELS_PER_CALL = {
    "gnn_csr2csc": None,  # depends on the number of radix passes, see launches_csr2csc
    "gnn_gat_fwd": 2, "gnn_gat_fwd_bf16": 2, "gnn_to_bf16": 1, "gnn_gat_fwd_act": 2, "gnn_gat_fwd_part": 2, "gnn_gat_bwd_col_part": 2,
    "gnn_gat_fwd_static_scratch": 2, "gnn_gat_bwd": 4, "gnn_gat_bwd_row": 2, "gnn_gat_bwd_col": 2,
    "gnn_gat_scores_fwd": 1, "gnn_gat_scores_bwd": 2,
    # weight split + GEMM; GEMM + split reduction (plus one transposing pre-pass per operand
    # whose row length is not a multiple of 4 floats, not counted here)
    "gnn_gemm_tf32x3": 2, "gnn_gemm_tf32x3_scores": 2, "gnn_gemm_tf32x3_tn": 2,
    "gnn_gat_bwd_col_edges": 2, "gnn_gat_bwd_pack": 1, "gnn_gat_bwd_pack_elu": 1, "gnn_gat_bwd_row_sum": 2, "gnn_invert_permutation": 1,
    "gnn_gat_edge_alpha": 1, "gnn_edgeconv_fwd": 1, "gnn_edgeconv_bwd": 1, "gnn_edgeconv_fwd_act": 1,
    "gnn_edgeconv_bwd_act": 1, "gnn_gmm_fwd": 2, "gnn_gmm_sum_fwd": 1, "gnn_gmm_sum_bwd": 1,
    "gnn_gaussian_fwd": 1, "gnn_gaussian_bwd": 2, "gnn_mhspmm": 2, "gnn_mhsddmm": 1,
    "gnn_sddmm_coo": 1, "gnn_mhtranspose": 1, "gnn_u_add_v_fwd": 1, "gnn_u_add_v_bwd": 1,
    "gnn_edge_softmax_fwd": 1, "gnn_edge_softmax_bwd": 1, "gnn_knn_graph": 1, "gnn_halo_push": 1, "gnn_halo_push_ranges": 1,
}


class CallTimer:
    """Optional per-entry-point timing with CUDA events on the launching stream.
    ``records`` holds (name, start_event, end_event) for every call made while the
    timer is installed; ``counts`` the number of calls per entry point."""

    def __init__(self, with_events: bool = True):
        self.with_events = with_events
        self.records: list[tuple[str, torch.cuda.Event, torch.cuda.Event]] = []
        self.counts: dict[str, int] = {}

    def totals_ms(self) -> dict[str, float]:
        out: dict[str, float] = {}
        for name, a, b in self.records:
            out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        return out


_timer: CallTimer | None = None


def install_timer(timer: CallTimer | None) -> None:
    global _timer
    _timer = timer


def call(name: str, *args) -> None:
    t = _timer
    if t is None:
        check(getattr(lib(), name)(*args), name)
        return
    t.counts[name] = t.counts.get(name, 0) + 1
    if not t.with_events:
        check(getattr(lib(), name)(*args), name)
        return
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    check(getattr(lib(), name)(*args), name)
    b.record()
    t.records.append((name, a, b))


def workspace_bytes(name: str, *args) -> int:
    out = C.c_size_t(0)
    check(getattr(lib(), name)(*args, C.byref(out)), name)
    return int(out.value)


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def require(t: torch.Tensor, dtype: torch.dtype, name: str, ndim: int | None = None,
            device: torch.device | None = None) -> torch.Tensor:
    """Argument validation that the reference does with C asserts
    (src/fused_gat/fused_gat_SM.cpp:22-36): CUDA device, dtype, contiguity."""
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (no CPU path exists)")
    if device is not None and t.device != device:
        raise ValueError(f"{name} is on {t.device}, expected {device}")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise ValueError(f"{name} must have {ndim} dims, got shape {tuple(t.shape)}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t


_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """A per-(device, stream) scratch buffer that only grows; contents are undefined."""
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = None
        _workspaces.pop(key, None)
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf

"""The C-ABI library loads without a GPU and exports every declared symbol."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    src = open(os.path.join(ROOT, "include", "gnn_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(gnn_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_exported():
    from ae_mlsys_gnn_b200 import _capi

    lib = ctypes.CDLL(_capi._build.build())
    names = _declared()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/gnn_b200.h but not exported"


def test_prototypes_cover_header():
    from ae_mlsys_gnn_b200 import _capi

    assert sorted(_capi.PROTOTYPES) == _declared()
    assert _capi.lib().gnn_abi_version() == 1


def test_argument_errors_without_gpu():
    """Argument validation happens before any CUDA call."""
    from ae_mlsys_gnn_b200 import _capi

    lib = _capi.lib()
    out = ctypes.c_size_t(0)
    assert lib.gnn_gat_fwd_workspace_bytes(1000, 4, 64, ctypes.byref(out)) == 0 and out.value > 0
    assert lib.gnn_gat_fwd_workspace_bytes(-1, 4, 64, ctypes.byref(out)) == -1
    assert "bad argument" in _capi.last_error()
    assert lib.gnn_csr2csc(None, None, -1, 0, 0, None, None, None, None, 0, None) == -1
    assert lib.gnn_edgeconv_fwd(0, None, None, None, 4, 4, None, None, None) == -1


def test_operators_refuse_cpu_tensors():
    import pytest
    import torch

    from ae_mlsys_gnn_b200.operators.fused_gat import gat_forward

    rp = torch.tensor([0, 1], dtype=torch.int32)
    ci = torch.tensor([0], dtype=torch.int32)
    with pytest.raises(ValueError, match="CUDA"):
        gat_forward(torch.zeros(1, 1), torch.zeros(1, 1), rp, ci, 0.2, torch.zeros(1, 1, 4))

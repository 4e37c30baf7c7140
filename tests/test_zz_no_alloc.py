"""gnn_gat_fwd_static_scratch: the GAT forward for hosts that must not allocate device
memory while they run a layer (a serving process whose pool owns the whole GPU, a plugin
inside another program's memory plan).  Its scratch is a fixed 16 MiB array inside the
library instead of a caller-provided workspace, so the only thing to check is that it
gives what gnn_gat_fwd gives — on two calls in a row, because the second call finds the
array holding the first call's leftovers.  Collected last (file name) so that a run that
stops at the first failure has already run every other test."""
import ctypes

import pytest
import torch

from tests.util import ATOL, RTOL, assert_close, power_law_graph

pytestmark = pytest.mark.gpu


def _run_pair(cuda, g, H, F, seed):
    from ae_mlsys_gnn_b200 import _capi as capi

    lib = capi.lib()
    gen = torch.Generator().manual_seed(seed)
    attn_row = torch.randn(g.n, H, generator=gen).to(cuda)
    attn_col = torch.randn(g.n, H, generator=gen).to(cuda)
    feat = torch.randn(g.n, H, F, generator=gen).to(cuda)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    stream = torch.cuda.current_stream(cuda).cuda_stream

    def outputs():
        return (torch.empty(g.n, H, F, device=cuda), torch.empty(g.n, H, device=cuda),
                torch.empty(g.n, H, device=cuda))

    ref_out = outputs()
    need = capi.workspace_bytes("gnn_gat_fwd_workspace_bytes", g.nnz, H, F)
    ws = torch.empty(need, dtype=torch.uint8, device=cuda)
    rc = lib.gnn_gat_fwd(rp.data_ptr(), ci.data_ptr(), g.n, g.nnz, attn_row.data_ptr(),
                         attn_col.data_ptr(), feat.data_ptr(), H, F, 0.2, ref_out[0].data_ptr(),
                         ref_out[1].data_ptr(), ref_out[2].data_ptr(), ws.data_ptr(), need, stream)
    assert rc == 0, capi.last_error()
    got = outputs()
    rc = lib.gnn_gat_fwd_static_scratch(rp.data_ptr(), ci.data_ptr(), g.n, g.nnz, attn_row.data_ptr(),
                                        attn_col.data_ptr(), feat.data_ptr(), H, F, 0.2,
                                        got[0].data_ptr(), got[1].data_ptr(), got[2].data_ptr(), stream)
    assert rc == 0, capi.last_error()
    torch.cuda.synchronize()
    for name, a, e in zip(("out", "edge_max", "edge_sum"), got, ref_out):
        assert_close(a, e, f"static-scratch {name}", rtol=RTOL, atol=ATOL)


def test_static_scratch_matches_workspace_variant_twice(cuda):
    # rows long enough to be split across chunks, so the scratch is really used;
    # the second call has another shape and finds the first call's data in the array
    _run_pair(cuda, power_law_graph(3000, 60, seed=21), 4, 64, 1)
    _run_pair(cuda, power_law_graph(2500, 45, seed=22), 1, 41, 2)


def test_static_scratch_refuses_oversized_problem(cuda):
    """Beyond 16 MiB of scratch the call is refused before anything is launched (no
    device pointer is touched, so dummy addresses are safe here)."""
    from ae_mlsys_gnn_b200 import _capi as capi

    lib = capi.lib()
    nnz, H, F = 200_000_000, 4, 128
    assert capi.workspace_bytes("gnn_gat_fwd_workspace_bytes", nnz, H, F) > (16 << 20)
    one = ctypes.c_void_p(256)
    rc = lib.gnn_gat_fwd_static_scratch(one, one, 10, nnz, one, one, one, H, F, 0.2, one, one, one, None)
    assert rc == -5
    assert "16 MiB" in capi.last_error()

"""The unfused operators that share the reference API, against the oracle."""
import pytest
import torch

from oracle import ops as ref
from tests.util import assert_close, crafted_graphs, power_law_graph

pytestmark = pytest.mark.gpu


def _sq(g):
    from tests.test_gat_gpu import _square

    return _square(g)


@pytest.mark.parametrize("name", ["tiny", "empty_rows", "hub", "random_200", "no_edges"])
@pytest.mark.parametrize("H", [1, 4, 3])
def test_edge_softmax(cuda, name, H):
    from ae_mlsys_gnn_b200.operators.edge_softmax import csr_edge_softmax

    g = crafted_graphs()[name]
    gen = torch.Generator().manual_seed(1)
    h = torch.randn(g.nnz, H, generator=gen) * 3
    gout = torch.randn(g.nnz, H, generator=gen)
    hd = h.to(cuda).requires_grad_(True)
    out = csr_edge_softmax(g.row_ptr.to(cuda), hd)
    out.backward(gout.to(cuda))
    hr = h.double().requires_grad_(True)
    eo = ref.edge_softmax(g.row_ptr, hr)
    eo.backward(gout.double())
    assert_close(out, eo, "edge_softmax")
    assert_close(hd.grad, hr.grad, "edge_softmax grad", scale_atol=True)


@pytest.mark.parametrize("H", [1, 4, 3, 8])
def test_edge_softmax_heavy_segments(cuda, H):
    """Segments long enough for the whole-CTA path (two in one CTA's group of rows, one at the
    very end), next to short ones; two runs are bit-identical."""
    from ae_mlsys_gnn_b200.operators.edge_softmax import csr_edge_softmax
    from tests.util import graph_from_degrees

    g = graph_from_degrees([3] * 10 + [5000] + [2] * 3 + [2048] + [7] * 20 + [0, 2047, 2500], n_cols=6000, seed=8)
    gen = torch.Generator().manual_seed(3)
    h = torch.randn(g.nnz, H, generator=gen) * 3
    gout = torch.randn(g.nnz, H, generator=gen)
    hd = h.to(cuda).requires_grad_(True)
    out = csr_edge_softmax(g.row_ptr.to(cuda), hd)
    out.backward(gout.to(cuda))
    hr = h.double().requires_grad_(True)
    eo = ref.edge_softmax(g.row_ptr, hr)
    eo.backward(gout.double())
    assert_close(out, eo, "edge_softmax")
    assert_close(hd.grad, hr.grad, "edge_softmax grad", scale_atol=True)
    hd2 = h.to(cuda).requires_grad_(True)
    out2 = csr_edge_softmax(g.row_ptr.to(cuda), hd2)
    out2.backward(gout.to(cuda))
    assert torch.equal(out, out2) and torch.equal(hd.grad, hd2.grad)


@pytest.mark.parametrize("name", ["tiny", "empty_rows", "hub", "random_200"])
@pytest.mark.parametrize("F", [1, 4, 33, 32, 8])
def test_u_add_v(cuda, name, F):
    from ae_mlsys_gnn_b200.operators.u_add_v import u_add_v_op

    g = _sq(crafted_graphs()[name])
    gen = torch.Generator().manual_seed(2)
    rv, cv = torch.randn(g.n, F, generator=gen), torch.randn(g.n, F, generator=gen)
    gout = torch.randn(g.nnz, F, generator=gen)
    rd, cd = rv.to(cuda).requires_grad_(True), cv.to(cuda).requires_grad_(True)
    out = u_add_v_op(g.row_ptr.to(cuda), g.col_ind.to(cuda), rd, cd)
    out.backward(gout.to(cuda))
    rr, cr = rv.double().requires_grad_(True), cv.double().requires_grad_(True)
    eo = ref.u_add_v(g.row_ptr, g.col_ind, rr, cr)
    eo.backward(gout.double())
    assert_close(out, eo, "u_add_v")
    assert_close(rd.grad, rr.grad, "grad_row", scale_atol=True)
    assert_close(cd.grad, cr.grad, "grad_col", scale_atol=True)


@pytest.mark.parametrize("H,F", [(1, 16), (4, 64), (3, 5), (8, 8), (16, 8), (2, 300), (1, 512)])
def test_mhspmm_autograd(cuda, H, F):
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc
    from ae_mlsys_gnn_b200.operators.mhspmm import csrmhspmm

    g = power_law_graph(300, 12, seed=4)
    gen = torch.Generator().manual_seed(3)
    feat, att = torch.randn(g.n, H, F, generator=gen), torch.randn(g.nnz, H, generator=gen)
    gout = torch.randn(g.n, H, F, generator=gen)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    cp, ri, pm = csr2csc(rp, ci)
    fd, ad = feat.to(cuda).requires_grad_(True), att.to(cuda).requires_grad_(True)
    out = csrmhspmm(rp, ci, cp, ri, pm, fd, ad)
    out.backward(gout.to(cuda))
    fr, ar = feat.double().requires_grad_(True), att.double().requires_grad_(True)
    eo = ref.mhspmm(g.row_ptr, g.col_ind, ar, fr)
    eo.backward(gout.double())
    assert_close(out, eo, "mhspmm", scale_atol=True)
    assert_close(fd.grad, fr.grad, "grad_feat", scale_atol=True)
    assert_close(ad.grad, ar.grad, "grad_att", scale_atol=True)


def test_mhspmm_wide_rows_forward(cuda):
    """Rows wider than the largest tile are processed in column slabs."""
    from ae_mlsys_gnn_b200.operators.mhspmm import mhspmm_forward

    g = power_law_graph(120, 9, seed=5)
    gen = torch.Generator().manual_seed(4)
    for H, F in [(1, 600), (2, 1100), (1, 301)]:
        feat, att = torch.randn(g.n, H, F, generator=gen), torch.randn(g.nnz, H, generator=gen)
        out = mhspmm_forward(g.row_ptr.to(cuda), g.col_ind.to(cuda), att.to(cuda), feat.to(cuda))
        assert_close(out, ref.mhspmm(g.row_ptr, g.col_ind, att, feat), f"mhspmm {H}x{F}", scale_atol=True)


@pytest.mark.parametrize("weighted", [False, True])
@pytest.mark.parametrize("sym", [False, True])
def test_csrspmm(cuda, weighted, sym):
    from ae_mlsys_gnn_b200.graphs import rmat_graph, uniform_graph
    from ae_mlsys_gnn_b200.operators.spmm import csrspmm

    g = rmat_graph(256, 1500, seed=1) if sym else uniform_graph(256, 2000, seed=1)
    gen = torch.Generator().manual_seed(5)
    x = torch.randn(g.n, 24, generator=gen)
    w = torch.rand(g.nnz, generator=gen) if weighted else None
    if sym and weighted:  # symmetric values: w(r,c) = w(c,r)
        rows = ref.rows_of(g.row_ptr)
        lo, hi = torch.minimum(rows, g.col_ind.long()), torch.maximum(rows, g.col_ind.long())
        w = ((lo * 7 + hi * 13) % 17).float() / 17 + 0.1
    gout = torch.randn(g.n, 24, generator=gen)
    xd = x.to(cuda).requires_grad_(True)
    wd = w.to(cuda).requires_grad_(True) if weighted else None
    out = csrspmm(g.row_ptr.to(cuda), g.col_ind.to(cuda), xd, wd, sym)
    out.backward(gout.to(cuda))
    xr = x.double().requires_grad_(True)
    wr = w.double().requires_grad_(True) if weighted else None
    eo = ref.mhspmm(g.row_ptr, g.col_ind, None if wr is None else wr[:, None], xr[:, None, :])[:, 0]
    eo.backward(gout.double())
    assert_close(out, eo, "spmm", scale_atol=True)
    assert_close(xd.grad, xr.grad, "grad_x", scale_atol=True)
    if weighted:
        assert_close(wd.grad, wr.grad, "grad_w", scale_atol=True)


@pytest.mark.parametrize("F", [1, 8, 30, 64, 130])
def test_sddmm(cuda, F):
    from ae_mlsys_gnn_b200.operators.spmm import coo_sddmm, csr_sddmm

    g = power_law_graph(200, 9, seed=6)
    gen = torch.Generator().manual_seed(6)
    a, b = torch.randn(g.n, F, generator=gen), torch.randn(g.n, F, generator=gen)
    rows = ref.rows_of(g.row_ptr).to(torch.int32)
    e = ref.coo_sddmm(rows, g.col_ind, a, b)
    got = csr_sddmm(g.row_ptr.to(cuda), g.col_ind.to(cuda), a.to(cuda), b.to(cuda))
    assert_close(got, e, "csr_sddmm", scale_atol=True)
    got = coo_sddmm(rows.to(cuda), g.col_ind.to(cuda), a.to(cuda), b.to(cuda))
    assert_close(got, e, "coo_sddmm", scale_atol=True)


def test_sparsetrans_and_mhtranspose(cuda):
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc, sparsetrans
    from ae_mlsys_gnn_b200.operators.mhspmm import mhtranspose_forward

    g = power_law_graph(500, 10, seed=8)
    vals = torch.randn(g.nnz, 4, generator=torch.Generator().manual_seed(1))
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    _, _, pm = csr2csc(rp, ci)
    _, _, epm = ref.csr2csc(g.row_ptr, g.col_ind)
    assert torch.equal(mhtranspose_forward(pm, vals.to(cuda)).cpu(), ref.mhtranspose(epm, vals))
    assert torch.equal(sparsetrans(rp, ci, vals[:, 0].contiguous().to(cuda)).cpu(), vals[:, 0][epm.long()])


@pytest.mark.parametrize("op", ["fused_gat_stash_op", "fused_gat_fusescatter", "fused_gat_op"])
def test_gat_variants_agree(cuda, op):
    import ae_mlsys_gnn_b200.operators.fused_gat as M
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc

    g = power_law_graph(400, 14, seed=9)
    gen = torch.Generator().manual_seed(9)
    H, F = 4, 16
    ar, ac = torch.randn(g.n, H, generator=gen), torch.randn(g.n, H, generator=gen)
    feat, gout = torch.randn(g.n, H, F, generator=gen), torch.randn(g.n, H, F, generator=gen)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    cp, ri, pm = csr2csc(rp, ci)
    dv = [t.to(cuda).requires_grad_(True) for t in (ar, ac, feat)]
    args = (dv[0], dv[1], rp, ci, cp, ri, 0.2, dv[2])
    out = getattr(M, op)(*args, pm) if op != "fused_gat_op" else M.fused_gat_op(*args)
    out.backward(gout.to(cuda))
    eo, em, es = ref.gat_forward(ar, ac, g.row_ptr, g.col_ind, 0.2, feat)
    ef, ear, eac = ref.gat_backward(0.2, g.row_ptr, g.col_ind, em, es, feat, ar, ac, gout)
    assert_close(out, eo, "out")
    assert_close(dv[2].grad, ef, "grad_feat", scale_atol=True)
    assert_close(dv[0].grad, ear, "grad_attn_row", scale_atol=True)
    assert_close(dv[1].grad, eac, "grad_attn_col", scale_atol=True)


def test_gat_edge_alpha(cuda):
    from ae_mlsys_gnn_b200.operators.fused_gat import gat_edge_alpha, gat_forward

    g = power_law_graph(300, 11, seed=10)
    gen = torch.Generator().manual_seed(10)
    H, F = 2, 8
    ar, ac, feat = torch.randn(g.n, H, generator=gen), torch.randn(g.n, H, generator=gen), torch.randn(g.n, H, F, generator=gen)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    _, m, s = gat_forward(ar.to(cuda), ac.to(cuda), rp, ci, 0.2, feat.to(cuda))
    relu, alpha = gat_edge_alpha(ar.to(cuda), ac.to(cuda), rp, ci, m, s, 0.2)
    _, em, es = ref.gat_forward(ar, ac, g.row_ptr, g.col_ind, 0.2, feat)
    er, ea = ref.gat_alpha(ar, ac, g.row_ptr, g.col_ind, 0.2, em, es)
    assert_close(relu, er, "edge_relu")
    assert_close(alpha, ea, "edge_softmax")

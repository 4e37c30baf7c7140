"""Parity of the fused GAT forward/backward (CUDA, through the C ABI) with the CPU
oracle.  Tolerance: rel 1e-4 / abs 1e-5 on fp32 outputs and gradients."""
import pytest
import torch

from oracle import ops as ref
from tests.util import assert_close, crafted_graphs, power_law_graph

pytestmark = pytest.mark.gpu

SHAPES = [(1, 8), (4, 64), (4, 128), (8, 8), (1, 7), (1, 41), (1, 47), (2, 16), (3, 12), (1, 128),
          (1, 256), (2, 100), (1, 5), (1, 13), (1, 30), (1, 61), (1, 63)]


def _inputs(g, H, F, seed, n_cols=None):
    gen = torch.Generator().manual_seed(seed)
    n_cols = g.n if n_cols is None else n_cols
    attn_row = torch.randn(g.n, H, generator=gen)
    attn_col = torch.randn(n_cols, H, generator=gen)
    feat = torch.randn(n_cols, H, F, generator=gen)
    gout = torch.randn(g.n, H, F, generator=gen)
    return attn_row, attn_col, feat, gout


def _n_cols(g):
    return max(g.n, int(g.col_ind.max().item()) + 1 if g.nnz else g.n)


@pytest.mark.parametrize("name", list(crafted_graphs().keys()))
@pytest.mark.parametrize("H,F", SHAPES)
def test_gat_forward_crafted(cuda, name, H, F):
    from ae_mlsys_gnn_b200.operators.fused_gat import gat_forward

    g = crafted_graphs()[name]
    nc = _n_cols(g)
    attn_row, attn_col, feat, _ = _inputs(g, H, F, 1, nc)
    out, m, s = gat_forward(attn_row.to(cuda), attn_col.to(cuda), g.row_ptr.to(cuda),
                            g.col_ind.to(cuda), 0.2, feat.to(cuda))
    eo, em, es = ref.gat_forward(attn_row, attn_col, g.row_ptr, g.col_ind, 0.2, feat)
    assert_close(out, eo, f"out[{name}]")
    assert_close(m, em, f"edge_max[{name}]", rtol=1e-6, atol=1e-6 )
    assert_close(s, es, f"edge_sum[{name}]")


def _square(g):
    """Crafted graphs may be rectangular; the fused backward API wants a square graph."""
    from ae_mlsys_gnn_b200.graphs import Graph

    nc = _n_cols(g)
    if nc == g.n:
        return g
    rp = torch.cat([g.row_ptr, g.row_ptr[-1:].expand(nc - g.n)])
    return Graph(nc, rp.contiguous(), g.col_ind)


@pytest.mark.parametrize("name", list(crafted_graphs().keys()))
@pytest.mark.parametrize("H,F", [(4, 64), (4, 128), (8, 8), (1, 7), (1, 47), (2, 16), (3, 12), (1, 13), (1, 30),
                                 (1, 61)])
def test_gat_backward_crafted(cuda, name, H, F):
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc
    from ae_mlsys_gnn_b200.operators.fused_gat import gat_backward, gat_forward

    g = _square(crafted_graphs()[name])
    attn_row, attn_col, feat, gout = _inputs(g, H, F, 2)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    cp, ri, _ = csr2csc(rp, ci)
    d = [t.to(cuda) for t in (attn_row, attn_col, feat, gout)]
    out, m, s = gat_forward(d[0], d[1], rp, ci, 0.2, d[2])
    gf, gar, gac = gat_backward(0.2, rp, ci, cp, ri, m, s, d[2], d[0], d[1], d[3])
    _, em, es = ref.gat_forward(attn_row, attn_col, g.row_ptr, g.col_ind, 0.2, feat)
    ef, ear, eac = ref.gat_backward(0.2, g.row_ptr, g.col_ind, em, es, feat, attn_row, attn_col, gout)
    assert_close(gf, ef, f"grad_feat[{name}]", scale_atol=True)
    assert_close(gar, ear, f"grad_attn_row[{name}]", scale_atol=True)
    assert_close(gac, eac, f"grad_attn_col[{name}]", scale_atol=True)


@pytest.mark.parametrize("H,F", [(4, 64), (1, 41), (4, 128)])
def test_gat_power_law(cuda, H, F):
    """A power-law graph large enough that many rows are split across chunks."""
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc
    from ae_mlsys_gnn_b200.operators.fused_gat import gat_backward, gat_forward

    g = power_law_graph(3000, 60, seed=3)
    attn_row, attn_col, feat, gout = _inputs(g, H, F, 3)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    cp, ri, _ = csr2csc(rp, ci)
    d = [t.to(cuda) for t in (attn_row, attn_col, feat, gout)]
    out, m, s = gat_forward(d[0], d[1], rp, ci, 0.2, d[2])
    eo, em, es = ref.gat_forward(attn_row, attn_col, g.row_ptr, g.col_ind, 0.2, feat)
    assert_close(out, eo, "out")
    assert_close(s, es, "edge_sum")
    gf, gar, gac = gat_backward(0.2, rp, ci, cp, ri, m, s, d[2], d[0], d[1], d[3])
    ef, ear, eac = ref.gat_backward(0.2, g.row_ptr, g.col_ind, em, es, feat, attn_row, attn_col, gout)
    assert_close(gf, ef, "grad_feat", scale_atol=True)
    assert_close(gar, ear, "grad_attn_row", scale_atol=True)
    assert_close(gac, eac, "grad_attn_col", scale_atol=True)


def test_gat_deterministic(cuda):
    """No atomics anywhere in forward or backward: two runs are bit-identical."""
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc
    from ae_mlsys_gnn_b200.operators.fused_gat import gat_backward, gat_forward

    g = power_law_graph(2000, 50, seed=5)
    attn_row, attn_col, feat, gout = _inputs(g, 4, 64, 5)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    cp, ri, _ = csr2csc(rp, ci)
    d = [t.to(cuda) for t in (attn_row, attn_col, feat, gout)]
    runs = []
    for _ in range(2):
        out, m, s = gat_forward(d[0], d[1], rp, ci, 0.2, d[2])
        runs.append((out, m, s) + gat_backward(0.2, rp, ci, cp, ri, m, s, d[2], d[0], d[1], d[3]))
    for a, b in zip(*runs):
        assert torch.equal(a, b)


def test_gat_autograd_layer(cuda):
    """GATConv layer (projection + fused op) against autograd of the DGL-style
    restatement, gradients of W / attn_l / attn_r / input included."""
    from ae_mlsys_gnn_b200.layers import GATConv
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc

    torch.manual_seed(0)
    g = power_law_graph(500, 20, seed=7)
    layer = GATConv(24, 16, 4).to(cuda)
    x = torch.randn(g.n, 24)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    cp, ri, _ = csr2csc(rp, ci)
    xd = x.to(cuda).requires_grad_(True)
    out = layer(rp, ci, cp, ri, xd)
    gout = torch.randn(out.shape, generator=torch.Generator().manual_seed(1))
    out.backward(gout.to(cuda))

    W = layer.W.detach().cpu().double().requires_grad_(True)
    al = layer.attn_l.detach().cpu().double().requires_grad_(True)
    ar = layer.attn_r.detach().cpu().double().requires_grad_(True)
    xr = x.double().requires_grad_(True)
    eo = ref.gat_layer_dgl(g.row_ptr, g.col_ind, xr, W, al, ar, 0.2)
    eo.backward(gout.double())
    assert_close(out, eo, "layer out")
    assert_close(layer.W.grad, W.grad, "W.grad", scale_atol=True)
    assert_close(layer.attn_l.grad, al.grad, "attn_l.grad", scale_atol=True)
    assert_close(layer.attn_r.grad, ar.grad, "attn_r.grad", scale_atol=True)
    assert_close(xd.grad, xr.grad, "x.grad", scale_atol=True)


def test_gat_backward_single_entry_point(cuda):
    """gnn_gat_bwd (both passes in one call) equals the two separately called passes."""
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc
    from ae_mlsys_gnn_b200.operators.fused_gat import (gat_backward, gat_backward_single_call,
                                                       gat_forward)

    g = power_law_graph(1500, 40, seed=8)
    attn_row, attn_col, feat, gout = _inputs(g, 4, 32, 8)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    cp, ri, _ = csr2csc(rp, ci)
    d = [t.to(cuda) for t in (attn_row, attn_col, feat, gout)]
    _, m, s = gat_forward(d[0], d[1], rp, ci, 0.2, d[2])
    a = gat_backward(0.2, rp, ci, cp, ri, m, s, d[2], d[0], d[1], d[3])
    b = gat_backward_single_call(0.2, rp, ci, cp, ri, m, s, d[2], d[0], d[1], d[3])
    for x, y in zip(a, b):
        assert torch.equal(x, y)


@pytest.mark.parametrize("H,F", [(4, 128), (4, 64), (8, 8), (1, 7), (1, 47), (3, 12), (2, 100)])
def test_gat_scores_kernels(cuda, H, F):
    """One-pass score kernels against the framework formulation of
    layers/gatconv_layer.py:52-53 and its autograd backward (fp64)."""
    from ae_mlsys_gnn_b200.operators.fused_gat import gat_scores_backward, gat_scores_forward

    gen = torch.Generator().manual_seed(H * 100 + F)
    n = 3001
    h = torch.randn(n, H, F, generator=gen)
    al, ar = torch.randn(1, H, F, generator=gen), torch.randn(1, H, F, generator=gen)
    gar, gac = torch.randn(n, H, generator=gen), torch.randn(n, H, generator=gen)
    gf = torch.randn(n, H, F, generator=gen)
    row, col = gat_scores_forward(h.to(cuda), al.to(cuda), ar.to(cuda))
    hd = h.double().requires_grad_(True)
    ald, ard = al.double().requires_grad_(True), ar.double().requires_grad_(True)
    er, ec = (ald * hd).sum(-1), (ard * hd).sum(-1)
    (er * gar.double()).sum().add((ec * gac.double()).sum()).backward()
    assert_close(row, er, "attn_row", scale_atol=True)
    assert_close(col, ec, "attn_col", scale_atol=True)
    gfd = gf.to(cuda).clone()
    gl, gr = gat_scores_backward(h.to(cuda), al.to(cuda), ar.to(cuda), gar.to(cuda), gac.to(cuda), gfd)
    assert_close(gfd, gf.double() + hd.grad, "grad_feat (in place)", scale_atol=True)
    assert_close(gl, ald.grad[0], "grad_attn_l", scale_atol=True)
    assert_close(gr, ard.grad[0], "grad_attn_r", scale_atol=True)


def test_gat_layer_unfused_scores_path(cuda):
    """GATConv with fuse_scores off is composed like the reference layer (framework ops
    around fused_gat_op) and must agree with the fused-scores path."""
    from ae_mlsys_gnn_b200.layers import GATConv
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc

    torch.manual_seed(3)
    g = power_law_graph(600, 20, seed=9)
    layer = GATConv(16, 8, 4).to(cuda)
    x = torch.randn(g.n, 16, device=cuda)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    cp, ri, _ = csr2csc(rp, ci)
    gout = torch.randn(g.n, 4, 8, device=cuda)
    res = []
    for fuse in (True, False):
        layer.fuse_scores = fuse
        layer.zero_grad()
        xd = x.clone().requires_grad_(True)
        out = layer(rp, ci, cp, ri, xd)
        out.backward(gout)
        res.append((out.detach(), xd.grad, layer.W.grad.clone(), layer.attn_l.grad.clone(),
                    layer.attn_r.grad.clone()))
    for name, a, b in zip(("out", "x.grad", "W.grad", "attn_l.grad", "attn_r.grad"), *res):
        assert_close(a, b, name, scale_atol=True)


@pytest.mark.parametrize("H,F", [(4, 128), (4, 64), (1, 47), (3, 12)])
@pytest.mark.parametrize("pieces", [2, 5])
def test_gat_column_pieces_match_single_launch(cuda, H, F, pieces):
    """Forward and column pass launched once per column / row piece of the graph, with the
    running state merged between launches, equal the single launch (same tolerance as
    against the oracle; the order of summation differs)."""
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc
    from ae_mlsys_gnn_b200.operators.fused_gat import (gat_backward_col, gat_backward_col_part,
                                                       gat_backward_row, gat_forward, gat_forward_part)
    from ae_mlsys_gnn_b200.partition import _split_by_piece

    g = power_law_graph(2500, 45, seed=12)
    # leave some rows without edges in some pieces, and some without any edge
    attn_row, attn_col, feat, gout = _inputs(g, H, F, 12)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    cp, ri, _ = csr2csc(rp, ci)
    d = [t.to(cuda) for t in (attn_row, attn_col, feat, gout)]
    out, m, s = gat_forward(d[0], d[1], rp, ci, 0.2, d[2])
    span = -(-g.n // pieces)
    seg = torch.repeat_interleave(torch.arange(g.n, device=cuda), (rp[1:] - rp[:-1]).long())
    parts = _split_by_piece(rp, ci.long(), seg, pieces, span)
    out2 = torch.full_like(out, float("nan"))
    m2, s2 = torch.full_like(m, float("nan")), torch.full_like(s, float("nan"))
    for c, (rp_c, ci_c) in enumerate(parts):
        gat_forward_part(d[0], d[1], rp_c, ci_c, 0.2, d[2], out2, m2, s2, c > 0, c == pieces - 1)
    assert_close(out2, out, "out by pieces")
    assert_close(s2, s, "edge_sum by pieces")
    assert torch.equal(m2, m)

    _, rowpack = gat_backward_row(0.2, rp, ci, m, s, d[2], d[0], d[1], d[3])
    gf, gac = gat_backward_col(0.2, cp, ri, d[2], d[1], rowpack, d[3])
    cseg = torch.repeat_interleave(torch.arange(g.n, device=cuda), (cp[1:] - cp[:-1]).long())
    cparts = _split_by_piece(cp, ri.long(), cseg, pieces, span)
    gf2, gac2 = torch.full_like(gf, float("nan")), torch.full_like(gac, float("nan"))
    for c, (cp_c, ri_c) in enumerate(cparts):
        gat_backward_col_part(0.2, cp_c, ri_c, d[2], d[1], rowpack, d[3], gf2, gac2, c > 0)
    assert_close(gf2, gf, "grad_feat by pieces", scale_atol=True)
    assert_close(gac2, gac, "grad_attn_col by pieces", scale_atol=True)


# ---- one-gather backward: forward output + per-edge gradients instead of the row pass ------

def _one_gather(cuda, g, H, F, seed):
    from ae_mlsys_gnn_b200.operators import fused_gat as G
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc

    attn_row, attn_col, feat, gout = _inputs(g, H, F, seed)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    cp, ri, pm = csr2csc(rp, ci)
    d = [t.to(cuda) for t in (attn_row, attn_col, feat, gout)]
    out, m, s = G.gat_forward(d[0], d[1], rp, ci, 0.2, d[2])
    pos = G.csr_positions(rp, ci, cp, ri)
    assert pos is not None and torch.equal(pm[pos.long()].cpu(), torch.arange(g.nnz, dtype=torch.int32))
    got = G.gat_backward_with_output(0.2, rp, ci, cp, ri, pos, m, s, d[2], d[0], d[1], out, d[3])
    two = G.gat_backward(0.2, rp, ci, cp, ri, m, s, d[2], d[0], d[1], d[3])
    _, em, es = ref.gat_forward(attn_row, attn_col, g.row_ptr, g.col_ind, 0.2, feat)
    exp = ref.gat_backward(0.2, g.row_ptr, g.col_ind, em, es, feat, attn_row, attn_col, gout)
    return got, two, exp


@pytest.mark.parametrize("name", list(crafted_graphs().keys()))
@pytest.mark.parametrize("H,F", [(4, 64), (4, 128), (8, 8), (1, 7), (1, 47), (2, 16), (3, 12), (1, 13), (1, 30),
                                 (1, 61)])
def test_gat_one_gather_backward_crafted(cuda, name, H, F):
    g = _square(crafted_graphs()[name])
    got, two, exp = _one_gather(cuda, g, H, F, 12)
    for a, b, e, what in zip(got, two, exp, ("grad_feat", "grad_attn_row", "grad_attn_col")):
        assert_close(a, e, f"{what}[{name}] vs oracle", scale_atol=True)
        assert_close(a, b, f"{what}[{name}] vs two-pass", scale_atol=True)


@pytest.mark.parametrize("H,F", [(4, 64), (1, 41), (4, 128), (8, 16)])
def test_gat_one_gather_backward_power_law(cuda, H, F):
    got, two, exp = _one_gather(cuda, power_law_graph(3000, 60, seed=3), H, F, 13)
    for a, b, e, what in zip(got, two, exp, ("grad_feat", "grad_attn_row", "grad_attn_col")):
        assert_close(a, e, f"{what} vs oracle", scale_atol=True)
        assert_close(a, b, f"{what} vs two-pass", scale_atol=True)


def test_gat_one_gather_pieces(cuda):
    """The three steps on their own: the per-row record, the per-edge gradients, the row sums."""
    from ae_mlsys_gnn_b200.operators import fused_gat as G
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc

    g = power_law_graph(1500, 40, seed=9)
    H, F = 4, 32
    attn_row, attn_col, feat, gout = _inputs(g, H, F, 14)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    cp, ri, pm = csr2csc(rp, ci)
    d = [t.to(cuda) for t in (attn_row, attn_col, feat, gout)]
    out, m, s = G.gat_forward(d[0], d[1], rp, ci, 0.2, d[2])
    pack = G.gat_backward_pack(out, d[3], d[0], m, s)
    _, old_pack = G.gat_backward_row(0.2, rp, ci, m, s, d[2], d[0], d[1], d[3])
    assert_close(pack, old_pack, "rowpack", scale_atol=True)
    S = (out.double() * d[3].double()).sum(-1)
    assert_close(pack[:, 3], S, "S = <grad_out, out>", scale_atol=True)
    gf, gac, eg = G.gat_backward_col_edges(0.2, cp, ri, d[2], d[1], pack, d[3])
    gf2, gac2 = G.gat_backward_col(0.2, cp, ri, d[2], d[1], pack, d[3])
    assert torch.equal(gf, gf2) and torch.equal(gac, gac2)
    # column sums of the per-edge gradients are grad_attn_col; row sums grad_attn_row
    col_of = torch.repeat_interleave(torch.arange(g.n, device=cuda), (cp[1:] - cp[:-1]).long())
    ref_col = torch.zeros(g.n, H, dtype=torch.float64, device=cuda).index_add_(0, col_of, eg.double())
    assert_close(gac, ref_col, "grad_attn_col from edge_grad", scale_atol=True)
    ref_row = torch.zeros(g.n, H, dtype=torch.float64, device=cuda).index_add_(0, ri.long(), eg.double())
    pos = G.invert_permutation(pm)
    assert_close(G.gat_backward_row_sum(rp, pos, eg), ref_row, "row sums", scale_atol=True)
    again = G.gat_backward_row_sum(rp, pos, eg)
    assert torch.equal(again, G.gat_backward_row_sum(rp, pos, eg)), "row sums are deterministic"


def test_gat_autograd_falls_back_for_foreign_csc(cuda):
    """A CSC that is not the one csr2csc builds (rows of a column in another order) is still
    handled: the autograd node takes the two-pass backward."""
    from ae_mlsys_gnn_b200.operators import fused_gat as G
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc

    g = power_law_graph(400, 12, seed=21)
    H, F = 2, 16
    attn_row, attn_col, feat, gout = _inputs(g, H, F, 15)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    cp, ri, _ = csr2csc(rp, ci)
    ri2 = ri.clone()
    for c in range(g.n):  # reverse the rows inside every column
        a, b = int(cp[c]), int(cp[c + 1])
        ri2[a:b] = ri[a:b].flip(0)
    assert G.csr_positions(rp, ci, cp, ri2) is None
    d = [t.to(cuda).requires_grad_(True) for t in (attn_row, attn_col, feat)]
    G.fused_gat_op(d[0], d[1], rp, ci, cp, ri2, 0.2, d[2]).backward(gout.to(cuda))
    _, em, es = ref.gat_forward(attn_row, attn_col, g.row_ptr, g.col_ind, 0.2, feat)
    ef, ear, eac = ref.gat_backward(0.2, g.row_ptr, g.col_ind, em, es, feat, attn_row, attn_col, gout)
    assert_close(d[2].grad, ef, "grad_feat", scale_atol=True)
    assert_close(d[0].grad, ear, "grad_attn_row", scale_atol=True)
    assert_close(d[1].grad, eac, "grad_attn_col", scale_atol=True)


def test_gat_long_run_of_isolated_nodes(cuda):
    """Thousands of consecutive rows (and columns) without edges in the middle of the graph:
    the chunk traversal jumps over the run instead of walking it; values are unchanged."""
    from ae_mlsys_gnn_b200.graphs import Graph

    base = power_law_graph(300, 10, seed=31)
    gap, n = 20000, 300 + 20000
    deg = (base.row_ptr[1:] - base.row_ptr[:-1]).long()
    full_deg = torch.cat([deg[:150], torch.zeros(gap, dtype=torch.long), deg[150:]])
    rp = torch.zeros(n + 1, dtype=torch.int32)
    rp[1:] = torch.cumsum(full_deg, 0).to(torch.int32)
    ci = base.col_ind.clone()
    ci[ci >= 150] += gap   # sources keep away from the gap as well
    g = Graph(n, rp.contiguous(), ci.contiguous())
    got, two, exp = _one_gather(cuda, g, 4, 16, 32)
    for a, b, e, what in zip(got, two, exp, ("grad_feat", "grad_attn_row", "grad_attn_col")):
        assert_close(a, e, f"{what} vs oracle", scale_atol=True)
        assert_close(b, e, f"{what} two-pass vs oracle", scale_atol=True)


# ---- ELU on the layer output, its backward folded into the per-row pack ------------------------

@pytest.mark.parametrize("H,F", [(4, 32), (1, 47), (2, 100)])
def test_gat_pack_elu(cuda, H, F):
    from ae_mlsys_gnn_b200.operators import fused_gat as G

    g = power_law_graph(900, 20, seed=17)
    attn_row, attn_col, feat, gact = _inputs(g, H, F, 18)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    d = [t.to(cuda) for t in (attn_row, attn_col, feat, gact)]
    out, m, s = G.gat_forward(d[0], d[1], rp, ci, 0.2, d[2])
    grad_pre, pack = G.gat_backward_pack_elu(out, d[3], d[0], m, s)
    o64, g64 = out.double(), d[3].double()
    exp_pre = g64 * torch.where(o64 > 0, torch.ones_like(o64), torch.exp(o64))
    assert_close(grad_pre, exp_pre, "grad_pre = grad_act * elu'(out)")
    assert_close(pack, G.gat_backward_pack(out, exp_pre.float(), d[0], m, s), "rowpack", scale_atol=True)


@pytest.mark.parametrize("foreign_csc", [False, True])
def test_gat_autograd_layer_with_elu(cuda, foreign_csc):
    """GATConv(activation="elu") against autograd of elu(DGL-style layer); also through the
    two-pass fallback (a CSC with another row order inside the columns)."""
    from ae_mlsys_gnn_b200.layers import GATConv
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc

    torch.manual_seed(1)
    g = power_law_graph(500, 20, seed=8)
    layer = GATConv(24, 16, 4, activation="elu").to(cuda)
    x = torch.randn(g.n, 24)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    cp, ri, _ = csr2csc(rp, ci)
    if foreign_csc:
        ri = ri.clone()
        for c in range(g.n):
            a, b = int(cp[c]), int(cp[c + 1])
            ri[a:b] = ri[a:b].flip(0)
    xd = x.to(cuda).requires_grad_(True)
    out = layer(rp, ci, cp, ri, xd)
    gout = torch.randn(out.shape, generator=torch.Generator().manual_seed(2))
    out.backward(gout.to(cuda))

    W = layer.W.detach().cpu().double().requires_grad_(True)
    al = layer.attn_l.detach().cpu().double().requires_grad_(True)
    ar = layer.attn_r.detach().cpu().double().requires_grad_(True)
    xr = x.double().requires_grad_(True)
    eo = torch.nn.functional.elu(ref.gat_layer_dgl(g.row_ptr, g.col_ind, xr, W, al, ar, 0.2))
    eo.backward(gout.double())
    assert_close(out, eo, "layer out")
    assert_close(layer.W.grad, W.grad, "W.grad", scale_atol=True)
    assert_close(layer.attn_l.grad, al.grad, "attn_l.grad", scale_atol=True)
    assert_close(layer.attn_r.grad, ar.grad, "attn_r.grad", scale_atol=True)
    assert_close(xd.grad, xr.grad, "x.grad", scale_atol=True)


def test_gat_forward_blocks_refuse_heads_wider_than_a_tile(cuda):
    """A head wider than the largest tile is processed in column slabs; launching such a shape
    block by block (state carried between launches) is refused instead of merging twice."""
    from ae_mlsys_gnn_b200 import _capi
    from ae_mlsys_gnn_b200.operators import fused_gat as G

    g = power_law_graph(200, 8, seed=4)
    H, F = 1, 640
    attn_row, attn_col, feat, _ = _inputs(g, H, F, 4)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    d = [t.to(cuda) for t in (attn_row, attn_col, feat)]
    out, m, s = G.gat_forward(d[0], d[1], rp, ci, 0.2, d[2])           # one launch per slab: fine
    eo, _, _ = ref.gat_forward(attn_row, attn_col, g.row_ptr, g.col_ind, 0.2, feat)
    assert_close(out, eo, "out 1x640")
    with pytest.raises(_capi.GnnError, match="column blocks"):
        G.gat_forward_part(d[0], d[1], rp, ci, 0.2, d[2], out, m, s, True, True)


@pytest.mark.parametrize("name", ["empty_rows", "hub", "long_rows", "random_200", "no_edges"])
@pytest.mark.parametrize("H,F", [(4, 128), (4, 64), (8, 8), (1, 47), (3, 12), (2, 100)])
def test_gat_forward_with_fused_elu(cuda, name, H, F):
    """gnn_gat_fwd_act: same out / edge_max / edge_sum as gnn_gat_fwd (bit for bit), and ELU(out)
    next to it; rows without edges give 0 in both."""
    from ae_mlsys_gnn_b200.operators import fused_gat as G

    g = crafted_graphs()[name]
    nc = _n_cols(g)
    attn_row, attn_col, feat, _ = _inputs(g, H, F, 21, nc)
    d = [t.to(cuda) for t in (attn_row, attn_col, feat)]
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    out, m, s = G.gat_forward(d[0], d[1], rp, ci, 0.2, d[2])
    out2, act, m2, s2 = G.gat_forward_act(d[0], d[1], rp, ci, 0.2, d[2])
    if H == 1 and F % 4:  # one narrow head: gnn_gat_fwd runs the sub-warp kernel, another summation order
        assert_close(out2, out, "out of the ELU variant")
    else:
        assert torch.equal(out, out2) and torch.equal(m, m2) and torch.equal(s, s2)
    assert_close(act, torch.nn.functional.elu(out2.double()), "elu(out)", rtol=1e-6, atol=2e-6)
    eo, _, _ = ref.gat_forward(attn_row, attn_col, g.row_ptr, g.col_ind, 0.2, feat)
    assert_close(act, torch.nn.functional.elu(eo), "elu(out) vs oracle")


@pytest.mark.parametrize("H,F", [(8, 128), (12, 8), (16, 40), (2, 300)])
def test_gat_layer_with_many_or_wide_heads(cuda, H, F):
    """More than 8 heads, or rows wider than one tile: forward and backward run head by head and
    the GATConv layer trains (the reference's fused_gat takes any H and F)."""
    from ae_mlsys_gnn_b200.layers import GATConv
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc

    torch.manual_seed(2)
    g = power_law_graph(300, 12, seed=11)
    layer = GATConv(10, F, H).to(cuda)
    x = torch.randn(g.n, 10)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    cp, ri, _ = csr2csc(rp, ci)
    xd = x.to(cuda).requires_grad_(True)
    out = layer(rp, ci, cp, ri, xd)
    gout = torch.randn(out.shape, generator=torch.Generator().manual_seed(3))
    out.backward(gout.to(cuda))
    W = layer.W.detach().cpu().double().requires_grad_(True)
    al = layer.attn_l.detach().cpu().double().requires_grad_(True)
    ar = layer.attn_r.detach().cpu().double().requires_grad_(True)
    xr = x.double().requires_grad_(True)
    eo = ref.gat_layer_dgl(g.row_ptr, g.col_ind, xr, W, al, ar, 0.2)
    eo.backward(gout.double())
    assert_close(out, eo, "layer out", scale_atol=True)
    assert_close(layer.W.grad, W.grad, "W.grad", scale_atol=True)
    assert_close(layer.attn_l.grad, al.grad, "attn_l.grad", scale_atol=True)
    assert_close(layer.attn_r.grad, ar.grad, "attn_r.grad", scale_atol=True)
    assert_close(xd.grad, xr.grad, "x.grad", scale_atol=True)


@pytest.mark.parametrize("name", ["empty_rows", "hub", "long_rows", "random_200"])
@pytest.mark.parametrize("H,F", [(4, 128), (4, 64), (8, 8), (1, 256), (2, 16), (1, 8)])
def test_gat_forward_bf16_gather(cuda, name, H, F):
    """Opt-in bfloat16 storage of the gathered rows: equals the fp32 kernel, and the oracle, on the
    rounded features within the usual fp32 tolerance (rounding the input is the only difference)."""
    from ae_mlsys_gnn_b200.operators import fused_gat as G

    g = crafted_graphs()[name]
    nc = _n_cols(g)
    attn_row, attn_col, feat, _ = _inputs(g, H, F, 31, nc)
    feat16 = feat.to(torch.bfloat16)
    d = [t.to(cuda) for t in (attn_row, attn_col, feat)]
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    conv = G.to_bf16(d[2])
    assert torch.equal(conv.cpu().view(torch.int16), feat16.view(torch.int16)), "round to nearest even"
    out, m, s = G.gat_forward_bf16(d[0], d[1], rp, ci, 0.2, conv)
    eo, em, es = ref.gat_forward(attn_row, attn_col, g.row_ptr, g.col_ind, 0.2, feat16.float())
    assert_close(out, eo, "out (bf16 gather)")
    assert_close(s, es, "edge_sum")
    out32, m32, s32 = G.gat_forward(d[0], d[1], rp, ci, 0.2, conv.float())
    assert_close(out, out32, "bf16 gather vs fp32 kernel on the rounded features")
    assert torch.equal(m, m32)

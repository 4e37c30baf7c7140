"""Parity at the chunk lengths the large benchmark graphs run.

Every edge-balanced kernel walks chunks of `chunk` consecutive edges per warp; the length
is chosen from the edge count: 32 below ~1.2 M edges, ~3,000-3,400 for the 10^8-edge
configurations.  With chunk 32 a piece of a row is never longer than one 32-edge batch, so
on small graphs the multi-batch paths (online softmax and accumulators carried across the
batches of one piece, the row-sum window carry, pieces of long rows merged across many
chunks) would never run under a checker.  gnn_debug_set_chunk forces the length, and the
comparisons against the CPU oracle are repeated for 32 / 64 / 416 / 3328 / 4096 on a graph
whose hub row and hub column span several chunks even at 4096.

One further test uses no hook: an R-MAT graph with more than 4 M edges picks chunk 128 by
itself, and is compared with the oracle and with the reference's own CUDA operator.

Tolerance: rel 1e-4 / abs 1e-5 (x max|expected| for sums with cancellation); integers exact.
"""
import functools

import numpy as np
import pytest
import torch

from oracle import ops as ref
from tests.util import assert_close

pytestmark = pytest.mark.gpu

CHUNKS = [32, 64, 416, 3328, 4096]
SHAPES = [(8, 8), (1, 7), (4, 64), (1, 41), (4, 128), (1, 47)]


@pytest.fixture
def chunk(request, cuda):
    from ae_mlsys_gnn_b200 import _capi

    c = request.param
    assert _capi.lib().gnn_debug_set_chunk(c) == 0
    yield c
    assert _capi.lib().gnn_debug_set_chunk(0) == 0


@functools.lru_cache(maxsize=None)
def hub_graph():
    """Symmetric graph of 12,000 nodes, ~80 K directed edges: one hub with 9,000 neighbours
    (its row and its column both span three chunks of 4,096), 60 rows of degree 200-700,
    the rest degree 0-3, and a run of 1,500 isolated nodes.  Mean degree of the non-empty heavy
    part is > 200; every long row appears as a long column too."""
    from ae_mlsys_gnn_b200.graphs import csr_from_edges

    rng = np.random.default_rng(11)
    n = 12000
    live = np.concatenate([np.arange(0, 9500), np.arange(11000, n)])  # [9500, 11000) stays isolated
    dst, src = [], []
    hub = 4321
    nb = rng.choice(9500, size=9000, replace=False)
    dst.append(np.full(nb.size, hub)); src.append(nb)
    heavy = rng.choice(live, size=60, replace=False)
    for r in heavy:
        d = int(rng.integers(200, 701))
        dst.append(np.full(d, r)); src.append(rng.choice(live, size=d, replace=False))
    light = rng.choice(live, size=2500, replace=False)
    for r in light:
        d = int(rng.integers(1, 4))
        dst.append(np.full(d, r)); src.append(rng.choice(live, size=d, replace=False))
    d, s = np.concatenate(dst), np.concatenate(src)
    d, s = np.concatenate([d, s]), np.concatenate([s, d])
    keep = d != s
    g = csr_from_edges(n, torch.from_numpy(d[keep]), torch.from_numpy(s[keep]), self_loops=False)
    deg = (g.row_ptr[1:] - g.row_ptr[:-1])
    assert int(deg.max()) > 2 * 4096 and int((deg == 0).sum()) > 1000
    return g


@functools.lru_cache(maxsize=None)
def _gat_case(H, F):
    g = hub_graph()
    gen = torch.Generator().manual_seed(1000 * H + F)
    ar, ac = torch.randn(g.n, H, generator=gen), torch.randn(g.n, H, generator=gen)
    x, go = torch.randn(g.n, H, F, generator=gen), torch.randn(g.n, H, F, generator=gen)
    eo, em, es = ref.gat_forward(ar, ac, g.row_ptr, g.col_ind, 0.2, x)
    eb = ref.gat_backward(0.2, g.row_ptr, g.col_ind, em, es, x, ar, ac, go)
    return (ar, ac, x, go), (eo, em, es), eb


def _dev(cuda, *ts):
    return [t.to(cuda) for t in ts]


@pytest.mark.parametrize("chunk", CHUNKS, indirect=True)
@pytest.mark.parametrize("H,F", SHAPES)
def test_gat_forward_and_backward(cuda, chunk, H, F):
    """Forward, the two-pass backward and the one-gather backward (pack / column pass with
    edge gradients / row sums) against the oracle."""
    from ae_mlsys_gnn_b200.operators import fused_gat as G
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc

    g = hub_graph()
    (ar, ac, x, go), (eo, em, es), eb = _gat_case(H, F)
    rp, ci, dar, dac, dx, dgo = _dev(cuda, g.row_ptr, g.col_ind, ar, ac, x, go)
    cp, ri, pm = csr2csc(rp, ci)
    ecp, eri, epm = ref.csr2csc(g.row_ptr, g.col_ind)
    assert torch.equal(cp.cpu(), ecp) and torch.equal(ri.cpu(), eri) and torch.equal(pm.cpu(), epm)
    out, m, s = G.gat_forward(dar, dac, rp, ci, 0.2, dx)
    assert_close(out, eo, "out")
    assert_close(m, em, "edge_max", rtol=1e-6, atol=1e-6)
    assert_close(s, es, "edge_sum")
    two = G.gat_backward(0.2, rp, ci, cp, ri, m, s, dx, dar, dac, dgo)
    pos = G.invert_permutation(pm)
    one = G.gat_backward_with_output(0.2, rp, ci, cp, ri, pos, m, s, dx, dar, dac, out, dgo)
    for a, b, e, what in zip(two, one, eb, ("grad_feat", "grad_attn_row", "grad_attn_col")):
        assert_close(a, e, f"two-pass {what}", scale_atol=True)
        assert_close(b, e, f"one-gather {what}", scale_atol=True)
    # same launch twice: bit-identical (no atomics, merge in chunk order)
    out2, m2, s2 = G.gat_forward(dar, dac, rp, ci, 0.2, dx)
    assert torch.equal(out, out2) and torch.equal(m, m2) and torch.equal(s, s2)
    # the variant that also stores ELU(out): same values, activation of split rows applied after the merge
    out3, act, m3, s3 = G.gat_forward_act(dar, dac, rp, ci, 0.2, dx)
    if H == 1 and F % 4:  # one narrow head: gnn_gat_fwd runs the sub-warp kernel, another summation order
        assert_close(out3, out, "out of the ELU variant")
    else:
        assert torch.equal(out, out3) and torch.equal(m, m3) and torch.equal(s, s3)
    assert_close(act, torch.nn.functional.elu(eo), "elu(out)")


@pytest.mark.parametrize("chunk", CHUNKS, indirect=True)
@pytest.mark.parametrize("H,F", [(4, 128), (1, 47), (4, 64)])
def test_gat_by_column_blocks(cuda, chunk, H, F):
    """gnn_gat_fwd_part and gnn_gat_bwd_col_edges(accumulate) over three column / row blocks of
    the graph, state merged between launches, against the oracle of the whole graph."""
    from ae_mlsys_gnn_b200.operators import fused_gat as G
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc
    from ae_mlsys_gnn_b200.partition import _split_by_piece

    g = hub_graph()
    (ar, ac, x, go), (eo, em, es), eb = _gat_case(H, F)
    rp, ci, dar, dac, dx, dgo = _dev(cuda, g.row_ptr, g.col_ind, ar, ac, x, go)
    cp, ri, _ = csr2csc(rp, ci)
    pieces, span = 3, -(-g.n // 3)
    seg = torch.repeat_interleave(torch.arange(g.n, device=cuda), (rp[1:] - rp[:-1]).long())
    out = torch.full((g.n, H, F), float("nan"), device=cuda)
    m, s = torch.full((g.n, H), float("nan"), device=cuda), torch.full((g.n, H), float("nan"), device=cuda)
    for c, (rp_c, ci_c) in enumerate(_split_by_piece(rp, ci.long(), seg, pieces, span)):
        G.gat_forward_part(dar, dac, rp_c, ci_c, 0.2, dx, out, m, s, c > 0, c == pieces - 1)
    assert_close(out, eo, "out by blocks")
    assert_close(s, es, "edge_sum by blocks")
    assert_close(m, em, "edge_max by blocks", rtol=1e-6, atol=1e-6)

    pack = G.gat_backward_pack(out, dgo, dar, m, s)
    cseg = torch.repeat_interleave(torch.arange(g.n, device=cuda), (cp[1:] - cp[:-1]).long())
    gf = torch.full((g.n, H, F), float("nan"), device=cuda)
    gac = torch.full((g.n, H), float("nan"), device=cuda)
    gar = torch.zeros((g.n, H), dtype=torch.float64, device=cuda)
    for c, (cp_c, ri_c) in enumerate(_split_by_piece(cp, ri.long(), cseg, pieces, span)):
        eg = G.gat_backward_col_edges_part(0.2, cp_c, ri_c, dx, dac, pack, dgo, gf, gac, c > 0)
        gar.index_add_(0, ri_c.long(), eg.double())
    assert_close(gf, eb[0], "grad_feat by blocks", scale_atol=True)
    assert_close(gac, eb[2], "grad_attn_col by blocks", scale_atol=True)
    assert_close(gar, eb[1], "grad_attn_row from the blocks' edge gradients", scale_atol=True)


@pytest.mark.parametrize("chunk", CHUNKS, indirect=True)
@pytest.mark.parametrize("K,D,F", [(3, 2, 16), (1, 3, 5), (4, 2, 32)])
def test_gmm_forward_and_autograd(cuda, chunk, K, D, F):
    import ae_mlsys_gnn_b200.operators.fused_gmmconv as M
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc

    g = hub_graph()
    gen = torch.Generator().manual_seed(7 + K)
    feat = torch.randn(g.n, K, F, generator=gen)
    pseudo = torch.rand(g.nnz, D, generator=gen)
    mu = torch.randn(K, D, generator=gen) * 0.3
    sig = torch.rand(K, D, generator=gen) + 0.5
    rp, ci = _dev(cuda, g.row_ptr, g.col_ind)
    cp, ri, pm = csr2csc(rp, ci)
    dv = [t.to(cuda).requires_grad_(True) for t in (feat, pseudo, mu, sig)]
    out = M.GmmConvFuse(rp, ci, cp, ri, pm, *dv)
    gout = torch.randn(out.shape, generator=gen)
    out.backward(gout.to(cuda))
    rv = [t.double().requires_grad_(True) for t in (feat, pseudo, mu, sig)]
    eo = ref.gmm_forward(g.row_ptr, g.col_ind, *rv)
    eo.backward(gout.double())
    assert_close(out, eo, "gmm out", scale_atol=True)
    for name, a, b in zip(("node_feat", "pseudo", "mu", "inv_sigma"), dv, rv):
        assert_close(a.grad, b.grad, f"grad {name}", scale_atol=True)


@pytest.mark.parametrize("chunk", CHUNKS, indirect=True)
@pytest.mark.parametrize("H,F", [(4, 64), (1, 47), (8, 8), (2, 300)])
def test_mhspmm_and_mhsddmm(cuda, chunk, H, F):
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc
    from ae_mlsys_gnn_b200.operators.mhspmm import csrmhspmm

    g = hub_graph()
    gen = torch.Generator().manual_seed(3 + F)
    feat, att = torch.randn(g.n, H, F, generator=gen), torch.randn(g.nnz, H, generator=gen)
    gout = torch.randn(g.n, H, F, generator=gen)
    rp, ci = _dev(cuda, g.row_ptr, g.col_ind)
    cp, ri, pm = csr2csc(rp, ci)
    fd, ad = feat.to(cuda).requires_grad_(True), att.to(cuda).requires_grad_(True)
    out = csrmhspmm(rp, ci, cp, ri, pm, fd, ad)
    out.backward(gout.to(cuda))  # grad_att is the mhsddmm of gout and feat
    fr, ar = feat.double().requires_grad_(True), att.double().requires_grad_(True)
    eo = ref.mhspmm(g.row_ptr, g.col_ind, ar, fr)
    eo.backward(gout.double())
    assert_close(out, eo, "mhspmm", scale_atol=True)
    assert_close(fd.grad, fr.grad, "grad_feat", scale_atol=True)
    assert_close(ad.grad, ar.grad, "grad_att (mhsddmm)", scale_atol=True)


@pytest.mark.parametrize("chunk", CHUNKS, indirect=True)
def test_u_add_v_and_edge_alpha(cuda, chunk):
    from ae_mlsys_gnn_b200.operators.fused_gat import gat_edge_alpha, gat_forward
    from ae_mlsys_gnn_b200.operators.u_add_v import u_add_v_op

    g = hub_graph()
    gen = torch.Generator().manual_seed(5)
    F = 6
    rv, cv = torch.randn(g.n, F, generator=gen), torch.randn(g.n, F, generator=gen)
    gout = torch.randn(g.nnz, F, generator=gen)
    rp, ci = _dev(cuda, g.row_ptr, g.col_ind)
    rd, cd = rv.to(cuda).requires_grad_(True), cv.to(cuda).requires_grad_(True)
    out = u_add_v_op(rp, ci, rd, cd)
    out.backward(gout.to(cuda))
    rr, cr = rv.double().requires_grad_(True), cv.double().requires_grad_(True)
    eo = ref.u_add_v(g.row_ptr, g.col_ind, rr, cr)
    eo.backward(gout.double())
    assert_close(out, eo, "u_add_v")
    assert_close(rd.grad, rr.grad, "grad_row", scale_atol=True)
    assert_close(cd.grad, cr.grad, "grad_col", scale_atol=True)

    H = 4
    (ar, ac, x, _), (_, em, es), _ = _gat_case(4, 64)
    dar, dac, dx = _dev(cuda, ar, ac, x)
    _, m, s = gat_forward(dar, dac, rp, ci, 0.2, dx)
    relu, alpha = gat_edge_alpha(dar, dac, rp, ci, m, s, 0.2)
    er, ea = ref.gat_alpha(ar, ac, g.row_ptr, g.col_ind, 0.2, em, es)
    assert relu.shape == (g.nnz, H)
    assert_close(relu, er, "edge_relu")
    assert_close(alpha, ea, "edge_softmax")


def test_rmat_4m_edges_automatic_chunk(cuda):
    """No hook: 262,144 nodes / > 4 M edges pick chunk 128 by themselves.  B200 kernels vs the
    fp64 oracle, and vs the reference's CUDA operator (one head, F = 32: the shape class where
    reading the reference kernels shows them in-bounds and race-free at any degree)."""
    from ae_mlsys_gnn_b200.graphs import rmat_graph
    from ae_mlsys_gnn_b200.operators import fused_gat as G
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc
    from oracle import build_ref

    g = rmat_graph(1 << 18, 2_400_000, seed=5)
    assert g.nnz > 4_000_000
    rp, ci = _dev(cuda, g.row_ptr, g.col_ind)
    cp, ri, pm = csr2csc(rp, ci)
    ecp, eri, epm = ref.csr2csc(g.row_ptr, g.col_ind)
    assert torch.equal(cp.cpu(), ecp) and torch.equal(ri.cpu(), eri) and torch.equal(pm.cpu(), epm)
    pos = G.invert_permutation(pm)
    for H, F, three_way in ((1, 8, False), (1, 32, True)):
        gen = torch.Generator().manual_seed(H * 100 + F)
        ar, ac = torch.randn(g.n, H, generator=gen), torch.randn(g.n, H, generator=gen)
        x, go = torch.randn(g.n, H, F, generator=gen), torch.randn(g.n, H, F, generator=gen)
        dar, dac, dx, dgo = _dev(cuda, ar, ac, x, go)
        out, m, s = G.gat_forward(dar, dac, rp, ci, 0.2, dx)
        two = G.gat_backward(0.2, rp, ci, cp, ri, m, s, dx, dar, dac, dgo)
        one = G.gat_backward_with_output(0.2, rp, ci, cp, ri, pos, m, s, dx, dar, dac, out, dgo)
        eo, em, es = ref.gat_forward(ar, ac, g.row_ptr, g.col_ind, 0.2, x)
        eb = ref.gat_backward(0.2, g.row_ptr, g.col_ind, em, es, x, ar, ac, go)
        assert_close(out, eo, f"out {H}x{F}")
        assert_close(s, es, f"edge_sum {H}x{F}")
        for a, b, e, what in zip(two, one, eb, ("grad_feat", "grad_attn_row", "grad_attn_col")):
            assert_close(a, e, f"two-pass {what} {H}x{F}", scale_atol=True)
            assert_close(b, e, f"one-gather {what} {H}x{F}", scale_atol=True)
        if three_way and build_ref.available("fused_gat_SM"):
            mod = build_ref.load_module("fused_gat_SM")
            r_out, r_max, r_sum = mod.gat_forward(dar, dac, rp, ci, 0.2, dx)
            rb = mod.gat_backward(0.2, rp, ci, cp, ri, m, s, dx, dar, dac, dgo)
            torch.cuda.synchronize()
            assert_close(r_out, eo, "reference vs oracle: out")
            assert_close(out, r_out, "B200 vs reference: out")
            assert torch.equal(m, r_max)
            assert_close(s, r_sum, "B200 vs reference: edge_sum")
            for a, r, e, what in zip(one, rb, eb, ("grad_feat", "grad_attn_row", "grad_attn_col")):
                assert_close(r, e, f"reference vs oracle: {what}", scale_atol=True)
                assert_close(a, r, f"B200 vs reference: {what}", scale_atol=True)

"""CPU checks of the oracle itself: independent formulations must agree."""
import numpy as np
import pytest
import torch

from oracle import ops as ref
from tests.util import assert_close, crafted_graphs, power_law_graph


@pytest.mark.parametrize("name", list(crafted_graphs().keys()))
def test_csr2csc_two_statements_agree(name):
    g = crafted_graphs()[name]
    nc = max(g.n, int(g.col_ind.max().item()) + 1 if g.nnz else g.n)
    a = ref.csr2csc_scipy(g.row_ptr, g.col_ind, nc)
    b = ref.csr2csc(g.row_ptr, g.col_ind, nc)
    for x, y in zip(a, b):
        assert torch.equal(x, y)
    col_ptr, row_ind, perm = a
    # rows ascend inside every column (no duplicate edges in these graphs)
    for c in range(nc):
        seg = row_ind[col_ptr[c]:col_ptr[c + 1]]
        assert torch.all(seg[1:] > seg[:-1])
    assert torch.equal(g.col_ind[perm.long()], torch.repeat_interleave(
        torch.arange(nc, dtype=torch.int32), (col_ptr[1:] - col_ptr[:-1]).long()))


def test_gat_hand_computed():
    """One row with two sources, one head, worked by hand."""
    row_ptr = torch.tensor([0, 2, 2], dtype=torch.int32)
    col_ind = torch.tensor([0, 1], dtype=torch.int32)
    attn_row = torch.tensor([[1.0], [0.0]])
    attn_col = torch.tensor([[1.0], [-3.0]])
    feat = torch.tensor([[[1.0, 2.0]], [[3.0, 5.0]]])
    out, m, s = ref.gat_forward(attn_row, attn_col, row_ptr, col_ind, 0.5, feat)
    e0, e1 = 2.0, -1.0                       # LeakyReLU(1+1), LeakyReLU(1-3) = -2*0.5
    w1 = np.exp(e1 - e0)
    a0, a1 = 1 / (1 + w1), w1 / (1 + w1)
    assert m[0, 0].item() == pytest.approx(2.0)
    assert s[0, 0].item() == pytest.approx(1 + w1)
    assert out[0, 0].tolist() == pytest.approx([a0 * 1 + a1 * 3, a0 * 2 + a1 * 5])
    assert m[1, 0].item() == pytest.approx(-1e38) and s[1, 0].item() == 0 and out[1].abs().sum() == 0


@pytest.mark.parametrize("H,F", [(1, 5), (4, 8)])
def test_gat_backward_matches_autograd(H, F):
    g = power_law_graph(120, 8, seed=1)
    gen = torch.Generator().manual_seed(0)
    ar = torch.randn(g.n, H, generator=gen, dtype=torch.float64).requires_grad_(True)
    ac = torch.randn(g.n, H, generator=gen, dtype=torch.float64).requires_grad_(True)
    x = torch.randn(g.n, H, F, generator=gen, dtype=torch.float64).requires_grad_(True)
    gout = torch.randn(g.n, H, F, generator=gen, dtype=torch.float64)
    rows, cols = ref.rows_of(g.row_ptr), g.col_ind.long()
    e = torch.nn.functional.leaky_relu(ar[rows] + ac[cols], 0.2)
    out = torch.zeros(g.n, H, F, dtype=torch.float64).index_add(
        0, rows, ref.edge_softmax(g.row_ptr, e)[:, :, None] * x[cols])
    out.backward(gout)
    eo, m, s = ref.gat_forward(ar.detach(), ac.detach(), g.row_ptr, g.col_ind, 0.2, x.detach())
    assert_close(eo, out, "forward", rtol=1e-12, atol=1e-12)
    gf, gar, gac = ref.gat_backward(0.2, g.row_ptr, g.col_ind, m, s, x.detach(), ar.detach(),
                                    ac.detach(), gout)
    assert_close(gf, x.grad, "grad_feat", rtol=1e-10, atol=1e-12)
    assert_close(gar, ar.grad, "grad_attn_row", rtol=1e-10, atol=1e-12)
    assert_close(gac, ac.grad, "grad_attn_col", rtol=1e-10, atol=1e-12)


@pytest.mark.parametrize("H,F", [(1, 5), (4, 8)])
def test_gat_one_gather_backward_identity(H, F):
    """What the one-gather backward rests on, in fp64 on the CPU: S[r,h] = sum_e a_e <G[r],h[c_e]>
    equals <G[r], out[r]>, and grad_attn_row / grad_attn_col are the row / column sums of the
    per-edge logit gradients a_e d_e (g_e - S[r]) (fused_backward_kernel, fused_gat_SM.cu:734-801)."""
    g = power_law_graph(150, 9, seed=4)
    gen = torch.Generator().manual_seed(3)
    ar = torch.randn(g.n, H, generator=gen, dtype=torch.float64)
    ac = torch.randn(g.n, H, generator=gen, dtype=torch.float64)
    x = torch.randn(g.n, H, F, generator=gen, dtype=torch.float64)
    gout = torch.randn(g.n, H, F, generator=gen, dtype=torch.float64)
    rows, cols = ref.rows_of(g.row_ptr), g.col_ind.long()
    out, m, s = ref.gat_forward(ar, ac, g.row_ptr, g.col_ind, 0.2, x)
    e, alpha = ref.gat_alpha(ar, ac, g.row_ptr, g.col_ind, 0.2, m, s)
    dots = (gout[rows] * x[cols]).sum(-1)
    S_edges = torch.zeros(g.n, H, dtype=torch.float64).index_add_(0, rows, alpha * dots)
    S_nodes = (gout * out).sum(-1)
    assert_close(S_nodes, S_edges, "S from the forward output", rtol=1e-10, atol=1e-12)
    ge = alpha * (dots - S_nodes[rows])
    ge = torch.where(e < 0, ge * 0.2, ge)
    _, gar, gac = ref.gat_backward(0.2, g.row_ptr, g.col_ind, m, s, x, ar, ac, gout)
    assert_close(torch.zeros(g.n, H, dtype=torch.float64).index_add_(0, rows, ge), gar, "row sums",
                 rtol=1e-10, atol=1e-12)
    assert_close(torch.zeros(g.n, H, dtype=torch.float64).index_add_(0, cols, ge), gac, "column sums",
                 rtol=1e-10, atol=1e-12)


def _bitrev5(x):
    return int(f"{x:05b}"[::-1], 2)


@pytest.mark.parametrize("k", [1, 5, 20, 32, 33, 70])
def test_edgeconv_tie_rule(k):
    """The butterfly simulation picks, among equal maxima, the later block of 32 and
    inside a block the position with the largest bit-reversed index."""
    gen = torch.Generator().manual_seed(k)
    n, F = 40, 6
    src = torch.randint(0, n, (n * k,), generator=gen, dtype=torch.int32)
    h_src = torch.randint(0, 3, (n, F), generator=gen).float()
    h_dst = torch.randint(0, 2, (n, F), generator=gen).float()
    out, idx = ref.edgeconv_forward(k, src, h_src, h_dst)
    s = src.view(n, k).long()
    vals = h_dst[:, None, :] + h_src[s]                     # (n,k,F)
    assert torch.equal(out, vals.max(1).values)
    for i in range(n):
        for f in range(F):
            best = max(range(k), key=lambda j: (vals[i, j, f].item(), j // 32, _bitrev5(j % 32)))
            assert idx[i, f].item() == s[i, best].item()


def test_edgeconv_matches_dgl_form():
    gen = torch.Generator().manual_seed(3)
    n, k, cin, cout = 50, 7, 4, 9
    x = torch.randn(n, cin, generator=gen)
    tw, pw = torch.randn(cout, cin, generator=gen), torch.randn(cout, cin, generator=gen)
    src = torch.randint(0, n, (n * k,), generator=gen, dtype=torch.int32)
    h_theta, h_phi = x @ tw.T, x @ pw.T
    out, _ = ref.edgeconv_forward(k, src, h_theta, h_phi - h_theta)
    assert_close(out, ref.edgeconv_layer_dgl(k, src, x, tw, pw), "edgeconv", rtol=1e-5, atol=1e-5)


def test_gmm_hand_computed():
    row_ptr = torch.tensor([0, 1, 2], dtype=torch.int32)
    col_ind = torch.tensor([1, 0], dtype=torch.int32)
    feat = torch.tensor([[[2.0]], [[3.0]]])
    pseudo = torch.tensor([[1.0], [0.0]])
    mu, sig = torch.tensor([[0.0]]), torch.tensor([[2.0]])
    out = ref.gmm_forward(row_ptr, col_ind, feat, pseudo, mu, sig)
    assert out[0, 0, 0].item() == pytest.approx(3.0 * np.exp(-0.5 * 4.0))
    assert out[1, 0, 0].item() == pytest.approx(2.0)


def test_golden_vectors():
    """The committed fixtures (tests/golden/make_golden.py) pin the oracle's outputs."""
    import os

    path = os.path.join(os.path.dirname(__file__), "golden", "oracle_golden.npz")
    z = np.load(path)
    from tests.golden.make_golden import compute

    fresh = compute()
    assert set(fresh) == set(z.files)
    for k in z.files:
        if z[k].dtype.kind in "iu":
            assert np.array_equal(z[k], fresh[k]), k
        else:
            np.testing.assert_allclose(fresh[k], z[k], rtol=1e-12, atol=1e-14, err_msg=k)

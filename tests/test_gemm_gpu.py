"""tcgen05 3xTF32 projection GEMM against an fp64 product; the tolerance is the one of
the fp32 operators (rel 1e-4, abs 1e-5 scaled by the largest output magnitude)."""
import pytest
import torch

from tests.util import assert_close

pytestmark = pytest.mark.gpu

SHAPES = [(128, 128, 32), (1000, 512, 100), (300, 47, 512), (4097, 512, 512), (130, 70, 36), (5, 3, 4),
          (257, 256, 64), (2048, 64, 128), (999, 41, 256),
          (40000, 512, 64),   # more output tiles than SMs: every CTA walks several tiles
          (150 * 128 + 5, 200, 96),
          (3000, 300, 128),   # 256-wide column tile with a partial second tile
          (2500, 768, 64), (20000, 256, 512), (700, 512, 544)]  # three wide tiles; K at / beyond one accumulator chain


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("n_by_k", [False, True])
def test_gemm_tf32x3(cuda, M, N, K, n_by_k):
    from ae_mlsys_gnn_b200.operators import dense

    gen = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=gen)
    b = torch.randn(N, K, generator=gen) if n_by_k else torch.randn(K, N, generator=gen)
    out = dense.gemm(a.to(cuda), b.to(cuda), n_by_k)
    dense.check_status()
    exp = a.double() @ (b.double().t() if n_by_k else b.double())
    assert_close(out, exp, f"gemm {M}x{N}x{K}", scale_atol=True)
    # a single TF32 pass would be off by ~1e-3 relative: make sure the compensation is on
    err = (out.cpu().double() - exp).abs().max().item() / exp.abs().max().item()
    assert err < 1e-5, f"relative error {err:.2e} is not fp32-level"


def test_gemm_large_magnitude_spread(cuda):
    """Entries spanning many orders of magnitude: the hi/lo split must stay exact."""
    from ae_mlsys_gnn_b200.operators import dense

    gen = torch.Generator().manual_seed(5)
    a = torch.randn(513, 128, generator=gen) * torch.logspace(-6, 6, 128)
    b = torch.randn(128, 96, generator=gen)
    out = dense.gemm(a.to(cuda), b.to(cuda), False)
    dense.check_status()
    assert_close(out, a.double() @ b.double(), "gemm spread", scale_atol=True)


def test_matmul_autograd_any_inner_dimension(cuda):
    from ae_mlsys_gnn_b200.operators import dense

    gen = torch.Generator().manual_seed(9)
    for K in (64, 30, 47):  # 30 and 47 are not multiples of 4: the operands are padded with zero columns
        x = torch.randn(700, K, generator=gen)
        w = torch.randn(K, 48, generator=gen)
        g = torch.randn(700, 48, generator=gen)
        xd, wd = x.to(cuda).requires_grad_(True), w.to(cuda).requires_grad_(True)
        dense.project(xd, wd).backward(g.to(cuda))
        xr, wr = x.double().requires_grad_(True), w.double().requires_grad_(True)
        (xr @ wr).backward(g.double())
        assert_close(xd.grad, xr.grad, "grad_x", scale_atol=True)
        assert_close(wd.grad, wr.grad, "grad_w", scale_atol=True)
        lin_w = torch.randn(48, K, generator=gen)
        out = dense.linear(x.to(cuda), lin_w.to(cuda))
        assert_close(out, x.double() @ lin_w.double().t(), "linear", scale_atol=True)
    # an output width of 47: the input gradient g (M x 47) @ w^T has the odd inner dimension
    x, w, g = torch.randn(5000, 64, generator=gen), torch.randn(64, 47, generator=gen), torch.randn(5000, 47, generator=gen)
    xd, wd = x.to(cuda).requires_grad_(True), w.to(cuda).requires_grad_(True)
    dense.project(xd, wd).backward(g.to(cuda))
    assert_close(xd.grad, g.double() @ w.double().t(), "grad_x (47 columns)", scale_atol=True)
    assert_close(wd.grad, x.double().t() @ g.double(), "grad_w (47 columns)", scale_atol=True)
    dense.check_status()


@pytest.mark.parametrize("M,K1,N1", [(5000, 100, 512), (4099, 512, 47), (70001, 64, 64), (33, 8, 130), (1, 5, 3),
                                     (300000, 512, 512), (9000, 47, 512), (64, 256, 384)])
def test_gemm_tn_weight_gradient(cuda, M, K1, N1):
    from ae_mlsys_gnn_b200.operators import dense

    gen = torch.Generator().manual_seed(M + K1)
    a, b = torch.randn(M, K1, generator=gen), torch.randn(M, N1, generator=gen)
    out = dense.gemm_tn(a.to(cuda), b.to(cuda))
    dense.check_status()
    assert_close(out, a.double().t() @ b.double(), f"gemm_tn {M}x{K1}x{N1}", scale_atol=True)


def test_matmul_autograd_large_uses_tensor_core_weight_gradient(cuda):
    from ae_mlsys_gnn_b200.operators import dense

    gen = torch.Generator().manual_seed(11)
    x, w, g = torch.randn(9000, 64, generator=gen), torch.randn(64, 96, generator=gen), torch.randn(9000, 96, generator=gen)
    xd, wd = x.to(cuda).requires_grad_(True), w.to(cuda).requires_grad_(True)
    dense.project(xd, wd).backward(g.to(cuda))
    dense.check_status()
    assert_close(wd.grad, x.double().t() @ g.double(), "grad_w", scale_atol=True)
    assert_close(xd.grad, g.double() @ w.double().t(), "grad_x", scale_atol=True)
    lw = torch.randn(96, 64, generator=gen).to(cuda).requires_grad_(True)
    dense.linear(x.to(cuda), lw).backward(g.to(cuda))
    assert_close(lw.grad, g.double().t() @ x.double(), "linear grad_w", scale_atol=True)


def test_gemm_tn_long_reduction(cuda):
    """Millions of rows: the tensor core truncates when it adds into its accumulator, so the
    kernel must not leave one accumulator running over the whole reduction (an unbroken
    chain comes out low by several 1e-4 of the value).  fp64 reference on the device."""
    from ae_mlsys_gnn_b200.operators import dense

    gen = torch.Generator(device=cuda).manual_seed(3)
    M = 2_000_003
    a = torch.randn(M, 128, device=cuda, generator=gen)
    b = torch.randn(M, 256, device=cuda, generator=gen).abs_()  # same-sign products in half of the rows
    a[: M // 2].abs_()
    out = dense.gemm_tn(a, b)
    dense.check_status()
    exp = a.double().t() @ b.double()
    assert_close(out, exp, "gemm_tn long reduction", scale_atol=True)
    bias = ((out.double() - exp) / exp)[exp.abs() > 0.1 * exp.abs().max()].mean().item()
    assert abs(bias) < 3e-5, f"systematic relative error {bias:.2e}"


def test_gemm_misaligned_view(cuda):
    """An operand that is a view starting 4 bytes into its storage cannot be read by TMA:
    the operator copies it first."""
    from ae_mlsys_gnn_b200.operators import dense

    gen = torch.Generator().manual_seed(21)
    buf = torch.randn(300 * 64 + 1, generator=gen).to(cuda)
    a = buf[1:].view(300, 64)
    assert a.data_ptr() % 16 != 0
    w = torch.randn(64, 40, generator=gen).to(cuda)
    out = dense.gemm_any_k(a, w, False)
    dense.check_status()
    assert_close(out, a.double() @ w.double(), "gemm on a misaligned view", scale_atol=True)


@pytest.mark.parametrize("M,K,H,F", [(5000, 100, 4, 128), (3001, 512, 4, 64), (777, 64, 8, 32), (4000, 96, 1, 47),
                                      (1500, 36, 2, 128), (900, 128, 1, 128), (2000, 32, 16, 32)])
def test_gemm_scores_epilogue(cuda, M, K, H, F):
    """Projection with the per-head attention scores formed in the epilogue: same product as the plain
    GEMM (bit for bit), scores against the float64 dot products of that product's rows."""
    from ae_mlsys_gnn_b200.operators import dense

    gen = torch.Generator().manual_seed(M + K + H)
    x = torch.randn(M, K, generator=gen).to(cuda)
    w = torch.randn(K, H * F, generator=gen).to(cuda)
    al = torch.randn(H, F, generator=gen).to(cuda)
    ar = torch.randn(H, F, generator=gen).to(cuda)
    assert dense.scores_supported(H, F)
    out, sl, sr = dense.gemm_any_k(x, w, False, scores=(al, ar))
    plain = dense.gemm_any_k(x, w, False)
    dense.check_status()
    assert torch.equal(out, plain)
    h = out.double().view(M, H, F)
    assert_close(sl, (h * al.double()).sum(-1), "score_l", scale_atol=True)
    assert_close(sr, (h * ar.double()).sum(-1), "score_r", scale_atol=True)


def test_weight_gradient_on_second_stream(cuda):
    """Two stacked projections whose weight-gradient GEMMs run on the second stream: the
    gradients read right after backward() (no explicit synchronisation by the caller) equal
    those of the in-order path bit for bit, over several passes that recycle the memory."""
    from ae_mlsys_gnn_b200.operators import dense

    gen = torch.Generator().manual_seed(11)
    x = torch.randn(20000, 96, generator=gen).to(cuda)
    w1 = torch.randn(96, 256, generator=gen).to(cuda)
    w2 = torch.randn(256, 64, generator=gen).to(cuda)
    g = torch.randn(20000, 64, generator=gen).to(cuda)

    def grads(side):
        a, b = w1.clone().requires_grad_(True), w2.clone().requires_grad_(True)
        xi = x.clone().requires_grad_(True)
        with dense.side_weight_grads(side):
            y = dense.project(torch.tanh(dense.project(xi, a)), b)
        y.backward(g)
        return a.grad.clone(), b.grad.clone(), xi.grad.clone()

    ref = grads(False)
    for _ in range(4):
        got = grads(True)
        for r, t in zip(ref, got):
            assert torch.equal(r, t)
    dense.check_status()
    assert_close(ref[1], (torch.tanh(x.double() @ w1.double())).t() @ g.double(), "grad_w2", scale_atol=True)


def test_projection_by_row_blocks(cuda):
    """The block-wise projection writes the same bits as the one-shot product, calls the hook
    once per block in order, and keeps the gradients of the whole product."""
    from ae_mlsys_gnn_b200.operators import dense

    gen = torch.Generator().manual_seed(12)
    M, K, N = 50000, 96, 512
    x = torch.randn(M, K, generator=gen).to(cuda)
    w = torch.randn(K, N, generator=gen).to(cuda)
    g = torch.randn(M, N, generator=gen).to(cuda)
    whole = dense.project(x, w)
    buf = torch.zeros(M + 100, N, device=cuda)
    seen = []
    blocks = [(0, 16384), (16384, 32768), (32768, 49152), (49152, M)]
    xi, wi = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    out = dense.project(xi, wi, out=dense.OutRows(buf, 0), row_blocks=blocks, after_block=lambda lo, hi: seen.append((lo, hi)))
    assert seen == blocks
    assert torch.equal(out, whole) and torch.equal(buf[:M], whole) and bool((buf[M:] == 0).all())
    out.backward(g)
    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    dense.project(xr, wr).backward(g)
    assert torch.equal(xi.grad, xr.grad) and torch.equal(wi.grad, wr.grad)
    dense.check_status()

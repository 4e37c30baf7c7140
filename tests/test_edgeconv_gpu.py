"""EdgeConv: values within tolerance, arg-max indices bit-exact (ties included)."""
import numpy as np
import pytest
import torch

from oracle import ops as ref
from tests.util import assert_close

pytestmark = pytest.mark.gpu


def _case(n, k, F, seed, ties=False):
    gen = torch.Generator().manual_seed(seed)
    src = torch.randint(0, n, (n * k,), generator=gen, dtype=torch.int32)
    if ties:
        # few distinct values, so equal maxima are the norm, not the exception
        h_src = torch.randint(0, 3, (n, F), generator=gen).float()
        h_dst = torch.randint(0, 2, (n, F), generator=gen).float()
    else:
        h_src = torch.randn(n, F, generator=gen)
        h_dst = torch.randn(n, F, generator=gen)
    return src, h_src, h_dst


@pytest.mark.parametrize("n,k,F", [(64, 20, 64), (50, 1, 3), (33, 5, 7), (40, 32, 16), (30, 33, 8),
                                   (20, 70, 12), (128, 20, 256), (64, 40, 128), (17, 20, 100),
                                   (9, 20, 1000), (10, 7, 250)])
@pytest.mark.parametrize("ties", [False, True])
def test_edgeconv_forward(cuda, n, k, F, ties):
    from ae_mlsys_gnn_b200.operators.fused_edgeconv import edgeconv_forward

    src, h_src, h_dst = _case(n, k, F, n * 1000 + k, ties)
    out, idx = edgeconv_forward(k, src.to(cuda), h_src.to(cuda), h_dst.to(cuda))
    eo, ei = ref.edgeconv_forward(k, src, h_src, h_dst)
    assert torch.equal(idx.cpu(), ei), "max_idx must be bit-exact"
    assert torch.equal(out.cpu(), eo), "a max of fp32 sums is exact"


def test_edgeconv_backward_and_autograd(cuda):
    from ae_mlsys_gnn_b200.layers import EdgeConv

    torch.manual_seed(0)
    n, k, cin, cout = 96, 20, 6, 32
    layer = EdgeConv(cin, cout).to(cuda)
    gen = torch.Generator().manual_seed(4)
    x = torch.randn(n, cin, generator=gen)
    src = torch.randint(0, n, (n * k,), generator=gen, dtype=torch.int32)
    xd = x.to(cuda).requires_grad_(True)
    out = layer(k, src.to(cuda), xd)
    gout = torch.randn(n, cout, generator=gen)
    out.backward(gout.to(cuda))

    tw = layer.theta.weight.detach().cpu().double().requires_grad_(True)
    pw = layer.phi.weight.detach().cpu().double().requires_grad_(True)
    xr = x.double().requires_grad_(True)
    eo = ref.edgeconv_layer_dgl(k, src, xr, tw, pw)
    eo.backward(gout.double())
    assert_close(out, eo, "EdgeConv out")
    assert_close(layer.theta.weight.grad, tw.grad, "theta.grad", scale_atol=True)
    assert_close(layer.phi.weight.grad, pw.grad, "phi.grad", scale_atol=True)
    assert_close(xd.grad, xr.grad, "x.grad", scale_atol=True)


def test_edgeconv_backward_scatter(cuda):
    from ae_mlsys_gnn_b200.operators.fused_edgeconv import edgeconv_backward

    gen = torch.Generator().manual_seed(9)
    n, F = 300, 48
    idx = torch.randint(-1, n, (n, F), generator=gen, dtype=torch.int32)
    g = torch.randn(n, F, generator=gen)
    got = edgeconv_backward(g.to(cuda), idx.to(cuda))
    assert_close(got, ref.edgeconv_backward(g, idx), "grad_src", scale_atol=True)


@pytest.mark.parametrize("n,k,F", [(64, 20, 64), (33, 5, 7), (30, 33, 8), (17, 20, 100)])
@pytest.mark.parametrize("ties", [False, True])
def test_edgeconv_leaky_forward_and_backward(cuda, n, k, F, ties):
    """LeakyReLU folded into the kernels: the output is bitwise leaky(max) of the plain forward
    (same arg-max), the backward equals autograd through the oracle's max followed by
    torch's leaky_relu."""
    from ae_mlsys_gnn_b200.operators.fused_edgeconv import edgeconv_forward, fused_edgeconv_op

    slope = 0.2
    src, h_src, h_dst = _case(n, k, F, n * 77 + k, ties)
    h_src = h_src - 1.0  # both signs of the maximum occur
    out, idx = edgeconv_forward(k, src.to(cuda), h_src.to(cuda), h_dst.to(cuda), slope)
    eo, ei = ref.edgeconv_forward(k, src, h_src, h_dst)
    assert torch.equal(idx.cpu(), ei)
    assert torch.equal(out.cpu(), torch.nn.functional.leaky_relu(eo, slope))

    hs = h_src.to(cuda).requires_grad_(True)
    hd = h_dst.to(cuda).requires_grad_(True)
    gen = torch.Generator().manual_seed(5)
    gout = torch.randn(n, F, generator=gen)
    fused_edgeconv_op(k, src.to(cuda), hs, hd, slope).backward(gout.to(cuda))
    g_pre = torch.where(eo > 0, gout, gout * slope)
    assert torch.equal(hd.grad.cpu(), g_pre)
    assert_close(hs.grad, ref.edgeconv_backward(g_pre, ei), "grad_src", scale_atol=True)

"""GMMConv operators against the oracle (values) and its autograd (gradients)."""
import pytest
import torch

from oracle import ops as ref
from tests.util import assert_close, crafted_graphs, power_law_graph

pytestmark = pytest.mark.gpu


def _inputs(g, K, D, F, seed):
    gen = torch.Generator().manual_seed(seed)
    feat = torch.randn(g.n, K, F, generator=gen)
    pseudo = torch.rand(g.nnz, D, generator=gen)
    mu = torch.randn(K, D, generator=gen) * 0.3
    sig = torch.rand(K, D, generator=gen) + 0.5
    return feat, pseudo, mu, sig


@pytest.mark.parametrize("name", ["tiny", "empty_rows", "hub", "long_rows", "no_edges"])
@pytest.mark.parametrize("K,D,F", [(3, 2, 16), (2, 1, 16), (1, 3, 5), (4, 2, 32), (8, 8, 8)])
def test_gmm_forward(cuda, name, K, D, F):
    from ae_mlsys_gnn_b200.graphs import Graph
    from ae_mlsys_gnn_b200.operators.fused_gmmconv import gmmconv

    g = crafted_graphs()[name]
    nc = max(g.n, int(g.col_ind.max().item()) + 1 if g.nnz else g.n)
    gen = torch.Generator().manual_seed(3)
    feat = torch.randn(nc, K, F, generator=gen)
    _, pseudo, mu, sig = _inputs(g, K, D, F, 4)
    out = gmmconv(g.row_ptr.to(cuda), g.col_ind.to(cuda), feat.to(cuda), pseudo.to(cuda),
                  mu.to(cuda), sig.to(cuda))
    eo = ref.gmm_forward(g.row_ptr, g.col_ind, feat, pseudo, mu, sig)
    assert_close(out, eo, f"gmm out[{name}]")


@pytest.mark.parametrize("K,D,F", [(3, 2, 16), (2, 1, 16), (1, 3, 5)])
@pytest.mark.parametrize("op", ["GmmConvFuse", "GmmConvStash", "GmmConvFuseEb"])
def test_gmm_autograd(cuda, K, D, F, op):
    import ae_mlsys_gnn_b200.operators.fused_gmmconv as M
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc

    g = power_law_graph(400, 15, seed=2)
    feat, pseudo, mu, sig = _inputs(g, K, D, F, 5)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    cp, ri, pm = csr2csc(rp, ci)
    dv = [t.to(cuda).requires_grad_(True) for t in (feat, pseudo, mu, sig)]
    out = getattr(M, op)(rp, ci, cp, ri, pm, *dv)
    gout = torch.randn(out.shape, generator=torch.Generator().manual_seed(6))
    out.backward(gout.to(cuda))
    rv = [t.double().requires_grad_(True) for t in (feat, pseudo, mu, sig)]
    eo = ref.gmm_forward(g.row_ptr, g.col_ind, *rv)
    eo.backward(gout.double())
    assert_close(out, eo, "out")
    for name, a, b in zip(("node_feat", "pseudo", "mu", "inv_sigma"), dv, rv):
        assert_close(a.grad, b.grad, f"grad {name}", scale_atol=True)


def test_gaussian(cuda):
    from ae_mlsys_gnn_b200.operators.fused_gmmconv import GaussianCp

    gen = torch.Generator().manual_seed(8)
    E, K, D = 1000, 3, 2
    p, mu, sg = torch.rand(E, D, generator=gen), torch.randn(K, D, generator=gen), torch.rand(K, D, generator=gen) + 0.2
    dv = [t.to(cuda).requires_grad_(True) for t in (p, mu, sg)]
    out = GaussianCp(*dv)
    gout = torch.randn(E, K, generator=gen)
    out.backward(gout.to(cuda))
    rv = [t.double().requires_grad_(True) for t in (p, mu, sg)]
    eo = ref.gaussian(*rv)
    eo.backward(gout.double())
    assert_close(out, eo, "gaussian")
    for name, a, b in zip(("pseudo", "mu", "inv_sigma"), dv, rv):
        assert_close(a.grad, b.grad, f"grad {name}", scale_atol=True)


def test_gmm_layer(cuda):
    from ae_mlsys_gnn_b200.layers import GMMConv
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc

    torch.manual_seed(1)
    g = power_law_graph(300, 10, seed=3)
    layer = GMMConv(20, 16, 2, 3, residual=True).to(cuda)
    gen = torch.Generator().manual_seed(2)
    x = torch.randn(g.n, 20, generator=gen)
    pseudo = torch.rand(g.nnz, 2, generator=gen)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    cp, ri, pm = csr2csc(rp, ci)
    out = layer(rp, ci, cp, ri, pm, x.to(cuda), pseudo.to(cuda))
    w = {k: v.detach().cpu().double() for k, v in layer.state_dict().items()}
    nf = (x.double() @ w["fc.weight"].T).view(g.n, 3, 16)
    eo = ref.gmm_forward(g.row_ptr, g.col_ind, nf, pseudo, w["mu"], w["inv_sigma"]).sum(1)
    eo = eo + x.double() @ w["res_fc.weight"].T + w["bias"]
    assert_close(out, eo, "GMMConv layer")


@pytest.mark.parametrize("n,K,F", [(300, 3, 16), (257, 2, 7), (64, 8, 64), (1, 1, 3), (0, 3, 16)])
@pytest.mark.parametrize("with_res,with_bias", [(True, True), (False, True), (True, False), (False, False)])
def test_kernel_sum(cuda, n, K, F, with_res, with_bias):
    """The layer's tail (sum over kernels + residual + bias) and its gradients against torch."""
    from ae_mlsys_gnn_b200.operators.fused_gmmconv import kernel_sum

    gen = torch.Generator().manual_seed(n * 31 + K)
    x = torch.randn(n, K, F, generator=gen)
    res = torch.randn(n, F, generator=gen) if with_res else None
    bias = torch.randn(F, generator=gen) if with_bias else None
    gout = torch.randn(n, F, generator=gen)

    def run(dev, dtype):
        leaves = [t.to(dev, dtype).requires_grad_(True) if t is not None else None for t in (x, res, bias)]
        if dev == "cpu":
            out = leaves[0].sum(1)
            if leaves[1] is not None:
                out = out + leaves[1]
            if leaves[2] is not None:
                out = out + leaves[2]
        else:
            out = kernel_sum(*leaves)
        out.backward(gout.to(dev, dtype))
        return out, [t.grad if t is not None else None for t in leaves]

    out, grads = run(cuda, torch.float32)
    eo, egrads = run("cpu", torch.float64)
    assert_close(out, eo, "kernel_sum")
    for name, a, b in zip(("x", "residual", "bias"), grads, egrads):
        if b is not None:
            assert_close(a, b, f"grad {name}", scale_atol=True)

"""csr2csc is integer work: outputs must be bit-identical to the oracle."""
import numpy as np
import pytest
import torch

from oracle import ops as ref
from tests.util import crafted_graphs, graph_from_degrees, power_law_graph

pytestmark = pytest.mark.gpu


def _check(cuda, g, n_cols=None):
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc

    nc = g.n if n_cols is None else n_cols
    cp, ri, pm = csr2csc(g.row_ptr.to(cuda), g.col_ind.to(cuda), n_cols=nc)
    ecp, eri, epm = ref.csr2csc_scipy(g.row_ptr, g.col_ind, n_cols=nc)
    assert torch.equal(cp.cpu(), ecp), "col_ptr"
    assert torch.equal(ri.cpu(), eri), "row_ind"
    assert torch.equal(pm.cpu(), epm), "permute"


@pytest.mark.parametrize("name", list(crafted_graphs().keys()))
def test_csr2csc_crafted(cuda, name):
    g = crafted_graphs()[name]
    nc = max(g.n, int(g.col_ind.max().item()) + 1 if g.nnz else g.n)
    _check(cuda, g, nc)


@pytest.mark.parametrize("n,mean", [(257, 5), (5000, 40), (70000, 12)])
def test_csr2csc_power_law(cuda, n, mean):
    _check(cuda, power_law_graph(n, mean, seed=n))


def test_csr2csc_wide_columns(cuda):
    """More than 2^16 and 2^24 columns: three and four radix passes."""
    rng = np.random.default_rng(0)
    _check(cuda, graph_from_degrees(rng.integers(0, 6, size=3000), n_cols=(1 << 16) + 77, seed=1),
           n_cols=(1 << 16) + 77)
    _check(cuda, graph_from_degrees(rng.integers(0, 4, size=2000), n_cols=(1 << 24) + 5, seed=2),
           n_cols=(1 << 24) + 5)


def test_csr2csc_duplicates_keep_csr_order(cuda):
    """Duplicate (row, col) entries: stability keeps their CSR order."""
    from ae_mlsys_gnn_b200.graphs import Graph

    row_ptr = torch.tensor([0, 4, 4, 7], dtype=torch.int32)
    col_ind = torch.tensor([2, 0, 2, 2, 1, 0, 0], dtype=torch.int32)
    _check(cuda, Graph(3, row_ptr, col_ind))


def test_csr2csc_involution(cuda):
    """Transposing twice gives back the CSR; composing the permutations gives identity."""
    from ae_mlsys_gnn_b200.operators.csr2csc import csr2csc

    g = power_law_graph(20000, 30, seed=11)
    rp, ci = g.row_ptr.to(cuda), g.col_ind.to(cuda)
    cp, ri, pm = csr2csc(rp, ci)
    rp2, ci2, pm2 = csr2csc(cp, ri)
    assert torch.equal(rp2, rp) and torch.equal(ci2, ci)
    assert torch.equal(pm[pm2.long()], torch.arange(g.nnz, device=cuda, dtype=torch.int32))

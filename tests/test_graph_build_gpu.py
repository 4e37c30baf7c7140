"""Graph construction kernels (COO -> CSR with dedup and self-loops, edge-balanced bounds, halo
plans) against SciPy / the host formulations: integer results, compared bit for bit."""
import numpy as np
import pytest
import scipy.sparse as sp
import torch

from oracle import ops as ref
from tests.util import power_law_graph

pytestmark = pytest.mark.gpu


def _scipy_csr(dst, src, n, self_loops):
    """What the reference's scripts do on the host (script/train/train_gatconv_our.py:82-91):
    remove self loops, add one per node, csr_matrix from (row = dst, col = src), duplicates summed."""
    d, s = dst.astype(np.int64), src.astype(np.int64)
    ok = (d >= 0) & (d < n) & (s >= 0) & (s < n)
    d, s = d[ok], s[ok]
    if self_loops:
        keep = d != s
        d, s = np.concatenate([d[keep], np.arange(n)]), np.concatenate([s[keep], np.arange(n)])
    m = sp.csr_matrix((np.ones(d.size), (d, s)), shape=(n, n))
    m.sum_duplicates()
    m.sort_indices()
    return m.indptr.astype(np.int32), m.indices.astype(np.int32)


@pytest.mark.parametrize("n,m,self_loops", [(5000, 200000, True), (5000, 200000, False), (70000, 300000, True),
                                             (257, 10, True), (40, 0, True), (40, 0, False), (3, 50, True)])
def test_coo_to_csr_matches_scipy(cuda, n, m, self_loops):
    from ae_mlsys_gnn_b200.operators.graph_build import coo_to_csr

    rng = np.random.default_rng(n + m)
    # skewed endpoints (many duplicates), some self loops, trailing nodes without any edge
    dst = np.minimum((rng.random(m) ** 2 * n * 0.9).astype(np.int64), n - 1)
    src = np.minimum((rng.random(m) ** 1.5 * n * 0.9).astype(np.int64), n - 1)
    if m > 20:
        src[:10] = dst[:10]         # explicit self loops
        dst[10:15] = -1             # out-of-range endpoints are dropped
        src[15:20] = n
    rp, ci = coo_to_csr(torch.from_numpy(dst.astype(np.int32)).to(cuda), torch.from_numpy(src.astype(np.int32)).to(cuda),
                        n, self_loops)
    erp, eci = _scipy_csr(dst, src, n, self_loops)
    assert torch.equal(rp.cpu(), torch.from_numpy(erp))
    assert torch.equal(ci.cpu(), torch.from_numpy(eci))


def test_generators_on_device_equal_host(cuda):
    """The benchmark's graph generators run through the device construction on a GPU; same seed,
    same pairs -> the same CSR as the host formulation."""
    from ae_mlsys_gnn_b200.graphs import csr_from_edges

    gen = torch.Generator().manual_seed(4)
    n = 3000
    d = torch.randint(0, n, (50000,), generator=gen)
    s = torch.randint(0, n, (50000,), generator=gen)
    for loops in (True, False):
        host = csr_from_edges(n, d, s, loops)
        dev = csr_from_edges(n, d.to(cuda), s.to(cuda), loops)
        assert torch.equal(host.row_ptr, dev.row_ptr.cpu()) and torch.equal(host.col_ind, dev.col_ind.cpu())


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_edge_balanced_bounds(cuda, world):
    from ae_mlsys_gnn_b200.operators.graph_build import edge_balanced_bounds as device_bounds
    from ae_mlsys_gnn_b200.partition import edge_balanced_bounds

    g = power_law_graph(3000, 25, seed=2)
    assert device_bounds(g.row_ptr.to(cuda), world) == edge_balanced_bounds(g.row_ptr, world)


@pytest.mark.parametrize("world", [2, 5, 8])
def test_halo_plans_on_device_equal_host(cuda, world):
    from ae_mlsys_gnn_b200.halo import build_halo_partition

    g = power_law_graph(1500, 14, seed=6)
    cp, ri, _ = ref.csr2csc(g.row_ptr, g.col_ind)
    dev = [t.to(cuda) for t in (g.row_ptr, g.col_ind, cp, ri)]
    for rank in range(world):
        h = build_halo_partition(g.row_ptr, g.col_ind, cp, ri, rank, world)
        d = build_halo_partition(*dev, rank, world)
        assert h.bounds == d.bounds
        for name in ("row_ptr", "col_ind", "col_ptr", "row_ind", "rs_ptr", "rs_pos"):
            assert torch.equal(getattr(h, name), getattr(d, name).cpu()), name
        for a, b in ((h.fwd, d.fwd), (h.bwd, d.bwd)):
            assert a.send_splits == b.send_splits and a.recv_splits == b.recv_splits
            assert a.halo_sizes == b.halo_sizes and a.dst_off == b.dst_off and a.active == b.active
            assert torch.equal(a.send_idx32, b.send_idx32.cpu())

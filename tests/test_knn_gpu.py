"""kNN graph kernel against the CPU oracle: source ids bit-equal, ties included."""
import pytest
import torch

from oracle import ops as ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,P,C,k", [(4, 1024, 3, 20), (3, 257, 3, 20), (2, 100, 2, 5), (2, 300, 16, 20),
                                     (1, 64, 3, 64), (5, 33, 7, 33), (2, 130, 4, 1), (1, 2000, 3, 20),
                                     (1, 500, 64, 20)])
def test_knn_matches_oracle(cuda, B, P, C, k):
    from ae_mlsys_gnn_b200.operators.knn import knn_graph

    pts = torch.randn(B, P, C, generator=torch.Generator().manual_seed(B * 1000 + P + C))
    got = knn_graph(pts.to(cuda), k)
    exp = ref.knn_graph(pts, k)
    assert got.dtype == torch.int32 and got.shape == (B * P * k,)
    assert torch.equal(got.cpu(), exp)
    # every point is its own nearest neighbour
    first = got.view(B * P, k)[:, 0].cpu()
    assert torch.equal(first, torch.arange(B * P, dtype=torch.int32))


def test_knn_ties_go_to_the_lower_index(cuda):
    """Points on a small integer grid, many of them duplicated: plenty of exactly equal distances."""
    from ae_mlsys_gnn_b200.operators.knn import knn_graph

    gen = torch.Generator().manual_seed(3)
    pts = torch.randint(0, 4, (3, 200, 3), generator=gen).float()
    got = knn_graph(pts.to(cuda), 20)
    assert torch.equal(got.cpu(), ref.knn_graph(pts, 20))


def test_knn_agrees_with_distance_matrix_formulation(cuda):
    """Same neighbour sets as the pairwise-distance-matrix + top-k formulation (random points:
    no exact ties, so only the arithmetic of the distance could differ)."""
    from ae_mlsys_gnn_b200.graphs import unit_ball_points
    from ae_mlsys_gnn_b200.operators.knn import knn_graph

    pts = unit_ball_points(4, 1024, seed=1)
    got = knn_graph(pts.to(cuda), 20).view(4, 1024, 20).cpu().long()
    d2 = torch.cdist(pts.double(), pts.double())
    exp = torch.topk(d2, 20, dim=-1, largest=False, sorted=True).indices + (torch.arange(4) * 1024).view(4, 1, 1)
    assert torch.equal(got.sort(-1).values, exp.sort(-1).values)


def test_knn_feeds_edgeconv(cuda):
    """DGCNN-style dynamic graph: kNN on the current features, then the fused EdgeConv."""
    from ae_mlsys_gnn_b200.operators.fused_edgeconv import edgeconv_forward
    from ae_mlsys_gnn_b200.operators.knn import knn_graph

    gen = torch.Generator().manual_seed(5)
    B, P, F, k = 2, 128, 16, 8
    feat = torch.randn(B, P, F, generator=gen)
    hs, hd = torch.randn(B * P, 8, generator=gen), torch.randn(B * P, 8, generator=gen)
    src = knn_graph(feat.to(cuda), k)
    out, idx = edgeconv_forward(k, src, hs.to(cuda), hd.to(cuda))
    eo, ei = ref.edgeconv_forward(k, ref.knn_graph(feat, k), hs, hd)
    assert torch.equal(out.cpu(), eo) and torch.equal(idx.cpu(), ei)

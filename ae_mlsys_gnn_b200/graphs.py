"""Seeded synthetic graphs and inputs with the shapes, sizes and value distributions
of the benchmark configurations (the public datasets the reference measures on —
Cora, Reddit, ModelNet40, PubMed, ogbn-products — are not available offline and are
not reproduced).

Every generator is deterministic for a given (seed, device type) and returns the
in-edge CSR the reference uses (row = destination, column = source,
script/train/train_gatconv_our.py:87-91): int32 ``row_ptr`` / ``col_ind``, column
ids ascending inside a row, no duplicate edges, exactly one self-loop per node.
The generators run on whatever device they are given; nothing here is on the timed
path.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch


@dataclass
class Graph:
    n: int
    row_ptr: torch.Tensor  # int32 [n+1]
    col_ind: torch.Tensor  # int32 [nnz]

    @property
    def nnz(self) -> int:
        return int(self.col_ind.numel())

    def to(self, device) -> "Graph":
        return Graph(self.n, self.row_ptr.to(device), self.col_ind.to(device))


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def csr_from_edges(n: int, dst: torch.Tensor, src: torch.Tensor, self_loops: bool = True) -> Graph:
    """Deduplicates (dst, src) pairs, optionally forces one self-loop per node, and
    builds the CSR sorted by (dst, src).  On a GPU this is the library's own construction
    (operators.graph_build.coo_to_csr: radix sorts, flags, scan, compaction); on the host the
    same result with framework ops."""
    dev = dst.device
    if dst.is_cuda and n < 2**31 - 2 and dst.numel() + n < 2**31 - 4096:
        from .operators.graph_build import coo_to_csr

        rp, ci = coo_to_csr(dst.to(torch.int32).contiguous(), src.to(torch.int32).contiguous(), n, self_loops)
        return Graph(n, rp, ci)
    dst = dst.long()
    src = src.long()
    if self_loops:
        keep = dst != src
        loops = torch.arange(n, device=dev)
        dst = torch.cat([dst[keep], loops])
        src = torch.cat([src[keep], loops])
    key = torch.unique(dst * n + src)  # sorted, duplicate-free
    dst = torch.div(key, n, rounding_mode="floor")
    src = key - dst * n
    counts = torch.bincount(dst, minlength=n)
    row_ptr = torch.zeros(n + 1, dtype=torch.int64, device=dev)
    row_ptr[1:] = torch.cumsum(counts, 0)
    return Graph(n, row_ptr.to(torch.int32), src.to(torch.int32))


def uniform_graph(n: int, n_edges: int, seed: int = 0, device="cpu") -> Graph:
    """``n_edges`` distinct directed edges with uniform-random endpoints (no
    self-loops among them) plus one self-loop per node (configs 1 and 4)."""
    g = _gen(seed, device)
    have = torch.empty(0, dtype=torch.int64, device=device)
    while have.numel() < n_edges:
        m = int((n_edges - have.numel()) * 1.2) + 16
        d = torch.randint(0, n, (m,), generator=g, device=device)
        s = torch.randint(0, n, (m,), generator=g, device=device)
        k = (d * n + s)[d != s]
        have = torch.unique(torch.cat([have, k]))
    if have.numel() > n_edges:  # drop a seeded random subset of the surplus
        perm = torch.randperm(have.numel(), generator=g, device=device)[:n_edges]
        have = have[perm]
    d = torch.div(have, n, rounding_mode="floor")
    return csr_from_edges(n, d, have - d * n)


def zipf_degree_weights(n: int, mean: float, max_deg: float, alpha: float = 0.6) -> torch.Tensor:
    """Expected-degree sequence w_i = c (i + i0)^-alpha with the requested mean and
    maximum (fp64, descending)."""
    i = torch.arange(1, n + 1, dtype=torch.float64)
    lo, hi = 0.0, float(n)
    target = max_deg / mean
    for _ in range(80):  # bisection on the offset: ratio max/mean falls as i0 grows
        mid = 0.5 * (lo + hi)
        w = (i + mid) ** (-alpha)
        if (w[0] / w.mean()).item() > target:
            lo = mid
        else:
            hi = mid
    w = (i + hi) ** (-alpha)
    return w * (mean / w.mean())


def chung_lu_graph(n: int, mean_deg: float, max_deg: float, seed: int = 0, device="cpu",
                   alpha: float = 0.6) -> Graph:
    """Chung–Lu sampling: n * mean_deg endpoint pairs, each endpoint drawn with
    probability proportional to a Zipf-like expected degree, duplicates and
    self-pairs dropped, self-loops added (config 2)."""
    g = _gen(seed, device)
    w = zipf_degree_weights(n, mean_deg, max_deg, alpha).to(device)
    cdf = torch.cumsum(w / w.sum(), 0)
    cdf[-1] = 1.0
    m = int(round(n * mean_deg))
    parts = []
    step = 1 << 25
    # node ids are shuffled so that degree is not monotone in the id
    relabel = torch.randperm(n, generator=g, device=device)
    for start in range(0, m, step):
        cnt = min(step, m - start)
        d = torch.searchsorted(cdf, torch.rand(cnt, generator=g, device=device, dtype=torch.float64))
        s = torch.searchsorted(cdf, torch.rand(cnt, generator=g, device=device, dtype=torch.float64))
        d = relabel[d.clamp_(max=n - 1)]
        s = relabel[s.clamp_(max=n - 1)]
        parts.append(torch.unique(d * n + s))
    key = torch.unique(torch.cat(parts))
    d = torch.div(key, n, rounding_mode="floor")
    return csr_from_edges(n, d, key - d * n)


def rmat_graph(n: int, n_pairs: int, abcd=(0.57, 0.19, 0.19, 0.05), seed: int = 0, device="cpu",
               symmetric: bool = True, relabel: bool = True) -> Graph:
    """R-MAT on ceil(log2 n) bits; pairs with an endpoint >= n are discarded, the rest
    symmetrised, deduplicated and given self-loops (config 5).  ``n_pairs`` is the
    number of generated (undirected) pairs before those steps.  With ``relabel`` the
    node ids are shuffled (seeded), as Graph500-style generators do, so that degree is
    not a function of the id."""
    g = _gen(seed, device)
    bits = max(1, math.ceil(math.log2(n)))
    a, b, c, _ = abcd
    parts = []
    step = 1 << 24
    for start in range(0, n_pairs, step):
        cnt = min(step, n_pairs - start)
        u = torch.zeros(cnt, dtype=torch.int64, device=device)
        v = torch.zeros(cnt, dtype=torch.int64, device=device)
        for _ in range(bits):
            r = torch.rand(cnt, generator=g, device=device)
            down = (r >= a + b).long()                      # quadrants c, d: row bit 1
            right = ((r >= a) & (r < a + b)) | (r >= a + b + c)  # quadrants b, d: col bit 1
            u = (u << 1) | down
            v = (v << 1) | right.long()
        ok = (u < n) & (v < n)
        u, v = u[ok], v[ok]
        k = u * n + v
        if symmetric:
            k = torch.cat([k, v * n + u])
        parts.append(torch.unique(k))
    key = torch.unique(torch.cat(parts))
    d = torch.div(key, n, rounding_mode="floor")
    s = key - d * n
    if relabel:
        perm = torch.randperm(n, generator=g, device=device)
        d, s = perm[d], perm[s]
    return csr_from_edges(n, d, s)


def knn_sources(points: torch.Tensor, k: int) -> torch.Tensor:
    """Per-cloud k nearest neighbours (Euclidean, the point itself included as the
    nearest).  ``points`` is (B, P, C); returns int32 source ids of shape (B*P*k,),
    the k sources of node i stored at [i*k, (i+1)*k) as the EdgeConv operator expects
    (src/fused_edgeconv/fused_edgeconv.cu:29-30), ids global (cloud offset added).
    On a GPU this is the kNN kernel (operators.knn); on the host (the CPU baseline's sample)
    the same rule written with framework ops: squared distance in float64 summed coordinate by
    coordinate, neighbours ordered by (distance, index)."""
    if points.is_cuda:
        from .operators.knn import knn_graph

        return knn_graph(points.float().contiguous(), k)
    B, P, C = points.shape
    x = points.double()
    d2 = torch.zeros(B, P, P, dtype=torch.float64)
    for c in range(C):
        diff = x[:, :, None, c] - x[:, None, :, c]
        d2 = d2 + diff * diff
    idx = torch.sort(d2, dim=-1, stable=True).indices[..., :k]
    idx = idx + (torch.arange(B) * P).view(B, 1, 1)
    return idx.reshape(-1).to(torch.int32)


def unit_ball_points(batch: int, n_points: int, seed: int = 0, device="cpu") -> torch.Tensor:
    """(batch, n_points, 3) points uniform in the unit ball (config 3)."""
    g = _gen(seed, device)
    v = torch.randn(batch, n_points, 3, generator=g, device=device)
    v = v / v.norm(dim=-1, keepdim=True)
    r = torch.rand(batch, n_points, 1, generator=g, device=device) ** (1.0 / 3.0)
    return v * r


def degree_pseudo(graph: Graph) -> torch.Tensor:
    """(E,2) pseudo-coordinates (1/sqrt(deg_src+1), 1/sqrt(deg_dst+1)) in CSR edge order,
    deg = in-degree (config 4; cf. script/train/train_gmmconv_our.py:124-130)."""
    rp = graph.row_ptr.long()
    deg = (rp[1:] - rp[:-1]).double()
    dst = torch.repeat_interleave(torch.arange(graph.n, device=rp.device), rp[1:] - rp[:-1])
    src = graph.col_ind.long()
    return torch.stack([1.0 / torch.sqrt(deg[src] + 1.0), 1.0 / torch.sqrt(deg[dst] + 1.0)], 1).float()


def bag_of_words(n: int, dim: int, p: float, seed: int = 0, device="cpu") -> torch.Tensor:
    """Binary features, each entry 1 with probability p (config 1)."""
    g = _gen(seed, device)
    return (torch.rand(n, dim, generator=g, device=device) < p).float()


def sparse_l1_features(n: int, dim: int, density: float, seed: int = 0, device="cpu") -> torch.Tensor:
    """`density` non-zeros ~ U(0,1), rows L1-normalised (config 4)."""
    g = _gen(seed, device)
    mask = torch.rand(n, dim, generator=g, device=device) < density
    x = torch.rand(n, dim, generator=g, device=device) * mask
    return x / x.sum(1, keepdim=True).clamp_min(1e-12)


def normal_features(n: int, dim: int, seed: int = 0, device="cpu") -> torch.Tensor:
    g = _gen(seed, device)
    return torch.randn(n, dim, generator=g, device=device)


def uniform_labels(n: int, n_classes: int, seed: int = 0, device="cpu") -> torch.Tensor:
    g = _gen(seed, device)
    return torch.randint(0, n_classes, (n,), generator=g, device=device)

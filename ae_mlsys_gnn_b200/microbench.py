"""Times one operator on a seeded synthetic graph and prints one JSON line.

  python -m ae_mlsys_gnn_b200.microbench --op gat_fwd --nodes 400000 --deg 50 --heads 4 --feat 128

Used for kernel work and as the small, self-terminating case for profiler captures
(few launches, under a few GB of device memory, gathered operand larger than L2).
"""
from __future__ import annotations

import argparse
import json

import torch

OPS = ("gat_fwd", "gat_fwd_act", "gat_fwd_bf16", "gat_bwd_pack_elu", "gat_bwd_row", "gat_bwd_col", "gat_bwd_col_edges", "gat_bwd_row_sum", "gat_bwd_pack", "csr2csc", "edgeconv_fwd", "gmm_fwd", "mhspmm", "mhsddmm",
       "gemm", "gemm_tn")


def dense_main(a):
    """Projection GEMM x (nodes, in) @ w (in, out), or its weight gradient x^T @ g."""
    import importlib

    D = importlib.import_module(".operators.dense", __package__)
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(a.seed)
    M, K, N = a.nodes, a.in_dim, a.out_dim
    x = torch.randn(M, K, device=dev, generator=gen)
    w = torch.randn(K, N, device=dev, generator=gen)
    g = torch.randn(M, N, device=dev, generator=gen)
    if a.op == "gemm":
        fn = lambda: D.gemm(x, w, False)
        nbytes = 4.0 * (M * K + K * N + M * N)
    else:
        fn = lambda: D.gemm_tn(x, g)
        nbytes = 4.0 * (M * K + M * N + K * N)
    flush = torch.empty(64 * 1024 * 1024, device=dev)
    for _ in range(a.warmup):
        fn()
    times = []
    for _ in range(a.iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    D.check_status()
    times.sort()
    med = times[len(times) // 2]
    print(json.dumps({"op": a.op, "nodes": M, "in_dim": K, "out_dim": N, "ms_median": med, "ms_min": times[0],
                      "algorithmic_gb": nbytes / 1e9, "gbs": nbytes / (med * 1e-3) / 1e9,
                      "tflops_fp32_equiv": 2.0 * M * K * N / (med * 1e-3) / 1e12}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", choices=OPS, default="gat_fwd")
    ap.add_argument("--graph", choices=("rmat", "chunglu", "uniform"), default="rmat")
    ap.add_argument("--nodes", type=int, default=400_000)
    ap.add_argument("--deg", type=int, default=50)
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--feat", type=int, default=128)
    ap.add_argument("--k", type=int, default=20)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--in-dim", type=int, default=512, help="gemm / gemm_tn: input width of the projection")
    ap.add_argument("--out-dim", type=int, default=512, help="gemm / gemm_tn: output width of the projection")
    a = ap.parse_args()
    if a.op in ("gemm", "gemm_tn"):
        return dense_main(a)

    from . import graphs as G
    import importlib

    T = importlib.import_module(".operators.csr2csc", __package__)
    EC = importlib.import_module(".operators.fused_edgeconv", __package__)
    GAT = importlib.import_module(".operators.fused_gat", __package__)
    GMM = importlib.import_module(".operators.fused_gmmconv", __package__)
    SP = importlib.import_module(".operators.mhspmm", __package__)

    dev = torch.device("cuda:0")
    n, H, F = a.nodes, a.heads, a.feat
    if a.graph == "rmat":
        g = G.rmat_graph(n, int(n * a.deg * 0.45), seed=a.seed, device=dev)
    elif a.graph == "chunglu":
        g = G.chung_lu_graph(n, a.deg, min(n // 2, a.deg * 40), seed=a.seed, device=dev)
    else:
        g = G.uniform_graph(n, n * a.deg, seed=a.seed, device=dev)
    nnz = g.nnz
    gen = torch.Generator(device=dev).manual_seed(a.seed)
    feat = torch.randn(n, H, F, device=dev, generator=gen)
    gout = torch.randn(n, H, F, device=dev, generator=gen)
    ar = torch.randn(n, H, device=dev, generator=gen)
    ac = torch.randn(n, H, device=dev, generator=gen)
    cp, ri, pm = T.csr2csc(g.row_ptr, g.col_ind)
    _, m, s = GAT.gat_forward(ar, ac, g.row_ptr, g.col_ind, 0.2, feat)
    _, rowpack = GAT.gat_backward_row(0.2, g.row_ptr, g.col_ind, m, s, feat, ar, ac, gout)
    HF = H * F
    if a.op == "gat_fwd":
        fn = lambda: GAT.gat_forward(ar, ac, g.row_ptr, g.col_ind, 0.2, feat)
        nbytes = 4.0 * nnz * (1 + H + HF) + 4.0 * n * (1 + 3 * H + HF)
    elif a.op == "gat_fwd_act":
        fn = lambda: GAT.gat_forward_act(ar, ac, g.row_ptr, g.col_ind, 0.2, feat)
        nbytes = 4.0 * nnz * (1 + H + HF) + 4.0 * n * (1 + 3 * H + 2 * HF)
    elif a.op == "gat_fwd_bf16":
        f16 = GAT.to_bf16(feat)
        fn = lambda: GAT.gat_forward_bf16(ar, ac, g.row_ptr, g.col_ind, 0.2, f16)
        nbytes = 4.0 * nnz * (1 + H) + 2.0 * nnz * HF + 4.0 * n * (1 + 3 * H + HF)
    elif a.op == "gat_bwd_pack_elu":
        out0 = GAT.gat_forward(ar, ac, g.row_ptr, g.col_ind, 0.2, feat)[0]
        fn = lambda: GAT.gat_backward_pack_elu(out0, gout, ar, m, s)
        nbytes = 4.0 * n * (3 * HF + 7 * H)
    elif a.op == "gat_bwd_row":
        fn = lambda: GAT.gat_backward_row(0.2, g.row_ptr, g.col_ind, m, s, feat, ar, ac, gout)
        nbytes = 4.0 * nnz * (1 + H + HF) + 4.0 * n * (1 + HF + 3 * H)
    elif a.op == "gat_bwd_col":
        fn = lambda: GAT.gat_backward_col(0.2, cp, ri, feat, ac, rowpack, gout)
        nbytes = 4.0 * nnz * (1 + 3 * H + HF) + 4.0 * n * (1 + HF + 3 * H)
    elif a.op == "gat_bwd_col_edges":
        fn = lambda: GAT.gat_backward_col_edges(0.2, cp, ri, feat, ac, rowpack, gout)
        nbytes = 4.0 * nnz * (1 + 4 * H + HF) + 4.0 * n * (1 + HF + 3 * H)
    elif a.op == "gat_bwd_row_sum":
        pos = GAT.invert_permutation(pm)
        eg = torch.randn(nnz, H, device=dev, generator=gen)
        fn = lambda: GAT.gat_backward_row_sum(g.row_ptr, pos, eg)
        nbytes = 4.0 * nnz * (1 + H) + 4.0 * n * (1 + H)
    elif a.op == "gat_bwd_pack":
        out0 = GAT.gat_forward(ar, ac, g.row_ptr, g.col_ind, 0.2, feat)[0]
        fn = lambda: GAT.gat_backward_pack(out0, gout, ar, m, s)
        nbytes = 4.0 * n * (2 * HF + 7 * H)
    elif a.op == "csr2csc":
        fn = lambda: T.csr2csc(g.row_ptr, g.col_ind)
        passes = (max(1, (n - 1).bit_length()) + 7) // 8
        nbytes = 4.0 * nnz * (passes * 5 + 4) + 8.0 * n
    elif a.op == "edgeconv_fwd":
        src = torch.randint(0, n, (n * a.k,), device=dev, dtype=torch.int32, generator=gen)
        hs, hd = feat.view(n, HF), gout.view(n, HF)
        fn = lambda: EC.edgeconv_forward(a.k, src, hs, hd)
        nbytes = 4.0 * n * a.k * (1 + HF) + 12.0 * n * HF
    elif a.op == "gmm_fwd":
        D = 2
        pseudo = torch.rand(nnz, D, device=dev, generator=gen)
        mu = torch.randn(H, D, device=dev, generator=gen) * 0.3
        sg = torch.rand(H, D, device=dev, generator=gen) + 0.5
        fn = lambda: GMM.gmmconv(g.row_ptr, g.col_ind, feat, pseudo, mu, sg)
        nbytes = 4.0 * nnz * (1 + D + HF) + 4.0 * n * (1 + HF)
    elif a.op == "mhspmm":
        att = torch.randn(nnz, H, device=dev, generator=gen)
        fn = lambda: SP.mhspmm_forward(g.row_ptr, g.col_ind, att, feat)
        nbytes = 4.0 * nnz * (1 + H + HF) + 4.0 * n * (1 + HF)
    else:
        fn = lambda: SP.mhsddmm_forward(g.row_ptr, g.col_ind, gout, feat)
        nbytes = 4.0 * nnz * (1 + H + HF) + 4.0 * n * (1 + HF)

    for _ in range(a.warmup):
        fn()
    torch.cuda.synchronize()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(a.iters)]
    for s0, s1 in ev:
        s0.record()
        fn()
        s1.record()
    torch.cuda.synchronize()
    ms = sorted(x.elapsed_time(y) for x, y in ev)
    med = ms[len(ms) // 2]
    print(json.dumps({"op": a.op, "graph": a.graph, "nodes": n, "edges": nnz, "heads": H, "feat": F,
                      "ms_median": med, "ms_min": ms[0], "algorithmic_gb": nbytes / 1e9,
                      "gbs": nbytes / med / 1e6}))


if __name__ == "__main__":
    main()

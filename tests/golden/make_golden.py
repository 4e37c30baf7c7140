"""Generates tests/golden/oracle_golden.npz: outputs of the CPU oracle (oracle/ops.py)
on small seeded inputs.  The reference repository ships no golden vectors of its
own; these fixtures freeze the oracle so that a later edit cannot silently change
what the CUDA kernels are compared against.  Run: python -m tests.golden.make_golden
"""
import os

import numpy as np
import torch

from oracle import ops as ref
from tests.util import power_law_graph


def compute():
    out = {}
    g = power_law_graph(64, 6, seed=42)
    gen = torch.Generator().manual_seed(42)
    H, F = 2, 4
    ar, ac = torch.randn(g.n, H, generator=gen), torch.randn(g.n, H, generator=gen)
    x, go = torch.randn(g.n, H, F, generator=gen), torch.randn(g.n, H, F, generator=gen)
    out["row_ptr"], out["col_ind"] = g.row_ptr.numpy(), g.col_ind.numpy()
    cp, ri, pm = ref.csr2csc_scipy(g.row_ptr, g.col_ind)
    out["col_ptr"], out["row_ind"], out["permute"] = cp.numpy(), ri.numpy(), pm.numpy()
    o, m, s = ref.gat_forward(ar, ac, g.row_ptr, g.col_ind, 0.2, x)
    gf, gar, gac = ref.gat_backward(0.2, g.row_ptr, g.col_ind, m, s, x, ar, ac, go)
    for k, v in dict(gat_out=o, gat_max=m, gat_sum=s, gat_grad_feat=gf, gat_grad_attn_row=gar,
                     gat_grad_attn_col=gac).items():
        out[k] = v.numpy()
    k = 5
    src = torch.randint(0, g.n, (g.n * k,), generator=gen, dtype=torch.int32)
    hs = torch.randint(0, 3, (g.n, 6), generator=gen).float()
    hd = torch.randint(0, 2, (g.n, 6), generator=gen).float()
    eo, ei = ref.edgeconv_forward(k, src, hs, hd)
    out["ec_src"], out["ec_out"], out["ec_idx"] = src.numpy(), eo.numpy(), ei.numpy()
    pseudo = torch.rand(g.nnz, 2, generator=gen)
    mu, sg = torch.randn(3, 2, generator=gen) * 0.3, torch.rand(3, 2, generator=gen) + 0.5
    nf = torch.randn(g.n, 3, 4, generator=gen)
    out["gmm_out"] = ref.gmm_forward(g.row_ptr, g.col_ind, nf, pseudo, mu, sg).numpy()
    return out


if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_golden.npz")
    np.savez_compressed(path, **compute())
    print("wrote", path)

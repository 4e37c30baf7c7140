"""Row-block partition and the partitioned GAT exchange logic, on CPU: two gloo ranks
with the oracle standing in for the CUDA kernels (the kernels themselves are covered by
the GPU tests; what is checked here is slicing, id remapping, the all-gathers, padding,
the loss normalisation and the gradient all-reduce)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ops as ref
from tests.util import assert_close, power_law_graph


def _pad(t, rows):
    if rows is None or rows <= t.shape[0]:
        return t
    out = t.new_zeros((rows,) + tuple(t.shape[1:]))
    out[: t.shape[0]] = t
    return out


class OracleKernels:
    """Same methods as partition._CudaKernels, computed by the CPU oracle."""

    @staticmethod
    def scores_forward(h, attn_l, attn_r):
        return (attn_l * h).sum(-1), (attn_r * h).sum(-1)

    @staticmethod
    def scores_backward(h, attn_l, attn_r, gar, gac, grad_feat):
        grad_feat += gar[:, :, None] * attn_l + gac[:, :, None] * attn_r
        return (gar[:, :, None] * h).sum(0), (gac[:, :, None] * h).sum(0)

    @staticmethod
    def forward_part(attn_row, attn_col_full, row_ptr, col_ind, slope, h_full, out, edge_max, edge_sum,
                     accumulate, finalize):
        n, H = attn_row.shape
        rows, cols = ref.rows_of(row_ptr), col_ind.long()
        e = ref.leaky_relu(attn_row.double()[rows] + attn_col_full.double()[cols], slope)
        m_p = torch.full((n, H), ref.NEG_BIG, dtype=torch.float64).scatter_reduce(
            0, rows[:, None].expand(-1, H), e, "amax", include_self=True)
        ex = torch.exp(e - m_p[rows])
        s_p = torch.zeros(n, H, dtype=torch.float64).index_add_(0, rows, ex)
        acc = torch.zeros((n,) + tuple(h_full.shape[1:]), dtype=torch.float64)
        acc.index_add_(0, rows, ex[:, :, None] * h_full.double()[cols])
        if accumulate:
            m_o, s_o = edge_max.double(), edge_sum.double()
            M = torch.maximum(m_o, m_p)
            fo, fn = torch.exp(m_o - M), torch.exp(m_p - M)
            acc = out[:n].double() * fo[:, :, None] + acc * fn[:, :, None]
            s_p = s_o * fo + s_p * fn
            m_p = M
        if finalize:
            acc = torch.where(s_p[:, :, None] > 0, acc / s_p[:, :, None].clamp_min(1e-300), acc)
        out[:n] = acc.float()
        edge_max.copy_(m_p.float())
        edge_sum.copy_(s_p.float())

    @staticmethod
    def backward_pack(out, grad_out, attn_row, edge_max, edge_sum, pad_to=None):
        n = edge_max.shape[0]
        S = (grad_out.double()[:n] * out.double()[:n]).sum(-1)
        es = edge_sum.double()
        inv = torch.where(es > 0, 1.0 / es.clamp_min(1e-300), torch.zeros_like(es))
        pack = torch.stack([attn_row.double()[:n], edge_max.double(), inv, torch.where(es > 0, S, torch.zeros_like(S))], 1)
        return _pad(pack.float(), pad_to)

    @staticmethod
    def backward_pack_elu(out, grad_act, attn_row, edge_max, edge_sum):
        n = edge_max.shape[0]
        o = out.double()[:n]
        grad_pre = (grad_act.double()[:n] * torch.where(o > 0, torch.ones_like(o), torch.exp(o))).float()
        return grad_pre, OracleKernels.backward_pack(out, grad_pre, attn_row, edge_max, edge_sum)

    @staticmethod
    def backward_col_edges_part(slope, col_ptr, row_ind, h_local, attn_col_local, rowpack_full, gout_full,
                                grad_feat, grad_attn_col, accumulate):
        cols, rows = ref.rows_of(col_ptr), row_ind.long()   # segments are the owned sources
        rp = rowpack_full.double()
        x = rp[rows, 0] + attn_col_local.double()[cols]
        e = torch.where(x > 0, x, x * slope)
        alpha = torch.exp(e - rp[rows, 1]) * rp[rows, 2]
        G = gout_full.double()[rows]
        n, H, F = h_local.shape
        gh = torch.zeros(n, H, F, dtype=torch.float64).index_add_(0, cols, alpha[:, :, None] * G)
        g = (G * h_local.double()[cols]).sum(-1)
        ge = alpha * (g - rp[rows, 3])
        ge = torch.where(e < 0, ge * slope, ge)
        gac = torch.zeros(n, H, dtype=torch.float64).index_add_(0, cols, ge)
        if accumulate:
            grad_feat[:n] += gh.float()
            grad_attn_col += gac.float()
        else:
            grad_feat[:n] = gh.float()
            grad_attn_col.copy_(gac.float())
        return ge.float()

    @staticmethod
    def backward_row_sum(ptr, pos, edge_grad):
        n = ptr.numel() - 1
        seg = ref.rows_of(ptr)
        out = torch.zeros(n, edge_grad.shape[1], dtype=torch.float64)
        out.index_add_(0, seg, edge_grad.double()[pos.long()])
        return out.float()


def test_edge_balanced_bounds():
    from ae_mlsys_gnn_b200.partition import edge_balanced_bounds

    g = power_law_graph(2000, 30, seed=1)
    for world in (1, 2, 4, 8):
        b = edge_balanced_bounds(g.row_ptr, world)
        assert b[0] == 0 and b[-1] == g.n and len(b) == world + 1
        assert all(b[i] <= b[i + 1] for i in range(world))
        rp = g.row_ptr.long()
        per = [int(rp[b[i + 1]] - rp[b[i]]) for i in range(world)]
        assert max(per) <= g.nnz / world + int((rp[1:] - rp[:-1]).max())


@pytest.mark.parametrize("pieces", [1, 3])
def test_partition_blocks_cover_graph(pieces):
    from ae_mlsys_gnn_b200.partition import build_partition

    g = power_law_graph(500, 12, seed=2)
    cp, ri, _ = ref.csr2csc(g.row_ptr, g.col_ind)
    world = 4
    parts = [build_partition(g.row_ptr, g.col_ind, cp, ri, r, world, pieces=pieces) for r in range(world)]
    p0 = parts[0]
    assert sum(p.n_local for p in parts) == g.n and p0.max_n == pieces * p0.cn
    assert sum(p.col_ind.numel() for p in parts) == g.nnz
    # position of every global node in the gathered (piece-major) index space
    pos = torch.cat([p0.gathered_positions(r) for r in range(world)])
    assert pos.unique().numel() == g.n and int(pos.max()) < world * p0.max_n
    inv = torch.full((world * p0.max_n,), -1, dtype=torch.long)
    inv[pos] = torch.arange(g.n)
    for r, p in enumerate(parts):
        lo, hi = p.bounds[r], p.bounds[r + 1]
        rp = g.row_ptr.long()
        # same edge set per row in the full local CSR and in the union of its pieces
        want = g.col_ind.long()[rp[lo]:rp[hi]]
        rows = ref.rows_of(p.row_ptr)
        got = inv[p.col_ind.long()]
        assert torch.equal(torch.sort(rows * g.n + got).values,
                           torch.sort(ref.rows_of(g.row_ptr)[rp[lo]:rp[hi]].sub(lo) * g.n + want).values)
        keys = []
        for c, (ptr_c, idx_c) in enumerate(p.csr_parts):
            assert ptr_c.numel() == p.n_local + 1
            assert torch.all(idx_c.long() // (world * p.cn) == c)
            keys.append(ref.rows_of(ptr_c) * g.n + inv[idx_c.long()])
        assert torch.equal(torch.sort(torch.cat(keys)).values, torch.sort(rows * g.n + got).values)
        assert sum(i.numel() for _, i in p.csc_parts) == int(cp.long()[hi] - cp.long()[lo])


def _worker(rank, world, port, results, pieces=3):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ae_mlsys_gnn_b200.partition import PartitionedGAT, build_partition

        torch.manual_seed(0)
        g = power_law_graph(300, 10, seed=3)
        cp, ri, _ = ref.csr2csc(g.row_ptr, g.col_ind)
        x = torch.randn(g.n, 12, generator=torch.Generator().manual_seed(1))
        y = torch.randint(0, 5, (g.n,), generator=torch.Generator().manual_seed(2))
        part = build_partition(g.row_ptr, g.col_ind, cp, ri, rank, world, pieces=pieces)
        model = PartitionedGAT(12, [8], [2], 5, 1, kernels=OracleKernels)
        if pieces == 1:  # also exercise "gather the inputs, project everywhere"
            for layer in model.gat_layers:
                layer.recompute_projection = True
        out = model(part, part.pad_rows(part.local_slice(x)))
        loss = model.loss(part, out, part.local_slice(y))
        loss.backward()
        model.all_reduce_grads(world)
        total = loss.detach().clone()
        dist.all_reduce(total)
        gathered = [torch.empty(part.max_n, out.shape[1]) for _ in range(world)]
        dist.all_gather(gathered, out.detach())
        if rank == 0:
            full = torch.cat([gathered[r][: part.bounds[r + 1] - part.bounds[r]] for r in range(world)])  # rank-major list
            results["out"] = full
            results["loss"] = total
            results["grads"] = {k: p.grad.clone() for k, p in model.named_parameters()}
            results["state"] = {k: v.clone() for k, v in model.state_dict().items()}
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("pieces", [3, 1])
def test_partitioned_gat_two_ranks_matches_single(pieces):
    import socket

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(2, port, results, pieces), nprocs=2, join=True)

    g = power_law_graph(300, 10, seed=3)
    x = torch.randn(g.n, 12, generator=torch.Generator().manual_seed(1))
    y = torch.randint(0, 5, (g.n,), generator=torch.Generator().manual_seed(2))
    st = {k: v.double().requires_grad_(True) for k, v in results["state"].items()}
    h = x.double()
    h = ref.gat_layer_dgl(g.row_ptr, g.col_ind, h, st["gat_layers.0.W"], st["gat_layers.0.attn_l"],
                          st["gat_layers.0.attn_r"], 0.2).flatten(1)
    h = torch.nn.functional.elu(h)
    out = ref.gat_layer_dgl(g.row_ptr, g.col_ind, h, st["gat_layers.1.W"], st["gat_layers.1.attn_l"],
                            st["gat_layers.1.attn_r"], 0.2).mean(1)
    loss = torch.nn.functional.cross_entropy(out, y)
    loss.backward()
    assert_close(results["out"], out, "partitioned logits")
    assert_close(results["loss"], loss, "loss")
    for k, gval in results["grads"].items():
        assert_close(gval, st[k].grad, f"grad {k}", scale_atol=True)


@pytest.mark.parametrize("pieces", [1, 3])
def test_partition_transposed_block_index(pieces):
    """rowsum_parts[c] lists, for every destination row of piece c (gathered order), the
    positions of its edges inside csc_parts[c], ascending."""
    from ae_mlsys_gnn_b200.partition import build_partition

    g = power_law_graph(400, 9, seed=4)
    cp, ri, _ = ref.csr2csc(g.row_ptr, g.col_ind)
    world = 3
    for r in range(world):
        p = build_partition(g.row_ptr, g.col_ind, cp, ri, r, world, pieces=pieces)
        span = world * p.cn
        assert len(p.rowsum_parts) == pieces
        for c, ((_, ri_c), (ptr, pos)) in enumerate(zip(p.csc_parts, p.rowsum_parts)):
            assert ptr.numel() == span + 1 and int(ptr[-1]) == ri_c.numel() == pos.numel()
            assert torch.equal(torch.sort(pos.long()).values, torch.arange(pos.numel()))
            rows_of_pos = ri_c.long()[pos.long()] - c * span
            seg = ref.rows_of(ptr)
            assert torch.equal(rows_of_pos, seg)
            for s in range(span):  # ascending inside every row
                a, b = int(ptr[s]), int(ptr[s + 1])
                assert torch.all(pos[a + 1: b] > pos[a: b - 1]) if b - a > 1 else True

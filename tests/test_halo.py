"""Halo partition (only the rows a block references are exchanged), on CPU: gloo ranks with
the oracle standing in for the CUDA kernels.  Checked: the plans (who sends which rows to
whom), the id remapping into [own | halo], the all-to-all exchanges in both directions, and
that a partitioned GAT model reproduces the single-process logits, loss and gradients."""
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ops as ref
from tests.test_partition import OracleKernels
from tests.util import assert_close, power_law_graph


@pytest.mark.parametrize("world", [1, 2, 5])
def test_halo_plans_cover_the_graph(world):
    from ae_mlsys_gnn_b200.halo import build_halo_partition

    g = power_law_graph(500, 12, seed=2)
    cp, ri, _ = ref.csr2csc(g.row_ptr, g.col_ind)
    parts = [build_halo_partition(g.row_ptr, g.col_ind, cp, ri, r, world) for r in range(world)]
    assert sum(p.n_local for p in parts) == g.n
    assert sum(p.col_ind.numel() for p in parts) == g.nnz == sum(p.row_ind.numel() for p in parts)
    rp = g.row_ptr.long()
    for r, p in enumerate(parts):
        lo, hi = p.bounds[r], p.bounds[r + 1]
        for plan, ptr, idx, gptr, gidx in ((p.fwd, p.row_ptr, p.col_ind, g.row_ptr, g.col_ind),
                                           (p.bwd, p.col_ptr, p.row_ind, cp, ri)):
            # what this rank receives from q is what q sends to it, in the same order
            for q, other in enumerate(parts):
                oplan = other.fwd if plan is p.fwd else other.bwd
                assert plan.recv_splits[q] == oplan.send_splits[r]
            # extended-space ids decode back to the global ids of the block's edges
            halo_global = []
            for q, other in enumerate(parts):
                oplan = other.fwd if plan is p.fwd else other.bwd
                off = sum(oplan.send_splits[:r])
                halo_global.append(oplan.send_idx[off: off + oplan.send_splits[r]] + other.bounds[q])
            table = torch.cat([torch.arange(lo, hi)] + halo_global)
            e0, e1 = int(gptr.long()[lo]), int(gptr.long()[hi])
            assert torch.equal(table[idx.long()], gidx.long()[e0:e1])
            assert torch.equal(ptr.long(), gptr.long()[lo: hi + 1] - e0)
            assert int(idx.max()) < p.n_local + plan.n_halo if idx.numel() else True
        # transposed index of the local CSC
        n_ext = p.n_local + p.bwd.n_halo
        assert p.rs_ptr.numel() == n_ext + 1 and int(p.rs_ptr[-1]) == p.row_ind.numel()
        assert torch.equal(p.row_ind.long()[p.rs_pos.long()], ref.rows_of(p.rs_ptr))


def _star_graph():
    """One hub row holds almost all edges: some ranks own no rows at all, most nodes are isolated."""
    from ae_mlsys_gnn_b200.graphs import Graph

    n = 64
    deg = torch.zeros(n, dtype=torch.long)
    deg[5], deg[60] = 40, 2
    rp = torch.zeros(n + 1, dtype=torch.int32)
    rp[1:] = torch.cumsum(deg, 0).to(torch.int32)
    ci = torch.cat([torch.arange(10, 50), torch.tensor([5, 63])]).to(torch.int32)
    return Graph(n, rp, ci)


def _graph(kind):
    return _star_graph() if kind == "star" else power_law_graph(300, 10, seed=3)


class SharedMemoryExchange:
    """Factory of a CPU stand-in for halo.PeerStoreExchange: the peers' buffers are slices of
    shared-memory tensors (one pool per rank, created before the ranks are spawned), the push is
    an index copy into the peers' pools at the offsets the real kernel is given, and completion
    is a barrier.  Exercises everything host-side of the peer-store exchange: halo sizes of all
    ranks, destination offsets, the two alternating buffers per exchange point."""

    def __init__(self, pools):
        self.pools = pools

    def __call__(self, part, group, small_group):
        from ae_mlsys_gnn_b200.halo import PeerStoreExchange

        pools = self.pools

        class _Buf:
            def __init__(self, off, nbytes, rank):
                self.off, self.nbytes, self.rank = off, nbytes, rank

            def view(self, shape, dtype=torch.float32):
                numel = 1
                for v in shape:
                    numel *= int(v)
                return pools[self.rank][self.off: self.off + numel].view(shape)

            def close(self):
                pass

        class _Exchange(PeerStoreExchange):
            def __init__(self, *a):
                super().__init__(*a)
                self._next = 0

            def _alloc(self, nbytes, device):
                floats = (nbytes + 3) // 4
                off, self._next = self._next, self._next + floats
                assert self._next <= pools[0].numel(), "test pool too small"
                return _Buf(off, nbytes, self.rank)

            def _push(self, x, plan, buf, row_bytes, n_local):
                row = row_bytes // 4
                xf = x.reshape(x.shape[0], row)
                pos = 0
                for q, cnt in enumerate(plan.send_splits):
                    if cnt:
                        start = buf.off + (self.n_locals[q] + plan.dst_off[q]) * row
                        pools[q][start: start + cnt * row] = xf[plan.send_idx[pos: pos + cnt].long()].reshape(-1)
                        pos += cnt
                pools[self.rank][buf.off: buf.off + n_local * row] = xf[:n_local].reshape(-1)

            def _push_rows(self, x, plan, buf, row_bytes, lo, hi):
                self.block_pushes = getattr(self, "block_pushes", 0) + 1
                row = row_bytes // 4
                xf = x.reshape(x.shape[0], row)
                begs, cnts = plan.ranges(lo, hi)
                pos = 0
                for q, total in enumerate(plan.send_splits):
                    if cnts[q]:
                        start = buf.off + (self.n_locals[q] + plan.dst_off[q] + begs[q] - pos) * row
                        rows = plan.send_idx[begs[q]: begs[q] + cnts[q]].long()
                        assert bool(((rows >= lo) & (rows < hi)).all())
                        pools[q][start: start + cnts[q] * row] = xf[rows].reshape(-1)
                    pos += total
                pools[self.rank][buf.off + lo * row: buf.off + hi * row] = xf[lo:hi].reshape(-1)

            def _complete(self, device):
                dist.barrier()

        return _Exchange(part, group, small_group)


def _worker(rank, world, port, results, recompute, graph="powerlaw", pools=None, overlap=False):
    import os

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ae_mlsys_gnn_b200.halo import HaloGAT, HaloGATConv, build_halo_partition, halo_exchange, halo_return_sum

        if overlap:  # small blocks of rows are pushed while the projection of the next block "runs"
            HaloGATConv.OVERLAP_MIN_ROWS, HaloGATConv.OVERLAP_MIN_WIDTH = 8, 1
        torch.manual_seed(0)
        g = _graph(graph)
        cp, ri, _ = ref.csr2csc(g.row_ptr, g.col_ind)
        x = torch.randn(g.n, 12, generator=torch.Generator().manual_seed(1))
        y = torch.randint(0, 5, (g.n,), generator=torch.Generator().manual_seed(2))
        part = build_halo_partition(g.row_ptr, g.col_ind, cp, ri, rank, world)
        # exchange round trip on a tensor whose value is its global row id
        ids = torch.arange(part.bounds[rank], part.bounds[rank + 1], dtype=torch.float32).view(-1, 1)
        ext, _ = halo_exchange(ids, part.fwd, part.n_local)
        lo, hi = part.bounds[rank], part.bounds[rank + 1]
        e0, e1 = int(g.row_ptr[lo]), int(g.row_ptr[hi])
        assert torch.equal(ext[part.col_ind.long(), 0].long(), g.col_ind.long()[e0:e1])
        back = halo_return_sum(torch.ones(part.n_local + part.bwd.n_halo, 1), part.bwd, part.n_local)
        exchange = "nccl" if pools is None else SharedMemoryExchange(pools)
        model = HaloGAT(12, [8], [2], 5, 1, kernels=OracleKernels, exchange=exchange)
        for layer in model.gat_layers:
            layer.recompute_projection = recompute
            if overlap:
                layer.overlap_blocks = 4
        for _ in range(3 if pools is not None else 1):  # several steps: both buffers of every exchange point
            model.zero_grad()
            out = model(part, part.local_slice(x))
            loss = model.loss(part, out, part.local_slice(y))
            loss.backward()
        if overlap and part.fwd.active and part.n_local >= 32:
            assert model.exchanger(part).block_pushes > 0, "the block-wise push was not exercised"
        model.all_reduce_grads(world)
        total = loss.detach().clone()
        dist.all_reduce(total)
        outs = [None] * world
        dist.all_gather_object(outs, out.detach())
        backs = [None] * world
        dist.all_gather_object(backs, back)
        if rank == 0:
            results["out"] = torch.cat(outs)
            results["back"] = torch.cat(backs)
            results["loss"] = total
            results["grads"] = {k: p.grad.clone() for k, p in model.named_parameters()}
            results["state"] = {k: v.clone() for k, v in model.state_dict().items()}
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
@pytest.mark.parametrize("world,recompute,graph,peer,overlap", [
    (2, False, "powerlaw", False, False), (3, True, "powerlaw", False, False), (8, "auto", "powerlaw", False, False),
    (4, False, "star", False, False),      # ranks with empty blocks still join every collective
    (2, False, "powerlaw", True, False), (3, True, "powerlaw", True, False), (4, "auto", "star", True, False),
    (2, False, "powerlaw", True, True), (3, False, "powerlaw", True, True), (4, False, "star", True, True)])
def test_halo_gat_matches_single(world, recompute, graph, peer, overlap):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mgr = mp.Manager()
    results = mgr.dict()
    pools = [torch.zeros(1 << 20).share_memory_() for _ in range(world)] if peer else None
    mp.spawn(_worker, args=(world, port, results, recompute, graph, pools, overlap), nprocs=world, join=True)

    g = _graph(graph)
    cp, ri, _ = ref.csr2csc(g.row_ptr, g.col_ind)
    # every node got 1 from its owner plus 1 from every other rank that has it in its backward halo
    assert results["back"].min() >= 1 and results["back"].max() <= world
    x = torch.randn(g.n, 12, generator=torch.Generator().manual_seed(1))
    y = torch.randint(0, 5, (g.n,), generator=torch.Generator().manual_seed(2))
    st = {k: v.double().requires_grad_(True) for k, v in results["state"].items()}
    h = ref.gat_layer_dgl(g.row_ptr, g.col_ind, x.double(), st["gat_layers.0.W"], st["gat_layers.0.attn_l"],
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


def test_halo_plans_with_empty_blocks_and_isolated_nodes():
    """A star graph: one hub row holds almost all edges, so some ranks own no rows at all and
    most nodes are referenced by nobody.  The plans must stay consistent."""
    from ae_mlsys_gnn_b200.graphs import Graph
    from ae_mlsys_gnn_b200.halo import build_halo_partition

    n = 64
    deg = torch.zeros(n, dtype=torch.long)
    deg[5] = 40          # the hub: in-edges from nodes 10..49
    deg[60] = 2          # a tail row
    rp = torch.zeros(n + 1, dtype=torch.int32)
    rp[1:] = torch.cumsum(deg, 0).to(torch.int32)
    ci = torch.cat([torch.arange(10, 50), torch.tensor([5, 63])]).to(torch.int32)
    g = Graph(n, rp, ci)
    cp, ri, _ = ref.csr2csc(g.row_ptr, g.col_ind)
    world = 4
    parts = [build_halo_partition(g.row_ptr, g.col_ind, cp, ri, r, world) for r in range(world)]
    assert sum(p.n_local for p in parts) == n
    for r, p in enumerate(parts):
        for q, other in enumerate(parts):
            assert p.fwd.recv_splits[q] == other.fwd.send_splits[r]
            assert p.bwd.recv_splits[q] == other.bwd.send_splits[r]
        assert p.fwd.send_splits[r] == 0 and p.bwd.recv_splits[r] == 0
        assert p.row_ptr.numel() == p.n_local + 1 == p.col_ptr.numel()
        if p.col_ind.numel():
            assert int(p.col_ind.max()) < p.n_local + p.fwd.n_halo
        if p.row_ind.numel():
            assert int(p.row_ind.max()) < p.n_local + p.bwd.n_halo
        assert p.rs_ptr.numel() == p.n_local + p.bwd.n_halo + 1
    assert sum(p.col_ind.numel() for p in parts) == g.nnz == sum(p.row_ind.numel() for p in parts)

"""Row-block partition of one graph over the GPUs of a node with a *halo* exchange: a rank
receives only the rows its block references, not every rank's rows.

The reference is single-GPU; nothing here has a counterpart in it.  ``partition.py`` moves
per-node tensors with all-gathers (every rank receives all N rows).  On a power-law graph cut
into 8 edge-balanced row blocks a block's edges touch only about 40 % of the other ranks' nodes
(config-5 R-MAT: 39 % at 8 ranks, 49 % at 4, 58 % at 2), and the exchange is the part of the
epoch that does not shrink with the number of GPUs.  Here:

* Rank g owns a contiguous block of rows (same edge-balanced bounds as ``partition.py``): its
  CSR rows for the forward, its CSC columns for the backward, both with ``n_local`` segments.
* Forward plan: the sources the block's CSR references outside the block, sorted by global id
  (hence grouped by owner).  They form the *halo*; per-node tensors of sources live in an
  extended index space [own rows | halo rows] and the CSR column ids are remapped into it.
  One ``all_to_all_single`` with per-peer row counts moves exactly those rows (the sender
  gathers them into a contiguous buffer first).
* Backward plan: the same for the destinations the block's CSC references (rows of grad_out
  and of the per-row pack).  The partial grad_attn_row of halo rows (sums of this rank's edge
  gradients) travels back to the owners with the reversed all-to-all and is added there peer
  by peer in rank order (indices are unique per peer: no atomics, deterministic).
* Kernels, autograd structure, loss normalisation and gradient all-reduce are those of
  ``partition.py`` (one gather pass in the backward, node-wise per-row pack).
"""
from __future__ import annotations

import dataclasses
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from .layers.gatconv_layer import _GATBase
from .operators import dense
from .partition import _CudaKernels, _transposed_index, edge_balanced_bounds


@dataclass
class ExchangePlan:
    """Which local rows go to which rank, and how many rows arrive from each."""
    send_idx: torch.Tensor   # int64, local row ids grouped by destination rank, ascending inside a group
    send_splits: list        # rows sent to rank q (0 for this rank)
    recv_splits: list        # rows received from rank q (0 for this rank)

    @property
    def n_halo(self) -> int:
        return int(sum(self.recv_splits))


@dataclass
class HaloPartition:
    rank: int
    world: int
    bounds: list              # global row boundaries, world+1 entries
    row_ptr: torch.Tensor     # local CSR, int32 [n_local+1]
    col_ind: torch.Tensor     # int32, ids in [0, n_local + fwd.n_halo)
    col_ptr: torch.Tensor     # local CSC, int32 [n_local+1]
    row_ind: torch.Tensor     # int32, ids in [0, n_local + bwd.n_halo)
    rs_ptr: torch.Tensor      # transposed index of the local CSC over its n_local + bwd.n_halo rows
    rs_pos: torch.Tensor
    fwd: ExchangePlan
    bwd: ExchangePlan

    @property
    def n_local(self) -> int:
        return self.bounds[self.rank + 1] - self.bounds[self.rank]

    @property
    def n_global(self) -> int:
        return self.bounds[-1]

    def local_slice(self, x_global: torch.Tensor) -> torch.Tensor:
        return x_global[self.bounds[self.rank]: self.bounds[self.rank + 1]]

    def pad_rows(self, x_local: torch.Tensor) -> torch.Tensor:
        """Per-rank tensors need no padding here (kept for callers written for partition.py)."""
        return x_local.contiguous()

    def index_tensors(self) -> dict:
        return {"row_ptr": self.row_ptr, "col_ind": self.col_ind, "col_ptr": self.col_ptr,
                "row_ind": self.row_ind, "rs_ptr": self.rs_ptr, "rs_pos": self.rs_pos,
                "fwd_send": self.fwd.send_idx, "bwd_send": self.bwd.send_idx}

    def with_index_tensors(self, d: dict) -> "HaloPartition":
        return dataclasses.replace(
            self, row_ptr=d["row_ptr"], col_ind=d["col_ind"], col_ptr=d["col_ptr"], row_ind=d["row_ind"],
            rs_ptr=d["rs_ptr"], rs_pos=d["rs_pos"],
            fwd=dataclasses.replace(self.fwd, send_idx=d["fwd_send"]),
            bwd=dataclasses.replace(self.bwd, send_idx=d["bwd_send"]))


def _outside(ids: torch.Tensor, lo: int, hi: int) -> torch.Tensor:
    """Sorted unique global ids of ``ids`` that lie outside [lo, hi)."""
    u = torch.unique(ids.long())
    return u[(u < lo) | (u >= hi)]


def _plan(ptr: torch.Tensor, idx: torch.Tensor, bounds: list, rank: int, world: int):
    """Exchange plan and remapped ids for the segment array (ptr, idx) of a square graph whose
    segments AND ids are global node ids: rank r works on segments [bounds[r], bounds[r+1])."""
    dev = idx.device
    p = ptr.long()
    b = torch.tensor(bounds, dtype=torch.long, device=dev)
    lo, hi = bounds[rank], bounds[rank + 1]
    needs = []  # what every rank's block references outside itself
    for q in range(world):
        e0, e1 = int(p[bounds[q]].item()), int(p[bounds[q + 1]].item())
        needs.append(_outside(idx[e0:e1], bounds[q], bounds[q + 1]))
    mine = needs[rank]
    recv_splits = torch.bincount(torch.bucketize(mine, b[1:-1], right=True), minlength=world).tolist() \
        if world > 1 else [0]
    send, send_splits = [], []
    for q in range(world):
        if q == rank:
            send_splits.append(0)
            continue
        want = needs[q]
        rows = want[(want >= lo) & (want < hi)] - lo
        send.append(rows)
        send_splits.append(int(rows.numel()))
    send_idx = torch.cat(send) if send else torch.zeros(0, dtype=torch.long, device=dev)
    # local segments and ids in the extended space [own | halo]
    e0, e1 = int(p[lo].item()), int(p[hi].item())
    local_ptr = (p[lo: hi + 1] - e0).to(torch.int32).contiguous()
    v = idx[e0:e1].long()
    own = (v >= lo) & (v < hi)
    ext = torch.where(own, v - lo, (hi - lo) + torch.searchsorted(mine, v))
    return ExchangePlan(send_idx.contiguous(), send_splits, recv_splits), local_ptr, ext.to(torch.int32).contiguous()


def build_halo_partition(row_ptr, col_ind, col_ptr, row_ind, rank: int, world: int,
                         bounds: list | None = None) -> HaloPartition:
    """Cuts the global CSR (row_ptr, col_ind) and CSC (col_ptr, row_ind) of a square graph into
    rank ``rank``'s block and builds both exchange plans.  Every rank calls it with the same
    global graph (the plans of the peers are derived from it, no communication)."""
    bounds = edge_balanced_bounds(row_ptr, world) if bounds is None else bounds
    fwd, rp, ci = _plan(row_ptr, col_ind, bounds, rank, world)
    bwd, cp, ri = _plan(col_ptr, row_ind, bounds, rank, world)
    n_local = bounds[rank + 1] - bounds[rank]
    rs_ptr, rs_pos = _transposed_index(ri, 0, n_local + bwd.n_halo)
    return HaloPartition(rank, world, bounds, rp, ci, cp, ri, rs_ptr, rs_pos, fwd, bwd)


# ---------------------------------------------------------------------------------------------
# exchanges

def halo_exchange(x: torch.Tensor, plan: ExchangePlan, n_local: int, group=None, async_op: bool = False):
    """(n_local, ...) per-node rows -> (n_local + n_halo, ...) [own rows | rows of the halo].
    Returns (extended tensor, work or None)."""
    x = x.contiguous()
    if plan.n_halo == 0 and sum(plan.send_splits) == 0:
        return x[:n_local], None
    ext = x.new_empty((n_local + plan.n_halo,) + tuple(x.shape[1:]))
    ext[:n_local] = x[:n_local]
    send = x.index_select(0, plan.send_idx)
    work = dist.all_to_all_single(ext[n_local:], send, output_split_sizes=plan.recv_splits,
                                  input_split_sizes=plan.send_splits, group=group, async_op=async_op)
    if async_op:
        return ext, (work, send)  # the send buffer must outlive the transfer
    return ext, None


def halo_return_sum(x_ext: torch.Tensor, plan: ExchangePlan, n_local: int, group=None) -> torch.Tensor:
    """Inverse direction for partial sums: the halo rows of ``x_ext`` go back to their owners
    and are added to the owners' rows, peer by peer in rank order."""
    total = x_ext[:n_local].clone()
    if plan.n_halo == 0 and sum(plan.send_splits) == 0:
        return total
    back = x_ext.new_empty((int(sum(plan.send_splits)),) + tuple(x_ext.shape[1:]))
    dist.all_to_all_single(back, x_ext[n_local:].contiguous(), output_split_sizes=plan.send_splits,
                           input_split_sizes=plan.recv_splits, group=group)
    off = 0
    for cnt in plan.send_splits:
        if cnt:
            idx = plan.send_idx[off: off + cnt]
            total[idx] = total[idx] + back[off: off + cnt]  # idx is unique inside a peer's group
            off += cnt
    return total


class HaloGATFunction(torch.autograd.Function):
    """Scores + fused GAT aggregation on a halo partition, one autograd node.
    ``h`` and the output have n_local rows."""

    @staticmethod
    def forward(ctx, h, attn_l, attn_r, part: HaloPartition, slope, kernels, group, small_group,
                h_halo=None):
        n = part.n_local
        h, attn_l, attn_r = h.contiguous(), attn_l.contiguous(), attn_r.contiguous()
        H, Fo = h.shape[1], h.shape[2]
        attn_row, attn_col = kernels.scores_forward(h, attn_l, attn_r)
        if h_halo is None:
            h_ext, pending = halo_exchange(h, part.fwd, n, group, async_op=True)
        else:  # the caller projected the halo inputs itself: nothing wide to move
            h_ext, pending = torch.cat([h, h_halo]), None
        ac_ext, _ = halo_exchange(attn_col, part.fwd, n, small_group)
        if pending is not None:
            pending[0].wait()
        out = h.new_empty((n, H, Fo))
        edge_max = h.new_empty((n, H))
        edge_sum = h.new_empty((n, H))
        kernels.forward_part(attn_row, ac_ext, part.row_ptr, part.col_ind, slope, h_ext, out, edge_max,
                             edge_sum, False, True)
        ctx.save_for_backward(attn_row, attn_col, h, edge_max, edge_sum, attn_l, attn_r, out)
        ctx.part, ctx.slope, ctx.kernels = part, slope, kernels
        ctx.group, ctx.small_group = group, small_group
        return out

    @staticmethod
    def backward(ctx, grad_out):
        attn_row, attn_col, h, edge_max, edge_sum, attn_l, attn_r, out = ctx.saved_tensors
        part, slope, kernels = ctx.part, ctx.slope, ctx.kernels
        n = part.n_local
        H, Fo = h.shape[1], h.shape[2]
        grad_out = grad_out.contiguous()
        # grad_out rows travel while the per-row pack (node-wise) is formed and exchanged
        gout_ext, pending = halo_exchange(grad_out, part.bwd, n, ctx.group, async_op=True)
        rowpack = kernels.backward_pack(out, grad_out, attn_row, edge_max, edge_sum)
        rp_ext, _ = halo_exchange(rowpack, part.bwd, n, ctx.small_group)
        if pending is not None:
            pending[0].wait()
        gh = h.new_empty((n, H, Fo))
        gac = h.new_empty((n, H))
        edge_grad = kernels.backward_col_edges_part(slope, part.col_ptr, part.row_ind, h, attn_col, rp_ext,
                                                    gout_ext, gh, gac, False)
        gar_ext = kernels.backward_row_sum(part.rs_ptr, part.rs_pos, edge_grad)
        gar = halo_return_sum(gar_ext, part.bwd, n, ctx.small_group)
        gl, gr = kernels.scores_backward(h, attn_l, attn_r, gar, gac, gh)
        return gh, gl.view_as(attn_l), gr.view_as(attn_r), None, None, None, None, None, None


class HaloGATConv(_GATBase):
    """GATConv (same parameters, same state_dict) on a HaloPartition.

    ``recompute_projection``: when the layer widens its input at least four times ("auto", the
    default; e.g. 100 -> 512) the narrow inputs of the halo are exchanged and projected on the
    receiving rank instead of exchanging the wide projected rows."""

    def __init__(self, in_feats, out_feats, num_heads, negative_slope=0.2, kernels=_CudaKernels,
                 group=None, small_group=None, recompute_projection="auto"):
        super().__init__(in_feats, out_feats, num_heads, negative_slope)
        self.kernels = kernels
        self.group = group
        self.small_group = small_group
        self.recompute_projection = recompute_projection

    def _recompute(self, part) -> bool:
        if part.world == 1:
            return False
        if self.recompute_projection == "auto":
            return 4 * self.in_feats <= self.out_feats * self.num_heads
        return bool(self.recompute_projection)

    def forward(self, part: HaloPartition, feat):
        h = dense.project(feat, self.W).view(-1, self.num_heads, self.out_feats)
        h_halo = None
        if self._recompute(part):
            with torch.no_grad():
                x_ext, _ = halo_exchange(feat.detach(), part.fwd, part.n_local, self.group)
                h_halo = dense.project(x_ext[part.n_local:].contiguous(), self.W.detach()).view(
                    -1, self.num_heads, self.out_feats)
        return HaloGATFunction.apply(h, self.attn_l, self.attn_r, part, self.negative_slope,
                                     self.kernels, self.group, self.small_group, h_halo)


class HaloGAT(nn.Module):
    """models.GAT on a halo partition: identical parameters; inputs / outputs hold the rank's
    n_local rows.  ``small_group`` is a second communicator over the same ranks for the small
    per-node tensors (created here when torch.distributed is initialised)."""

    def __init__(self, in_dim, hidden, heads, num_classes, out_heads=1, negative_slope=0.2,
                 activation="elu", kernels=_CudaKernels, group=None, small_group=None):
        super().__init__()
        if (small_group is None and dist.is_available() and dist.is_initialized()
                and dist.get_world_size() > 1):
            small_group = dist.new_group(ranks=list(range(dist.get_world_size())))
        if isinstance(hidden, int):
            hidden = [hidden] * len(heads)
        dims_in = [in_dim] + [h * f for h, f in zip(heads, hidden)]
        self.gat_layers = nn.ModuleList(
            [HaloGATConv(dims_in[i], hidden[i], heads[i], negative_slope, kernels, group, small_group)
             for i in range(len(heads))])
        self.gat_layers.append(
            HaloGATConv(dims_in[-1], num_classes, out_heads, negative_slope, kernels, group, small_group))
        self.activation = activation
        self.group = group

    def forward(self, part: HaloPartition, inputs):
        h = inputs
        for layer in self.gat_layers[:-1]:
            h = layer(part, h).flatten(1)
            if self.activation == "elu":
                h = F.elu(h)
        return self.gat_layers[-1](part, h).mean(1)

    def loss(self, part: HaloPartition, logits, labels_local):
        """Cross-entropy averaged over ALL nodes of the graph (sum over the owned rows divided
        by the global node count), so that summing gradients over ranks gives the single-GPU
        gradient."""
        picked = F.log_softmax(logits, dim=1).gather(1, labels_local.view(-1, 1))
        return -picked.sum() / part.n_global

    def all_reduce_grads(self, world: int):
        if world == 1:
            return
        grads = [p.grad for p in self.parameters() if p.grad is not None]
        flat = torch.cat([g.reshape(-1) for g in grads])
        dist.all_reduce(flat, group=self.group)
        off = 0
        for g in grads:
            g.copy_(flat[off: off + g.numel()].view_as(g))
            off += g.numel()

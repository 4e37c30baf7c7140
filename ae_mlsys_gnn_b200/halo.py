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
* Two ways to move the rows (``exchange=`` of the model):
  "peer" (GPUs of one node): the owner stores the rows straight into the halo region of the
  receiver's buffer through peer-mapped pointers (``peer.py``, gnn_halo_push: one kernel, plain
  stores over NVLink), then a one-element all-reduce on the same stream orders "every rank's
  stores are complete" before the consumer kernel.  Every exchange point of the model owns two
  buffers used in turn, so a rank can never overwrite rows a slower peer still reads: between
  two uses of the same buffer lies the completion all-reduce of the use in between.
  "nccl": gather into a send buffer + ``all_to_all_single`` (also what the gloo tests run).
"""
from __future__ import annotations

import dataclasses
import math
import os
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
    # for the peer-store exchange: the halo size of EVERY rank, and for every destination rank q
    # the row of q's halo region at which this rank's rows start (what q receives from the
    # ranks before this one)
    halo_sizes: list = None
    dst_off: list = None
    send_idx32: torch.Tensor = None  # send_idx as int32 (kernel argument)
    # Whether ANY rank has rows to receive.  Every rank derives it from the replicated global
    # graph, so all ranks agree on whether the collective of this plan is issued at all: a rank
    # with nothing to send or receive itself (an empty block, only isolated nodes) still joins.
    active: bool = True
    # host copy of send_idx and the ranges already looked up in it (for pushing a row block early)
    send_host: object = None
    range_cache: dict = dataclasses.field(default_factory=dict)

    @property
    def n_halo(self) -> int:
        return int(sum(self.recv_splits))

    def ranges(self, lo: int, hi: int):
        """For every destination rank q, (begin, count) of the part of its group of ``send_idx`` whose
        rows lie in [lo, hi) -- the groups are ascending, so the part is contiguous."""
        got = self.range_cache.get((lo, hi))
        if got is None:
            import numpy as np

            if self.send_host is None:
                self.send_host = self.send_idx.detach().cpu().numpy()
            begs, cnts, pos = [], [], 0
            for c in self.send_splits:
                grp = self.send_host[pos: pos + c]
                a, b = int(np.searchsorted(grp, lo, "left")), int(np.searchsorted(grp, hi, "left"))
                begs.append(pos + a)
                cnts.append(b - a)
                pos += c
            got = self.range_cache[(lo, hi)] = (begs, cnts)
        return got


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
                "fwd_send": self.fwd.send_idx32, "bwd_send": self.bwd.send_idx32}

    def with_index_tensors(self, d: dict) -> "HaloPartition":
        return dataclasses.replace(
            self, row_ptr=d["row_ptr"], col_ind=d["col_ind"], col_ptr=d["col_ptr"], row_ind=d["row_ind"],
            rs_ptr=d["rs_ptr"], rs_pos=d["rs_pos"],
            fwd=dataclasses.replace(self.fwd, send_idx=d["fwd_send"], send_idx32=d["fwd_send"]),
            bwd=dataclasses.replace(self.bwd, send_idx=d["bwd_send"], send_idx32=d["bwd_send"]))


def _outside(ids: torch.Tensor, lo: int, hi: int) -> torch.Tensor:
    """Sorted unique global ids of ``ids`` that lie outside [lo, hi)."""
    u = torch.unique(ids.long())
    return u[(u < lo) | (u >= hi)]


def _plan_device(ptr: torch.Tensor, idx: torch.Tensor, bounds: list, rank: int, world: int):
    """``_plan`` for a graph on a GPU, with the library's own kernels: one pass over the edges marks
    what every block references outside itself, a scan turns the marks into positions (which give
    every count and offset of the plans), a compaction lists the ids, a last kernel remaps this
    block's ids.  One small device-to-host copy."""
    from .operators import graph_build as gb

    dev = idx.device
    n = ptr.numel() - 1
    lo, hi = bounds[rank], bounds[rank + 1]
    positions, needs = gb.halo_needs(ptr, idx, bounds)
    bd = torch.tensor(bounds, dtype=torch.long, device=dev)
    at = (torch.arange(world, device=dev)[:, None] * n + bd[None, :]).reshape(-1)
    fetch = torch.cat([positions[at].long(), ptr[bd[[rank, rank + 1]]].long()]).tolist()
    table = [fetch[q * (world + 1): (q + 1) * (world + 1)] for q in range(world)]  # table[q][r]: needs of q below bounds[r]
    e0, e1 = fetch[-2], fetch[-1]
    halo_sizes = [table[q][world] - table[q][0] for q in range(world)]
    recv_splits = [table[rank][r + 1] - table[rank][r] for r in range(world)]
    send_splits = [0 if q == rank else table[q][rank + 1] - table[q][rank] for q in range(world)]
    dst_off = [0 if q == rank else table[q][rank] - table[q][0] for q in range(world)]
    parts = [needs[table[q][rank]: table[q][rank + 1]] for q in range(world) if q != rank]
    send32 = (torch.cat(parts) - lo).to(torch.int32).contiguous() if parts else \
        torch.zeros(0, dtype=torch.int32, device=dev)
    local_ptr = (ptr[lo: hi + 1] - e0).to(torch.int32).contiguous()
    ext = gb.halo_remap(idx[e0:e1].contiguous(), lo, hi, positions, rank, n)
    plan = ExchangePlan(send32.long(), send_splits, recv_splits, active=any(h > 0 for h in halo_sizes),
                        halo_sizes=halo_sizes, dst_off=dst_off, send_idx32=send32)
    return plan, local_ptr, ext


def _plan(ptr: torch.Tensor, idx: torch.Tensor, bounds: list, rank: int, world: int):
    """Exchange plan and remapped ids for the segment array (ptr, idx) of a square graph whose
    segments AND ids are global node ids: rank r works on segments [bounds[r], bounds[r+1])."""
    if idx.is_cuda and ptr.dtype == torch.int32 and idx.dtype == torch.int32:
        return _plan_device(ptr.contiguous(), idx.contiguous(), bounds, rank, world)
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
    halo_sizes = [int(t.numel()) for t in needs]
    dst_off = []
    for q in range(world):
        if q == rank or world == 1:
            dst_off.append(0)
        else:  # rows of q's halo owned by the ranks before this one
            dst_off.append(int((needs[q] < lo).sum().item()))
    # local segments and ids in the extended space [own | halo]
    e0, e1 = int(p[lo].item()), int(p[hi].item())
    local_ptr = (p[lo: hi + 1] - e0).to(torch.int32).contiguous()
    v = idx[e0:e1].long()
    own = (v >= lo) & (v < hi)
    ext = torch.where(own, v - lo, (hi - lo) + torch.searchsorted(mine, v))
    active = any(int(t.numel()) > 0 for t in needs)
    plan = ExchangePlan(send_idx.contiguous(), send_splits, recv_splits, active=active, halo_sizes=halo_sizes,
                        dst_off=dst_off, send_idx32=send_idx.to(torch.int32).contiguous())
    return plan, local_ptr, ext.to(torch.int32).contiguous()


def build_halo_partition(row_ptr, col_ind, col_ptr, row_ind, rank: int, world: int,
                         bounds: list | None = None) -> HaloPartition:
    """Cuts the global CSR (row_ptr, col_ind) and CSC (col_ptr, row_ind) of a square graph into
    rank ``rank``'s block and builds both exchange plans.  Every rank calls it with the same
    global graph (the plans of the peers are derived from it, no communication)."""
    if bounds is None:
        if row_ptr.is_cuda and row_ptr.dtype == torch.int32:
            from .operators.graph_build import edge_balanced_bounds as device_bounds

            bounds = device_bounds(row_ptr.contiguous(), world)
        else:
            bounds = edge_balanced_bounds(row_ptr, world)
    fwd, rp, ci = _plan(row_ptr, col_ind, bounds, rank, world)
    bwd, cp, ri = _plan(col_ptr, row_ind, bounds, rank, world)
    n_local = bounds[rank + 1] - bounds[rank]
    rs_ptr, rs_pos = _transposed_index(ri, 0, n_local + bwd.n_halo)
    return HaloPartition(rank, world, bounds, rp, ci, cp, ri, rs_ptr, rs_pos, fwd, bwd)


# ---------------------------------------------------------------------------------------------
# exchanges

def halo_exchange(x: torch.Tensor, plan: ExchangePlan, n_local: int, group=None, async_op: bool = False):
    """(n_local, ...) per-node rows -> (n_local + n_halo, ...) [own rows | rows of the halo] with
    one all-to-all.  Returns (extended tensor, work or None)."""
    x = x.contiguous()
    if not plan.active:  # no rank references a row outside its block: no collective anywhere
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
    if not plan.active:
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


class NcclExchange:
    """Moves halo rows with ``all_to_all_single`` (any backend of torch.distributed).

    Protocol of both exchange classes: ``open`` hands out the extended tensors [own | halo] of
    one exchange point, the caller fills rows [0, n_local) (ideally the producing kernel writes
    there directly), ``push`` moves those rows into the other ranks' halo regions and returns
    once everything enqueued afterwards may read the halo rows.  ``exchange`` = open + copy +
    push for tensors that already exist."""

    def __init__(self, part: "HaloPartition", group=None, small_group=None):
        self.group, self.small_group = group, small_group

    def open(self, key, tails, plan: ExchangePlan, n_local: int, device):
        rows = n_local + (plan.n_halo if plan.active else 0)
        return [torch.empty((rows,) + tuple(t), dtype=torch.float32, device=device) for t in tails]

    def push(self, key, exts, plan: ExchangePlan, n_local: int):
        if not plan.active:
            return
        pending = []
        for i, ext in enumerate(exts):  # the first, wide tensor on the main communicator, the rest on the second
            send = ext[:n_local].index_select(0, plan.send_idx)
            work = dist.all_to_all_single(ext[n_local:], send, output_split_sizes=plan.recv_splits,
                                          input_split_sizes=plan.send_splits,
                                          group=self.group if i == 0 else self.small_group,
                                          async_op=(i == 0 and len(exts) > 1))
            if work is not None and i == 0 and len(exts) > 1:
                pending.append((work, send))
        for work, _ in pending:
            work.wait()

    def exchange(self, key, tensors, plan: ExchangePlan, n_local: int):
        exts = self.open(key, [t.shape[1:] for t in tensors], plan, n_local, tensors[0].device)
        for e, t in zip(exts, tensors):
            e[:n_local] = t[:n_local]
        self.push(key, exts, plan, n_local)
        return exts


class PeerStoreExchange(NcclExchange):
    """Moves halo rows with one store kernel per tensor into peer-mapped buffers (see the module
    docstring).  ``open`` / ``push`` are collective and must be called by every rank with the same
    sequence of keys; the buffers of a key are allocated at its first use."""

    def __init__(self, part: "HaloPartition", group=None, small_group=None):
        self.part = part
        self.group, self.small_group = group, small_group
        self.rank, self.world = part.rank, part.world
        self.n_locals = [part.bounds[q + 1] - part.bounds[q] for q in range(part.world)]
        self._slots = {}   # key -> [buffers of use 0, buffers of use 1, next use]
        self._open = {}    # key -> buffers handed out by the last open()
        self._early = {}   # key -> indices of the tensors whose rows push_rows() has already moved
        self._flag = None
        self._side = None

    # -- overridable pieces (a CPU stand-in for tests replaces them) -------------------------
    def _alloc(self, nbytes, device):
        from .peer import PeerBuffer

        return PeerBuffer(nbytes, device, self.group)

    def _push(self, ext, plan, buf, row_bytes, n_local):
        """Stores the rows of ``ext`` (this rank's buffer) listed in the plan into the peers' buffers."""
        from .peer import halo_push

        offs = [0]
        for c in plan.send_splits:
            offs.append(offs[-1] + int(c))
        dst = [0 if q == self.rank or plan.send_splits[q] == 0
               else buf.ptrs[q] + (self.n_locals[q] + plan.dst_off[q]) * row_bytes for q in range(self.world)]
        halo_push(ext, plan.send_idx32, offs, dst, 0, 0)

    def _push_rows(self, ext, plan, buf, row_bytes, lo, hi):
        """The part of ``_push`` whose rows lie in [lo, hi)."""
        from .peer import halo_push_ranges

        begs, cnts = plan.ranges(lo, hi)
        pos, dst = 0, []
        for q, c in enumerate(plan.send_splits):
            dst.append(0 if cnts[q] == 0 else
                       buf.ptrs[q] + (self.n_locals[q] + plan.dst_off[q] + begs[q] - pos) * row_bytes)
            pos += c
        halo_push_ranges(ext, plan.send_idx32, begs, cnts, dst)

    def _side_stream(self, device):
        """(main, side) streams for pushes that overlap their producer; (None, None) where streams do not apply."""
        if torch.device(device).type != "cuda":
            return None, None
        if self._side is None:
            self._side = torch.cuda.Stream(device=device)
        return torch.cuda.current_stream(device), self._side

    def _complete(self, device):
        """Every rank's push kernels are complete before anything enqueued after this call runs."""
        if self._flag is None:
            self._flag = torch.zeros(1, dtype=torch.float32, device=device)
        dist.all_reduce(self._flag, group=self.small_group)

    # ----------------------------------------------------------------------------------------
    def open(self, key, tails, plan: ExchangePlan, n_local: int, device):
        if not plan.active:
            return [torch.empty((n_local,) + tuple(t), dtype=torch.float32, device=device) for t in tails]
        rows_max = max(n + h for n, h in zip(self.n_locals, plan.halo_sizes))
        row_bytes = [4 * math.prod(t) for t in tails]
        slot = self._slots.get(key)
        if slot is None:
            slot = [[self._alloc(rows_max * rb, device) for rb in row_bytes] for _ in range(2)] + [0]
            self._slots[key] = slot
        bufs = slot[slot[2]]
        slot[2] ^= 1
        for buf, rb in zip(bufs, row_bytes):
            if rows_max * rb > buf.nbytes:
                raise ValueError(f"exchange {key!r}: rows changed width since its buffers were allocated")
        self._open[key] = (bufs, row_bytes)
        rows = n_local + plan.n_halo
        return [buf.view((rows,) + tuple(t), torch.float32) for buf, t in zip(bufs, tails)]

    def push_rows(self, key, i: int, ext, plan: ExchangePlan, lo: int, hi: int):
        """Moves the rows [lo, hi) of tensor ``i`` of the exchange point now, on a second stream that
        waits for what the caller has enqueued so far: a producer that fills the tensor block by block
        (a GEMM over row blocks) overlaps the transfer of one block with the computation of the next.
        Every row of the tensor must be covered by such calls before ``push``, which then skips it."""
        if not plan.active:
            return
        bufs, row_bytes = self._open[key]
        main, side = self._side_stream(ext.device)
        if side is not None:
            side.wait_stream(main)
            with torch.cuda.stream(side):
                self._push_rows(ext, plan, bufs[i], row_bytes[i], lo, hi)
        else:
            self._push_rows(ext, plan, bufs[i], row_bytes[i], lo, hi)
        self._early.setdefault(key, set()).add(i)

    def push(self, key, exts, plan: ExchangePlan, n_local: int):
        if not plan.active:
            return
        bufs, row_bytes = self._open.pop(key)
        early = self._early.pop(key, ())
        for i, (ext, buf, rb) in enumerate(zip(exts, bufs, row_bytes)):
            if i not in early:
                self._push(ext, plan, buf, rb, n_local)
        if early:
            main, side = self._side_stream(exts[0].device)
            if side is not None:
                main.wait_stream(side)
        self._complete(exts[0].device)

    def close(self):
        for slot in self._slots.values():
            for use in slot[:2]:
                for buf in use:
                    buf.close()
        self._slots = {}


def make_exchange(kind, part, group=None, small_group=None):
    if kind in (None, "nccl", "halo"):
        return NcclExchange(part, group, small_group)
    if kind == "peer":
        return PeerStoreExchange(part, group, small_group)
    if callable(kind):
        return kind(part, group, small_group)
    raise ValueError(f"unknown exchange {kind!r}")


class HaloGATFunction(torch.autograd.Function):
    """Scores + fused GAT aggregation (+ optional ELU) on a halo partition, one autograd node.
    ``h`` (n_local rows) is the front of ``h_ext`` ([own | halo] rows).  ``ac_ext`` is the buffer of
    the extended source scores opened together with ``h_ext``; None means the halo rows of ``h_ext``
    are already there (the caller projected the halo's inputs) and only the scores travel.  ``exch`` moves the rows; ``key`` names this layer's exchange points."""

    @staticmethod
    def forward(ctx, h, attn_l, attn_r, part: HaloPartition, slope, kernels, exch, key, activation, h_ext,
                ac_ext):
        halo_ready = ac_ext is None
        n = part.n_local
        attn_l, attn_r = attn_l.contiguous(), attn_r.contiguous()
        H, Fo = h.shape[1], h.shape[2]
        attn_row, attn_col = kernels.scores_forward(h, attn_l, attn_r)
        if halo_ready:
            (ac_ext,) = exch.exchange((key, "fwd_attn"), [attn_col], part.fwd, n)
        else:  # h_ext and ac_ext came from one exch.open((key, "fwd"), ...): one push, one completion
            ac_ext[:n] = attn_col
            exch.push((key, "fwd"), [h_ext, ac_ext], part.fwd, n)
        act = None
        if activation == "elu" and hasattr(kernels, "forward_act"):  # ELU stored by the forward kernel
            out, act, edge_max, edge_sum = kernels.forward_act(attn_row, ac_ext, part.row_ptr, part.col_ind,
                                                               slope, h_ext)
        else:
            out = h.new_empty((n, H, Fo))
            edge_max = h.new_empty((n, H))
            edge_sum = h.new_empty((n, H))
            kernels.forward_part(attn_row, ac_ext, part.row_ptr, part.col_ind, slope, h_ext, out, edge_max,
                                 edge_sum, False, True)
            if activation == "elu":
                act = F.elu(out)
        ctx.save_for_backward(attn_row, attn_col, h, edge_max, edge_sum, attn_l, attn_r, out)
        ctx.part, ctx.slope, ctx.kernels = part, slope, kernels
        ctx.exch, ctx.key, ctx.activation = exch, key, activation
        return out if act is None else act

    @staticmethod
    def backward(ctx, grad_out):
        attn_row, attn_col, h, edge_max, edge_sum, attn_l, attn_r, out = ctx.saved_tensors
        part, slope, kernels, exch = ctx.part, ctx.slope, ctx.kernels, ctx.exch
        n = part.n_local
        H, Fo = h.shape[1], h.shape[2]
        grad_out = grad_out.contiguous()
        # the rows the column pass gathers (gradient w.r.t. the pre-activation output, per-row
        # record) are produced straight into the front of the exchange buffers
        gout_ext, rp_ext = exch.open((ctx.key, "bwd"), [(H, Fo), (4, H)], part.bwd, n, h.device)
        direct = getattr(kernels, "writes_into", False)
        if ctx.activation == "elu":  # the ELU backward rides on the node-wise per-row pack
            if direct:
                kernels.backward_pack_elu(out, grad_out, attn_row, edge_max, edge_sum, grad_pre=gout_ext,
                                          rowpack=rp_ext)
            else:
                g, rp = kernels.backward_pack_elu(out, grad_out, attn_row, edge_max, edge_sum)
                gout_ext[:n], rp_ext[:n] = g, rp
        else:
            gout_ext[:n] = grad_out
            if direct:
                kernels.backward_pack(out, grad_out, attn_row, edge_max, edge_sum, rowpack=rp_ext)
            else:
                rp_ext[:n] = kernels.backward_pack(out, grad_out, attn_row, edge_max, edge_sum)
        exch.push((ctx.key, "bwd"), [gout_ext, rp_ext], part.bwd, n)
        gh = h.new_empty((n, H, Fo))
        gac = h.new_empty((n, H))
        edge_grad = kernels.backward_col_edges_part(slope, part.col_ptr, part.row_ind, h, attn_col, rp_ext,
                                                    gout_ext, gh, gac, False)
        gar_ext = kernels.backward_row_sum(part.rs_ptr, part.rs_pos, edge_grad)
        gar = halo_return_sum(gar_ext, part.bwd, n, exch.small_group)
        gl, gr = kernels.scores_backward(h, attn_l, attn_r, gar, gac, gh)
        return gh, gl.view_as(attn_l), gr.view_as(attn_r), None, None, None, None, None, None, None, None


class HaloGATConv(_GATBase):
    """GATConv (same parameters, same state_dict) on a HaloPartition.

    ``recompute_projection``: when the layer widens its input at least four times ("auto", the
    default; e.g. 100 -> 512) the narrow inputs of the halo are exchanged and projected on the
    receiving rank instead of exchanging the wide projected rows."""

    OVERLAP_MIN_ROWS = 16384  # per block: below this a block's GEMM no longer fills the GPU
    OVERLAP_MIN_WIDTH = 128   # floats per row: narrow rows travel in no time

    def __init__(self, in_feats, out_feats, num_heads, negative_slope=0.2, kernels=_CudaKernels,
                 recompute_projection="auto", activation=None, key=0, overlap_blocks=1, side_weight_grads=False):
        super().__init__(in_feats, out_feats, num_heads, negative_slope)
        self.kernels = kernels
        # Both options move work beside the main stream (see forward); measured on 2 and 4 GPUs they
        # change the epoch by less than the run-to-run spread, because a GEMM and a push kernel that
        # run at the same time slow each other down by about what the overlap hides: off by default.
        self.overlap_blocks = int(os.environ.get("GNN_B200_OVERLAP_BLOCKS", overlap_blocks))
        self.side_weight_grads = bool(int(os.environ.get("GNN_B200_SIDE_WEIGHT_GRADS", int(side_weight_grads))))
        self.recompute_projection = recompute_projection
        self.activation = activation
        self.key = key

    def _recompute(self, part) -> bool:
        if part.world == 1:
            return False
        if self.recompute_projection == "auto":
            return 4 * self.in_feats <= self.out_feats * self.num_heads
        return bool(self.recompute_projection)

    def forward(self, part: HaloPartition, feat, exch):
        n, H, Fo = part.n_local, self.num_heads, self.out_feats
        W, attn_l, attn_r = self.W, self.attn_l, self.attn_r
        # One head of odd width (the 47-wide output layer): zero weight columns up to the next multiple of
        # 4 floats give the projected rows, the rows that travel and their gradients a 16-byte pitch (128-bit
        # accesses in the sparse kernels and in the push); the extra columns are zero and are cut off below.
        pad = (-Fo) % 4 if H == 1 else 0
        if pad:
            W = F.pad(W, (0, pad))
            attn_l, attn_r = F.pad(attn_l, (0, pad)), F.pad(attn_r, (0, pad))
            Fo = Fo + pad
        out = self._forward(part, feat, exch, W, attn_l, attn_r, n, H, Fo)
        return out[:, :, : Fo - pad] if pad else out

    def _forward(self, part, feat, exch, W, attn_l, attn_r, n, H, Fo):
        if self._recompute(part):
            # the narrow inputs travel first; both projections write into one [own | halo] tensor
            with torch.no_grad():
                (x_ext,) = exch.exchange((self.key, "fwd_x"), [feat.detach()], part.fwd, n)
            h_ext = feat.new_empty((x_ext.shape[0], H, Fo))
            with dense.side_weight_grads(self.side_weight_grads and part.world > 1):  # X^T G beside the next exchange
                h = dense.project(feat, W, out=dense.OutRows(h_ext, 0)).view(-1, H, Fo)
            if x_ext.shape[0] > n:
                with torch.no_grad():
                    dense.project(x_ext[n:], W.detach(), out=dense.OutRows(h_ext, n))
            ac_ext = None  # only the scores of the halo are still to be exchanged
        else:
            h_ext, ac_ext = exch.open((self.key, "fwd"), [(H, Fo), (H,)], part.fwd, n, feat.device)
            # wide rows: the projection runs block by block and every finished block of rows starts
            # travelling to the ranks that need it while the next block is computed
            blocks = after = None
            if (self.overlap_blocks > 1 and hasattr(exch, "push_rows") and part.fwd.active
                    and n >= self.overlap_blocks * self.OVERLAP_MIN_ROWS and H * Fo >= self.OVERLAP_MIN_WIDTH):
                step = -(-n // self.overlap_blocks)
                step = -(-step // 128) * 128  # whole GEMM tiles
                blocks = [(lo, min(lo + step, n)) for lo in range(0, n, step)]
                key = (self.key, "fwd")

                def after(lo, hi):
                    exch.push_rows(key, 0, h_ext, part.fwd, lo, hi)
            with dense.side_weight_grads(self.side_weight_grads and part.world > 1):
                h = dense.project(feat, W, out=dense.OutRows(h_ext, 0), row_blocks=blocks,
                                  after_block=after).view(-1, H, Fo)
        return HaloGATFunction.apply(h, attn_l, attn_r, part, self.negative_slope,
                                     self.kernels, exch, self.key, self.activation, h_ext, ac_ext)


class HaloGAT(nn.Module):
    """models.GAT on a halo partition: identical parameters; inputs / outputs hold the rank's
    n_local rows.  ``exchange``: "peer" (stores into peer-mapped buffers, GPUs of one node),
    "nccl" (all-to-all; any backend), or a factory ``f(part, group, small_group)``.
    ``small_group`` is a second communicator over the same ranks for the small per-node tensors
    (created here when torch.distributed is initialised)."""

    def __init__(self, in_dim, hidden, heads, num_classes, out_heads=1, negative_slope=0.2,
                 activation="elu", kernels=_CudaKernels, group=None, small_group=None, exchange="nccl"):
        super().__init__()
        if (small_group is None and dist.is_available() and dist.is_initialized()
                and dist.get_world_size() > 1):
            small_group = dist.new_group(ranks=list(range(dist.get_world_size())))
        if isinstance(hidden, int):
            hidden = [hidden] * len(heads)
        dims_in = [in_dim] + [h * f for h, f in zip(heads, hidden)]
        self.gat_layers = nn.ModuleList(
            [HaloGATConv(dims_in[i], hidden[i], heads[i], negative_slope, kernels, activation=activation, key=i)
             for i in range(len(heads))])
        self.gat_layers.append(
            HaloGATConv(dims_in[-1], num_classes, out_heads, negative_slope, kernels, key=len(heads)))
        self.activation = activation
        self.group, self.small_group = group, small_group
        self.exchange = exchange
        self._exch = None  # created for the first partition seen

    def exchanger(self, part: HaloPartition):
        # (an end-to-end step hands in the same partition with freshly uploaded index tensors:
        # the plan's sizes are what the buffers depend on, and those do not change)
        if self._exch is None:
            self._exch = make_exchange(self.exchange, part, self.group, self.small_group)
        return self._exch

    def forward(self, part: HaloPartition, inputs):
        exch = self.exchanger(part)
        h = inputs
        for layer in self.gat_layers[:-1]:
            h = layer(part, h, exch).flatten(1)
        return self.gat_layers[-1](part, h, exch).mean(1)

    def close(self):
        if self._exch is not None and hasattr(self._exch, "close"):
            self._exch.close()
        self._exch = None

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

"""Peer-mapped device buffers of the ranks of one node, and the halo push over them.

The reference is single-GPU; nothing here has a counterpart in it.  ``PeerBuffer`` is one
allocation of the same size on every rank of a process group, mapped into every other rank's
address space (gnn_peer_alloc / gnn_peer_open, i.e. CUDA IPC handles exchanged once through
the process group).  ``halo_push`` is the kernel that stores rows of a local tensor into the
peers' buffers (ordinary stores over NVLink; no TMA, no multicast).  torch only owns the
views: the memory is the library's, wrapped through ``__cuda_array_interface__``.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _capi as capi

HANDLE_BYTES = 64
MAX_PEERS = 8

_TYPESTR = {torch.float32: "<f4", torch.int32: "<i4", torch.uint8: "|u1"}


class _Span:
    """A typed window of raw device memory for torch.as_tensor."""

    def __init__(self, ptr: int, shape, dtype, owner):
        self.__cuda_array_interface__ = {"shape": tuple(int(s) for s in shape), "typestr": _TYPESTR[dtype],
                                         "data": (int(ptr), False), "version": 2}
        self._owner = owner  # keeps the allocation alive as long as any view exists


class PeerBuffer:
    """``nbytes`` of device memory on every rank of ``group``; ``ptrs[q]`` is rank q's
    allocation as seen from this process (``ptrs[rank]`` the local one).  Collective: every
    rank of the group must construct it at the same point of its program."""

    def __init__(self, nbytes: int, device: torch.device, group=None):
        self.device = torch.device(device)
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > MAX_PEERS:
            raise ValueError(f"at most {MAX_PEERS} ranks can share peer buffers")
        self.nbytes = int(max(nbytes, 256))
        ptr = C.c_void_p()
        handle = (C.c_ubyte * HANDLE_BYTES)()
        with torch.cuda.device(self.device):
            capi.check(capi.lib().gnn_peer_alloc(self.nbytes, C.byref(ptr), handle), "gnn_peer_alloc")
        self._own = int(ptr.value)
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.ptrs = []
        self._opened = []
        for q, h in enumerate(handles):
            if q == self.rank:
                self.ptrs.append(self._own)
                continue
            p = C.c_void_p()
            buf = (C.c_ubyte * HANDLE_BYTES).from_buffer_copy(h)
            with torch.cuda.device(self.device):
                capi.check(capi.lib().gnn_peer_open(buf, C.byref(p)), "gnn_peer_open")
            self.ptrs.append(int(p.value))
            self._opened.append(int(p.value))

    def view(self, shape, dtype=torch.float32, byte_offset: int = 0) -> torch.Tensor:
        """The local allocation (from ``byte_offset``) as a tensor of ``shape``."""
        numel = 1
        for s in shape:
            numel *= int(s)
        if byte_offset + numel * torch.empty((), dtype=dtype).element_size() > self.nbytes:
            raise ValueError("view exceeds the peer buffer")
        if numel == 0:
            return torch.empty(tuple(shape), dtype=dtype, device=self.device)
        return torch.as_tensor(_Span(self._own + byte_offset, shape, dtype, self), device=self.device)

    def close(self, collective: bool = True):
        """Unmaps the peers' allocations, waits for every rank to have done so (``collective``:
        every rank calls close at the same point), frees the own one."""
        if self._own is None:
            return
        torch.cuda.synchronize(self.device)
        with torch.cuda.device(self.device):
            for p in self._opened:
                capi.lib().gnn_peer_close(p)
            self._opened = []
            if collective and dist.is_initialized():
                dist.barrier(group=self.group)
            capi.lib().gnn_peer_free(self._own)
        self._own = None


def halo_push(x: torch.Tensor, send_idx: torch.Tensor, send_off: list, dst_ptrs: list, own_dst_ptr: int,
              n_own: int) -> None:
    """Stores row ``send_idx[i]`` of ``x`` (float32, rows contiguous) to ``dst_ptrs[q] + (i - send_off[q]) * row``
    for the i of rank q's group, and rows [0, n_own) of ``x`` to ``own_dst_ptr`` (0: skip).  ``dst_ptrs`` are
    raw device addresses (mapped peer memory), already advanced to where this rank's rows go."""
    capi.require(x, torch.float32, "x")
    dev = x.device
    world = len(dst_ptrs)
    row = 1
    for s in x.shape[1:]:
        row *= int(s)
    if send_idx.numel():
        capi.require(send_idx, torch.int32, "send_idx", 1, dev)
    off = (C.c_int64 * (world + 1))(*[int(v) for v in send_off])
    dst = (C.c_void_p * world)(*[C.c_void_p(int(p)) if p else C.c_void_p(None) for p in dst_ptrs])
    with torch.cuda.device(dev):
        capi.call("gnn_halo_push", capi.ptr(x), row, capi.ptr(send_idx) if send_idx.numel() else None, off, dst,
                  world, own_dst_ptr if own_dst_ptr else None, int(n_own), capi.stream_ptr(dev))


def halo_push_ranges(x: torch.Tensor, send_idx: torch.Tensor, begs: list, cnts: list, dst_ptrs: list) -> None:
    """``halo_push`` for part of a send list: rank q receives rows ``send_idx[begs[q] : begs[q] + cnts[q]]``
    of ``x`` at ``dst_ptrs[q]`` onwards (the caller advances the pointer to where the range lands)."""
    capi.require(x, torch.float32, "x")
    dev = x.device
    world = len(dst_ptrs)
    row = 1
    for s in x.shape[1:]:
        row *= int(s)
    if sum(int(c) for c in cnts) == 0:
        return
    capi.require(send_idx, torch.int32, "send_idx", 1, dev)
    beg = (C.c_int64 * world)(*[int(v) for v in begs])
    cnt = (C.c_int64 * world)(*[int(v) for v in cnts])
    dst = (C.c_void_p * world)(*[C.c_void_p(int(p)) if p else C.c_void_p(None) for p in dst_ptrs])
    with torch.cuda.device(dev):
        capi.call("gnn_halo_push_ranges", capi.ptr(x), row, capi.ptr(send_idx), beg, cnt, dst, world, None, 0,
                  capi.stream_ptr(dev))


def probe(device, group=None) -> bool:
    """Whether peer-mapped buffers work between the ranks of ``group`` on this node: every rank
    stores one row into every other rank's buffer and checks what it received.  Collective; all
    ranks return the same answer (False if any rank failed at any step)."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    ok = torch.ones(1, dtype=torch.float32, device=device)
    buf = None
    try:
        buf = PeerBuffer(16 * world, device, group)
    except Exception:
        ok.zero_()
    dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
    if ok.item() < 1:  # some rank could not allocate or map: no rank pushes
        if buf is not None:
            buf.close(collective=False)  # the ranks that failed hold no buffer to close
        return False
    try:
        mine = torch.full((1, 4), float(rank + 1), dtype=torch.float32, device=device)
        own = buf.view((world, 4))
        own.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=group)
        idx = torch.zeros(world - 1, dtype=torch.int32, device=device)
        offs, dst = [0], []
        for q in range(world):
            offs.append(offs[-1] + (0 if q == rank else 1))
            dst.append(0 if q == rank else buf.ptrs[q] + 16 * rank)
        halo_push(mine, idx, offs, dst, 0, 0)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)
        got = own[:, 0].tolist()
        for q in range(world):
            if q != rank and got[q] != float(q + 1):
                ok.zero_()
    except Exception:
        ok.zero_()
    dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
    buf.close()
    return bool(ok.item() >= 1)

"""Dense node-feature projection on the tensor cores (no counterpart module in the
reference, which calls torch.matmul / nn.Linear: layers/gatconv_layer.py:50,
layers/edgeconv_layer.py:37-38, layers/gmmconv_layer.py:68).

``matmul_tf32x3(x, w)`` computes ``x @ w`` with the error-compensated 3xTF32 tcgen05
kernel (fp32-level accuracy); its backward uses the same kernel for grad_x and, with the
node axis as the reduction axis, for grad_w.  ``project`` picks it whenever the shape is
supported; the shapes it does not take (fewer rows than one tile pays for, non-fp32) go to
the framework's fp32 GEMM, and every such call is counted (``fallback_calls``) so that a
run can report how much of its dense work left the tensor-core kernel.

Error contract of the kernel: every barrier wait inside it is bounded; when one expires the
CTA gives up and sets a status word instead of hanging, and the output of that launch is
incomplete.  ``check_status()`` reads the word (a device synchronisation) and raises; call it
wherever the step synchronises anyway (after reading the loss, at the end of a timed loop).
"""
from __future__ import annotations

import torch

from .. import _capi as capi

F32 = torch.float32
enabled = True  # set False to force the cuBLAS fp32 path

_status: dict[int, torch.Tensor] = {}
_fallbacks = {"calls": 0}


# ---- weight gradients off the critical path -------------------------------------------------
# The weight gradient of a projection (X^T G) is needed only when the optimizer runs, while
# grad_x is what the rest of the backward pass waits for.  Inside ``side_weight_grads()`` the
# projections record that their weight-gradient GEMM may run on a second stream: the backward
# then enqueues it there, after grad_x, and the stream that ran the backward waits for all of
# them when the backward pass ends (an engine callback), so callers see ordinary semantics.
# Used by the partitioned model, where the GEMM fills the time in which the next layer's halo
# exchange keeps the SMs nearly idle.
_side = {"on": False, "streams": {}, "pending": [], "queued": False}


class side_weight_grads:
    def __init__(self, on: bool = True):
        self.on = on

    def __enter__(self):
        self.prev = _side["on"]
        _side["on"] = self.on
        return self

    def __exit__(self, *exc):
        _side["on"] = self.prev


def _side_stream(dev: torch.device) -> "torch.cuda.Stream":
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    st = _side["streams"].get(idx)
    if st is None:
        st = torch.cuda.Stream(device=dev)
        _side["streams"][idx] = st
    return st


def join_weight_grads() -> None:
    """The current stream waits for every weight-gradient GEMM enqueued on the second stream."""
    _side["queued"] = False
    pending, _side["pending"] = _side["pending"], []
    for dev, ev in pending:
        torch.cuda.current_stream(dev).wait_event(ev)


def fallback_calls() -> int:
    """Dense products that went to the framework GEMM instead of the tensor-core kernel so far."""
    return _fallbacks["calls"]


def _note_fallback():
    _fallbacks["calls"] += 1


def _status_word(dev: torch.device) -> torch.Tensor:
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _status[idx] = t
    return t


def check_status(dev=None) -> None:
    """Synchronises and raises if any GEMM launched so far reported an expired wait."""
    for idx, t in _status.items():
        if dev is not None and torch.device(dev).index not in (None, idx):
            continue
        if int(t.item()) != 0:
            t.zero_()
            raise capi.GnnError("gnn_gemm_tf32x3: a barrier wait expired inside the kernel")


def supported(m: int, n: int, k: int, a: torch.Tensor) -> bool:
    """Whether ``gemm_any_k`` takes an (m, k) x (k, n) product of ``a``'s kind: fp32 on a GPU.
    (The kernel itself wants k % 4 == 0 and 16-byte aligned rows; ``gemm_any_k`` pads.)"""
    k4 = k + (-k) % 4
    return (enabled and a.is_cuda and a.dtype == F32 and m > 0
            and bool(capi.lib().gnn_gemm_tf32x3_supported(m, n, k4)))


class OutRows:
    """Where a product is to be written: rows [start, start + M) of ``base`` (rows, N), e.g. the
    front of a buffer whose remaining rows other ranks fill.  Not a tensor argument on purpose:
    autograd then sees the returned view as an ordinary fresh output of the product."""

    def __init__(self, base: torch.Tensor, start: int = 0):
        self.base, self.start = base, int(start)

    def rows(self, m: int, n: int) -> torch.Tensor:
        width = 1
        for d in self.base.shape[1:]:
            width *= int(d)
        flat = self.base.view(self.base.shape[0], width)
        if flat.shape[1] != n or self.start + m > flat.shape[0] or not flat.is_contiguous():
            raise ValueError("output rows do not fit the given buffer")
        return flat[self.start: self.start + m]


def scores_supported(heads: int, head_w: int) -> bool:
    """Whether the GEMM's epilogue can form the per-head attention scores for this output shape."""
    return bool(capi.lib().gnn_gemm_tf32x3_scores_supported(int(heads), int(head_w)))


def gemm(a: torch.Tensor, b: torch.Tensor, b_is_n_by_k: bool, out: "OutRows | None" = None, scores=None):
    """a (M,K) times b, where b is (K,N) or, with ``b_is_n_by_k``, (N,K).
    ``scores`` = (attn_l, attn_r) of shape (H, F) with H*F == N: also returns the (M, H) dot products
    of every output row's heads with them, formed in the kernel's epilogue -> (out, score_l, score_r)."""
    dev = a.device
    capi.require(a, F32, "a", 2)
    capi.require(b, F32, "b", 2, dev)
    M, K = a.shape
    N = b.shape[0] if b_is_n_by_k else b.shape[1]
    if (b.shape[1] if b_is_n_by_k else b.shape[0]) != K:
        raise ValueError(f"inner dimensions differ: a is {tuple(a.shape)}, b is {tuple(b.shape)}")
    out = torch.empty((M, N), dtype=F32, device=dev) if out is None else out.rows(M, N)
    nbytes = capi.workspace_bytes("gnn_gemm_tf32x3_workspace_bytes", M, N, K)
    ws = capi.workspace(dev, nbytes)
    if scores is None:
        with torch.cuda.device(dev):
            capi.call("gnn_gemm_tf32x3", capi.ptr(a), capi.ptr(b), int(b_is_n_by_k), capi.ptr(out), M, N, K,
                      capi.ptr(ws), ws.numel(), capi.ptr(_status_word(dev)), capi.stream_ptr(dev))
        return out
    al, ar = (capi.require(t, F32, "attn", 2, dev) for t in scores)
    H, Fw = al.shape
    if H * Fw != N or ar.shape != al.shape:
        raise ValueError("attention vectors must be (H, F) with H * F equal to the output width")
    sl = torch.empty((M, H), dtype=F32, device=dev)
    sr = torch.empty((M, H), dtype=F32, device=dev)
    with torch.cuda.device(dev):
        capi.call("gnn_gemm_tf32x3_scores", capi.ptr(a), capi.ptr(b), int(b_is_n_by_k), capi.ptr(out), M, N, K,
                  capi.ptr(al), capi.ptr(ar), H, Fw, capi.ptr(sl), capi.ptr(sr), capi.ptr(ws), ws.numel(),
                  capi.ptr(_status_word(dev)), capi.stream_ptr(dev))
    return out, sl, sr


def gemm_any_k(a: torch.Tensor, b: torch.Tensor, b_is_n_by_k: bool, out: "OutRows | None" = None, scores=None):
    """``gemm`` for any inner dimension: TMA reads rows whose length is a multiple of 4 floats,
    so other lengths (an input width of 602, a gradient with 47 columns) are padded with zero
    columns first -- one copy of ``a``, far cheaper than leaving the product to an fp32 SIMT GEMM."""
    pad = (-a.shape[1]) % 4
    if pad:
        a = torch.nn.functional.pad(a, (0, pad))
        b = torch.nn.functional.pad(b, (0, pad) if b_is_n_by_k else (0, 0, 0, pad))
    a = a.contiguous()
    if a.data_ptr() % 16:  # a view that starts at an odd offset of its storage
        a = a.clone()
    return gemm(a, b.contiguous(), b_is_n_by_k, out, scores)


def gemm_tn(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a^T @ b for a (M,K1), b (M,N1): the weight gradient of a projection."""
    dev = a.device
    capi.require(a, F32, "a", 2)
    capi.require(b, F32, "b", 2, dev)
    M, K1 = a.shape
    if b.shape[0] != M:
        raise ValueError("a and b must have the same number of rows")
    N1 = b.shape[1]
    out = torch.empty((K1, N1), dtype=F32, device=dev)
    nbytes = capi.workspace_bytes("gnn_gemm_tf32x3_tn_workspace_bytes", M, K1, N1)
    ws = capi.workspace(dev, nbytes)
    with torch.cuda.device(dev):
        capi.call("gnn_gemm_tf32x3_tn", capi.ptr(a), capi.ptr(b), capi.ptr(out), M, K1, N1, capi.ptr(ws),
                  ws.numel(), capi.ptr(_status_word(dev)), capi.stream_ptr(dev))
    return out


# below this many rows the transposes + split-K launch cost more than the framework GEMM
TN_MIN_ROWS = 4096


class _MatmulFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, w_is_out_by_in, out=None, row_blocks=None, after_block=None):
        x = x.contiguous()
        w = w.contiguous()
        ctx.save_for_backward(x, w)
        ctx.w_is_out_by_in = w_is_out_by_in
        ctx.side = _side["on"] and x.is_cuda
        if not row_blocks or out is None:
            return gemm_any_k(x, w, w_is_out_by_in, out)
        # one product per block of rows, each written to its rows of ``out``; ``after_block(lo, hi)``
        # runs once a block is enqueued (e.g. to start moving those rows elsewhere)
        n_out = w.shape[0] if w_is_out_by_in else w.shape[1]
        for lo, hi in row_blocks:
            gemm_any_k(x[lo:hi], w, w_is_out_by_in, OutRows(out.base, out.start + lo))
            if after_block is not None:
                after_block(lo, hi)
        return out.rows(x.shape[0], n_out)

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        g = g.contiguous()
        gx = gw = None
        if ctx.needs_input_grad[0]:
            # grad_x = g @ w^T (w given K x N) or g @ w (w given N x K)
            n_out = g.shape[1]
            if supported(g.shape[0], x.shape[1], n_out, g):
                gx = gemm_any_k(g, w, not ctx.w_is_out_by_in)
            else:
                _note_fallback()
                gx = g @ (w if ctx.w_is_out_by_in else w.t())
        if ctx.needs_input_grad[1]:
            def weight_grad():
                if enabled and x.shape[0] >= TN_MIN_ROWS and x.data_ptr() % 16 == 0 and g.data_ptr() % 16 == 0:
                    return gemm_tn(g, x) if ctx.w_is_out_by_in else gemm_tn(x, g)
                _note_fallback()
                return (g.t() @ x) if ctx.w_is_out_by_in else (x.t() @ g)

            if ctx.side:
                dev = g.device
                main, side = torch.cuda.current_stream(dev), _side_stream(dev)
                side.wait_stream(main)  # x, g (and grad_x, enqueued first) are in stream order before it
                with torch.cuda.stream(side):
                    gw = weight_grad()
                    ev = torch.cuda.Event()
                    ev.record(side)
                x.record_stream(side)
                g.record_stream(side)
                gw.record_stream(main)
                _side["pending"].append((dev, ev))
                if not _side["queued"]:  # once per backward pass: join when the pass ends
                    _side["queued"] = True
                    torch.autograd.Variable._execution_engine.queue_callback(join_weight_grads)
            else:
                gw = weight_grad()
        return gx, gw, None, None, None, None


def matmul_tf32x3(x, w, out=None, row_blocks=None, after_block=None):
    """x (M,K) @ w (K,N)."""
    return _MatmulFunction.apply(x, w, False, out, row_blocks, after_block)


def project(x, w, out: "OutRows | None" = None, row_blocks=None, after_block=None):
    """x @ w, on the tensor cores for CUDA fp32 matrices.  ``out``: rows of an existing buffer to
    write the product into (the returned tensor is then that view).  ``row_blocks`` (list of
    (lo, hi) covering the rows, needs ``out``): the product is enqueued block by block and
    ``after_block(lo, hi)`` is called after each, so that a consumer of finished rows (a transfer)
    can start while the next block is computed; the backward is that of the whole product."""
    if x.dim() == 2 and supported(x.shape[0], w.shape[1], w.shape[0], x):
        return matmul_tf32x3(x, w, out, row_blocks, after_block)
    _note_fallback()
    res = torch.matmul(x, w)
    if out is not None:
        dst = out.rows(res.shape[0], res.shape[1])
        dst.copy_(res.detach())
    if row_blocks and after_block is not None:
        for lo, hi in row_blocks:
            after_block(lo, hi)
    return res


def linear(x, weight):
    """nn.Linear without bias: x (M,K) @ weight(N,K)^T."""
    if x.dim() == 2 and supported(x.shape[0], weight.shape[0], weight.shape[1], x):
        return _MatmulFunction.apply(x, weight, True)
    _note_fallback()
    return torch.nn.functional.linear(x, weight)

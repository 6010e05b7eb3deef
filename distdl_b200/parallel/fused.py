"""Fused compute + collective GEMMs of the native backend (sequence-parallel
tensor parallelism): all-gather -> GEMM and GEMM -> reduce-scatter in ONE
kernel each, traffic issued from inside the kernel over peer-mapped memory
(see ``csrc/gemm_fused.cu``).  They stand where the reference runs
``ncclAllGather`` + permute copy + ``F.linear`` and ``F.linear`` + permute copy
+ ``ncclReduceScatter`` back to back on one stream
(``src/distdl/nn/linear_ag.py:462-486``, ``src/distdl/nn/linear_rs.py:339-364``).

The two are each other's adjoint: the backward of ``ag_linear`` is a
``gemm_rs`` of the output gradient (plus a local weight-gradient GEMM against
the gathered activation that the forward kept), the backward of ``linear_rs``
is an ``ag_gemm`` of the output gradient.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .. import _native
from ..ops._util import ptr, stream_ptr
from ..ops.gemm import _major, grad_target, weight_grad
from . import symm

c_void_p, c_int, c_ll, c_uint = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_uint
_PP, _IP, _UP = ctypes.POINTER(c_void_p), ctypes.POINTER(c_int), ctypes.POINTER(c_uint)
_native.declare("dd_ag_gemm", [c_int, c_int, _PP, c_void_p, c_void_p, c_int, c_ll, c_void_p, c_ll, c_void_p, c_int,
                               c_int, c_int, c_int, c_int, c_void_p, c_uint, _PP, _IP, _UP, c_void_p, c_uint, c_int,
                               c_void_p, _UP, c_void_p])
_native.declare("dd_gemm_rs", [c_int, c_int, c_void_p, c_ll, c_void_p, c_int, c_ll, _PP, c_void_p, c_void_p, c_void_p,
                               c_int, c_int, c_int, c_int, c_int, _PP, _IP, _UP, _UP, c_void_p, c_uint, c_void_p,
                               c_uint, c_int, c_void_p])
_native.declare("dd_fused_reduce_ctas", [])
_native.declare("dd_gemm_rs_folds", [c_int, c_int])
_native.declare("dd_fused_gemm_ctas", [])

ENABLED = os.environ.get("DISTDL_FUSED", "1") != "0"


class _State:
    """Host-side bookkeeping of the counter flags used by the fused kernels."""

    def __init__(self):
        self.h = symm.heap()
        W = self.h.world
        self.ag_signals = [0] * W                       # AG signals received so far from each peer
        self.rs_delivered = [[0] * W, [0] * W]          # per staging parity
        self.rs_consumed = [[0] * W, [0] * W]
        self.rs_calls = 0
        self.epoch = 0
        lib = _native.lib()
        self.sm = lib.dd_fused_gemm_ctas()      # grid of the fused GEMM kernels (completion counters count CTAs)
        self.reduce_ctas = lib.dd_fused_reduce_ctas()
        # misc region: [0, 64) counters, then the row-block ready words
        self.misc = self.h.region_tensor("misc", self.h.regions["misc"][1], torch.int32)
        self.misc.zero_()
        self.done = [0, 0, 0]                           # ag pull, rs gemm, rs reduce (totals so far)
        # after the counters: ready words, then the per-block piece counters of the pull
        self.ready_words = (self.misc.numel() - 64) // 2
        # the shard staging is double buffered: a call only has to know that the readers
        # of the call before the previous one are through, which the previous call's
        # kernel has already checked
        self.ag_calls = {}
        self.ag_last_team = None
        self.ag_unconfirmed = None

    def counter_ptr(self, i):
        return self.h.region_ptr("misc", offset=4 * i)

    def ready_ptr(self):
        return self.h.region_ptr("misc", offset=4 * 64)

    def ready_cnt_ptr(self):
        return self.h.region_ptr("misc", offset=4 * (64 + self.ready_words))


_state = None


def state() -> _State:
    global _state
    if _state is None:
        _state = _State()
    return _state


PAD_AG_WORD = 1024      # word offset of the ag_gemm signals inside a signal pad


def _confirm_readers(st, limit_s: float = 2.0):
    """Host-side bounded wait until the peers of the last double-buffered ``ag_gemm``
    have signalled that they are done reading this process's shard."""
    import time
    _team, expected = st.ag_unconfirmed
    pad = symm._wrap_device_pointer(st.h._local_pad.value, symm.SIGNAL_PAD_BYTES // 4, torch.int32, st.h.device)
    torch.cuda.current_stream().synchronize()
    t0 = time.time()
    for r, want in expected.items():
        while ((int(pad[PAD_AG_WORD + r].item()) & 0xFFFFFFFF) - (want & 0xFFFFFFFF)) & 0x80000000:
            if time.time() - t0 > limit_s:
                raise RuntimeError(f"peer {r} did not finish reading the all-gather shard within {limit_s} s")
            time.sleep(0.0005)
    st.ag_unconfirmed = None


def _team_arrays(h, ranks):
    n = len(ranks)
    pads = (c_void_p * n)(*[h.pad_ptrs[r] for r in ranks])
    writers = (c_int * n)(*[int(r) for r in ranks])
    return pads, writers


def ag_gemm(x_local: torch.Tensor, w: torch.Tensor, bias, ranks):
    """``y = gather_seq(x_local) @ w.T (+ bias)``.

    ``x_local`` [batch, s_local, K] bf16 (this member's sequence shard), ``w``
    an [N, K] view (row- or column-contiguous).  Returns ``(y [batch, P*s_local, N],
    G [batch, P*s_local, K])`` where ``G`` is the gathered activation."""
    symm.require_healthy()
    st = state()
    h = st.h
    ranks = list(ranks)
    P, me = len(ranks), ranks.index(h.rank)
    b, s_local, K = x_local.shape
    N = w.shape[0]
    nbytes = x_local.numel() * 2
    half = h.regions["ag_shard"][1] // 2 // 256 * 256
    # The shard staging is double buffered: this call's kernel then only checks, before
    # it exits, that the readers of the PREVIOUS call are through (they are, in
    # practice), instead of waiting for its own readers.  That is sound while
    # consecutive calls use the same team; on a change of team the host first confirms
    # the readers of the last double-buffered call.
    team = tuple(ranks)
    if st.ag_unconfirmed is not None and (st.ag_unconfirmed[0] != team or nbytes > half):
        _confirm_readers(st)
    double = nbytes <= half and st.ag_last_team == team
    parity = st.ag_calls.get(team, 0) & 1 if nbytes <= half else 0
    if nbytes <= half:
        st.ag_calls[team] = st.ag_calls.get(team, 0) + 1
    st.ag_last_team = team if nbytes <= half else None
    off = parity * half
    stage = h.region_tensor("ag_shard", nbytes, torch.bfloat16, offset=off)
    stage.copy_(x_local.reshape(-1))
    M = b * P * s_local
    if M // 128 > st.ready_words:
        raise ValueError("too many row blocks for the ready-word region")
    G = torch.empty(b, P * s_local, K, dtype=torch.bfloat16, device=x_local.device)
    y = torch.empty(b, P * s_local, N, dtype=torch.bfloat16, device=x_local.device)
    shards = (c_void_p * P)(*[h.region_ptr("ag_shard", r, off) for r in ranks])
    pads, writers = _team_arrays(h, ranks)
    expect = (c_uint * P)(*[(st.ag_signals[r] + 1) & 0xFFFFFFFF for r in ranks])
    # "done pulling" of this call, or (double buffered) of the previous call
    end_expect = (c_uint * P)(*[(st.ag_signals[r] + (0 if double else 2)) & 0xFFFFFFFF for r in ranks])
    st.epoch += 1
    st.done[0] += st.sm
    w_mn, ldw, _ = _major(w)
    _native.launch_count += 1
    _native.check(_native.lib().dd_ag_gemm(
        P, me, shards, G.data_ptr(), w.data_ptr(), w_mn, ldw, y.data_ptr(), N, ptr(bias),
        int(bias is not None and bias.dtype == torch.float32), b, s_local, N, K, st.ready_ptr(), st.epoch, pads,
        writers, expect, st.counter_ptr(0), st.done[0] & 0xFFFFFFFF, 0, st.ready_cnt_ptr(), end_expect,
        stream_ptr()), "dd_ag_gemm")
    for r in ranks:
        if r != h.rank:
            st.ag_signals[r] += 2
    # readers of this call are confirmed by the next call's kernel, if there is one
    st.ag_unconfirmed = (team, {r: st.ag_signals[r] for r in ranks if r != h.rank}) if nbytes <= half else None
    return y, G


def gemm_rs(x: torch.Tensor, w: torch.Tensor, bias, ranks, batch: int, s_local: int):
    """``reduce_scatter_seq(x @ w.T (+ bias))``: ``x`` [batch * P * s_local, K] bf16
    (rows ordered [batch, seq]), returns this member's [batch, s_local, N]."""
    symm.require_healthy()
    st = state()
    h = st.h
    ranks = list(ranks)
    P, me = len(ranks), ranks.index(h.rank)
    M, K = x.shape
    N = w.shape[0]
    assert M == batch * P * s_local and x.stride(1) == 1
    rows = batch * s_local
    slot_bytes = rows * N * 2
    parity = st.rs_calls & 1
    st.rs_calls += 1
    region = f"rs{parity}"
    if P * slot_bytes > h.regions[region][1]:
        raise ValueError("partial products do not fit the reduce-scatter staging region")
    slots = (c_void_p * P)(*[h.region_ptr(region, r, offset=me * slot_bytes) for r in ranks])
    pads, writers = _team_arrays(h, ranks)
    consumed = (c_uint * P)(*[st.rs_consumed[parity][r] & 0xFFFFFFFF for r in ranks])
    delivered = (c_uint * P)(*[(st.rs_delivered[parity][r] + 1) & 0xFFFFFFFF for r in ranks])
    out = torch.empty(batch, s_local, N, dtype=torch.bfloat16, device=x.device)
    st.done[1] += st.sm
    # the reduction's completion counter counts the GEMM's CTAs when the fold runs inside the GEMM
    folds = bool(_native.lib().dd_gemm_rs_folds(batch, s_local))
    st.done[2] += st.sm if folds else st.reduce_ctas
    w_mn, ldw, _ = _major(w)
    _native.launch_count += 1 if folds else 2
    _native.check(_native.lib().dd_gemm_rs(
        P, me, x.data_ptr(), x.stride(0), w.data_ptr(), w_mn, ldw, slots, h.region_ptr(region), out.data_ptr(),
        ptr(bias), batch, s_local, N, K, parity, pads, writers, consumed, delivered, st.counter_ptr(1),
        st.done[1] & 0xFFFFFFFF, st.counter_ptr(2), st.done[2] & 0xFFFFFFFF, 0, stream_ptr()), "dd_gemm_rs")
    for r in ranks:
        if r != h.rank:
            st.rs_delivered[parity][r] += 1
            st.rs_consumed[parity][r] += 1
    return out


class AgLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, ranks):
        y, G = ag_gemm(x, w, bias, ranks)
        ctx.save_for_backward(G, w)
        ctx.wgrad = grad_target(w)
        ctx.ranks, ctx.has_bias = ranks, bias is not None
        ctx.shape = x.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        G, w = ctx.saved_tensors
        b, s_local, K = ctx.shape
        N = w.shape[0]
        dy2 = dy.reshape(-1, N)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[1]:
            dw = weight_grad(dy2, G.reshape(-1, K), target=ctx.wgrad)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.sum(0, dtype=torch.float32).to(dy.dtype)
        if ctx.needs_input_grad[0]:
            dx = gemm_rs(dy2, w.t(), None, ctx.ranks, b, s_local)
        return dx, dw, db, None


class LinearRsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, ranks):
        b, s, K = x.shape
        P = len(ranks)
        x2 = x.reshape(-1, K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        out = gemm_rs(x2, w, bias, ranks, b, s // P)
        ctx.save_for_backward(x2, w)
        ctx.wgrad = grad_target(w)
        ctx.ranks, ctx.has_bias = ranks, bias is not None
        ctx.shape = x.shape
        return out

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        b, s, K = ctx.shape
        N = w.shape[0]
        dyc = dy.contiguous()
        # dx = gather(dy) @ w ; the gathered dy also feeds the weight gradient
        dx, Gdy = ag_gemm(dyc, w.t(), None, ctx.ranks)
        dw = db = None
        if ctx.needs_input_grad[1]:
            dw = weight_grad(Gdy.reshape(-1, N), x2, target=ctx.wgrad)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = Gdy.reshape(-1, N).sum(0, dtype=torch.float32).to(dy.dtype)
        return dx.reshape(b, s, K), dw, db, None


# ------------------------------------------------------------------ uneven shards
# The kernels work on shards of equal length, a multiple of 128 rows.  Members whose shards
# differ (the balanced split of a sequence that does not divide by the team size) or are not
# a multiple of 128 run the same kernels on PADDED shards: every member's rows sit at the head
# of a slot of ``s_pad`` rows (zero filled), the padded rows take part in the GEMM and are
# dropped afterwards.  The reference pads unequal shards by one slice for its all-gather in
# the same spirit (``src/distdl/backends/nccl_cupy/functional/all_gather.py:86-99``).

def _pad_segments(t, extents, s_pad):
    """[b, sum(extents), F] -> [b, P * s_pad, F]: member i's rows at [i * s_pad, i * s_pad + extents[i])."""
    b, _, F = t.shape
    out = torch.zeros(b, len(extents) * s_pad, F, dtype=t.dtype, device=t.device)
    at = 0
    for i, e in enumerate(extents):
        out[:, i * s_pad:i * s_pad + e].copy_(t[:, at:at + e])
        at += e
    return out


def _unpad_segments(t, extents, s_pad):
    """The inverse of :func:`_pad_segments`."""
    return torch.cat([t[:, i * s_pad:i * s_pad + e] for i, e in enumerate(extents)], dim=1)


class AgLinearPaddedFn(torch.autograd.Function):
    """:class:`AgLinearFn` for members with different (or not tile-aligned) shard lengths."""

    @staticmethod
    def forward(ctx, x, w, bias, ranks, extents, s_pad):
        b, s_local, K = x.shape
        xp = torch.zeros(b, s_pad, K, dtype=x.dtype, device=x.device)
        xp[:, :s_local].copy_(x)
        y_pad, G = ag_gemm(xp, w, bias, ranks)
        ctx.save_for_backward(G, w)
        ctx.wgrad = grad_target(w)
        ctx.cfg = (ranks, bias is not None, tuple(extents), s_pad, s_local, b, K)
        return _unpad_segments(y_pad, extents, s_pad)

    @staticmethod
    def backward(ctx, dy):
        G, w = ctx.saved_tensors
        ranks, has_bias, extents, s_pad, s_local, b, K = ctx.cfg
        N = w.shape[0]
        dy2 = _pad_segments(dy, extents, s_pad).reshape(-1, N)       # zero rows where G has zero rows
        dx = dw = db = None
        if ctx.needs_input_grad[1]:
            dw = weight_grad(dy2, G.reshape(-1, K), target=ctx.wgrad)
        if has_bias and ctx.needs_input_grad[2]:
            db = dy.reshape(-1, N).sum(0, dtype=torch.float32).to(dy.dtype)
        if ctx.needs_input_grad[0]:
            dx = gemm_rs(dy2, w.t(), None, ranks, b, s_pad)[:, :s_local].contiguous()
        return dx, dw, db, None, None, None


class LinearRsPaddedFn(torch.autograd.Function):
    """:class:`LinearRsFn` for members with different (or not tile-aligned) shard lengths."""

    @staticmethod
    def forward(ctx, x, w, bias, ranks, extents, s_pad, me):
        b, S, K = x.shape
        x2 = _pad_segments(x, extents, s_pad).reshape(-1, K)
        out = gemm_rs(x2, w, bias, ranks, b, s_pad)[:, :extents[me]].contiguous()
        ctx.save_for_backward(x2, w)
        ctx.wgrad = grad_target(w)
        ctx.cfg = (ranks, bias is not None, tuple(extents), s_pad, me, b, K)
        return out

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        ranks, has_bias, extents, s_pad, me, b, K = ctx.cfg
        N = w.shape[0]
        dyp = torch.zeros(b, s_pad, N, dtype=dy.dtype, device=dy.device)
        dyp[:, :extents[me]].copy_(dy)
        dx_pad, Gdy = ag_gemm(dyp, w.t(), None, ranks)
        dw = db = None
        if ctx.needs_input_grad[1]:
            dw = weight_grad(Gdy.reshape(-1, N), x2, target=ctx.wgrad)
        if has_bias and ctx.needs_input_grad[2]:
            db = Gdy.reshape(-1, N).sum(0, dtype=torch.float32).to(dy.dtype)
        return _unpad_segments(dx_pad, extents, s_pad), dw, db, None, None, None, None


def _balanced(n, P):
    return [n // P + (1 if i < n % P else 0) for i in range(P)]


def _team_of(layer, P_part, dim):
    key = "_fused_team"
    team = getattr(layer, key, None)
    if team is None:
        team = tuple(P_part.create_allreduction_partition((dim,)).ranks)
        object.__setattr__(layer, key, team)
    return team


def _usable(t, w, P):
    return (ENABLED and t.is_cuda and t.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and t.dim() == 3
            and w.dim() == 2 and w.shape[0] % 8 == 0 and w.shape[1] % 8 == 0
            and 1 < P <= 8 and symm.heap_ready())


def _fits(batch, s_pad, P, K, N):
    """Shard staging and row-block bookkeeping of the kernels hold this geometry."""
    h = symm.heap()
    return (batch * s_pad * max(K, N) * 2 <= h.regions["ag_shard"][1] and
            P * batch * s_pad * max(K, N) * 2 <= h.regions["rs0"][1] and
            batch * P * s_pad // 128 <= state().ready_words)


def maybe_ag_linear(layer, input, weight, bias):
    """Fused path of the column-parallel layers; ``None`` when it does not apply
    (input not sequence-sharded, shapes not tile-aligned, one worker, ...)."""
    P_x = layer.P_x
    dim = P_x.dim
    if layer.gather_dim != dim - 2 or dim != 3:
        return None
    P = int(P_x.shape[-2])
    if not _usable(input, weight, P):
        return None
    if bias is not None and bias.dtype != torch.bfloat16:
        return None
    ranks = _team_of(layer, P_x, layer.gather_dim)
    x = input if input.is_contiguous() else input.contiguous()
    # the members' shard lengths: the balanced split of the gathered length, which the layer's
    # all-gather module learns in its (collective, once per input structure) set-up
    ag = layer.all_gather
    ag._distdl_forward_pre_hook(ag, (input,))
    total = int(ag.output_tensor_structure.shape[layer.gather_dim])
    extents = _balanced(total, P)
    if extents[list(ranks).index(symm.heap().rank)] != input.shape[1]:
        return None
    if len(set(extents)) == 1 and extents[0] % 128 == 0:
        return AgLinearFn.apply(x, weight, bias, ranks)
    s_pad = -(-max(extents) // 128) * 128
    if not _fits(input.shape[0], s_pad, P, weight.shape[1], weight.shape[0]):
        return None
    return AgLinearPaddedFn.apply(x, weight, bias, ranks, tuple(extents), s_pad)


def maybe_linear_rs(layer, input, weight, bias):
    """Fused path of the row-parallel layers; ``None`` when it does not apply."""
    P_y = layer.P_y
    dim = P_y.dim
    if layer.scatter_dim != dim - 2 or dim != 3:
        return None
    P = int(P_y.shape[-2])
    if input.dim() != 3:
        return None
    if not _usable(input, weight, P):
        return None
    if bias is not None and bias.dtype != torch.bfloat16:
        return None
    ranks = _team_of(layer, P_y, layer.scatter_dim)
    extents = _balanced(int(input.shape[1]), P)
    if len(set(extents)) == 1 and extents[0] % 128 == 0:
        return LinearRsFn.apply(input, weight, bias, ranks)
    s_pad = -(-max(extents) // 128) * 128
    if not _fits(input.shape[0], s_pad, P, weight.shape[1], weight.shape[0]):
        return None
    return LinearRsPaddedFn.apply(input, weight, bias, ranks, tuple(extents), s_pad,
                                  list(ranks).index(symm.heap().rank))

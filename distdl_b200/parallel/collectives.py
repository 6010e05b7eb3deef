"""Host wrappers of the native device collectives (all-reduce, all-gather,
reduce-scatter, all-to-all) over the symmetric heap.

Each call copies the operand into the local staging buffer (a local
HBM-to-HBM copy), then launches ONE kernel on every GPU of the team that pulls
what it needs from the peers' staging buffers over NVLink and synchronises
through flag counters.  Message sizes above the staging capacity are processed
in slices.  Replaces the NCCL calls of the reference's ``nccl_cupy`` backend
(``src/distdl/backends/nccl_cupy/functional/all_sum_reduce.py:73-76``,
``all_gather.py:101-109``, ``reduce_scatter.py:117-125``).
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from .. import _native
from ..ops._util import stream_ptr
from ..utilities import streams
from . import symm

ONE_SHOT_BYTES = 256 * 1024
_DT = {torch.bfloat16: 0, torch.float32: 1}


def available(ranks) -> bool:
    if not (dist.is_available() and dist.is_initialized() and torch.cuda.is_available()):
        return False
    if not _native.available() or len(ranks) > 8:
        return False
    return True


def team(ranks):
    """Makes sure the heap exists (collective over all processes on first call)."""
    return symm.heap()


def _launch(name, h, ranks, *args):
    symm.require_healthy()
    steps = ctypes.c_int(0)
    targs = h.team_args(ranks)
    _native.launch_count += 1
    _native.check(getattr(_native.lib(), name)(*targs, *args, ctypes.byref(steps), stream_ptr()), name)
    h.advance(ranks, steps.value)


MC_ONE_SHOT_BYTES = 512 * 1024


def _all_reduce_multicast(mc, h, flat, out):
    """The job-wide all-reduce through the NVLink multicast region: the input is copied into this
    GPU's copy of the region, one kernel reads the sums with ``multimem.ld_reduce`` (and, for large
    messages, spreads them with ``multimem.st``)."""
    symm.require_healthy()
    es = flat.element_size()
    half = (mc.nbytes // 2) // 256 * 256
    n, done = flat.numel(), 0
    pads = (ctypes.c_void_p * h.world)(*h.pad_ptrs)
    lib = _native.lib()
    while done < n:
        cnt = min(n - done, half // es)
        nbytes = (cnt * es + 15) // 16 * 16
        stage = mc.local_tensor(nbytes, flat.dtype)
        if cnt * es != nbytes:
            stage[cnt:].zero_()
        stage[:cnt].copy_(flat[done:done + cnt])
        one_shot = int(nbytes <= MC_ONE_SHOT_BYTES)
        direct = cnt * es == nbytes
        dst = out[done:done + cnt] if direct else torch.empty(nbytes // es, dtype=flat.dtype, device=flat.device)
        steps = ctypes.c_int(0)
        _native.launch_count += 1
        _native.check(lib.dd_mc_allreduce(h.world, h.rank, pads, (mc.steps_done + 1) & 0xFFFFFFFF, 0, half,
                                          dst.data_ptr(), nbytes, _DT[flat.dtype], one_shot, mc.ctas,
                                          ctypes.byref(steps), stream_ptr()), "dd_mc_allreduce")
        mc.steps_done += steps.value
        if not direct:
            out[done:done + cnt].copy_(dst[:cnt])
        done += cnt


def all_reduce(x: torch.Tensor, ranks) -> torch.Tensor:
    """Team-wide sum of ``x`` (bf16 or fp32; fp32 accumulation); returns a new tensor."""
    h = symm.heap()
    ranks = list(ranks)
    flat = x.contiguous().view(-1)
    if flat.dtype not in _DT:
        flat = flat.float()
    out = torch.empty_like(flat)
    mc = symm.multicast_region() if len(ranks) == h.world else None
    if mc is not None:
        _all_reduce_multicast(mc, h, flat, out)
        return out.view(x.shape).to(x.dtype)
    es = flat.element_size()
    per = 16 // es
    cap = h.staging_bytes // 16 * 16
    n = flat.numel()
    done = 0
    while done < n:
        cnt = min(n - done, cap // es)
        nbytes = (cnt * es + 15) // 16 * 16
        stage = h.staging_tensor(nbytes, flat.dtype)
        if cnt % per:
            stage[cnt:].zero_()
        stage[:cnt].copy_(flat[done:done + cnt])
        if cnt * es == nbytes:
            dst = out[done:done + cnt]
            _launch("dd_allreduce", h, ranks, dst.data_ptr(), nbytes, _DT[flat.dtype], int(nbytes <= ONE_SHOT_BYTES))
        else:
            tmp = torch.empty(nbytes // es, dtype=flat.dtype, device=flat.device)
            _launch("dd_allreduce", h, ranks, tmp.data_ptr(), nbytes, _DT[flat.dtype], int(nbytes <= ONE_SHOT_BYTES))
            out[done:done + cnt].copy_(tmp[:cnt])
        done += cnt
    return out.view(x.shape).to(x.dtype)


def all_gather(x: torch.Tensor, ranks) -> torch.Tensor:
    """Stacks every member's ``x`` (equal shapes) along a new leading axis."""
    h = symm.heap()
    ranks = list(ranks)
    P = len(ranks)
    flat = x.contiguous().view(-1).view(torch.uint8)
    nbytes_total = flat.numel()
    out = torch.empty(P, nbytes_total, dtype=torch.uint8, device=x.device)
    cap = h.staging_bytes // 16 * 16
    done = 0
    while done < nbytes_total:
        cnt = min(nbytes_total - done, cap)
        padded = (cnt + 15) // 16 * 16
        stage = h.staging_tensor(padded, torch.uint8)
        stage[:cnt].copy_(flat[done:done + cnt])
        if padded == cnt and P * cnt == out.numel():
            _launch("dd_allgather", h, ranks, out.data_ptr(), padded)
        else:
            tmp = torch.empty(P, padded, dtype=torch.uint8, device=x.device)
            _launch("dd_allgather", h, ranks, tmp.data_ptr(), padded)
            out[:, done:done + cnt].copy_(tmp[:, :cnt])
        done += cnt
    return out.view(x.dtype).view((P,) + tuple(x.shape))


_native.declare("dd_gather_pull", [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p,
                                   ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p])


_native.declare("dd_rs_pull_f32", [ctypes.c_int, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.c_size_t,
                                   ctypes.c_float, ctypes.c_void_p])
_native.declare("dd_grad_rs_adamw", [ctypes.c_int, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.c_void_p,
                                     ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_float,
                                     ctypes.c_float, ctypes.c_float, ctypes.c_float, ctypes.c_float, ctypes.c_int,
                                     ctypes.c_void_p, ctypes.c_float, ctypes.c_void_p])
_native.declare("dd_gather_pull_ce", [ctypes.c_int, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.c_size_t,
                                      ctypes.c_void_p])
# messages of at least this many bytes per member go through the copy engines
GATHER_CE_BYTES = int(os.environ.get("DISTDL_GATHER_CE_BYTES", str(1 << 20)))


def _pull(P, first, srcs, out, nbytes, stream):
    if nbytes >= GATHER_CE_BYTES:
        _native.check(_native.lib().dd_gather_pull_ce(P, srcs, out.data_ptr(), nbytes, stream), "dd_gather_pull_ce")
    else:
        _native.check(_native.lib().dd_gather_pull(P, first, srcs, out.data_ptr(), nbytes, 0, stream), "dd_gather_pull")


def gather_in_place(x: torch.Tensor, ranks):
    """All-gather of a tensor that lives at the same offset of a registered parameter
    region on every member (ZeRO shards in the optimizer's flat buffer): the peers'
    copies are read where they are, without staging copy, flags or waits.  Returns the
    stacked ``[P, ...]`` result, or ``None`` when ``x`` is not such a tensor.  The
    caller guarantees that no member writes its shard meanwhile (the optimizer brackets
    its update with barriers)."""
    nbytes = x.numel() * x.element_size()
    if not x.is_contiguous() or nbytes == 0 or nbytes % 16 or x.data_ptr() % 16:
        return None
    reg = symm.find_param_region(x.data_ptr(), nbytes)
    if reg is None:
        return None
    ranks = list(ranks)
    P = len(ranks)
    off = x.data_ptr() - reg.local_ptr
    srcs = (ctypes.c_void_p * P)(*[reg.ptrs[r] + off for r in ranks])
    out = torch.empty((P,) + tuple(x.shape), dtype=x.dtype, device=x.device)
    first = ranks.index(reg.heap.rank)
    _native.launch_count += 1
    side = streams.side_stream(x.device)
    main = torch.cuda.current_stream(x.device)
    if side is None or side.cuda_stream == main.cuda_stream:
        _pull(P, first, srcs, out, nbytes, main.cuda_stream)
        return out
    # wait-free copy: runs on the side stream, after what is queued so far (the memory of
    # `out` may have been in use by earlier kernels of this stream)
    side.wait_stream(main)
    _pull(P, first, srcs, out, nbytes, side.cuda_stream)
    out.record_stream(side)
    if not streams.is_deferred():
        main.wait_stream(side)
    return out


def _as_one(rows):
    """The flat slices as one ``[P, n]`` tensor when they sit back to back in memory (the slices of
    one contiguous tensor, the usual case), else the list unchanged."""
    n, es = rows[0].numel(), rows[0].element_size()
    base = rows[0].data_ptr()
    if n and all(r.numel() == n and r.data_ptr() == base + i * n * es for i, r in enumerate(rows)):
        return torch.as_strided(rows[0], (len(rows), n), (n, 1))
    return rows


def _stage_rows(stage, rows, done, cnt):
    """stage[i, :cnt] = rows[i][done:done + cnt]: one copy when the rows are one tensor."""
    if isinstance(rows, torch.Tensor):
        stage[:, :cnt].copy_(rows[:, done:done + cnt])
    else:
        for i, r in enumerate(rows):
            stage[i, :cnt].copy_(r[done:done + cnt])


def reduce_scatter(x, ranks) -> torch.Tensor:
    """``x`` is ``[P, ...]`` (or a list of ``P`` equally shaped tensors): member ``i`` receives the
    team-wide sum of ``x[i]``.  Slices that are 16-byte aligned are pushed from where they are into
    the owners' staging buffers by the kernel itself; others are copied into this GPU's staging
    buffer first and pulled."""
    h = symm.heap()
    ranks = list(ranks)
    P = len(ranks)
    assert len(x) == P
    dtype_in = x[0].dtype
    rows = [x[i].contiguous().view(-1) for i in range(P)]
    if dtype_in not in _DT:
        rows = [r.float() for r in rows]
    rows = _as_one(rows)
    dt = rows[0].dtype
    es = rows[0].element_size()
    chunk = rows[0].numel()
    out = torch.empty(chunk, dtype=dt, device=rows[0].device)
    mc = symm.multicast_region() if P == h.world else None
    if mc is not None:
        _reduce_scatter_multicast(mc, h, rows, out)
        return out.view(x[0].shape).to(dtype_in)
    cap_elems = (h.staging_bytes // P) // 16 * 16 // es
    done = 0
    if (chunk * es) % 16 == 0 and all(rows[i].data_ptr() % 16 == 0 for i in range(P)):
        # no staging copy: every member pushes its slices straight into the owners' staging buffers
        while done < chunk:
            cnt = min(chunk - done, cap_elems)
            ptrs = (ctypes.c_void_p * P)(*[rows[i].data_ptr() + done * es for i in range(P)])
            _launch("dd_reducescatter_push", h, ranks, ptrs, out[done:done + cnt].data_ptr(), cnt * es, _DT[dt])
            done += cnt
        return out.view(x[0].shape).to(dtype_in)
    while done < chunk:
        cnt = min(chunk - done, cap_elems)
        padded = (cnt * es + 15) // 16 * 16
        pe = padded // es
        stage = h.staging_tensor(P * padded, dt).view(P, pe)
        if pe != cnt:
            stage[:, cnt:].zero_()
        _stage_rows(stage, rows, done, cnt)
        if pe == cnt:
            _launch("dd_reducescatter", h, ranks, out[done:done + cnt].data_ptr(), padded, _DT[dt])
        else:
            tmp = torch.empty(pe, dtype=dt, device=out.device)
            _launch("dd_reducescatter", h, ranks, tmp.data_ptr(), padded, _DT[dt])
            out[done:done + cnt].copy_(tmp[:cnt])
        done += cnt
    return out.view(x[0].shape).to(dtype_in)


def _reduce_scatter_multicast(mc, h, xs, out):
    """Job-wide reduce-scatter (``xs``: the P flat slices) through the multicast region: every GPU stages
    its whole input in its copy, then reads the sum of its own slice with ``multimem.ld_reduce``."""
    symm.require_healthy()
    P = h.world
    dt = xs[0].dtype
    es = xs[0].element_size()
    n = xs[0].numel()
    cap = (mc.nbytes // P) // 256 * 256
    pads = (ctypes.c_void_p * P)(*h.pad_ptrs)
    lib = _native.lib()
    done = 0
    while done < n:
        cnt = min(n - done, cap // es)
        padded = (cnt * es + 15) // 16 * 16
        pe = padded // es
        stage = mc.local_tensor(P * padded, dt).view(P, pe)
        if pe != cnt:
            stage[:, cnt:].zero_()
        _stage_rows(stage, xs, done, cnt)
        direct = pe == cnt
        dst = out[done:done + cnt] if direct else torch.empty(pe, dtype=dt, device=out.device)
        steps = ctypes.c_int(0)
        _native.launch_count += 1
        _native.check(lib.dd_mc_allreduce(P, h.rank, pads, (mc.steps_done + 1) & 0xFFFFFFFF, 0, 0, dst.data_ptr(),
                                          padded, _DT[dt], 2, mc.ctas, ctypes.byref(steps), stream_ptr()),
                      "dd_mc_allreduce")
        mc.steps_done += steps.value
        if not direct:
            out[done:done + cnt].copy_(dst[:cnt])
        done += cnt


def reduce_scatter_accumulate_(x: torch.Tensor, acc: torch.Tensor, ranks, scale: float = 1.0) -> bool:
    """``acc += scale * reduce_scatter(x)`` in one kernel: ``x`` is bf16 ``[P, n]``,
    ``acc`` a flat fp32 buffer of ``n`` elements (16-byte aligned, ``n % 8 == 0``).
    Returns False (doing nothing) when the operands do not qualify."""
    h = symm.heap()
    ranks = list(ranks)
    P = len(ranks)
    if (x.dtype != torch.bfloat16 or acc.dtype != torch.float32 or x.shape[0] != P or not acc.is_contiguous()
            or acc.data_ptr() % 16):
        return False
    n = x[0].numel()
    if n % 8 or acc.numel() != n or P * n * 2 > h.staging_bytes // 16 * 16:
        return False
    symm.require_healthy()
    stage = h.staging_tensor(P * n * 2, torch.bfloat16)
    stage.copy_(x.reshape(-1))
    steps = ctypes.c_int(0)
    targs = h.team_args(ranks)
    _native.launch_count += 1
    _native.check(_native.lib().dd_reducescatter_acc(*targs, acc.data_ptr(), n * 2, float(scale), ctypes.byref(steps),
                                                     stream_ptr()), "dd_reducescatter_acc")
    h.advance(ranks, steps.value)
    return True


def all_to_all(x: torch.Tensor, ranks) -> torch.Tensor:
    """``x`` is ``[P, ...]`` with equal blocks: block ``i`` goes to member ``i``;
    returns ``[P, ...]`` whose block ``i`` came from member ``i``."""
    h = symm.heap()
    ranks = list(ranks)
    P = len(ranks)
    xs = x.contiguous().view(P, -1).view(torch.uint8)
    chunk = xs.shape[1]
    out = torch.empty(P, chunk, dtype=torch.uint8, device=x.device)
    cap = (h.staging_bytes // P) // 16 * 16
    done = 0
    while done < chunk:
        cnt = min(chunk - done, cap)
        padded = (cnt + 15) // 16 * 16
        stage = h.staging_tensor(P * padded, torch.uint8).view(P, padded)
        stage[:, :cnt].copy_(xs[:, done:done + cnt])
        if padded == cnt and cnt == chunk:
            _launch("dd_alltoall", h, ranks, out.data_ptr(), padded)
        else:
            tmp = torch.empty(P, padded, dtype=torch.uint8, device=x.device)
            _launch("dd_alltoall", h, ranks, tmp.data_ptr(), padded)
            out[:, done:done + cnt].copy_(tmp[:, :cnt])
        done += cnt
    return out.view(x.dtype).view(x.shape)


def _nbytes(shape, dtype) -> int:
    n = 1
    for s_ in shape:
        n *= int(s_)
    return n * torch.empty((), dtype=dtype).element_size()


def exchange_split(team_size: int, staging_bytes: int, sends, recvs):
    """Which messages of this member travel inside the one-kernel exchange.

    The kernel is launched by EVERY member of the team on every exchange (it opens with a
    barrier over the team), so nothing about that launch depends on the messages.  What is
    decided here, per message, is whether it rides in the kernel or goes through the
    library's point-to-point path beside it.  A message rides in the kernel when it fits a
    staging slot and is the only message of its ordered pair; both ends of a pair know the
    message's size and how many messages the pair has, so the two ends always decide alike
    and no agreement round is needed.  ``sends`` = [(rank, tensor)], ``recvs`` =
    [(rank, shape, dtype)].  Returns ``(send_native, recv_native)``: one bool per entry."""
    slot = (staging_bytes // team_size) // 256 * 256
    n_to, n_from = {}, {}
    for dst, _ in sends:
        n_to[dst] = n_to.get(dst, 0) + 1
    for src, _, _ in recvs:
        n_from[src] = n_from.get(src, 0) + 1
    send_native = [n_to[dst] == 1 and t.numel() * t.element_size() <= slot for dst, t in sends]
    recv_native = [n_from[src] == 1 and _nbytes(shape, dtype) <= slot for src, shape, dtype in recvs]
    return send_native, recv_native


def exchange(team, sends, recvs):
    """Point-to-point messages inside ``team`` in one kernel.  ``sends`` =
    [(world_rank, tensor)], ``recvs`` = [(world_rank, shape, dtype)]; at most one
    message per ordered pair, each within its staging slot (the messages that
    :func:`exchange_split` marks; both lists may be empty, the member then only takes part
    in the kernel's barriers).  Returns the received tensors in the order of ``recvs``."""
    h = symm.heap()
    team = list(team)
    P = len(team)
    slot = (h.staging_bytes // P) // 256 * 256
    ok_s, ok_r = exchange_split(P, h.staging_bytes, sends, recvs)
    if not (all(ok_s) and all(ok_r)):
        raise ValueError("exchange: a message does not fit its staging slot, or two messages share a pair")
    symm.require_healthy()
    outs, dsts, nbytes = [], [0] * P, [0] * P
    for src, shape, dtype in recvs:
        nb = _nbytes(shape, dtype)
        padded = (nb + 15) // 16 * 16
        raw = torch.empty(padded, dtype=torch.uint8, device=h.device)
        outs.append(raw[:nb].view(dtype).view(tuple(int(s_) for s_ in shape)))
        i = team.index(src)
        dsts[i], nbytes[i] = raw.data_ptr(), (padded if nb else 0)
    for dst, t in sends:
        nb = t.numel() * t.element_size()
        if nb == 0:
            continue
        j = team.index(dst)
        stage = h.staging_tensor(slot * P, torch.uint8)[j * slot: j * slot + nb]
        stage.view(t.dtype).view(t.shape).copy_(t)            # the "pack": strided source -> contiguous slot
    steps = ctypes.c_int(0)
    targs = h.team_args(team)
    _native.launch_count += 1
    _native.check(_native.lib().dd_exchange(*targs, (ctypes.c_void_p * P)(*dsts), (ctypes.c_ulonglong * P)(*nbytes),
                                            slot, ctypes.byref(steps), stream_ptr()), "dd_exchange")
    h.advance(team, steps.value)
    return outs


def barrier(ranks):
    h = symm.heap()
    _launch("dd_team_barrier", h, list(ranks))

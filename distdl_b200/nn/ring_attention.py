"""Ring attention: exact self-attention over a sequence split across workers, with the key /
value blocks travelling around a ring while every worker keeps its queries.

New relative to the reference (which has no attention code).  Complements
:class:`~distdl_b200.nn.DistributedSelfAttention` (head <-> sequence all-to-all), which
needs the head count to divide by the sequence-parallel size; the ring form has no such
constraint and moves K / V only.

Worker ``r`` of ``S`` holds queries, keys and values of sequence block ``r``.  In step ``t`` it
attends its queries to block ``(r - t) mod S`` (for causal attention: fully if that block is
earlier, with the triangular mask if it is its own, not at all if it is later), then passes
the block on to worker ``r + 1``.  Partial results are merged with their log-sum-exp:

    lse = logaddexp(lse_a, lse_b),   out = out_a * exp(lse_a - lse) + out_b * exp(lse_b - lse)

The backward pass sends the blocks around once more, each with its gradient accumulator:
with the GLOBAL output and log-sum-exp the flash-attention backward of one (query block, key
block) pair yields exactly that pair's contribution to dQ, dK and dV.  The per-pair kernels are
the library's attention forward / backward (tcgen05 flash attention for bf16 CUDA tensors, a
PyTorch formulation otherwise); the ring hops use the transport's point-to-point exchange
(one kernel over peer memory on the native backend).
"""
import math

import torch

from .. import ops
from ..ops._util import use_native
from .module import Module


def _native_ok(q, seq):
    return use_native(q) and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128) and seq % 128 == 0


def _pair_forward(q, k, v, batch, seq, causal, scale):
    """(out [tokens, Hq, D], lse [batch, Hq, seq]) of one query block against one key block."""
    if _native_ok(q, seq):
        return ops.attention_forward(q, k, v, batch, seq, causal, scale)
    tokens, Hq, D = q.shape
    Hkv = k.shape[1]
    qh = q.reshape(batch, seq, Hq, D).transpose(1, 2).float()
    kh = k.reshape(batch, seq, Hkv, D).transpose(1, 2).float().repeat_interleave(Hq // Hkv, dim=1)
    vh = v.reshape(batch, seq, Hkv, D).transpose(1, 2).float().repeat_interleave(Hq // Hkv, dim=1)
    s = (qh @ kh.transpose(-1, -2)) * scale
    if causal:
        s = s.masked_fill(torch.ones(seq, seq, dtype=torch.bool, device=q.device).triu(1), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    out = torch.exp(s - lse.unsqueeze(-1)) @ vh
    return out.transpose(1, 2).reshape(tokens, Hq, D).to(q.dtype), lse


def _pair_backward(dout, q, k, v, out, lse, batch, seq, causal, scale):
    """Contribution of one (query block, key block) pair to (dq, dk, dv), given the GLOBAL
    ``out`` and ``lse`` of the query block."""
    if _native_ok(q, seq):
        return ops.attention_backward(dout, q, k, v, out, lse, batch, seq, causal, scale)
    tokens, Hq, D = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    qh = q.reshape(batch, seq, Hq, D).transpose(1, 2).float()
    kh = k.reshape(batch, seq, Hkv, D).transpose(1, 2).float().repeat_interleave(g, dim=1)
    vh = v.reshape(batch, seq, Hkv, D).transpose(1, 2).float().repeat_interleave(g, dim=1)
    doh = dout.reshape(batch, seq, Hq, D).transpose(1, 2).float()
    oh = out.reshape(batch, seq, Hq, D).transpose(1, 2).float()
    s = (qh @ kh.transpose(-1, -2)) * scale
    if causal:
        s = s.masked_fill(torch.ones(seq, seq, dtype=torch.bool, device=q.device).triu(1), float("-inf"))
    p = torch.exp(s - lse.unsqueeze(-1))
    delta = (doh * oh).sum(-1, keepdim=True)
    dv = p.transpose(-1, -2) @ doh
    ds = p * (doh @ vh.transpose(-1, -2) - delta) * scale
    dq = ds @ kh
    dk = ds.transpose(-1, -2) @ qh
    dk = dk.reshape(batch, Hkv, g, seq, D).sum(2)
    dv = dv.reshape(batch, Hkv, g, seq, D).sum(2)
    back = lambda t, h: t.transpose(1, 2).reshape(tokens, h, D).to(q.dtype)  # noqa: E731
    return back(dq, Hq), back(dk, Hkv), back(dv, Hkv)


def _lse_rows(lse, tokens, Hq):
    """[batch, Hq, seq] -> [tokens, Hq, 1] (the layout of the outputs)."""
    return lse.permute(0, 2, 1).reshape(tokens, Hq, 1)


class _RingAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, batch, seq, causal, scale, ranks, me, transport):
        S = len(ranks)
        nxt, prv = ranks[(me + 1) % S], ranks[(me - 1) % S]
        tokens, Hq, D = q.shape
        out = torch.zeros(tokens, Hq, D, dtype=torch.float32, device=q.device)
        lse = torch.full((batch, Hq, seq), float("-inf"), dtype=torch.float32, device=q.device)
        kb, vb = k.contiguous(), v.contiguous()
        for t in range(S):
            j = (me - t) % S                           # the block that is here in this step
            if not causal or j <= me:
                o_t, lse_t = _pair_forward(q, kb, vb, batch, seq, causal and j == me, scale)
                new = torch.logaddexp(lse, lse_t)
                out = out * torch.exp(_lse_rows(lse - new, tokens, Hq)) + \
                    o_t.float() * torch.exp(_lse_rows(lse_t - new, tokens, Hq))
                lse = new
            if t + 1 < S:
                kv = transport.exchange([(nxt, torch.stack([kb, vb]))], [(prv, (2,) + tuple(kb.shape), kb.dtype)],
                                        team=list(ranks))[0].to(q.device)
                kb, vb = kv[0], kv[1]
        out = out.to(q.dtype)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cfg = (batch, seq, causal, scale, tuple(ranks), me, transport)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        batch, seq, causal, scale, ranks, me, transport = ctx.cfg
        S = len(ranks)
        nxt, prv = ranks[(me + 1) % S], ranks[(me - 1) % S]
        dout = dout.contiguous()
        dq = torch.zeros_like(q, dtype=torch.float32)
        # the travelling bundle: K, V of some block and the gradients gathered for it so far
        kb, vb = k.contiguous(), v.contiguous()
        dkb = torch.zeros_like(kb, dtype=torch.float32)
        dvb = torch.zeros_like(vb, dtype=torch.float32)
        for t in range(S):
            j = (me - t) % S
            if not causal or j <= me:
                dq_t, dk_t, dv_t = _pair_backward(dout, q, kb, vb, out, lse, batch, seq, causal and j == me, scale)
                dq += dq_t.float()
                dkb += dk_t.float()
                dvb += dv_t.float()
            # pass the bundle on; after the last step it is back at the owner of its block
            bundle = torch.stack([kb.float(), vb.float(), dkb, dvb])
            got = transport.exchange([(nxt, bundle)], [(prv, tuple(bundle.shape), bundle.dtype)],
                                     team=list(ranks))[0].to(q.device)
            kb, vb, dkb, dvb = got[0].to(k.dtype), got[1].to(v.dtype), got[2], got[3]
        return dq.to(q.dtype), dkb.to(k.dtype), dvb.to(v.dtype), None, None, None, None, None, None, None


class DistributedRingAttention(Module):
    r"""``forward(q, k, v) -> out`` with ``q [b, s_local, Hq, D]``, ``k, v [b, s_local, Hkv, D]`` on
    ``P_seq = [B, S, H, 1]`` (equal sequence blocks, block ``i`` on the worker with sequence index
    ``i``; ``H`` > 1 when the heads are additionally split over tensor-parallel workers, each of
    which then runs its own ring).  Exact attention over the whole sequence, causal by global
    position if ``causal``.

    ``zigzag=True`` selects the load-balanced layout for causal attention: the sequence is cut into
    ``2S`` chunks and the worker with sequence index ``r`` holds chunks ``r`` and ``2S - 1 - r``
    (concatenated, so ``s_local`` is two chunks).  With contiguous blocks the last worker attends to
    ``S`` blocks and the first to one; with this layout every worker does the same work in every
    step of the ring."""

    def __init__(self, P_seq, causal=True, scale=None, zigzag=False):
        super().__init__()
        self.P_seq = P_seq
        self.causal, self.scale, self.zigzag = causal, scale, zigzag
        if not P_seq.active:
            return
        if P_seq.dim != 4 or int(P_seq.shape[3]) != 1:
            raise ValueError("DistributedRingAttention expects a partition of shape [B, S, H, 1]")
        ring = P_seq.create_allreduction_partition((1,))
        self.ranks = tuple(int(r) for r in ring.ranks)          # ordered by sequence index
        from ..backends.common import world
        self.me = self.ranks.index(world.world_rank())
        if self.me != int(P_seq.index[1]):
            raise RuntimeError("ring order does not follow the sequence index of the partition")

    def forward(self, q, k, v):
        if not self.P_seq.active:
            return q
        b, s, hq, d = q.shape
        hkv = k.shape[2]
        scale = self.scale if self.scale is not None else 1.0 / math.sqrt(d)
        transport = self._distdl_backend.transport()
        if self.zigzag and self.causal and len(self.ranks) > 1:
            if s % 2:
                raise ValueError("the zigzag layout holds two chunks per worker: the local length must be even")
            o = _ZigzagRingAttnFn.apply(q.reshape(b * s, hq, d), k.reshape(b * s, hkv, d), v.reshape(b * s, hkv, d),
                                        b, s, scale, self.ranks, self.me, transport)
            return o.reshape(b, s, hq, d)
        # without a causal mask attention does not depend on the order of the keys: the plain ring serves
        # both layouts
        o = _RingAttnFn.apply(q.reshape(b * s, hq, d), k.reshape(b * s, hkv, d), v.reshape(b * s, hkv, d), b, s,
                              self.causal, scale, self.ranks, self.me, transport)
        return o.reshape(b, s, hq, d)


def _halves(t, batch, c):
    """[batch * 2c, H, D] (tokens batch-major, two chunks of c per sequence) -> the two chunks."""
    H, D = t.shape[1], t.shape[2]
    t4 = t.reshape(batch, 2, c, H, D)
    return t4[:, 0].reshape(batch * c, H, D).contiguous(), t4[:, 1].reshape(batch * c, H, D).contiguous()


def _join(lo, hi, batch, c):
    H, D = lo.shape[1], lo.shape[2]
    return torch.stack([lo.reshape(batch, c, H, D), hi.reshape(batch, c, H, D)], dim=1).reshape(batch * 2 * c, H, D)


def _zigzag_pairs(j, me):
    """(query half, key half, triangular mask?) combinations that a worker computes while the K / V
    of worker ``j`` are with it.  Worker ``r`` holds chunks ``r`` (half 0) and ``2S - 1 - r`` (half 1)
    of the 2S chunks of the sequence, so every visit costs two or three chunk pairs: the causal
    work is the same on every worker."""
    if j == me:
        return [(0, 0, True), (1, 0, False), (1, 1, True)]
    if j < me:
        return [(0, 0, False), (1, 0, False)]        # both of my chunks come after j's early chunk only
    return [(1, 0, False), (1, 1, False)]            # only my late chunk comes after j's chunks


class _ZigzagRingAttnFn(torch.autograd.Function):
    """Causal ring attention on the load-balanced ("zigzag") layout."""

    @staticmethod
    def forward(ctx, q, k, v, batch, seq, scale, ranks, me, transport):
        S, c = len(ranks), seq // 2
        nxt, prv = ranks[(me + 1) % S], ranks[(me - 1) % S]
        Hq, D = q.shape[1], q.shape[2]
        qh = _halves(q, batch, c)
        out = [torch.zeros(batch * c, Hq, D, dtype=torch.float32, device=q.device) for _ in range(2)]
        lse = [torch.full((batch, Hq, c), float("-inf"), dtype=torch.float32, device=q.device) for _ in range(2)]
        kb, vb = k.contiguous(), v.contiguous()
        for t in range(S):
            j = (me - t) % S
            kh, vh = _halves(kb, batch, c), _halves(vb, batch, c)
            for a, b, tri in _zigzag_pairs(j, me):
                o_t, lse_t = _pair_forward(qh[a], kh[b], vh[b], batch, c, tri, scale)
                new = torch.logaddexp(lse[a], lse_t)
                out[a] = out[a] * torch.exp(_lse_rows(lse[a] - new, batch * c, Hq)) + \
                    o_t.float() * torch.exp(_lse_rows(lse_t - new, batch * c, Hq))
                lse[a] = new
            if t + 1 < S:
                kv = transport.exchange([(nxt, torch.stack([kb, vb]))], [(prv, (2,) + tuple(kb.shape), kb.dtype)],
                                        team=list(ranks))[0].to(q.device)
                kb, vb = kv[0], kv[1]
        res = _join(out[0], out[1], batch, c).to(q.dtype)
        ctx.save_for_backward(q, k, v, res, lse[0], lse[1])
        ctx.cfg = (batch, seq, scale, tuple(ranks), me, transport)
        return res

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse0, lse1 = ctx.saved_tensors
        batch, seq, scale, ranks, me, transport = ctx.cfg
        S, c = len(ranks), seq // 2
        nxt, prv = ranks[(me + 1) % S], ranks[(me - 1) % S]
        qh, oh, lse = _halves(q, batch, c), _halves(out, batch, c), (lse0, lse1)
        dh = _halves(dout.contiguous(), batch, c)
        dq = [torch.zeros_like(qh[0], dtype=torch.float32) for _ in range(2)]
        kb, vb = k.contiguous(), v.contiguous()
        dkb = torch.zeros_like(kb, dtype=torch.float32)
        dvb = torch.zeros_like(vb, dtype=torch.float32)
        for t in range(S):
            j = (me - t) % S
            kh, vh = _halves(kb, batch, c), _halves(vb, batch, c)
            dkh, dvh = list(_halves(dkb, batch, c)), list(_halves(dvb, batch, c))
            for a, b, tri in _zigzag_pairs(j, me):
                dq_t, dk_t, dv_t = _pair_backward(dh[a], qh[a], kh[b], vh[b], oh[a], lse[a], batch, c, tri, scale)
                dq[a] += dq_t.float()
                dkh[b] = dkh[b] + dk_t.float()
                dvh[b] = dvh[b] + dv_t.float()
            dkb, dvb = _join(dkh[0], dkh[1], batch, c), _join(dvh[0], dvh[1], batch, c)
            bundle = torch.stack([kb.float(), vb.float(), dkb, dvb])
            got = transport.exchange([(nxt, bundle)], [(prv, tuple(bundle.shape), bundle.dtype)],
                                     team=list(ranks))[0].to(q.device)
            kb, vb, dkb, dvb = got[0].to(k.dtype), got[1].to(v.dtype), got[2], got[3]
        dq_all = _join(dq[0], dq[1], batch, c)
        return dq_all.to(q.dtype), dkb.to(k.dtype), dvb.to(v.dtype), None, None, None, None, None, None

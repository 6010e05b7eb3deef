"""SwiGLU, GELU and rotary-embedding kernels (new relative to the reference,
which has no activation or attention code; they are required by the
GPT-2 / Llama / Mixtral model shapes)."""
from __future__ import annotations


import torch

from .. import _native
from ._util import stream_ptr, use_native


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        F = gu.shape[-1] // 2
        g2 = gu.reshape(-1, 2 * F)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        out = torch.empty(g2.shape[0], F, dtype=gu.dtype, device=gu.device)
        _native.call("dd_swiglu_fwd", g2.data_ptr(), out.data_ptr(), g2.shape[0], F, stream_ptr())
        ctx.save_for_backward(g2)
        ctx.shape = gu.shape
        return out.view(*gu.shape[:-1], F)

    @staticmethod
    def backward(ctx, dout):
        (g2,) = ctx.saved_tensors
        F = g2.shape[-1] // 2
        d2 = dout.reshape(-1, F)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        dgu = torch.empty_like(g2)
        _native.call("dd_swiglu_bwd", d2.data_ptr(), g2.data_ptr(), dgu.data_ptr(), g2.shape[0], F, stream_ptr())
        return dgu.view(ctx.shape)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up for a tensor whose last dimension is ``[gate | up]``."""
    F = gate_up.shape[-1] // 2
    if use_native(gate_up) and gate_up.dtype == torch.bfloat16 and F % 8 == 0:
        return _SwiGLUFn.apply(gate_up)
    g, u = gate_up[..., :F], gate_up[..., F:]
    return torch.nn.functional.silu(g) * u


class _GeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        xc = x.contiguous()
        y = torch.empty_like(xc)
        _native.call("dd_gelu_fwd", xc.data_ptr(), y.data_ptr(), xc.numel(), stream_ptr())
        ctx.save_for_backward(xc)
        return y

    @staticmethod
    def backward(ctx, dy):
        (xc,) = ctx.saved_tensors
        dyc = dy.contiguous()
        dx = torch.empty_like(xc)
        _native.call("dd_gelu_bwd", dyc.data_ptr(), xc.data_ptr(), dx.data_ptr(), xc.numel(), stream_ptr())
        return dx


def gelu(x: torch.Tensor) -> torch.Tensor:
    """tanh-approximated GELU (the GPT-2 activation)."""
    if use_native(x) and x.dtype == torch.bfloat16 and x.numel() % 8 == 0:
        return _GeluFn.apply(x)
    return torch.nn.functional.gelu(x, approximate="tanh")


_rope_cache = {}


def rope_table(seq: int, head_dim: int, theta: float, device) -> torch.Tensor:
    """[seq, head_dim/2, 2] fp32 table of (cos, sin)."""
    key = (seq, head_dim, theta, str(device))
    t = _rope_cache.get(key)
    if t is None:
        inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
        ang = torch.outer(torch.arange(seq, dtype=torch.float64), inv)
        t = torch.stack([ang.cos(), ang.sin()], dim=-1).float().to(device).contiguous()
        _rope_cache[key] = t
    return t


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, table, seq, nheads, layout):
        # qkv: contiguous, read as [tokens, heads_total, hd] = layout; rotates heads [0, nheads) in place.
        ctx.mark_dirty(qkv)
        tokens, ht, hd = layout
        _native.call("dd_rope", qkv.data_ptr(), table.data_ptr(), tokens, seq, ht, nheads, hd, 1.0, stream_ptr())
        ctx.table, ctx.seq, ctx.nheads, ctx.layout = table, seq, nheads, layout
        return qkv

    @staticmethod
    def backward(ctx, d):
        # the incoming gradient belongs to this node alone (the rotated tensor has one producer and
        # its consumers' gradients were summed into a fresh tensor): rotate it back in place
        d = d.contiguous()
        tokens, ht, hd = ctx.layout
        _native.call("dd_rope", d.data_ptr(), ctx.table.data_ptr(), tokens, ctx.seq, ht, ctx.nheads, hd, -1.0,
                     stream_ptr())
        return d, None, None, None, None


def rope_table_ranges(ranges, head_dim: int, theta: float, device) -> torch.Tensor:
    """Table for a local sequence made of several position ranges ``((start, length), ...)``."""
    key = (tuple(ranges), head_dim, theta, str(device))
    t = _rope_cache.get(key)
    if t is None:
        full = rope_table(max(a + n for a, n in ranges), head_dim, theta, device)
        t = torch.cat([full[a:a + n] for a, n in ranges]).contiguous()
        _rope_cache[key] = t
    return t


def rope_(qkv: torch.Tensor, seq: int, nheads: int, theta: float = 500000.0, offset: int = 0,
          ranges=None, layout=None) -> torch.Tensor:
    """Applies rotary position embedding (rotate-half convention) to the first
    ``nheads`` heads of ``qkv`` [tokens, heads_total, head_dim]; position of a
    token is ``offset`` plus its index modulo ``seq`` (``offset`` > 0 for a worker that holds a
    later block of a sequence split across workers), or, with ``ranges = ((start, length), ...)``
    adding up to ``seq``, the positions of those ranges one after the other.  In place on CUDA.

    ``layout = (tokens, heads_total, head_dim)``: ``qkv`` is the projection's own output in
    whatever shape it has (say ``[batch, seq, heads_total * head_dim]``) and is only READ in that
    layout.  Prefer this form: rotating a reshaped VIEW in place makes autograd copy the whole
    gradient twice in the backward pass."""
    if layout is not None:
        if use_native(qkv) and qkv.dtype == torch.bfloat16 and layout[2] % 16 == 0 and qkv.is_contiguous():
            tokens, ht, hd = (int(v) for v in layout)
            if ranges is not None:
                table = rope_table_ranges(tuple((int(a), int(n)) for a, n in ranges), hd, theta, qkv.device)
            else:
                table = rope_table(offset + seq, hd, theta, qkv.device)
                if offset:
                    table = table[offset:]
            return _RopeFn.apply(qkv, table, seq, nheads, (tokens, ht, hd))
        shape = qkv.shape
        return rope_(qkv.reshape(layout), seq, nheads, theta, offset, ranges).reshape(shape)
    tokens, ht, hd = qkv.shape
    if ranges is not None:
        table = rope_table_ranges(tuple((int(a), int(n)) for a, n in ranges), hd, theta, qkv.device)
    else:
        table = rope_table(offset + seq, hd, theta, qkv.device)
        if offset:
            table = table[offset:]                            # rows [offset, offset + seq)
    if use_native(qkv) and qkv.dtype == torch.bfloat16 and hd % 16 == 0 and qkv.is_contiguous():
        return _RopeFn.apply(qkv, table, seq, nheads, (tokens, ht, hd))
    pos = torch.arange(tokens, device=qkv.device) % seq
    cos = table[pos, :, 0].unsqueeze(1)
    sin = table[pos, :, 1].unsqueeze(1)
    x = qkv[:, :nheads].float()
    a, b = x[..., : hd // 2], x[..., hd // 2:]
    rot = torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).to(qkv.dtype)
    return torch.cat([rot, qkv[:, nheads:]], dim=1)

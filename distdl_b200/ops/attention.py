"""Flash attention (causal or full, grouped-query) on tcgen05 tensor cores.

New relative to the reference, which has no attention code; required by the
decoder model shapes.  Forward and backward never materialise the
[seq, seq] score matrix: scores live in TMEM, probabilities pass through
shared memory as bf16, and only the output and the per-row log-sum-exp reach
HBM.  Tensors use the layout ``[tokens, heads, head_dim]`` so that the packed
output of a fused QKV projection is consumed in place (strided views).
"""
from __future__ import annotations

import math
import os

import torch

from .. import _native
from ._util import stream_ptr, use_native

_native.declare("dd_attn_fwd", [_native.c_void_p, _native.c_ll, _native.c_ll, _native.c_void_p, _native.c_ll,
                                _native.c_ll, _native.c_void_p, _native.c_ll, _native.c_ll, _native.c_void_p,
                                _native.c_void_p, _native.c_int, _native.c_int, _native.c_int, _native.c_int,
                                _native.c_int, _native.c_int, _native.c_float, _native.c_void_p])
_native.declare("dd_attn_fwd2", [_native.c_void_p, _native.c_ll, _native.c_ll, _native.c_void_p, _native.c_ll,
                                 _native.c_ll, _native.c_void_p, _native.c_ll, _native.c_ll, _native.c_void_p,
                                 _native.c_void_p, _native.c_int, _native.c_int, _native.c_int, _native.c_int,
                                 _native.c_int, _native.c_int, _native.c_float, _native.c_void_p])
_BWD_ARGS = [_native.c_void_p, _native.c_ll, _native.c_ll, _native.c_void_p, _native.c_ll,
             _native.c_ll, _native.c_void_p, _native.c_ll, _native.c_ll, _native.c_void_p,
             _native.c_void_p, _native.c_void_p, _native.c_void_p, _native.c_void_p,
             _native.c_ll, _native.c_ll, _native.c_void_p, _native.c_ll, _native.c_ll,
             _native.c_void_p, _native.c_ll, _native.c_ll, _native.c_int, _native.c_int,
             _native.c_int, _native.c_int, _native.c_int, _native.c_int, _native.c_float,
             _native.c_void_p]
_native.declare("dd_attn_bwd2", _BWD_ARGS)
_native.declare("dd_attn_bwd", [_native.c_void_p, _native.c_ll, _native.c_ll, _native.c_void_p, _native.c_ll,
                                _native.c_ll, _native.c_void_p, _native.c_ll, _native.c_ll, _native.c_void_p,
                                _native.c_void_p, _native.c_void_p, _native.c_void_p, _native.c_void_p,
                                _native.c_ll, _native.c_ll, _native.c_void_p, _native.c_ll, _native.c_ll,
                                _native.c_void_p, _native.c_ll, _native.c_ll, _native.c_int, _native.c_int,
                                _native.c_int, _native.c_int, _native.c_int, _native.c_int, _native.c_float,
                                _native.c_void_p])


def _strides(t):
    # [tokens, heads, D] view with unit stride in D
    assert t.stride(2) == 1
    return t.stride(0), t.stride(1)


def attention_forward(q, k, v, batch, seq, causal=True, scale=None):
    """Returns (out [tokens, Hq, D], lse [batch, Hq, seq])."""
    tokens, Hq, D = q.shape
    Hkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = torch.empty(tokens, Hq, D, dtype=q.dtype, device=q.device)
    lse = torch.empty(batch, Hq, seq, dtype=torch.float32, device=q.device)
    # head dim 128 / 64 and sequences of whole 256-row pairs run the two-tile kernel (scores and
    # probabilities in tensor memory, two query tiles alternating on the tensor cores)
    two_tile = D in (64, 128) and seq % 256 == 0 and os.environ.get("DISTDL_ATTN_FWD2", "1") != "0"
    _native.call("dd_attn_fwd2" if two_tile else "dd_attn_fwd", q.data_ptr(), *_strides(q), k.data_ptr(), *_strides(k),
                 v.data_ptr(), *_strides(v), out.data_ptr(), lse.data_ptr(), batch, seq, Hq, Hkv, D, int(causal),
                 float(scale), stream_ptr())
    return out, lse


def attention_backward(dout, q, k, v, out, lse, batch, seq, causal=True, scale=None, dq=None, dk=None, dv=None):
    """Gradients of :func:`attention_forward`; writes into ``dq/dk/dv`` views when given."""
    tokens, Hq, D = q.shape
    Hkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if dq is None:
        dq = torch.empty(tokens, Hq, D, dtype=q.dtype, device=q.device)
    if dk is None:
        dk = torch.empty(tokens, Hkv, D, dtype=q.dtype, device=q.device)
    if dv is None:
        dv = torch.empty(tokens, Hkv, D, dtype=q.dtype, device=q.device)
    dout = dout.contiguous()
    # the kernels that keep P / dS in tensor memory (scratch: delta and the base-2 lse)
    in_tmem = D in (64, 128) and os.environ.get("DISTDL_ATTN_BWD2", "1") != "0"
    delta = torch.empty(2 if in_tmem else 1, batch, Hq, seq, dtype=torch.float32, device=q.device)
    _native.call("dd_attn_bwd2" if in_tmem else "dd_attn_bwd", q.data_ptr(), *_strides(q), k.data_ptr(), *_strides(k),
                 v.data_ptr(), *_strides(v), out.data_ptr(), dout.data_ptr(), lse.data_ptr(), delta.data_ptr(),
                 dq.data_ptr(), *_strides(dq), dk.data_ptr(), *_strides(dk), dv.data_ptr(), *_strides(dv), batch, seq,
                 Hq, Hkv, D, int(causal), float(scale), stream_ptr())
    return dq, dk, dv


class _AttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, batch, seq, causal, scale):
        out, lse = attention_forward(q, k, v, batch, seq, causal, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cfg = (batch, seq, causal, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        batch, seq, causal, scale = ctx.cfg
        dq, dk, dv = attention_backward(dout, q, k, v, out, lse, batch, seq, causal, scale)
        return dq, dk, dv, None, None, None, None


def _reference(q, k, v, batch, seq, causal, scale):
    tokens, Hq, D = q.shape
    Hkv = k.shape[1]
    qh = q.reshape(batch, seq, Hq, D).transpose(1, 2)
    kh = k.reshape(batch, seq, Hkv, D).transpose(1, 2)
    vh = v.reshape(batch, seq, Hkv, D).transpose(1, 2)
    # grouped-query heads are handled by the library kernel itself on CUDA (no expanded copy of K / V)
    if Hkv != Hq and not q.is_cuda:
        kh = kh.repeat_interleave(Hq // Hkv, dim=1)
        vh = vh.repeat_interleave(Hq // Hkv, dim=1)
    o = torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=causal, scale=scale,
                                                         enable_gqa=Hkv != Hq and q.is_cuda)
    return o.transpose(1, 2).reshape(tokens, Hq, D)


def attention(q, k, v, batch: int, seq: int, causal: bool = True, scale: float = None):
    """Scaled-dot-product attention over ``[tokens = batch*seq, heads, head_dim]``
    tensors (strided views allowed); ``k``/``v`` may have fewer heads (GQA)."""
    D = q.shape[-1]
    native = (use_native(q) and q.dtype == torch.bfloat16 and D in (64, 128) and seq % 128 == 0
              and os.environ.get("DISTDL_ATTN_IMPL", "native") == "native")
    if native:
        return _AttnFn.apply(q, k, v, batch, seq, causal, scale)
    return _reference(q, k, v, batch, seq, causal, scale)


class _PackedAttnFn(torch.autograd.Function):
    """Attention on a packed ``[tokens, Hq + 2*Hkv, D]`` projection output; the
    backward kernels write dq / dk / dv straight into one packed gradient."""

    @staticmethod
    def forward(ctx, qkv, Hq, Hkv, batch, seq, causal, scale):
        q, k, v = qkv[:, :Hq], qkv[:, Hq:Hq + Hkv], qkv[:, Hq + Hkv:]
        out, lse = attention_forward(q, k, v, batch, seq, causal, scale)
        ctx.save_for_backward(qkv, out, lse)
        ctx.cfg = (Hq, Hkv, batch, seq, causal, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        Hq, Hkv, batch, seq, causal, scale = ctx.cfg
        q, k, v = qkv[:, :Hq], qkv[:, Hq:Hq + Hkv], qkv[:, Hq + Hkv:]
        dqkv = torch.empty_like(qkv)
        attention_backward(dout, q, k, v, out, lse, batch, seq, causal, scale, dq=dqkv[:, :Hq],
                           dk=dqkv[:, Hq:Hq + Hkv], dv=dqkv[:, Hq + Hkv:])
        return dqkv, None, None, None, None, None, None


def attention_packed(qkv, Hq: int, Hkv: int, batch: int, seq: int, causal: bool = True, scale: float = None):
    """Attention over a packed projection ``[tokens, Hq + 2*Hkv, head_dim]`` (heads
    ordered q..., k..., v...).  Returns ``[tokens, Hq, head_dim]``."""
    D = qkv.shape[-1]
    native = (use_native(qkv) and qkv.dtype == torch.bfloat16 and D in (64, 128) and seq % 128 == 0
              and qkv.is_contiguous() and os.environ.get("DISTDL_ATTN_IMPL", "native") == "native")
    if native:
        return _PackedAttnFn.apply(qkv, Hq, Hkv, batch, seq, causal, scale)
    return _reference(qkv[:, :Hq], qkv[:, Hq:Hq + Hkv], qkv[:, Hq + Hkv:], batch, seq, causal, scale)

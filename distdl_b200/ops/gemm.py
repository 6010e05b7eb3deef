"""bf16 GEMM on tcgen05 tensor cores (TMEM accumulators, TMA-fed) and the
autograd ``linear`` built on it.

The native kernel computes ``D[b,m,n] (+)= sum_k A[b,m,k] * B[b,n,k] (+ bias[n])``
with each operand either K-major or MN-major, so forward (``x @ w.T``),
data-gradient (``dy @ w``) and weight-gradient (``dy.T @ x``) run without
transposition copies.  It stands where the reference calls
``torch.nn.functional.linear`` / ``torch.einsum`` (cuBLAS):
``src/distdl/nn/linear_ag.py:486``, ``src/distdl/nn/linear_rs.py:361``,
``src/distdl/nn/linear_ag_zero.py:35-61``.
"""
from __future__ import annotations

import torch

from .. import _native
from ._util import ptr, stream_ptr, use_native

F_OUT_F32 = 1
F_ACCUMULATE = 2
F_BIAS = 4
F_BIAS_F32 = 8


def _major(t: torch.Tensor):
    """Classifies a 2-D/3-D operand view [.., rows, k]: returns (mn_major, ld, batch_stride)."""
    if t.stride(-1) == 1:
        return 0, t.stride(-2), (t.stride(0) if t.dim() == 3 else 0)
    if t.stride(-2) == 1:
        return 1, t.stride(-1), (t.stride(0) if t.dim() == 3 else 0)
    raise ValueError("GEMM operand needs unit stride in one of its last two dimensions")


def gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor = None, *, bias: torch.Tensor = None,
         accumulate: bool = False, out_dtype: torch.dtype = None, max_ctas: int = 0) -> torch.Tensor:
    """``out[.., m, n] (+)= a[.., m, k] @ b[.., n, k].T (+ bias)`` on bf16 operands.

    ``a`` and ``b`` are *views*: pass ``w`` for ``x @ w.T``, ``w.t()`` for
    ``dy @ w``, and ``dy.t(), x.t()`` for ``dy.T @ x``; any combination of
    row-/column-contiguous views with 16-byte-aligned leading dimensions is
    accepted.  ``out`` may be bf16 or fp32 and may be a strided row-major view.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "bf16 operands required"
    assert a.dim() == b.dim() and a.dim() in (2, 3)
    M, K = a.shape[-2], a.shape[-1]
    N = b.shape[-2]
    assert b.shape[-1] == K, f"contraction mismatch {a.shape} x {b.shape}"
    batch = a.shape[0] if a.dim() == 3 else 1
    if out is None:
        shape = (batch, M, N) if a.dim() == 3 else (M, N)
        out = torch.empty(shape, dtype=out_dtype or torch.bfloat16, device=a.device)
        assert not accumulate
    assert out.stride(-1) == 1
    if M == 0 or N == 0:
        return out
    if K == 0:
        if not accumulate:
            out.zero_()
        return out
    a_mn, lda, sa = _major(a)
    b_mn, ldb, sb = _major(b)
    flags = 0
    if out.dtype == torch.float32:
        flags |= F_OUT_F32
    else:
        assert out.dtype == torch.bfloat16
    if accumulate:
        flags |= F_ACCUMULATE
    if bias is not None:
        flags |= F_BIAS
        if bias.dtype == torch.float32:
            flags |= F_BIAS_F32
        assert bias.is_contiguous() and bias.numel() == N
    ldd = out.stride(-2)
    sd = out.stride(0) if out.dim() == 3 else 0
    _native.call("dd_gemm_bf16", a.data_ptr(), a_mn, lda, sa, b.data_ptr(), b_mn, ldb, sb, out.data_ptr(), ldd, sd,
                 ptr(bias), M, N, K, batch, flags, max_ctas, stream_ptr())
    return out


def grad_target(w: torch.Tensor):
    """What a weight-gradient GEMM needs to know about the weight ``w`` ([out, in], possibly a
    transposed view), as a small tuple that a backward pass can keep without keeping ``w``
    itself alive: ``(main_grad, transposed_storage)``."""
    return getattr(w, "main_grad", None), (not w.is_contiguous() and w.t().is_contiguous())


def weight_grad(dy2: torch.Tensor, x2: torch.Tensor, w: torch.Tensor = None, target=None):
    """Gradient of ``y = x @ w.T`` with respect to ``w`` ([out, in]) from
    ``dy2 [tokens, out]`` and ``x2 [tokens, in]``; give either ``w`` or ``target =
    grad_target(w)``.

    * ``w.main_grad`` (an fp32 tensor in the layout of ``w``, possibly a
      transposed view): the GEMM epilogue accumulates into it and ``None`` is
      returned, so no bf16 gradient is ever written.
    * ``w`` a transposed view of a contiguous ``[in, out]`` tensor: the gradient
      is produced in that storage order (``x^T dy``) and returned as the matching
      view, so autograd's transpose back is free instead of a strided copy.
    """
    mg, transposed = target if target is not None else grad_target(w)
    if mg is not None:
        if mg.is_contiguous():
            gemm(dy2.t(), x2.t(), out=mg, accumulate=True)
        else:
            gemm(x2.t(), dy2.t(), out=mg.t(), accumulate=True)
        return None
    if transposed:
        return gemm(x2.t(), dy2.t()).t()
    return gemm(dy2.t(), x2.t())


class _LinearFn(torch.autograd.Function):
    """y = x @ w.T + b with all three GEMMs on the native kernel.

    When the weight carries a ``main_grad`` fp32 buffer (set by the optimizer
    for gradient accumulation) the weight gradient is accumulated straight into
    it from the GEMM epilogue and ``None`` is returned for ``w.grad``.
    """

    @staticmethod
    def forward(ctx, x, w, b):
        x2 = x.reshape(-1, x.shape[-1])
        # the result is allocated in its final shape (never a view), so that
        # in-place ops such as the rotary embedding may follow
        y = torch.empty(*x.shape[:-1], w.shape[0], dtype=x.dtype, device=x.device)
        gemm(x2, w, out=y.view(-1, w.shape[0]), bias=b)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = b is not None
        # (not the weight itself: a gathered ZeRO weight must not be held from forward to backward)
        ctx.wgrad = grad_target(w)
        ctx.b_main_grad = getattr(b, "main_grad", None) if b is not None else None
        ctx.xshape = x.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w.t()).view(ctx.xshape)
        if ctx.needs_input_grad[1]:
            dw = weight_grad(dy2, x2, target=ctx.wgrad)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            mg = ctx.b_main_grad
            s = dy2.sum(0, dtype=torch.float32)
            if mg is not None:
                mg.add_(s)
            else:
                db = s.to(dy.dtype)
        return dx, dw, db


def linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor = None) -> torch.Tensor:
    """Drop-in for ``torch.nn.functional.linear`` (bf16 CUDA operands run the tcgen05 kernel)."""
    if use_native(x, w) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.dim() == 2 \
            and w.shape[1] % 8 == 0 and (w.shape[0] % 8 == 0):
        return _LinearFn.apply(x, w, b)
    return torch.nn.functional.linear(x, w, b)


def matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a @ b`` for 2-D / 3-D bf16 CUDA tensors through the native kernel (no autograd)."""
    return gemm(a, b.transpose(-1, -2))

"""RMSNorm with ZeRO-sharded affine parameters
(``src/distdl/nn/rmsnorm_zero.py:22-347``)."""
from .. import ops
from ._zero_norm import _ZeroNormBase


class DistributedRMSNormZero(_ZeroNormBase):
    r"""``y = x * rsqrt(mean(x^2) + eps) * weight (+ bias)`` over the (local) last
    dimension; weight and optional bias split evenly over all workers of
    ``P_x`` and all-gathered on use.  Raises if the normalised dimension is
    partitioned.  Runs the fused RMSNorm kernel of this library."""

    def __init__(self, P_x, normalized_shape, elementwise_affine=True, bias=False, eps=1e-5, collect_state=False,
                 device=None, dtype=None, scale_backward=None, auto_clear_buffer=True):
        super().__init__()
        if not P_x.active:
            self.P_x = P_x
            return
        self.eps = eps
        names = ("weight", "bias") if bias else ("weight",)
        self._setup_zero_params(P_x, normalized_shape, names, elementwise_affine, collect_state, device, dtype,
                                scale_backward, auto_clear_buffer)

    def forward(self, input, residual=None):
        """With ``residual``: returns ``(input + residual, norm(input + residual))``, the add fused
        into the norm kernel."""
        if not self.P_x.active:
            return input if residual is None else (input, input)
        w, b = self._gathered()
        if residual is not None:
            if len(self.normalized_shape) != 1:
                s = input + residual
                x = s.reshape(*s.shape[: s.dim() - len(self.normalized_shape)], -1)
                return s, ops.rms_norm(x, w, self.eps, b).reshape(s.shape)
            return ops.add_rms_norm(input, residual, w, self.eps, b)
        if len(self.normalized_shape) != 1:
            x = input.reshape(*input.shape[: input.dim() - len(self.normalized_shape)], -1)
            return ops.rms_norm(x, w, self.eps, b).reshape(input.shape)
        return ops.rms_norm(input, w, self.eps, b)

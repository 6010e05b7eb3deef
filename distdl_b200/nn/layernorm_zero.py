"""LayerNorm with ZeRO-sharded affine parameters
(``src/distdl/nn/layernorm_zero.py:21-307``)."""
import torch

from .. import ops
from ._zero_norm import _ZeroNormBase


class DistributedLayerNormZero(_ZeroNormBase):
    r"""LayerNorm whose normalised dimensions are local to every worker; the
    affine weight and bias are split evenly over all workers of ``P_x`` and
    all-gathered on use (FSDP).  The normalisation itself is the fused
    LayerNorm kernel of this library (the reference calls the optional
    ``flash_attn`` fused norm here)."""

    def __init__(self, P_x, normalized_shape, elementwise_affine=True, eps=1e-5, collect_state=False, device=None,
                 dtype=None, scale_backward=None, auto_clear_buffer=True):
        super().__init__()
        if not P_x.active:
            self.P_x = P_x
            return
        self.eps = eps
        self._setup_zero_params(P_x, normalized_shape, ("weight", "bias"), elementwise_affine, collect_state, device,
                                dtype, scale_backward, auto_clear_buffer)

    def forward(self, input, residual=None):
        """With ``residual``: returns ``(input + residual, norm(input + residual))``, the add fused
        into the norm kernel."""
        if not self.P_x.active:
            return input if residual is None else (input, input)
        w, b = self._gathered()
        if residual is not None and len(self.normalized_shape) == 1:
            return ops.add_layer_norm(input, residual, w, b, self.eps)
        if residual is not None:
            input = input + residual
            return input, self.forward(input)
        if len(self.normalized_shape) == 1:
            return ops.layer_norm(input, w, b, self.eps)
        shape = self.normalized_shape
        return torch.nn.functional.layer_norm(input, shape, None if w is None else w.reshape(shape),
                                              None if b is None else b.reshape(shape), self.eps)

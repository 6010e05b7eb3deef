"""General 2-D tensor-parallel linear layer (``src/distdl/nn/linear.py:11-108``)."""
import math

import torch

from .. import ops
from ..utilities.slicing import compute_subshape
from .broadcast import Broadcast
from .module import Module
from .sum_reduce import SumReduce


class DistributedLinear(Module):
    r"""``y = x W^T + b`` with ``W`` on a 2-D grid ``P_w = [P_fo, P_fi]``.

    The input lives on ``P_x = [1, P_fi]`` (features split), the output on
    ``P_y = [1, P_fo]``.  Forward: broadcast ``x`` down the columns of ``P_w``,
    local ``torch.nn.Linear`` on every weight block (bias only in column 0, so
    it enters the sum once), sum-reduce along the rows onto ``P_y`` (the
    partition is read transposed).
    """

    def __init__(self, P_x, P_y, P_w, in_features, out_features, bias=True, checkpoint=False, device=None,
                 dtype=None):
        super().__init__()
        self.P_x, self.P_y, self.P_w = P_x, P_y, P_w
        self.in_features, self.out_features = in_features, out_features
        self.use_bias = bias
        if P_w.active:
            local_out = int(compute_subshape(P_w.shape[0], P_w.index[0], [out_features])[0])
            local_in = int(compute_subshape(P_w.shape[1], P_w.index[1], [in_features])[0])
            has_bias = bias and int(P_w.index[-1]) == 0
            self.sublinear = torch.nn.Linear(local_in, local_out, bias=has_bias, device=device or P_w.device,
                                             dtype=dtype)
            bound = 1 / math.sqrt(in_features)
            with torch.no_grad():
                self.sublinear.weight.uniform_(-bound, bound)
                if has_bias:
                    self.sublinear.bias.uniform_(-bound, bound)
        self.x_broadcast = Broadcast(P_x, P_w, preserve_batch=True)
        self.y_sum_reduce = SumReduce(P_w, P_y, transpose_src=True, preserve_batch=True)

    def forward(self, input):
        if not (self.P_x.active or self.P_y.active or self.P_w.active):
            return input
        x = self.x_broadcast(input)
        if self.P_w.active:
            x = ops.linear(x, self.sublinear.weight, self.sublinear.bias)
        return self.y_sum_reduce(x)

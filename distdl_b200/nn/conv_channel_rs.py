"""Channel-parallel convolutions in the reduce-scatter form
(``src/distdl/nn/conv_channel_rs.py:64-1123``): the tensor-parallel analogue of
``DistributedLinearReduceScatter``."""
from .broadcast import Broadcast
from .conv_channel_ag import _ChannelConvNd, _make
from .reduce_scatter import ReduceScatter


class _ChannelReduceScatterConv(_ChannelConvNd):
    r"""Weight split over its *input* channels on ``P_weight = [1, M, 1, ...]``; every
    worker convolves its channel slice of the input ``[batch/D, in/M, ...]``, the
    partial results are reduce-scattered along the channel dimension into
    ``[batch/D, out/M, ...]``.  The bias lives on one worker and is added on the
    first tensor-parallel column only, so it enters the sum once."""

    shard = "in"

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        if not self.P_x.active:
            return
        self.reduce_scatter = ReduceScatter(self.P_x, axes_reduce_scatter=(1,))
        if self.use_bias:
            # first tensor-parallel column, all data-parallel rows
            from ._linear_common import derived_partition
            dim = self.P_x.dim
            idx = [slice(0, int(s)) for s in self.P_x.shape]
            idx[1] = slice(0, 1)
            shape = [int(s) for s in self.P_x.shape]
            shape[1] = 1
            self.P_apply_bias = derived_partition(self.P_x, idx, shape)
            if self.P_apply_bias.active:
                self.broadcast_bias = Broadcast(self.P_bias, self.P_apply_bias, preserve_batch=False)

    def forward(self, input):
        if not self.P_x.active:
            return input
        w = self.broadcast_weight(self.weight)
        b = None
        if self.use_bias and self.P_apply_bias.active:
            b = self.broadcast_bias(self.bias)
        y = self._conv(input, w, b)
        return self.reduce_scatter(y)


_DOC = "Channel reduce-scatter {}convolution, {}-D (see the base class)."
for _nd in (1, 2, 3):
    for _transposed in (False, True):
        _name = f"DistributedChannelReduceScatterConv{'Transpose' if _transposed else ''}{_nd}d"
        globals()[_name] = _make(_ChannelReduceScatterConv, _nd, _transposed, _name,
                                 _DOC.format("transposed " if _transposed else "", _nd))
del _nd, _transposed, _name

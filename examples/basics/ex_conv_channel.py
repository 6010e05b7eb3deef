"""Channel-parallel convolutions on [batch, channel, length] tensors.

* DistributedChannelConv1d: input channels split on P_x, output channels on P_y, kernel blocks on the
  2 x 2 grid P_w (broadcast, convolve, sum-reduce);
* DistributedChannelAllGatherConv1d -> DistributedChannelReduceScatterConv1d: the tensor-parallel pair
  (out channels split, then in channels split) on a [data 2, model 2, 1] grid."""
import torch
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
from distdl_b200.nn import (DistributedChannelAllGatherConv1d, DistributedChannelConv1d,  # noqa: E402
                            DistributedChannelReduceScatterConv1d)
from distdl_b200.utilities.torch import zero_volume_tensor  # noqa: E402

P_x, P_y = cart(P_world, [0, 1], [1, 2, 1]), cart(P_world, [0, 1], [1, 2, 1])
P_w = cart(P_world, [0, 1, 2, 3], [2, 2, 1])
conv = DistributedChannelConv1d(P_x, P_y, P_w, in_channels=4, out_channels=6, kernel_size=3, padding=1)
x = torch.randn(2, 2, 9, requires_grad=True) if P_x.active else zero_volume_tensor(requires_grad=True)
y = conv(x)
say(P_world, "channel conv: x", tuple(x.shape), "-> y", tuple(y.shape))

P = cart(P_world, [0, 1, 2, 3], [2, 2, 1])
up = DistributedChannelAllGatherConv1d(P, 4, 8, 3, padding=1)
down = DistributedChannelReduceScatterConv1d(P, 8, 4, 3, padding=1)
x = torch.randn(3, 2, 9, requires_grad=True)                      # [batch / 2, channels / 2, length]
y = down(torch.relu(up(x)))
y.sum().backward()
say(P_world, "all-gather / reduce-scatter pair: kernel shards", tuple(up.weight.shape), tuple(down.weight.shape),
    "y", tuple(y.shape))

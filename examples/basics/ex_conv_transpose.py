"""Transposed convolutions: spatially partitioned (halo exchange of the input, local transposed
convolution, crop) and channel-partitioned (all-gather form)."""
import torch
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
from distdl_b200.nn import (DistributedChannelAllGatherConvTranspose2d,  # noqa: E402
                            DistributedFeatureConvTranspose2d)

P_space = cart(P_world, [0, 1, 2, 3], [1, 1, 2, 2])
up = DistributedFeatureConvTranspose2d(P_space, 3, 2, kernel_size=4, stride=2, padding=1)
x = torch.randn(1, 3, 5, 4, requires_grad=True)                   # this worker's spatial block
y = up(x)
y.sum().backward()
say(P_world, "feature-partitioned: x", tuple(x.shape), "-> y", tuple(y.shape))

P_chan = cart(P_world, [0, 1, 2, 3], [2, 2, 1, 1])
upc = DistributedChannelAllGatherConvTranspose2d(P_chan, 4, 6, kernel_size=2, stride=2)
x = torch.randn(1, 2, 5, 5, requires_grad=True)                   # [batch / 2, channels / 2, h, w]
y = upc(x)
say(P_world, "channel-partitioned: x", tuple(x.shape), "-> y", tuple(y.shape))

"""Spatially partitioned convolution, pooling and upsampling on a 2x2 grid."""
import torch
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
P = cart(P_world, [0, 1, 2, 3], [1, 1, 2, 2])
from distdl_b200.nn import DistributedAvgPool2d, DistributedFeatureConv2d, DistributedUpsample  # noqa: E402

x = torch.randn(1, 3, 8, 8)                              # local 8x8 tile of a 16x16 image
y = DistributedFeatureConv2d(P, 3, 4, 3, padding=1)(x)
y = DistributedAvgPool2d(P, 2, stride=2)(y)
y = DistributedUpsample(P, scale_factor=2, mode="linear")(y)
say(P_world, "output tile", tuple(y.shape))

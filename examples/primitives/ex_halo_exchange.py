"""HaloExchange of width-1 halos on a 1x1x2x2 partition; corners propagate."""
import numpy as np
import torch
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
P = cart(P_world, [0, 1, 2, 3], [1, 1, 2, 2])
from distdl_b200.nn import HaloExchange  # noqa: E402

halo = np.array([[0, 0], [0, 0], [int(P.index[2] > 0), int(P.index[2] < 1)], [int(P.index[3] > 0), int(P.index[3] < 1)]])
shape = [1, 1, 3 + halo[2].sum(), 3 + halo[3].sum()]
x = torch.zeros(*shape)
x[:, :, halo[2][0]:shape[2] - halo[2][1], halo[3][0]:shape[3] - halo[3][1]] = rank + 1
y = HaloExchange(P, halo, halo, halo)(x)
say(P_world, "\n", y[0, 0].int().tolist())

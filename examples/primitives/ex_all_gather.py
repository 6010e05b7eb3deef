"""AllGather along tensor dimension 1 (uneven shards: 7 columns over 2 workers)."""
import torch
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
P = cart(P_world, [0, 1, 2, 3], [2, 2])
from distdl_b200.nn import AllGather  # noqa: E402

cols = 4 if P.index[1] == 0 else 3
y = AllGather(P, axes_all_gather=(1,))(torch.full((2, cols), float(rank)))
say(P_world, "y =", y.tolist())

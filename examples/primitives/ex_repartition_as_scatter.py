"""Repartition as a scatter: a tensor that lives on worker 0 is dealt out over a 2 x 2 decomposition
(balanced: the first workers along a dimension get the extra entries)."""
import torch
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import cart, say, start

P_world, rank = start()
P_root, P_y = cart(P_world, [0], [1, 1]), cart(P_world, [0, 1, 2, 3], [2, 2])
from distdl_b200.nn import Repartition  # noqa: E402
from distdl_b200.utilities.torch import zero_volume_tensor  # noqa: E402

x = torch.arange(35.0).reshape(5, 7).requires_grad_() if rank == 0 else zero_volume_tensor(requires_grad=True)
y = Repartition(P_root, P_y, preserve_batch=False)(x)
say(P_world, "y", y.tolist())

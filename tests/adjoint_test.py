"""Dot-product (adjoint) test: for y = F(x) and dx = F*(dy) the identity
<y, dy> == <x, dx> must hold when the inner products are summed over all
workers.  This is the universal oracle of the primitive and layer tests, as in
the reference (``tests/adjoint_test.py:11-56``)."""
import numpy as np
import torch
import torch.distributed as dist


def _global_sum(v):
    t = torch.tensor([float(v)], dtype=torch.float64)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t)
    return t.item()


def check_adjoint_test_tight(x, dx, y, dy, rtol=1e-6):
    def dot(a, b):
        if a is None or b is None or a.numel() == 0 or b.numel() == 0:
            return 0.0
        return float((a.detach().double() * b.detach().double()).sum())
    x_dx, y_dy = _global_sum(dot(x, dx)), _global_sum(dot(y, dy))
    nx, ndx = np.sqrt(_global_sum(dot(x, x))), np.sqrt(_global_sum(dot(dx, dx)))
    ny, ndy = np.sqrt(_global_sum(dot(y, y))), np.sqrt(_global_sum(dot(dy, dy)))
    denom = max(ny * ndy, nx * ndx)
    if denom == 0:
        assert x_dx == y_dy
        return
    assert abs(x_dx - y_dy) / denom < rtol, f"adjoint mismatch: <x,dx>={x_dx} <y,dy>={y_dy} denom={denom}"

"""Shared start-up of the examples: initialise ``torch.distributed`` from the
torchrun environment (gloo on CPU, NCCL with a GPU) and pick the backend.

    torchrun --nproc-per-node 4 --master-addr 127.0.0.1 examples/primitives/ex_repartition.py
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

import distdl_b200  # noqa: E402
from distdl_b200.backends.common import world  # noqa: E402


def start(cpu=True):
    """Returns (P_world, rank).  ``cpu=True`` keeps tensors on the host (gloo plumbing path)."""
    use_gpu = torch.cuda.is_available() and not cpu
    world.init_process_group_from_env("nccl" if use_gpu else "gloo")
    distdl_b200.config.set_backend("native" if use_gpu else "mpi", "cupy" if use_gpu else "numpy")
    P_world = distdl_b200.backends.backend.Partition()
    return P_world, world.world_rank()


def cart(P_world, ranks, shape):
    return P_world.create_partition_inclusive(ranks).create_cartesian_topology_partition(shape)


def say(P, *what):
    """Rank-ordered printing."""
    P.print_sequential(" ".join(str(w) for w in what))

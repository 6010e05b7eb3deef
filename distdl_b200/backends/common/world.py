"""Process-level view of the job: world rank/size and the control-plane group.

The reference forms every team of workers with MPI communicators
(``src/distdl/backends/common/partition.py:82-126``).  Here a team is just an
ordered tuple of world ranks; this module supplies the two things that still
need a live connection between processes:

* ``world_rank()`` / ``world_size()`` from ``torch.distributed`` (1 process when
  it is not initialised, so single-process use needs no launcher);
* a CPU (gloo) *control-plane* group over all processes, used for small
  metadata messages (tensor shapes, dtype ids) and by the CPU data path.  When
  the default group is NCCL, a gloo group is created beside it the first time
  it is needed -- a collective call, so every process must reach it (creating
  the world partition is such a point in an SPMD program).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

PROC_NULL = -1

_control_group = None
_control_ready = False


def initialized() -> bool:
    return dist.is_available() and dist.is_initialized()


def world_rank() -> int:
    return dist.get_rank() if initialized() else 0


def world_size() -> int:
    return dist.get_world_size() if initialized() else 1


def control_group():
    """gloo group over all processes (``None`` in a single-process run)."""
    global _control_group, _control_ready
    if not initialized():
        return None
    if _control_ready:
        return _control_group
    backend = dist.get_backend()
    if "gloo" in str(backend):
        _control_group = dist.group.WORLD
    else:
        _control_group = dist.new_group(backend="gloo")
    _control_ready = True
    return _control_group


def init_process_group_from_env(backend: str = None, timeout_s: float = 600.0):
    """Initialises ``torch.distributed`` from RANK / WORLD_SIZE / MASTER_* (the
    variables ``torchrun`` sets).  ``backend`` defaults to NCCL with a CUDA device
    and gloo otherwise.  Binds the process to ``cuda:LOCAL_RANK``."""
    import datetime

    if initialized():
        return
    if "RANK" not in os.environ or "WORLD_SIZE" not in os.environ:
        return
    has_cuda = torch.cuda.is_available()
    if backend is None:
        backend = "nccl" if has_cuda else "gloo"
    kwargs = {}
    if has_cuda:
        local = int(os.environ.get("LOCAL_RANK", os.environ["RANK"])) % torch.cuda.device_count()
        torch.cuda.set_device(local)
        if backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=timeout_s), **kwargs)


def reset_for_tests():
    """Forgets the cached control-plane group (after ``destroy_process_group``)."""
    global _control_group, _control_ready
    _control_group = None
    _control_ready = False

"""Backend selection (``src/distdl/config.py:8-76`` in the reference).

Three environment variables are honoured:

``DISTDL_BACKEND_COMM``
    ``mpi`` (CPU transport; gloo point-to-point here), ``nccl`` (library
    collectives through ``torch.distributed``) or ``native`` (hand-written
    sm_100a kernels over NVLink peer memory, NCCL where no kernel exists).
``DISTDL_BACKEND_ARRAY``
    ``numpy`` (tensors on the host) or ``cupy`` / ``torch`` (tensors on the GPU).
``DISTDL_CHECK_INPUT_CHANGED``
    ``1`` (default) re-runs a module's set-up when its input structure changes.

Without any variable set, the backend is ``native`` on a machine with a CUDA
device and the CPU backend otherwise.
"""
from __future__ import annotations

import os

import torch

from .logger import logger

BACKEND_COMM_ENVAR_NAME = "DISTDL_BACKEND_COMM"
BACKEND_ARRAY_ENVAR_NAME = "DISTDL_BACKEND_ARRAY"
CHECK_INPUT_CHANGED_ENVAR_NAME = "DISTDL_CHECK_INPUT_CHANGED"

_COMM = ("mpi", "nccl", "native")
_ARRAY = ("numpy", "cupy", "torch")

backend_comm = None
backend_array = None
check_input_changed = True


def get_default_comm():
    v = os.environ.get(BACKEND_COMM_ENVAR_NAME)
    if v is None:
        return "native" if torch.cuda.is_available() else "mpi"
    v = v.lower()
    if v not in _COMM:
        logger.warning(f"Unknown {BACKEND_COMM_ENVAR_NAME}={v!r}; using 'mpi'.")
        return "mpi"
    return v


def get_default_array(comm=None):
    v = os.environ.get(BACKEND_ARRAY_ENVAR_NAME)
    if v is None:
        return "numpy" if (comm or get_default_comm()) == "mpi" else "cupy"
    v = v.lower()
    if v not in _ARRAY:
        logger.warning(f"Unknown {BACKEND_ARRAY_ENVAR_NAME}={v!r}; using 'numpy'.")
        return "numpy"
    return v


def get_default_check_input_changed():
    v = os.environ.get(CHECK_INPUT_CHANGED_ENVAR_NAME)
    if v is None:
        return True
    if v.strip() in ("0", "false", "False"):
        return False
    if v.strip() in ("1", "true", "True"):
        return True
    logger.warning(f"Unknown {CHECK_INPUT_CHANGED_ENVAR_NAME}={v!r}; using True.")
    return True


def array_is_device() -> bool:
    return backend_array in ("cupy", "torch")


def set_backend(backend_comm=None, backend_array=None, check_input_changed=None):
    """Selects the process-global backend; returns the backend module.

    ``backend_comm`` in {mpi, nccl, native}; ``backend_array`` in {numpy, cupy,
    torch}.  Unsupported combinations fall back to ``mpi``/``numpy`` with a
    warning, as the reference does."""
    from . import backends
    g = globals()
    comm = (backend_comm or get_default_comm()).lower()
    array = (backend_array or get_default_array(comm)).lower()
    if array == "torch":
        array = "cupy"
    name = f"{comm}_{array}"
    mod = backends.supported_backends.get(name)
    if mod is None:
        logger.warning(f"Backend {name} is not available; falling back to mpi_numpy.")
        comm, array, name = "mpi", "numpy", "mpi_numpy"
        mod = backends.supported_backends[name]
    g["backend_comm"], g["backend_array"] = comm, array
    g["check_input_changed"] = (get_default_check_input_changed() if check_input_changed is None
                                else bool(check_input_changed))
    backends.backend = mod
    return mod

"""Backend registry (``src/distdl/backends/__init__.py:7-19`` in the reference).

``supported_backends`` maps ``<comm>_<array>`` to a backend module; ``backend``
is the process-global active one (set by :func:`distdl_b200.config.set_backend`).
"""
import importlib

from ..logger import logger

backend = None

_MODULES = {
    "mpi_numpy": "cpu_p2p",
    "mpi_cupy": "cpu_p2p",
    "nccl_cupy": "nccl_group",
    "native_cupy": "native_b200",
}
supported_backends = {}
for _key, _mod in _MODULES.items():
    try:
        supported_backends[_key] = importlib.import_module(f"{__name__}.{_mod}")
    except Exception as e:  # pragma: no cover - import problems are reported, not fatal
        logger.warning(f"Backend {_key} could not be loaded: {e}")
        supported_backends[_key] = None

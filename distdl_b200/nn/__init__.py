"""Distributed layers (``src/distdl/nn/__init__.py`` in the reference)."""
from .all_gather import AllGather  # noqa: F401
from .all_sum_reduce import AllSumReduce  # noqa: F401
from .broadcast import Broadcast  # noqa: F401
from .halo_exchange import HaloExchange  # noqa: F401
from .module import Module  # noqa: F401
from .reduce_scatter import ReduceScatter  # noqa: F401
from .repartition import Repartition  # noqa: F401
from .sum_reduce import SumReduce  # noqa: F401
from .transpose import DistributedTranspose  # noqa: F401

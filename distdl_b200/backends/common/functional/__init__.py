"""Backend-generic implementations of the seven adjoint-paired primitives."""
from ._base import bind_functional  # noqa: F401
from .all_gather import AllGatherFunction  # noqa: F401
from .all_sum_reduce import AllSumReduceFunction  # noqa: F401
from .broadcast import BroadcastFunction  # noqa: F401
from .halo_exchange import HaloAccumulateFunction, HaloExchangeFunction  # noqa: F401
from .reduce_scatter import ReduceScatterFunction  # noqa: F401
from .repartition import RepartitionFunction  # noqa: F401
from .sum_reduce import SumReduceFunction  # noqa: F401

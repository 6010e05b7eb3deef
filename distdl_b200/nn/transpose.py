"""Deprecated name of :class:`Repartition` (``src/distdl/nn/transpose.py:1-7``)."""
from .repartition import Repartition


class DistributedTranspose(Repartition):
    pass

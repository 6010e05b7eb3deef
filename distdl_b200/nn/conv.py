"""Selector that picks the distributed convolution matching the partitions
(``src/distdl/nn/conv.py:14-81``)."""
import numpy as np

from .conv_channel import DistributedChannelConv1d, DistributedChannelConv2d, DistributedChannelConv3d
from .conv_feature import DistributedFeatureConv1d, DistributedFeatureConv2d, DistributedFeatureConv3d
from .conv_general import DistributedGeneralConv1d, DistributedGeneralConv2d, DistributedGeneralConv3d


class DistributedConvSelector:
    """Only ``P_x`` given: spatial ("feature") partitioning.  ``P_x``, ``P_y`` and
    ``P_w`` given: channel partitioning when every spatial partition dimension is
    1, the general layer otherwise.  Anything else raises ``ValueError``."""

    DistributedChannelConvType = None
    DistributedFeatureConvType = None
    DistributedGeneralConvType = None

    def __new__(cls, P_x, P_y=None, P_w=None, buffer_manager=None, *args, **kwargs):
        if P_y is None and P_w is None:
            return cls.DistributedFeatureConvType(P_x, *args, buffer_manager=buffer_manager, **kwargs)
        if P_y is not None and P_w is not None:
            if np.all(np.asarray(P_x.shape[2:]) == 1) and np.all(np.asarray(P_y.shape[2:]) == 1):
                return cls.DistributedChannelConvType(P_x, P_y, P_w, *args, **kwargs)
            return cls.DistributedGeneralConvType(P_x, P_y, P_w, *args, buffer_manager=buffer_manager, **kwargs)
        raise ValueError("Cannot determine valid matching class.")


class DistributedConv1d(DistributedConvSelector):
    DistributedChannelConvType = DistributedChannelConv1d
    DistributedFeatureConvType = DistributedFeatureConv1d
    DistributedGeneralConvType = DistributedGeneralConv1d


class DistributedConv2d(DistributedConvSelector):
    DistributedChannelConvType = DistributedChannelConv2d
    DistributedFeatureConvType = DistributedFeatureConv2d
    DistributedGeneralConvType = DistributedGeneralConv2d


class DistributedConv3d(DistributedConvSelector):
    DistributedChannelConvType = DistributedChannelConv3d
    DistributedFeatureConvType = DistributedFeatureConv3d
    DistributedGeneralConvType = DistributedGeneralConv3d

"""Index arithmetic shared by the halo-exchanging layers."""
from .conv_mixin import ConvMixin  # noqa: F401
from .halo_mixin import HaloMixin  # noqa: F401
from .interpolate_mixin import InterpolateMixin  # noqa: F401
from .pooling_mixin import PoolingMixin  # noqa: F401

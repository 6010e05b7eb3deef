"""Functional layer: zero-volume corrector and the native interpolation op."""
from . import interpolate  # noqa: F401
from .zero_volume_corrector import ZeroVolumeCorrectorFunction  # noqa: F401

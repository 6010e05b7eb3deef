"""Functional layer: zero-volume corrector and the native interpolation op."""
from .zero_volume_corrector import ZeroVolumeCorrectorFunction  # noqa: F401

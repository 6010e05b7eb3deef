"""Native interpolation op (constant / multilinear, global coordinates)."""
from .interpolate import InterpolateFunction, interpolate  # noqa: F401

"""Which input entries an interpolated output range depends on
(``src/distdl/nn/mixins/interpolate_mixin.py:9-343``).

Conventions follow ``torch.nn.functional.interpolate``: with
``align_corners=False`` an output index ``i`` samples the input coordinate
``(i + 0.5) / scale - 0.5`` (clamped at 0), with ``align_corners=True`` the
coordinate ``i * (in - 1) / (out - 1)``; ``nearest`` takes ``floor(i / scale)``.
"""
import numpy as np


class InterpolateMixin:
    @staticmethod
    def _scale(in_size, out_size, align_corners, scale_factor=None):
        if align_corners:
            return (in_size - 1) / (out_size - 1) if out_size > 1 else 0.0
        if scale_factor is not None and scale_factor > 0:
            return 1.0 / scale_factor
        return in_size / out_size

    def _source_coordinate(self, i, in_size, out_size, mode, align_corners, scale_factor=None):
        r = self._scale(in_size, out_size, align_corners, scale_factor)
        if mode == "nearest":
            return float(np.floor(i * (1.0 / scale_factor if scale_factor else in_size / out_size)))
        if align_corners:
            return i * r
        return max(0.0, (i + 0.5) * r - 0.5)

    def _compute_needed_start(self, y_global_idx, x_global_shape, y_global_shape, scale_factor, mode, align_corners):
        """First input index (per dimension) read by output index ``y_global_idx``."""
        out = []
        for i, n_in, n_out, sf in zip(y_global_idx, x_global_shape, y_global_shape, scale_factor):
            c = self._source_coordinate(int(i), int(n_in), int(n_out), mode, align_corners, sf)
            out.append(int(min(n_in - 1, np.floor(c + 1e-4 if mode != "nearest" else c))))
        return np.asarray(out, dtype=int)

    def _compute_needed_stop(self, y_global_idx, x_global_shape, y_global_shape, scale_factor, mode, align_corners):
        """One past the last input index read by output index ``y_global_idx``."""
        out = []
        for i, n_in, n_out, sf in zip(y_global_idx, x_global_shape, y_global_shape, scale_factor):
            c = self._source_coordinate(int(i), int(n_in), int(n_out), mode, align_corners, sf)
            lo = int(min(n_in - 1, np.floor(c + 1e-4 if mode != "nearest" else c)))
            hi = lo if mode == "nearest" else min(n_in - 1, lo + 1)
            out.append(hi + 1)
        return np.asarray(out, dtype=int)

    def _compute_needed_range(self, y_start, y_stop, x_global_shape, y_global_shape, scale_factor, mode,
                              align_corners):
        """[start, stop) of the input entries needed for outputs [y_start, y_stop)."""
        y_last = np.maximum(np.asarray(y_stop) - 1, np.asarray(y_start))
        lo = self._compute_needed_start(y_start, x_global_shape, y_global_shape, scale_factor, mode, align_corners)
        hi = self._compute_needed_stop(y_last, x_global_shape, y_global_shape, scale_factor, mode, align_corners)
        return lo, hi

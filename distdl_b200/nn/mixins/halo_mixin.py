"""Halo sizes of a sliding-window operator on a partitioned tensor
(``src/distdl/nn/mixins/halo_mixin.py:7-207``).

For the worker at a given grid index the mixin answers: how many entries does
it need from its left / right neighbour in every dimension (``halo_shape``),
how many will it receive and send (``recv_buffer_shape`` /
``send_buffer_shape``; a worker sends what its neighbour's halo asks for), and
which part of the halo-padded local tensor the local operator has to be applied
to (``needed_ranges``; when the windows of a worker start beyond its own first
entries -- strided operators -- the left "halo" is negative, i.e. entries to
drop).  The host class supplies ``_compute_min_input_range`` /
``_compute_max_input_range`` (conv / pooling mixins).
"""
import numpy as np

from ...utilities.slicing import compute_start_index, compute_subshape


class HaloMixin:
    @staticmethod
    def _lpad(a, n, value):
        a = np.atleast_1d(np.asarray(a, dtype=int))
        return np.concatenate([np.full(n - len(a), value, dtype=int), a])

    def _compute_exchange_info(self, x_global_shape, kernel_size, stride, padding, dilation, partition_active,
                               partition_shape, partition_index, subtensor_shapes=None):
        if not partition_active:
            return None, None, None, None
        x_global_shape = np.asarray(x_global_shape, dtype=int)
        n = len(x_global_shape)
        k, s = self._lpad(kernel_size, n, 1), self._lpad(stride, n, 1)
        p, d = self._lpad(padding, n, 0), self._lpad(dilation, n, 1)
        P = [int(v) for v in partition_shape]
        idx = [int(v) for v in partition_index]

        def halo(index, nonneg=True):
            return self._compute_halo_shape(P, index, x_global_shape, k, s, p, d, require_nonnegative=nonneg,
                                            subtensor_shapes=subtensor_shapes)
        halo_shape = halo(idx)
        recv = halo_shape.copy()
        send = np.zeros_like(halo_shape)
        for dim in range(n):
            if idx[dim] - 1 >= 0:
                left = list(idx)
                left[dim] -= 1
                send[dim, 0] = halo(left)[dim, 1]
            if idx[dim] + 1 < P[dim]:
                right = list(idx)
                right[dim] += 1
                send[dim, 1] = halo(right)[dim, 0]
        if subtensor_shapes is not None:
            local = np.asarray(subtensor_shapes[tuple(idx)], dtype=int)
        else:
            local = compute_subshape(P, idx, x_global_shape)
        needed = self._compute_needed_ranges(local, halo(idx, nonneg=False))
        return halo_shape.astype(int), recv.astype(int), send.astype(int), needed.astype(int)

    def _compute_local_start_index(self, index, subtensor_shapes, x_local_shape):
        start = np.zeros(len(x_local_shape), dtype=int)
        for dim in range(len(x_local_shape)):
            for i in range(int(index[dim])):
                probe = tuple(i if j == dim else 0 for j in range(len(x_local_shape)))
                start[dim] += int(subtensor_shapes[probe][dim])
        return start

    def _compute_needed_ranges(self, tensor_shape, halo_shape):
        tensor_shape = np.asarray(tensor_shape, dtype=int)
        out = np.zeros_like(halo_shape, dtype=int)
        out[:, 0] = -np.minimum(0, halo_shape[:, 0])
        out[:, 1] = tensor_shape + np.maximum(0, halo_shape[:, 0]) + np.maximum(0, halo_shape[:, 1])
        return out

    def _compute_out_shape(self, in_shape, kernel_size, stride, padding, dilation):
        in_shape = np.asarray(in_shape)
        return np.floor((in_shape + 2 * padding - dilation * (kernel_size - 1) - 1) / stride + 1).astype(in_shape.dtype)

    def _compute_halo_shape(self, shape, index, x_global_shape, kernel_size, stride, padding, dilation,
                            require_nonnegative=True, subtensor_shapes=None):
        x_global_shape = np.asarray(x_global_shape, dtype=int)
        if subtensor_shapes is not None:
            x_local = np.asarray(subtensor_shapes[tuple(index)], dtype=int)
            x_start = self._compute_local_start_index(index, subtensor_shapes, x_local)
        else:
            x_local = compute_subshape(shape, index, x_global_shape)
            x_start = compute_start_index(shape, index, x_global_shape)
        y_global = self._compute_out_shape(x_global_shape, kernel_size, stride, padding, dilation)
        y_local = compute_subshape(shape, index, y_global)
        y_start = compute_start_index(shape, index, y_global)
        # first / last input entries the local outputs read, clipped to the tensor
        need_lo = np.maximum(0, self._compute_min_input_range(y_start, kernel_size, stride, padding, dilation))
        need_hi = np.minimum(x_global_shape - 1,
                             self._compute_max_input_range(y_start + y_local - 1, kernel_size, stride, padding,
                                                           dilation))
        left = x_start - need_lo
        right = need_hi - (x_start + x_local - 1)
        if require_nonnegative:
            left, right = np.maximum(left, 0), np.maximum(right, 0)
        return np.stack([left, right], axis=1).astype(int)

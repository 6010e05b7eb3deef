"""Input index range of a pooling window (``src/distdl/nn/mixins/pooling_mixin.py:6-64``);
the same arithmetic as a convolution."""


class PoolingMixin:
    def _compute_min_input_range(self, idx, kernel_size, stride, padding, dilation):
        return stride * idx - padding

    def _compute_max_input_range(self, idx, kernel_size, stride, padding, dilation):
        return stride * idx + dilation * (kernel_size - 1) - padding

"""Input index range touched by a convolution kernel centred on an output index
(``src/distdl/nn/mixins/conv_mixin.py:6-64``)."""


class ConvMixin:
    def _compute_min_input_range(self, idx, kernel_size, stride, padding, dilation):
        """Left-most input index read for output index ``idx``."""
        return stride * idx - padding

    def _compute_max_input_range(self, idx, kernel_size, stride, padding, dilation):
        """Right-most input index read for output index ``idx``."""
        return stride * idx + dilation * (kernel_size - 1) - padding

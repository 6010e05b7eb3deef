"""Base class of every distributed layer.

A forward pre-hook runs the layer's set-up lazily, on the first call and again
whenever the structure of the input (shape, dtype, requires_grad) changes
(``src/distdl/nn/module.py:34-56``, ``:101-112``); set
``DISTDL_CHECK_INPUT_CHANGED=0`` to skip the re-check.  The backend that is
active when the layer is built is captured on the instance.
"""
import torch

from .. import backends, config


class Module(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self._distdl_backend = backends.backend
        self._distdl_is_setup = False
        self.register_forward_pre_hook(self._distdl_forward_pre_hook)

    @staticmethod
    def _distdl_forward_pre_hook(self, input):
        if self._distdl_module_requires_reset(input):
            if self._distdl_is_setup:
                self._distdl_module_teardown(input)
            self._distdl_module_setup(input)

    def _distdl_module_setup(self, input):
        """Layer-specific set-up from the structure of ``input``."""

    def _distdl_module_teardown(self, input):
        """Releases whatever set-up allocated."""

    def _distdl_input_changed(self, input):
        """Layer-specific definition of "the input changed"."""
        return False

    def _distdl_module_requires_reset(self, input):
        if not self._distdl_is_setup:
            return True
        return bool(config.check_input_changed) and bool(self._distdl_input_changed(input))


def reset_setup(module: torch.nn.Module):
    """Makes every distributed layer below ``module`` run its set-up again at its next call.

    Set-up is collective, but a layer re-runs it only when THIS worker sees its input structure change.
    When shapes change in a way some workers cannot see (a new sequence length that leaves one worker's
    shard as long as before; a worker that feeds zero-volume tensors), call this on all workers before
    the next forward pass, so that all of them take part."""
    for m in module.modules():
        if isinstance(m, Module) and m._distdl_is_setup:
            m._distdl_module_teardown(None)
            m._distdl_is_setup = False

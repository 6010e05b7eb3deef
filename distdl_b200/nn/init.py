"""Initialisers for partitioned tensors (``src/distdl/nn/init.py``).

The element-wise initialisers are those of ``torch.nn.init``.  The Xavier and
Kaiming families take the partition of the tensor first and compute fan-in /
fan-out from the *global* tensor shape, so the distribution does not depend on
how many workers hold the tensor.
"""
import math

import torch
from torch.nn.init import (_no_grad_normal_, _no_grad_uniform_, calculate_gain, constant_, dirac_, eye_,  # noqa: F401
                           normal_, ones_, trunc_normal_, uniform_, zeros_)

from ..backends.common.tensor_comm import assemble_global_tensor_structure
from ..utilities.torch import TensorStructure


def _calculate_fan_in_and_fan_out(shape):
    shape = list(shape)
    # partition-rank-padded weights carry singleton dims: drop them for the fan computation
    if len(shape) < 2:
        raise ValueError("Fan in and fan out can not be computed for tensor with fewer than 2 dimensions")
    num_input_fmaps, num_output_fmaps = shape[1], shape[0]
    receptive = 1
    for s in shape[2:]:
        receptive *= s
    return num_input_fmaps * receptive, num_output_fmaps * receptive


def _global_shape(P_tensor, tensor):
    if P_tensor is None or P_tensor.size == 1 or not P_tensor.active:
        return list(tensor.shape)
    return list(assemble_global_tensor_structure(TensorStructure(tensor), P_tensor).shape)


def _linear_like_fans(shape):
    """Fans of a weight whose partition-padding singleton dims are ignored:
    the last two non-singleton extents are (out, in) for linear weights; conv
    weights ([out, in, *k]) keep torch's rule."""
    core = [s for s in shape if s != 1]
    if len(core) == 2 and len(shape) > 2 and shape[0] == 1:
        return core[1], core[0]
    if len(core) < 2:
        core = (list(shape) + [1, 1])[:2] if len(shape) < 2 else list(shape)
        return _calculate_fan_in_and_fan_out(core)
    return _calculate_fan_in_and_fan_out(shape)


def _calculate_correct_fan(P_tensor, tensor, mode):
    mode = mode.lower()
    if mode not in ("fan_in", "fan_out"):
        raise ValueError(f"Mode {mode} not supported, please use one of fan_in, fan_out")
    fan_in, fan_out = _linear_like_fans(_global_shape(P_tensor, tensor))
    return fan_in if mode == "fan_in" else fan_out


def xavier_uniform_(P_tensor, tensor, gain=1.0):
    fan_in, fan_out = _linear_like_fans(_global_shape(P_tensor, tensor))
    a = math.sqrt(3.0) * gain * math.sqrt(2.0 / float(fan_in + fan_out))
    return _no_grad_uniform_(tensor, -a, a) if tensor.numel() else tensor


def xavier_normal_(P_tensor, tensor, gain=1.0):
    fan_in, fan_out = _linear_like_fans(_global_shape(P_tensor, tensor))
    std = gain * math.sqrt(2.0 / float(fan_in + fan_out))
    return _no_grad_normal_(tensor, 0.0, std) if tensor.numel() else tensor


def kaiming_uniform_(P_tensor, tensor, a=0, mode="fan_in", nonlinearity="leaky_relu"):
    fan = _calculate_correct_fan(P_tensor, tensor, mode)
    if tensor.numel() == 0:
        return tensor
    std = calculate_gain(nonlinearity, a) / math.sqrt(fan)
    bound = math.sqrt(3.0) * std
    with torch.no_grad():
        return tensor.uniform_(-bound, bound)


def kaiming_normal_(P_tensor, tensor, a=0, mode="fan_in", nonlinearity="leaky_relu"):
    fan = _calculate_correct_fan(P_tensor, tensor, mode)
    if tensor.numel() == 0:
        return tensor
    std = calculate_gain(nonlinearity, a) / math.sqrt(fan)
    with torch.no_grad():
        return tensor.normal_(0, std)

"""Convolutions on spatially partitioned tensors ("feature"-distributed):
halo exchange, then the local library convolution
(``src/distdl/nn/conv_feature.py:16-431``)."""
import numpy as np
import torch
import torch.nn.functional as F

from ..utilities.slicing import assemble_slices
from ..utilities.torch import TensorStructure, distdl_padding_to_torch_padding, zero_volume_tensor
from .broadcast import Broadcast
from .halo_exchange import HaloExchange
from .mixins.conv_mixin import ConvMixin
from .mixins.halo_mixin import HaloMixin
from .module import Module


def _per_dim(v, nd):
    """A scalar or per-dimension setting as an integer array with one entry per spatial dimension."""
    a = np.atleast_1d(np.asarray(v, dtype=int))
    return a * np.ones(nd, dtype=int) if np.ndim(v) == 0 else a


class DistributedFeatureConvBase(Module, HaloMixin, ConvMixin):
    r"""Convolution of a tensor ``[batch, channel, *space]`` whose *spatial*
    dimensions are split over ``P_x = [1, 1, *P_space]``.

    Weights and bias live on worker 0 and are broadcast to all workers each
    forward.  Every worker zero-pads its sub-tensor where it touches the global
    boundary, allocates ghost regions towards its neighbours, fills them with a
    :class:`HaloExchange`, crops what its own output windows do not need
    (strided kernels) and applies the local convolution with ``padding=0``.
    Halo widths are computed from the actual (possibly unbalanced) sub-tensor
    shapes.  The local convolution is the library (cuDNN) kernel: convolution is
    not one of this framework's hand-written hot paths.
    """

    TorchConvType = None
    num_dimensions = None
    transposed = False

    def __init__(self, P_x, in_channels, out_channels, kernel_size, stride=1, padding=0, padding_mode="zeros",
                 dilation=1, groups=1, bias=True, buffer_manager=None, collect_state=False, device=None, dtype=None):
        super().__init__()
        self.P_x = P_x
        self.buffer_manager = buffer_manager or self._distdl_backend.BufferManager()
        if not P_x.active:
            return
        nd = self.num_dimensions
        exp = lambda v: _per_dim(v, nd)  # noqa: E731
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride = exp(kernel_size), exp(stride)
        self.padding, self.dilation = exp(padding), exp(dilation)
        self.padding_mode, self.groups, self.use_bias = padding_mode, groups, bias
        self.collect_state = collect_state
        device = device if device is not None else P_x.device
        self.conv_layer = self.TorchConvType(in_channels, out_channels, tuple(int(k) for k in self.kernel_size),
                                             stride=tuple(int(s) for s in self.stride), padding=0,
                                             dilation=tuple(int(d) for d in self.dilation), groups=groups, bias=bias,
                                             device=device, dtype=dtype)
        dims = P_x.dim
        self.global_padding = np.concatenate([np.zeros(dims - nd, dtype=int), self.padding])
        self.P_wb_cart = P_x.create_partition_inclusive([0]).create_cartesian_topology_partition([1])
        w0, b0 = self.conv_layer.weight.detach(), (self.conv_layer.bias.detach() if bias else None)
        del self.conv_layer.weight
        self.conv_layer.weight = None
        if bias:
            del self.conv_layer.bias
            self.conv_layer.bias = None
        if self.P_wb_cart.active:
            self.weight = torch.nn.Parameter(w0.clone())
            if bias:
                self.bias = torch.nn.Parameter(b0.clone())
            else:
                self.register_buffer("bias", None)
        else:
            # zero-volume stand-ins must require grad, or autograd would skip the adjoint of the broadcast here
            self.register_buffer("weight", zero_volume_tensor(device=device, dtype=w0.dtype, requires_grad=True))
            self.register_buffer("bias", zero_volume_tensor(device=device, dtype=w0.dtype, requires_grad=True)
                                 if bias else None)
        self.w_broadcast = Broadcast(self.P_wb_cart, P_x, preserve_batch=False)
        if bias:
            self.b_broadcast = Broadcast(self.P_wb_cart, P_x, preserve_batch=False)
        self.halo_layer = None
        self.needed_slices = None
        self.pad_tuple = None
        self._register_state_dict_hook(self.gather_state_dict)
        self._register_load_state_dict_pre_hook(self.scatter_state_dict)

    def gather_state_dict(self, module, destination, prefix, *args):
        """``collect_state=True``: only the worker that stores the kernel keeps ``weight`` / ``bias``
        in its state dict (``src/distdl/nn/conv_feature.py:215-226``)."""
        if getattr(self, "collect_state", False) and self.P_x.active and not self.P_wb_cart.active:
            destination.pop(prefix + "weight", None)
            destination.pop(prefix + "bias", None)
        return destination

    def scatter_state_dict(self, destination, prefix, *args):
        """``collect_state=True``: the other workers load their zero-volume stand-ins, whatever
        (if anything) the given state dict holds for this layer (``:228-243``)."""
        if getattr(self, "collect_state", False) and self.P_x.active and not self.P_wb_cart.active:
            destination[prefix + "weight"] = self.weight.detach().clone()
            if self.use_bias:
                destination[prefix + "bias"] = self.bias.detach().clone()
            else:
                destination.pop(prefix + "bias", None)
        return destination

    def _compute_local_padding(self, padding):
        """The global zero padding only applies where a worker touches the boundary."""
        local = np.array(padding, dtype=int)
        idx, shape = self.P_x.index, self.P_x.shape
        for d in range(self.P_x.dim):
            if idx[d] != 0:
                local[d, 0] = 0
            if idx[d] != shape[d] - 1:
                local[d, 1] = 0
        return local

    def _distdl_module_setup(self, input):
        self._distdl_is_setup = True
        self._input_tensor_structure = TensorStructure(input[0])
        if not self.P_x.active:
            return
        be = self._distdl_backend
        ts = TensorStructure(input[0])
        g = be.assemble_global_tensor_structure(ts, self.P_x)
        shapes = be.tensor_decomposition.compute_subtensor_shapes_unbalanced(ts, self.P_x)
        halo, recv, send, needed = self._compute_exchange_info(
            g.shape, self.kernel_size, self.stride, self.padding, self.dilation, True, self.P_x.shape,
            self.P_x.index, subtensor_shapes=shapes)
        dims = self.P_x.dim
        gpad = np.repeat(self.global_padding.reshape(dims, 1), 2, axis=1)
        local_pad = self._compute_local_padding(gpad)
        # the halo computed above counts the global padding as missing input at
        # the boundary: ghost regions exist only towards real neighbours
        self.halo_shape = halo
        total = local_pad + halo
        self.pad_tuple = distdl_padding_to_torch_padding(total)
        self.local_pad = local_pad
        # the exchange sees the padded tensor: the boundary padding counts as bulk offset
        halo_with_pad = halo + local_pad
        self.halo_layer = HaloExchange(self.P_x, halo_with_pad, recv, send, self.buffer_manager)
        # crop: negative halos mean leading entries this worker's windows never read
        lo = needed[:, 0]
        hi = needed[:, 1] + local_pad[:, 0] + local_pad[:, 1]
        self.needed_slices = assemble_slices(lo, hi)

    def _distdl_module_teardown(self, input):
        self.halo_layer = None
        self.needed_slices = None
        self._distdl_is_setup = False

    def _distdl_input_changed(self, input):
        return self._input_tensor_structure != TensorStructure(input[0])

    def _local_conv(self, x, w, b):
        fn = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[self.num_dimensions]
        return fn(x, w, b, stride=tuple(int(s) for s in self.stride), padding=0,
                  dilation=tuple(int(d) for d in self.dilation), groups=self.groups)

    def forward(self, input):
        if not self.P_x.active:
            return input
        w = self.w_broadcast(self.weight)
        b = self.b_broadcast(self.bias) if self.use_bias else None
        x = F.pad(input, self.pad_tuple, mode="constant", value=0)
        x = self.halo_layer(x)
        x = x[self.needed_slices]
        return self._local_conv(x, w, b)


class DistributedFeatureConv1d(DistributedFeatureConvBase):
    TorchConvType, num_dimensions = torch.nn.Conv1d, 1


class DistributedFeatureConv2d(DistributedFeatureConvBase):
    TorchConvType, num_dimensions = torch.nn.Conv2d, 2


class DistributedFeatureConv3d(DistributedFeatureConvBase):
    TorchConvType, num_dimensions = torch.nn.Conv3d, 3


class _FeatureConvTransposeBase(Module):
    r"""Transposed convolution of a tensor ``[batch, channel, *space]`` whose spatial dimensions
    are split over ``P_x = [1, 1, *P_space]``; any kernel size, stride, padding, output padding,
    dilation and groups.

    Input entry ``i`` contributes to the output entries ``i * stride - padding + dilation * j``,
    ``j < kernel``.  A worker that holds the input block ``[a, b)`` owns the output entries
    ``[a * stride - padding, b * stride - padding)`` (the last worker: up to the end; everything
    clipped to the global output).  It applies the local, unpadded transposed convolution to its
    block; where the kernel is longer than the stride, the last ``dilation * (kernel - 1) + 1 -
    stride`` entries of the result belong to the right-hand neighbour and are ADDED to its block
    by a halo exchange in accumulate mode (the adjoint of the exchange that the forward
    convolution does); the global padding is then cropped on the boundary workers and the bias
    added.  The outputs are therefore not balanced: the first worker is ``padding`` entries
    short, the last one carries the tail.

    (The reference routes the transposed classes through the halo arithmetic of the forward
    convolution, ``src/distdl/nn/conv_feature.py:442-465``, which is only meaningful when kernel
    and stride coincide, as in its example.)"""

    num_dimensions = None

    def __init__(self, P_x, in_channels, out_channels, kernel_size, stride=1, padding=0, output_padding=0, groups=1,
                 bias=True, dilation=1, buffer_manager=None, collect_state=False, device=None, dtype=None):
        super().__init__()
        self.P_x = P_x
        self.buffer_manager = buffer_manager or self._distdl_backend.BufferManager()
        if not P_x.active:
            return
        nd = self.num_dimensions
        exp = lambda v: tuple(int(a) for a in _per_dim(v, nd))  # noqa: E731
        self.in_channels, self.out_channels = in_channels, out_channels
        self.kernel_size, self.stride, self.padding = exp(kernel_size), exp(stride), exp(padding)
        self.output_padding, self.dilation, self.groups = exp(output_padding), exp(dilation), groups
        self.collect_state = collect_state
        if any(int(p) != 1 for p in P_x.shape[:P_x.dim - nd]):
            raise ValueError("only the spatial dimensions may be partitioned")
        device = device if device is not None else P_x.device
        cls = {1: torch.nn.ConvTranspose1d, 2: torch.nn.ConvTranspose2d, 3: torch.nn.ConvTranspose3d}[nd]
        ref = cls(in_channels, out_channels, self.kernel_size, stride=self.stride, padding=self.padding,
                  output_padding=self.output_padding, groups=groups, bias=bias, dilation=self.dilation, device=device,
                  dtype=dtype)
        self.use_bias = bias
        self.P_wb_cart = P_x.create_partition_inclusive([0]).create_cartesian_topology_partition([1])
        if self.P_wb_cart.active:
            self.weight = torch.nn.Parameter(ref.weight.detach().clone())
            self.bias = torch.nn.Parameter(ref.bias.detach().clone()) if bias else None
        else:
            self.register_buffer("weight",
                                 zero_volume_tensor(device=device, dtype=ref.weight.dtype, requires_grad=True))
            self.register_buffer("bias", zero_volume_tensor(device=device, dtype=ref.weight.dtype, requires_grad=True)
                                 if bias else None)
        self.w_broadcast = Broadcast(self.P_wb_cart, P_x, preserve_batch=False)
        if bias:
            self.b_broadcast = Broadcast(self.P_wb_cart, P_x, preserve_batch=False)
        # spill of a local result into the right-hand neighbour's entries, per spatial dimension
        self.spill = tuple(max(0, d * (k - 1) + 1 - s) for k, s, d in zip(self.kernel_size, self.stride, self.dilation))
        self.halo_layer = None
        self._register_state_dict_hook(DistributedFeatureConvBase.gather_state_dict.__get__(self))
        self._register_load_state_dict_pre_hook(DistributedFeatureConvBase.scatter_state_dict.__get__(self))

    def _distdl_module_setup(self, input):
        self._distdl_is_setup = True
        self._input_tensor_structure = TensorStructure(input[0])
        if not self.P_x.active:
            return
        be = self._distdl_backend
        nd, dim = self.num_dimensions, self.P_x.dim
        ts = TensorStructure(input[0])
        shapes = np.asarray(be.tensor_decomposition.compute_subtensor_shapes_unbalanced(ts, self.P_x), dtype=int)
        from ..utilities.tensor_decomposition import compute_subtensor_start_indices
        starts = compute_subtensor_start_indices(shapes)
        idx = tuple(int(i) for i in self.P_x.index)
        halo = np.zeros((dim, 2), dtype=int)
        recv = np.zeros((dim, 2), dtype=int)
        send = np.zeros((dim, 2), dtype=int)
        self.extend, self.crop = [], []
        exchange = False
        for i in range(nd):
            d = dim - nd + i
            column = shapes[idx[:d] + (slice(None),) + idx[d + 1:]][:, d]      # extents of all workers along d
            n, a, l_in = int(shapes[idx][d]), int(starts[idx][d]), int(column.sum())
            P, me = int(self.P_x.shape[d]), idx[d]
            k, s, p, op, dil, r = (self.kernel_size[i], self.stride[i], self.padding[i], self.output_padding[i],
                                   self.dilation[i], self.spill[i])
            last = me == P - 1
            l_out = (l_in - 1) * s - 2 * p + dil * (k - 1) + op + 1
            if r and P > 1:
                exchange = True
                if not last:
                    # the last r entries are the ghost region that travels to the right-hand neighbour
                    if int(column[me + 1]) * s < r:
                        raise ValueError("a worker's block is too small for the kernel of this transposed convolution")
                    halo[d, 1], recv[d, 1] = r, r
                if me > 0:
                    send[d, 0] = r                 # ... and arrives on the first r entries there
            # local result -> [own entries (n * s) | spill (r)], plus the output padding at the very end
            z_len = (n - 1) * s + dil * (k - 1) + 1
            length = max(z_len, n * s + r) + (op if last else 0)
            self.extend.append(length - z_len)
            # entry j sits at global output position a * s - p + j; keep what is inside [0, l_out) and owned
            own_end = length if last else n * s
            lo = min(max(0, p - a * s), own_end)
            hi = max(lo, min(own_end, l_out - (a * s - p)))
            self.crop.append((lo, hi))
        self.halo_layer = None
        if exchange:
            self.halo_layer = HaloExchange(self.P_x, halo, recv, send, self.buffer_manager, accumulate=True)

    def _distdl_module_teardown(self, input):
        self.halo_layer = None
        self._distdl_is_setup = False

    def _distdl_input_changed(self, input):
        return self._input_tensor_structure != TensorStructure(input[0])

    def forward(self, input):
        if not self.P_x.active:
            return input
        w = self.w_broadcast(self.weight)
        b = self.b_broadcast(self.bias) if self.use_bias else None
        nd = self.num_dimensions
        fn = {1: F.conv_transpose1d, 2: F.conv_transpose2d, 3: F.conv_transpose3d}[nd]
        z = fn(input, w, None, stride=self.stride, padding=0, output_padding=0, groups=self.groups,
               dilation=self.dilation)
        if any(self.extend):
            pad = []
            for e in reversed(self.extend):
                pad += [0, e]
            z = F.pad(z, pad)
        if self.halo_layer is not None:
            z = self.halo_layer(z)
        sl = [slice(None)] * (z.dim() - nd) + [slice(lo, hi) for lo, hi in self.crop]
        y = z[tuple(sl)]
        if b is not None:
            y = y + b.reshape([1, -1] + [1] * nd)
        return y


class DistributedFeatureConvTranspose1d(_FeatureConvTransposeBase):
    num_dimensions = 1


class DistributedFeatureConvTranspose2d(_FeatureConvTransposeBase):
    num_dimensions = 2


class DistributedFeatureConvTranspose3d(_FeatureConvTransposeBase):
    num_dimensions = 3

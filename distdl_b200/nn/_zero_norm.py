"""Shared base of the ZeRO-sharded norm layers: affine parameters are split
evenly over *all* workers of ``P_x`` along the feature dimension and
all-gathered on use."""
import numpy as np
import torch

from ..utilities.slicing import compute_subshape
from ..utilities.torch import zero_volume_tensor
from ._linear_common import KeptBufferGuard, PrefetchStream, deliver_grad, root_partition
from .all_gather import AllGather
from .module import Module
from .reduce_scatter import ReduceScatter
from .repartition import Repartition


class _ZeroNormBase(Module):
    def _setup_zero_params(self, P_x, normalized_shape, names, elementwise_affine, collect_state, device, dtype,
                           scale_backward, auto_clear_buffer):
        self.P_x = P_x
        if isinstance(normalized_shape, int):
            normalized_shape = (normalized_shape,)
        self.normalized_shape = tuple(int(s) for s in normalized_shape)
        self.elementwise_affine, self.collect_state, self.dtype = elementwise_affine, collect_state, dtype
        self.scale_backward, self.auto_clear_buffer = scale_backward, auto_clear_buffer
        self.param_names = names if elementwise_affine else ()
        dim, nn = P_x.dim, len(self.normalized_shape)
        for d in range(dim - nn, dim):
            if int(P_x.shape[d]) != 1:
                raise ValueError("The normalised dimensions must not be partitioned for ZeRO norm layers.")
        device = device if device is not None else P_x.device
        self._device = device
        if not elementwise_affine:
            for n in ("weight", "bias"):
                self.register_parameter(n, None)
            return
        # parameters sharded 1/P_x.size along the last dim on a flat [size, 1, ...] partition
        shape = [int(P_x.size)] + [1] * (dim - 1)
        self.P_w = P_x.create_partition_inclusive(range(P_x.size)).create_cartesian_topology_partition(shape)
        self.allgather = AllGather(self.P_w, axes_all_gather=(0,), scale_backward=scale_backward)
        self.reduce_scatter = ReduceScatter(self.P_w, axes_reduce_scatter=(0,))
        nfeat = int(np.prod(self.normalized_shape))
        self.num_features = nfeat
        local = int(compute_subshape(P_x.size, self.P_w.index[0], [nfeat])[0])
        pshape = [local] + [1] * (dim - 1)
        for n in ("weight", "bias"):
            if n in names:
                init = torch.ones if n == "weight" else torch.zeros
                setattr(self, n, torch.nn.Parameter(init(tuple(pshape), device=device, dtype=dtype)))
            else:
                self.register_parameter(n, None)
        self.prefetch = PrefetchStream(device)
        self._kept = KeptBufferGuard()
        self.buffers_gathered = None
        self._register_state_dict_hook(self.gather_state_dict)
        self._register_load_state_dict_pre_hook(self.scatter_state_dict)
        if collect_state:
            self.P_root = root_partition(P_x)
            self.gather = Repartition(self.P_w, self.P_root, preserve_batch=False)
            self.scatter = Repartition(self.P_root, self.P_w, preserve_batch=False)

    def reset_parameters(self):
        """Weight to one, bias to zero (``src/distdl/nn/layernorm_zero.py:162-165``)."""
        with torch.no_grad():
            for n in self.param_names:
                getattr(self, n).fill_(1.0 if n == "weight" else 0.0)
        self.buffers_gathered = None

    def extra_repr(self):
        return f"normalized_shape={self.normalized_shape}"

    def gather_state_dict(self, module, destination, prefix, *args):
        if not (self.collect_state and self.P_x.active):
            return destination
        for name in reversed(self.param_names):
            key = prefix + name
            t = self.gather(destination.pop(key).detach())
            if self.P_root.active:
                destination[key] = t.reshape(self.normalized_shape)
        return destination

    def scatter_state_dict(self, destination, prefix, *args):
        if not (self.collect_state and self.P_x.active):
            return destination
        dim = self.P_x.dim
        for name in self.param_names:
            key = prefix + name
            t = destination.pop(key, None)
            if self.P_root.active:
                t = t.reshape([self.num_features] + [1] * (dim - 1)).to(self._device)
            else:
                t = zero_volume_tensor(device=self._device, dtype=self.dtype)
            destination[key] = self.scatter(t)
        return destination

    def _collect(self):
        out = {}
        for n in self.param_names:
            full = self.allgather(getattr(self, n)).reshape(self.num_features)
            if not self.auto_clear_buffer:
                full = full.detach().requires_grad_(True)
                if full.is_cuda and full.dtype == torch.bfloat16:
                    # the fused norm backward accumulates dw / db of every micro-batch here in fp32
                    full.main_grad = torch.zeros(self.num_features, dtype=torch.float32, device=full.device)
            out[n] = full
        self.buffers_gathered = out

    def collect_weights(self):
        if not hasattr(self, "prefetch"):
            return          # a worker outside the layer's partition holds nothing
        if not self.elementwise_affine:
            return
        params = [getattr(self, n) for n in self.param_names]
        if self.buffers_gathered is not None and not self.auto_clear_buffer and self._kept.stale(*params):
            self.buffers_gathered = None
        if self.buffers_gathered is None:
            self.prefetch.run(self._collect)
            self._kept.remember(*params)

    prefetch_weights = collect_weights

    def wait_for_streams(self):
        if not hasattr(self, "prefetch"):
            return          # a worker outside the layer's partition holds nothing
        if self.elementwise_affine:
            self.prefetch.wait()

    def clear_weight_buffer(self):
        if not hasattr(self, "prefetch"):
            return          # a worker outside the layer's partition holds nothing
        if self.buffers_gathered is not None and not self.auto_clear_buffer:
            for n, full in self.buffers_gathered.items():
                g = full.grad
                if g is None:
                    g = getattr(full, "main_grad", None)
                if g is None:
                    continue
                g = g if self.scale_backward is None else g / self.scale_backward
                gl = self.reduce_scatter(g.reshape([self.num_features] + [1] * (self.P_x.dim - 1)))
                p = getattr(self, n)
                deliver_grad(p, gl)
        self.buffers_gathered = None

    def _gathered(self):
        if not self.elementwise_affine:
            return None, None
        self.collect_weights()
        self.wait_for_streams()
        g = self.buffers_gathered
        w, b = g.get("weight"), g.get("bias")
        if self.auto_clear_buffer:
            self.buffers_gathered = None
        return w, b

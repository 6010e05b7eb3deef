"""Losses on partitioned tensors (``src/distdl/nn/loss.py:10-257``)."""
import numpy as np
import torch

from ..functional.zero_volume_corrector import ZeroVolumeCorrectorFunction
from .module import Module
from .sum_reduce import SumReduce


class DistributedLossBase(Module):
    r"""Local torch loss with ``reduction='sum'``, sum-reduced onto worker 0 of
    ``P_x`` and normalised there by the global element count (``mean``) or the
    global batch size (``batchmean``).  The value lives on worker 0; the other
    workers receive a dummy scalar that they can call ``.backward()`` on, whose
    adjoint injects "nothing" (the adjoint of the sum-reduction broadcasts the
    true gradient to them)."""

    BaseLossLayer = None
    _valid_reductions = ("none", "mean", "sum", "batchmean")

    def __init__(self, P_x, reduction="mean", **kwargs):
        super().__init__()
        if reduction not in self._valid_reductions:
            raise ValueError(f"Invalid reduction mode: {reduction}.")
        self.P_x, self.reduction = P_x, reduction
        self.base_loss_function = self.BaseLossLayer(reduction="none" if reduction == "none" else "sum", **kwargs)
        if reduction == "none":
            return
        self.P_0 = P_x.create_partition_inclusive([0]).create_cartesian_topology_partition([1] * P_x.dim)
        self.sum_reduce = SumReduce(P_x, self.P_0, preserve_batch=False)
        self.normalization_factor = 1

    def _distdl_module_setup(self, input):
        self._distdl_is_setup = True
        if not self.P_x.active or self.reduction in ("none", "sum"):
            return
        local = np.array([int(np.prod(input[0].shape))], dtype=float)
        if self.reduction == "batchmean":
            # batch entries are counted once per batch-dimension worker
            first = all(int(i) == 0 for i in self.P_x.index[1:])
            local = np.array([float(input[0].shape[0]) if first else 0.0])
        self.normalization_factor = float(self.P_x.allreduce_data(local)[0])

    def forward(self, input, target):
        if not self.P_x.active:
            return input.clone()
        loss = self.base_loss_function(input, target)
        if self.reduction == "none":
            return loss
        loss = self.sum_reduce(loss.reshape([1] * self.P_x.dim))
        if self.P_0.active:
            if self.reduction != "sum":
                loss = loss / self.normalization_factor
            loss = loss.reshape(())
        return ZeroVolumeCorrectorFunction.apply(loss)


class DistributedL1Loss(DistributedLossBase):
    BaseLossLayer = torch.nn.L1Loss
    _valid_reductions = ("none", "mean", "sum")


class DistributedMSELoss(DistributedLossBase):
    BaseLossLayer = torch.nn.MSELoss
    _valid_reductions = ("none", "mean", "sum")


class DistributedPoissonNLLLoss(DistributedLossBase):
    BaseLossLayer = torch.nn.PoissonNLLLoss
    _valid_reductions = ("none", "mean", "sum")


class DistributedBCELoss(DistributedLossBase):
    BaseLossLayer = torch.nn.BCELoss
    _valid_reductions = ("none", "mean", "sum")


class DistributedBCEWithLogitsLoss(DistributedLossBase):
    BaseLossLayer = torch.nn.BCEWithLogitsLoss
    _valid_reductions = ("none", "mean", "sum")


class DistributedKLDivLoss(DistributedLossBase):
    BaseLossLayer = torch.nn.KLDivLoss
    _valid_reductions = ("none", "mean", "sum", "batchmean")

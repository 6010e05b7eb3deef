"""A decoder cut into pipeline stages.

``PipelinedDecoder(cfg, pp, dp, tp, cp)`` takes ``pp * dp * cp * tp`` workers: world ranks
``[s * G, (s + 1) * G)`` with ``G = dp * cp * tp`` form stage ``s`` and hold its share of the blocks
(:func:`~distdl_b200.models.decoder.stage_layers`), sharded inside the stage exactly like a whole
decoder (tensor / sequence / context parallel, ZeRO over the stage's data-parallel workers).  The
worker at position ``g`` of a stage hands its activation shard ``[micro, seq_local, d_model]`` to the
worker at position ``g`` of the next stage (:class:`~distdl_b200.parallel.PipelineStage`: NCCL
point-to-point on GPUs, gloo on CPU), and :meth:`PipelinedDecoder.forward_backward` runs one
optimizer step's micro-batches through the one-forward-one-backward schedule.

The reference has no pipeline parallelism (and no model code).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..parallel.pipeline import PipelineStage, run_1f1b
from ..utilities.slicing import compute_subshape
from .decoder import Decoder, DecoderConfig, ParallelLayout


class PipelinedDecoder:
    def __init__(self, cfg: DecoderConfig, pp: int, dp: int, tp: int, cp: int = 1, P_world=None):
        from .. import backends
        P_world = P_world if P_world is not None else backends.backend.Partition()
        group = dp * cp * tp
        if pp * group != P_world.size:
            raise ValueError(f"pp*dp*cp*tp = {pp * group} does not match the {P_world.size} workers")
        if pp > cfg.n_layers:
            raise ValueError("more pipeline stages than layers")
        self.cfg, self.pp = cfg, pp
        rank = int(P_world.rank)
        self.stage_index, self.position = rank // group, rank % group
        P_stage = P_world.create_partition_inclusive(range(self.stage_index * group, (self.stage_index + 1) * group))
        self.layout = ParallelLayout(dp, tp, P_world=P_stage, cp=cp)
        self.model = Decoder(cfg, self.layout, stage=(self.stage_index, pp))
        # world ranks of the workers at this position in every stage, in stage order
        self.chain = [int(P_world.ranks[s * group + self.position]) for s in range(pp)]
        self._pipe = None
        self._pipe_key = None

    @property
    def first(self):
        return self.stage_index == 0

    @property
    def last(self):
        return self.stage_index == self.pp - 1

    def parameters(self):
        return self.model.parameters()

    def _stage(self, micro, seq):
        lay, cfg = self.layout, self.cfg
        s_local = int(compute_subshape(lay.tp, lay.tp_index, [seq // lay.cp])[0])
        key = (micro, seq)                               # what every worker sees, not this worker's shard
        if self._pipe_key != key:
            if self._pipe_key is not None:
                from ..nn import reset_setup
                reset_setup(self.model)                  # a new block shape: all layers set up again together
            p = next(self.model.parameters())
            self._pipe = PipelineStage(self.model, self.chain, act_shape=(micro, s_local, cfg.d_model),
                                       act_dtype=cfg.dtype, device=p.device)
            self._pipe_key = key
        return self._pipe

    def forward_backward(self, tokens: torch.Tensor, micro_batch: int, scale: float):
        """Forward and backward of every micro-batch of ``tokens [b_local, seq + 1]`` (inputs
        ``[:, :-1]``, targets ``[:, 1:]``; every stage is given the same tensor, the first uses the
        inputs and the last the targets).  Gradients accumulate in the parameters.  Returns the
        summed loss times ``scale`` on the last stage, zero elsewhere."""
        self.model.train()
        B, seq = tokens.shape[0], tokens.shape[1] - 1
        if B % micro_batch:
            raise ValueError("the local batch must divide into micro-batches")
        n = B // micro_batch
        stage = self._stage(micro_batch, seq)
        chunks = [tokens[i * micro_batch:(i + 1) * micro_batch] for i in range(n)]
        total = run_1f1b(stage,
                         [c[:, :-1] for c in chunks] if self.first else None,
                         [c[:, 1:] for c in chunks] if self.last else None,
                         (lambda h, t: self.model.loss_from_hidden(h, t, scale, unit_grad=True)) if self.last else None,
                         n_micro=n)
        if total is None:
            p = next(self.model.parameters())
            total = torch.zeros((), dtype=torch.float32, device=p.device)
        return total.float()

    def global_loss(self, total: torch.Tensor) -> torch.Tensor:
        """Sum of the per-worker losses over the whole job (every worker gets it)."""
        total = total.clone()
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(total)
        return total

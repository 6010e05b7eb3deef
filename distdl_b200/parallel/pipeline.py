"""Pipeline parallelism: point-to-point hand-off of activations between stages
and a 1F1B micro-batch schedule.

The reference has no pipeline support (disjoint partitions plus ``Repartition``
could hand activations over, but there is no schedule).  Here the stage
boundaries use the library point-to-point path of ``torch.distributed`` (NCCL
send/recv on GPUs, gloo on CPU), issued on a side stream so that the transfer of
micro-batch ``i`` overlaps the compute of micro-batch ``i + 1``.

``PipelineStage`` wraps the module of one stage; ``run_1f1b`` drives the
schedule: warm-up forwards, steady one-forward-one-backward, cool-down
backwards.  Gradients accumulate in the parameters as with any micro-batching;
the loss (last stage) is returned as the sum over micro-batches.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist


class _Channel:
    """Ordered sends / receives with one neighbour, on a side stream on GPUs."""

    def __init__(self, peer: int, device: torch.device, group=None):
        self.peer, self.device, self.group = peer, device, group
        self.stream = torch.cuda.Stream(device=device) if device.type == "cuda" else None
        self._pending = []

    def send(self, t: torch.Tensor):
        t = t.detach().contiguous()
        if self.stream is None:
            self._pending.append((dist.isend(t, self.peer, group=self.group), t))
            return
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream):
            t.record_stream(self.stream)
            self._pending.append((dist.isend(t, self.peer, group=self.group), t))

    def recv(self, shape, dtype) -> torch.Tensor:
        out = torch.empty(tuple(shape), dtype=dtype, device=self.device)
        if self.stream is None:
            dist.recv(out, self.peer, group=self.group)
            return out
        with torch.cuda.stream(self.stream):
            work = dist.irecv(out, self.peer, group=self.group)
            work.wait()
        torch.cuda.current_stream(self.device).wait_stream(self.stream)
        return out

    def flush(self):
        for work, _ in self._pending:
            work.wait()
        self._pending.clear()
        if self.stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)


class PipelineStage:
    """One stage of a pipeline over the ordered world ranks ``stage_ranks``.

    ``module`` maps the stage input to the stage output; the first stage gets the
    micro-batch itself, the last stage's output goes to ``loss_fn(output,
    target)``.  ``act_shape`` / ``act_dtype`` describe the activation of ONE
    micro-batch that crosses a stage boundary (all boundaries alike)."""

    def __init__(self, module: torch.nn.Module, stage_ranks: Sequence[int], act_shape, act_dtype=torch.float32,
                 device: Optional[torch.device] = None, group=None):
        self.module = module
        self.ranks = list(stage_ranks)
        self.rank = dist.get_rank()
        self.index = self.ranks.index(self.rank)
        self.first, self.last = self.index == 0, self.index == len(self.ranks) - 1
        self.act_shape, self.act_dtype = tuple(act_shape), act_dtype
        if device is None:
            p = next(module.parameters(), None)
            device = p.device if p is not None else torch.device("cpu")
        self.device = device
        self.prev = None if self.first else _Channel(self.ranks[self.index - 1], device, group)
        self.next = None if self.last else _Channel(self.ranks[self.index + 1], device, group)

    # one micro-batch forward: returns (input that needs a gradient or None, output)
    def forward_step(self, micro_input):
        if self.first:
            x = micro_input
        else:
            x = self.prev.recv(self.act_shape, self.act_dtype).requires_grad_(True)
        y = self.module(x)
        if not self.last:
            self.next.send(y)
        return x, y

    def backward_step(self, x, y, loss=None):
        if self.last:
            loss.backward()
        else:
            gy = self.next.recv(self.act_shape, self.act_dtype)
            y.backward(gy)
        if not self.first:
            self.prev.send(x.grad)

    def flush(self):
        for ch in (self.prev, self.next):
            if ch is not None:
                ch.flush()


def run_1f1b(stage: PipelineStage, micro_inputs: Optional[List[torch.Tensor]], micro_targets: Optional[List] = None,
             loss_fn: Optional[Callable] = None, n_micro: Optional[int] = None) -> Optional[torch.Tensor]:
    """Runs one optimizer step's worth of micro-batches through the pipeline with
    the one-forward-one-backward schedule.  ``micro_inputs`` is needed on the
    first stage, ``micro_targets`` and ``loss_fn`` on the last; every stage passes
    the same ``n_micro`` (or a list of that length).  Returns the summed loss on
    the last stage, ``None`` elsewhere."""
    n = n_micro if n_micro is not None else len(micro_inputs if micro_inputs is not None else micro_targets)
    S = len(stage.ranks)
    warm = min(S - 1 - stage.index, n)
    queue = []                                   # (x, y, loss) of forwards whose backward is pending
    total = None
    fwd = 0

    def do_forward():
        nonlocal fwd, total
        x, y = stage.forward_step(micro_inputs[fwd] if stage.first else None)
        loss = None
        if stage.last:
            loss = loss_fn(y, micro_targets[fwd])
            total = loss.detach() if total is None else total + loss.detach()
        queue.append((x, y, loss))
        fwd += 1

    for _ in range(warm):
        do_forward()
    for _ in range(n - warm):
        do_forward()
        x, y, loss = queue.pop(0)
        stage.backward_step(x, y, loss)
    while queue:
        x, y, loss = queue.pop(0)
        stage.backward_step(x, y, loss)
    stage.flush()
    return total

"""Rank-0 JSONL metrics sink: one line per training step (step, loss, step time as the
maximum over ranks, tokens/s of the whole job, learning rate, gradient norm) plus
free-form records.  The reference has logging only (``src/distdl/logger.py``)."""
from __future__ import annotations

import json
import time

import torch
import torch.distributed as dist


class MetricsSink:
    def __init__(self, path: str, every: int = 1):
        self.path, self.every = path, max(1, int(every))
        self.rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        self._fh = open(path, "a", buffering=1) if self.rank == 0 else None
        self._t_last = None

    def record(self, **fields):
        if self._fh is not None:
            fields.setdefault("time", time.time())
            self._fh.write(json.dumps(fields) + "\n")

    def step(self, step: int, loss, tokens: int, lr: float = None, grad_norm=None, device=None):
        """Call once per optimizer step.  Reads ``loss`` (a device scalar) only on steps that
        are logged; the step time is the wall time between logged calls divided by the
        number of steps in between, reduced with MAX over the ranks."""
        now = time.time()
        if step % self.every:
            return
        ms = None
        if self._t_last is not None:
            t = torch.tensor([(now - self._t_last[0]) * 1e3 / max(1, step - self._t_last[1])], device=device or "cpu")
            if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        self._t_last = (now, step)
        self.record(step=int(step), loss=float(loss), ms_per_step=ms,
                    tokens_per_s=(tokens / (ms / 1e3)) if ms else None, lr=lr,
                    grad_norm=None if grad_norm is None else float(grad_norm))

    def close(self):
        if self._fh is not None:
            self._fh.close()
            self._fh = None

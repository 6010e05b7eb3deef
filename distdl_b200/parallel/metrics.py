"""Rank-0 JSONL metrics sink: one line per training step (step, loss, step time as the
maximum over ranks, tokens/s of the whole job, learning rate, gradient norm; with
``flops_per_token`` also the model TFLOP/s per GPU and, with ``peak_tflops``, the fraction of
that peak; with ``device_waits`` the milliseconds this rank's fused kernels spent waiting for
other GPUs since the last logged step, by kind) plus free-form records.  The reference has
logging only (``src/distdl/logger.py``)."""
from __future__ import annotations

import json
import time

import torch
import torch.distributed as dist


class MetricsSink:
    def __init__(self, path: str, every: int = 1, flops_per_token: float = None, peak_tflops: float = None,
                 device_waits: bool = False):
        self.path, self.every = path, max(1, int(every))
        self.flops_per_token, self.peak_tflops, self.device_waits = flops_per_token, peak_tflops, device_waits
        self.world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
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
        tps = (tokens / (ms / 1e3)) if ms else None
        extra = {}
        if self.flops_per_token and tps:
            extra["model_tflops_per_gpu"] = tps * self.flops_per_token / self.world / 1e12
            if self.peak_tflops:
                extra["fraction_of_peak"] = extra["model_tflops_per_gpu"] / self.peak_tflops
        if self.device_waits and torch.cuda.is_available():
            from .. import _native
            waits = _native.read_wait_ns()          # reads and clears; synchronises the device
            extra["wait_ms"] = {k: v / 1e6 for k, v in waits.items() if v}
        self.record(step=int(step), loss=float(loss), ms_per_step=ms, tokens_per_s=tps, lr=lr,
                    grad_norm=None if grad_norm is None else float(grad_norm), **extra)

    def close(self):
        if self._fh is not None:
            self._fh.close()
            self._fh = None

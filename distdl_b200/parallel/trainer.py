"""Training step driver: pinned-host input staging, micro-batching with fp32
gradient accumulation, fused optimizer step, device-side loss."""
from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

from .optimizer import FlatAdamW, cosine_lr


class Trainer:
    """``Trainer(model, ...).step(tokens_host)`` runs one optimizer step.

    ``tokens_host`` is this worker's ``[local_batch, seq + 1]`` int64 token block
    in pinned host memory (tensor-parallel peers of one data-parallel group must
    be given the same block).  Inputs are ``tokens[:, :-1]``, targets
    ``tokens[:, 1:]``.  The local batch is cut into ``micro_batch`` sequences
    per forward/backward.  Returns the mean token loss of the global batch as a
    device scalar (read it with ``.item()`` when the host needs it).
    """

    def __init__(self, model, global_tokens_per_step: int, micro_batch: int = 1, lr: float = 3e-4,
                 weight_decay: float = 0.1, max_grad_norm: float = 1.0, warmup_steps: int = 10,
                 total_steps: int = 1000, device=None, metrics=None, health_check_every: int = 50, heartbeat=None):
        # a models.PipelinedDecoder: this process trains its stage, micro-batches run through the 1F1B schedule
        self.pipeline = model if hasattr(model, "forward_backward") else None
        if self.pipeline is not None:
            model = self.pipeline.model
        self.model = model
        self.heartbeat = heartbeat      # a parallel.health.Heartbeat: checked before every step, so that a
                                        # missing rank raises RankFailure here instead of hanging a collective
        self.health_check_every = health_check_every   # steps between reads of the device status record
        self.metrics = metrics          # a parallel.metrics.MetricsSink, or None
        self.micro_batch = micro_batch
        self.global_tokens = global_tokens_per_step
        self.opt = FlatAdamW(model, lr=lr, weight_decay=weight_decay, max_grad_norm=max_grad_norm)
        self.base_lr, self.warmup_steps, self.total_steps = lr, warmup_steps, total_steps
        self.device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
                                 else torch.device("cpu"))
        self._dev_tokens = None
        self._last_shape = None
        self.steps_done = 0

    def stage(self, tokens_host: torch.Tensor) -> torch.Tensor:
        """Asynchronous host -> device copy into a reused device buffer."""
        if self._dev_tokens is None or self._dev_tokens.shape != tokens_host.shape:
            self._dev_tokens = torch.empty(tokens_host.shape, dtype=tokens_host.dtype, device=self.device)
        self._dev_tokens.copy_(tokens_host, non_blocking=True)
        return self._dev_tokens

    def step_device(self, tokens: torch.Tensor) -> torch.Tensor:
        if self.heartbeat is not None:
            self.heartbeat.check()
        if self._last_shape is not None and tuple(tokens.shape) != self._last_shape:
            # a new block shape is seen by every process, but not every process's shard changes with it:
            # make all layers set up again together
            from ..nn import reset_setup
            reset_setup(self.model)
        self._last_shape = tuple(tokens.shape)
        self.model.train()
        self.opt.set_lr(cosine_lr(self.steps_done, self.base_lr, self.warmup_steps, self.total_steps))
        total = torch.zeros((), dtype=torch.float32, device=tokens.device)
        scale = 1.0 / float(self.global_tokens)
        B = tokens.shape[0]
        if self.pipeline is not None:
            total += self.pipeline.forward_backward(tokens, self.micro_batch, scale).to(total.device)
        else:
            for lo in range(0, B, self.micro_batch):
                mb = tokens[lo:lo + self.micro_batch]
                if lo + self.micro_batch >= B:
                    self.opt.begin_last_micro_batch()     # gradients are final block by block from here on
                # the loss is back-propagated as it is (gradient 1), which the fused cross-entropy may rely on
                loss = self.model.loss(mb[:, :-1], mb[:, 1:], scale=scale, unit_grad=True)
                loss.backward()
                total += loss.detach().float()
        self.opt.step()
        self.steps_done += 1
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(total)
        if (self.health_check_every and tokens.is_cuda and self.steps_done % self.health_check_every == 0):
            from . import symm
            symm.check_health()       # raises DeviceTimeout if a kernel gave up waiting for a peer
        if self.metrics is not None:
            self.metrics.step(self.steps_done, total, self.global_tokens, lr=self.opt.lr,
                              grad_norm=self.opt.last_grad_norm, device=tokens.device)
        return total

    def step(self, tokens_host: torch.Tensor) -> torch.Tensor:
        return self.step_device(self.stage(tokens_host))

    # ------------------------------------------------------------ checkpoints
    def save_checkpoint(self, directory: str, extra: dict = None):
        """Writes ``rank<r>.pt`` (this worker's shards: model ``state_dict``, fp32 master
        weights and moments, step counters, RNG states) and, on rank 0, ``manifest.json``
        (world size, step, parallel layout and model configuration when the model has
        them).  Collective: every worker calls it; returns after all files are written."""
        os.makedirs(directory, exist_ok=True)
        rank = dist.get_rank() if dist.is_initialized() else 0
        world = dist.get_world_size() if dist.is_initialized() else 1
        state = {"model": self.model.state_dict(), "optimizer": self.opt.state_dict(), "steps_done": self.steps_done,
                 "rng_cpu": torch.get_rng_state(),
                 "rng_cuda": torch.cuda.get_rng_state() if torch.cuda.is_available() else None}
        torch.save(state, os.path.join(directory, f"rank{rank}.pt"))
        if rank == 0:
            layout = getattr(self.model, "layout", None)
            cfg = getattr(self.model, "cfg", None)
            manifest = {"world_size": world, "steps_done": self.steps_done,
                        "layout": None if layout is None else {"dp": layout.dp, "tp": layout.tp,
                                                               "cp": getattr(layout, "cp", 1)},
                        "model": None if cfg is None else {k: (str(v) if isinstance(v, torch.dtype) else v)
                                                           for k, v in vars(cfg).items()},
                        "files": [f"rank{r}.pt" for r in range(world)], "extra": extra or {}}
            with open(os.path.join(directory, "manifest.json"), "w") as fh:
                json.dump(manifest, fh, indent=1)
        if dist.is_initialized() and world > 1:
            dist.barrier()

    def load_checkpoint(self, directory: str) -> dict:
        """Restores what :meth:`save_checkpoint` wrote on the same worker grid; returns the
        manifest.  (To move between grids, save the model with ``collect_state=True``
        layers and load that serial ``state_dict``.)"""
        rank = dist.get_rank() if dist.is_initialized() else 0
        world = dist.get_world_size() if dist.is_initialized() else 1
        with open(os.path.join(directory, "manifest.json")) as fh:
            manifest = json.load(fh)
        if manifest["world_size"] != world:
            raise ValueError(f"checkpoint was written by {manifest['world_size']} workers, this job has {world}")
        state = torch.load(os.path.join(directory, f"rank{rank}.pt"), map_location=self.device, weights_only=False)
        self.model.load_state_dict(state["model"])
        self.opt.load_state_dict(state["optimizer"])
        self.steps_done = int(state["steps_done"])
        torch.set_rng_state(state["rng_cpu"].cpu())
        if state.get("rng_cuda") is not None and torch.cuda.is_available():
            torch.cuda.set_rng_state(state["rng_cuda"].cpu())
        if dist.is_initialized() and world > 1:
            dist.barrier()
        return manifest


    # ------------------------------------------- checkpoints that move between worker grids
    def save_model_collected(self, path: str):
        """Writes the SERIAL model state (one file, written by the first worker) of a model whose layers
        were built with ``collect_state=True`` (``DecoderConfig.collect_state``), together with the step
        count.  Collective.  The file loads on any worker grid with :meth:`load_model_collected`."""
        state = self.model.state_dict()                     # collective: the hooks gather onto worker 0
        rank = dist.get_rank() if dist.is_initialized() else 0
        if rank == 0:
            if not state:
                raise ValueError("the model has no collected state: build its layers with collect_state=True")
            torch.save({"model": {k: v.detach().cpu() for k, v in state.items()}, "steps_done": self.steps_done},
                       path)
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()

    def load_model_collected(self, path: str, keep_step_count: bool = True):
        """Loads a file written by :meth:`save_model_collected`, on this job's worker grid whatever grid
        wrote it: the first worker reads it, the layers' hooks scatter it.  The optimizer restarts from
        these weights with cleared moments (they were sharded for the old grid)."""
        rank = dist.get_rank() if dist.is_initialized() else 0
        meta = [None]
        if rank == 0:
            blob = torch.load(path, map_location="cpu", weights_only=False)
            self.model.load_state_dict(blob["model"])
            meta[0] = int(blob["steps_done"])
        else:
            self.model.load_state_dict({})
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.broadcast_object_list(meta, src=0)
        self.opt.sync_master_from_params(reset_moments=True)
        if keep_step_count:
            self.steps_done = meta[0]                       # the learning-rate schedule continues


class SyntheticTokens:
    """Uniform random token blocks in pinned host memory.  Every call of
    :meth:`next` draws fresh tokens into the next of a few pinned buffers
    (round-robin, so a buffer is not rewritten while its asynchronous copy may
    still be in flight); the stream of blocks depends on (seed, data-parallel
    index) only, so tensor-parallel peers see identical data."""

    def __init__(self, local_batch, seq, vocab, dp_index=0, seed=0, n_buffers=4):
        self.vocab = vocab
        self.gen = torch.Generator().manual_seed(seed * 100003 + dp_index * 1009 + 17)
        self.blocks = []
        for _ in range(n_buffers):
            t = torch.empty((local_batch, seq + 1), dtype=torch.int64)
            if torch.cuda.is_available():
                t = t.pin_memory()
            torch.randint(0, vocab, t.shape, generator=self.gen, out=t)
            self.blocks.append(t)
        self.i = 0

    def next(self):
        t = self.blocks[self.i % len(self.blocks)]
        if self.i >= len(self.blocks):
            torch.randint(0, self.vocab, t.shape, generator=self.gen, out=t)
        self.i += 1
        return t

    @property
    def bytes_per_block(self):
        return self.blocks[0].numel() * self.blocks[0].element_size()

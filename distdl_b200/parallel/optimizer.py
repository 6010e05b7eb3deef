"""Mixed-precision AdamW over flat buffers.

The bf16 working parameters of a model are re-homed as views into one flat
bf16 buffer; fp32 master weights, both Adam moments and the fp32 gradient
accumulator are flat buffers of the same length.  Because every distributed
layer stores each parameter element on exactly one worker (ZeRO shards, or the
owning data-parallel row), these buffers *are* the sharded optimizer state: no
extra partitioning step is needed.  One fused kernel per parameter group does
the whole update (moments, decoupled weight decay, master update, bf16
refresh, gradient clearing).  Gradients reach the accumulator through
post-accumulate hooks, so micro-batches are summed in fp32.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from .. import _native, ops
from ..ops._util import stream_ptr, use_native


class FlatAdamW:
    def __init__(self, model: torch.nn.Module, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1,
                 max_grad_norm=1.0, no_decay=("norm", "bias")):
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.step_count = 0
        self._release = getattr(model, "release_gathered", None)
        params = [(n, p) for n, p in model.named_parameters() if p.requires_grad and p.numel() > 0]
        decay = [(n, p) for n, p in params if not any(k in n for k in no_decay)]
        plain = [(n, p) for n, p in params if any(k in n for k in no_decay)]
        self.groups = []
        ordered = decay + plain
        if not ordered:
            self.total = 0
            return
        device, dtype = ordered[0][1].device, ordered[0][1].dtype
        offsets, off = [], 0
        for _, p in ordered:
            offsets.append(off)
            off += (p.numel() + 7) // 8 * 8          # 16-byte alignment of every bf16 view
        self.total = off
        n_decay = offsets[len(decay)] if len(decay) < len(ordered) else off
        self.param_flat = torch.zeros(off, dtype=dtype, device=device)
        self.master = torch.zeros(off, dtype=torch.float32, device=device)
        self.exp_avg = torch.zeros(off, dtype=torch.float32, device=device)
        self.exp_avg_sq = torch.zeros(off, dtype=torch.float32, device=device)
        self.grad = torch.zeros(off, dtype=torch.float32, device=device)
        self._hooks = []
        self.names = []
        for (name, p), o in zip(ordered, offsets):
            n = p.numel()
            view = self.param_flat[o:o + n].view(p.shape)
            view.copy_(p.data)
            p.data = view
            self.master[o:o + n].copy_(view.reshape(-1))
            p.main_grad_view = self.grad[o:o + n]
            self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(p)))
            self.names.append((name, o, n))
        self.groups = [(0, n_decay, weight_decay), (n_decay, off - n_decay, 0.0)]
        self._norm_sq = torch.zeros(1, dtype=torch.float32, device=device)
        self._clip = torch.ones(1, dtype=torch.float32, device=device)
        self.last_grad_norm = None

    @staticmethod
    def _make_hook(p):
        def hook(param):
            g = param.grad
            if g is None:
                return
            ops.optim.accumulate_f32_(param.main_grad_view, g)
            param.grad = None
        return hook

    def set_lr(self, lr):
        self.lr = lr

    def step(self, grad_scale: float = 1.0):
        """Applies one AdamW update from the accumulated fp32 gradients (which are
        cleared).  With ``max_grad_norm`` the global gradient norm is computed
        over all workers and the clipping coefficient stays on the device.
        A model that keeps gathered ZeRO parameters across micro-batches
        (``release_gathered``) is asked to flush their gradients first."""
        if self._release is not None:
            self._release()
        if self.total == 0:
            if self.max_grad_norm and dist.is_initialized() and dist.get_world_size() > 1:
                dist.all_reduce(torch.zeros(1, device="cuda" if torch.cuda.is_available() else "cpu"))
            return
        self.step_count += 1
        clip_ptr = None
        if self.max_grad_norm:
            self._norm_sq.zero_()
            ops.sumsq_(self.grad, self._norm_sq)
            if dist.is_initialized() and dist.get_world_size() > 1:
                dist.all_reduce(self._norm_sq)
            norm = self._norm_sq.sqrt() * grad_scale
            self.last_grad_norm = norm
            torch.clamp(self.max_grad_norm / (norm + 1e-6), max=1.0, out=self._clip)
            clip_ptr = self._clip
        b1, b2 = self.betas
        for start, length, wd in self.groups:
            if length == 0:
                continue
            sl = slice(start, start + length)
            ops.adamw_step_(self.master[sl], self.exp_avg[sl], self.exp_avg_sq[sl], self.grad[sl],
                            self.param_flat[sl], lr=self.lr, beta1=b1, beta2=b2, eps=self.eps, weight_decay=wd,
                            step=self.step_count, grad_scale_tensor=clip_ptr, grad_scale=grad_scale, zero_grad=True)

    def zero_grad(self):
        if self.total:
            self.grad.zero_()

    # ------------------------------------------------------------ checkpoints
    def state_dict(self):
        """Per-worker (sharded) optimizer state."""
        return {"step": self.step_count, "master": self.master, "exp_avg": self.exp_avg,
                "exp_avg_sq": self.exp_avg_sq, "layout": list(self.names)}

    def load_state_dict(self, sd):
        self.step_count = int(sd["step"])
        if self.total:
            self.master.copy_(sd["master"])
            self.exp_avg.copy_(sd["exp_avg"])
            self.exp_avg_sq.copy_(sd["exp_avg_sq"])
            self.param_flat.copy_(self.master)


def cosine_lr(step, base_lr, warmup, total, min_ratio=0.1):
    if step < warmup:
        return base_lr * (step + 1) / max(1, warmup)
    t = min(1.0, (step - warmup) / max(1, total - warmup))
    return base_lr * (min_ratio + (1 - min_ratio) * 0.5 * (1 + math.cos(math.pi * t)))

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
import os

import torch
import torch.distributed as dist

from .. import _native, ops
from ..ops._util import stream_ptr


class FlatAdamW:
    def __init__(self, model: torch.nn.Module, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1,
                 max_grad_norm=1.0, no_decay=("norm", "bias")):
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.max_grad_norm = max_grad_norm
        self.step_count = 0
        self._by_block, self._armed, self._block_done, self._updated_ranges, self._all_blocks = {}, False, set(), [], []
        self._release = getattr(model, "release_gathered", None)
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        decay = [(n, p) for n, p in named if not any(k in n for k in no_decay)]
        plain = [(n, p) for n, p in named if any(k in n for k in no_decay)]
        self.groups = []
        ordered = decay + plain
        multi = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
        # Slot sizes: with identical parameter lists on every process the slots take the
        # largest local size, so that a parameter sits at the SAME offset everywhere (the
        # native transport then gathers ZeRO shards by reading the peers' buffers in place).
        sizes = [p.numel() for _, p in ordered]
        self.uniform_layout = False
        if multi:
            # every process takes part, also one that holds no trainable parameter (an inactive worker)
            table = [None] * dist.get_world_size()
            dist.all_gather_object(table, [(n, p.numel()) for n, p in ordered])
            if all([n for n, _ in t] == [n for n, _ in table[0]] for t in table):
                sizes = [max(t[i][1] for t in table) for i in range(len(ordered))]
                self.uniform_layout = True
                if not ordered:
                    self.total = 0          # no process has a parameter: all of them leave here together
                    self._symmetric, self._full, self._full_any = False, [], False
                    return
            else:
                sizes = self._grouped_sizes(ordered, table, sizes)
        if not self.uniform_layout:
            keep = [i for i, (_, p) in enumerate(ordered) if p.numel() > 0]
            n_dec = sum(1 for i in keep if i < len(decay))
            ordered = [ordered[i] for i in keep]
            sizes = [sizes[i] for i in keep]
            decay = ordered[:n_dec]
        if not multi and (not ordered or sum(sizes) == 0):
            self.total = 0
            self._symmetric, self._full, self._full_any = False, [], False
            return
        have = [p for _, p in ordered if p.numel() > 0]
        ref = have[0] if have else (ordered[0][1] if ordered else None)
        if ref is not None:
            device, dtype = ref.device, ref.dtype
        else:                                  # a process without parameters still joins the collective steps below
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() \
                else torch.device("cpu")
            dtype = None
        offsets, off = [], 0
        for sz in sizes:
            offsets.append(off)
            off += (sz + 7) // 8 * 8          # 16-byte alignment of every bf16 view
        self.total = off
        n_decay = offsets[len(decay)] if len(decay) < len(ordered) else off
        self.param_flat = self._alloc_params(off, dtype, device, multi)
        self.master = torch.zeros(off, dtype=torch.float32, device=device)
        self.exp_avg = torch.zeros(off, dtype=torch.float32, device=device)
        self.exp_avg_sq = torch.zeros(off, dtype=torch.float32, device=device)
        self.grad = torch.zeros(off, dtype=torch.float32, device=device)
        self._hooks = []
        self.names = []
        for (name, p), o in zip(ordered, offsets):
            n = p.numel()
            if n == 0:
                continue
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
        self._setup_full_grads(ordered)
        self._setup_overlap(model, ordered)
        self._publish()

    def _grouped_sizes(self, ordered, table, sizes):
        """Parameter lists that differ between processes (pipeline stages): processes with the same
        list form a group, and the slots take the largest size within the group.  That keeps every
        parameter at one offset throughout its group, which is enough for the in-place gathers as long
        as no ZeRO gather team reaches outside its group; every process checks its own teams and the
        layout is used only if all of them agree (the decision must be the same everywhere, because
        allocating the peer-mapped buffer is collective)."""
        rank = dist.get_rank()
        names = [[n for n, _ in t] for t in table]
        group = [r for r in range(len(table)) if names[r] == names[rank]]
        ok = True
        for _, p in ordered:
            gather = getattr(p, "zero_gather", None)
            if gather is None or not gather.P_x.active:
                continue
            team = gather.P_x.create_allreduction_partition(gather.axes_all_gather).ranks
            ok = ok and all(int(r) in group for r in team)
        verdicts = [None] * len(table)
        dist.all_gather_object(verdicts, bool(ok))
        if not all(verdicts):
            return sizes
        self.uniform_layout = True
        self.layout_group = group
        return [max(table[r][i][1] for r in group) for i in range(len(ordered))]

    def _alloc_params(self, numel, dtype, device, multi):
        """The flat bf16 parameter buffer; in peer-mapped memory on the native backend.  Allocating
        peer-mapped memory is collective, so the processes first agree on it: each reports whether
        its own parameters qualify (a process without parameters always does) and the peer-mapped
        buffer is used only if all do."""
        self._symmetric = False
        if multi:
            local_ok = bool(self.uniform_layout and device.type == "cuda" and dtype in (torch.bfloat16, None)
                            and dist.get_world_size() <= 8 and os.environ.get("DISTDL_SYMM_PARAMS", "1") != "0")
            if local_ok:
                from . import symm
                local_ok = symm.heap_ready()
            votes = [None] * dist.get_world_size()
            dist.all_gather_object(votes, local_ok)
            if all(votes):
                from . import symm
                region = symm.SymmetricRegion(symm.heap(), numel * 2)
                symm.register_param_region(region)
                self._region = region
                self._symmetric = True
                return region.tensor(numel, torch.bfloat16)
        return torch.zeros(numel, dtype=dtype or torch.float32, device=device)

    def _setup_full_grads(self, ordered):
        """Unsharded fp32 gradient accumulators for the ZeRO weight matrices (peer-mapped):
        the weight-gradient GEMMs of all micro-batches add into them and ``step()``
        reduce-scatters them once, each worker reading its slice of every peer's
        accumulator in place, instead of one reduce-scatter per layer and micro-batch."""
        self._full = []
        self._full_any = False              # some process has such accumulators: all join the step's barriers
        self._full_region = None
        if not self._symmetric or os.environ.get("DISTDL_FULL_GRADS", "1") == "0":
            return
        plan, off = [], 0
        for _, p in ordered:
            gather = getattr(p, "zero_gather", None)
            if gather is None or p.numel() == 0 or p.numel() % 8 or not hasattr(p, "main_grad_view"):
                continue
            axis = gather.axes_all_gather[0]
            if int(gather.P_x.shape[axis]) <= 1 or gather.scale_backward is not None or not gather.P_x.active:
                continue
            team = tuple(int(r) for r in gather.P_x.create_allreduction_partition(gather.axes_all_gather).ranks)
            if len(team) <= 1 or len(team) > 8:
                continue
            plan.append((p, off, p.numel(), team, team.index(dist.get_rank())))
            off += len(team) * p.numel()
        # the allocation is collective: every process takes part as soon as one needs it, and the
        # slot layout must agree within every team (same model structure everywhere)
        needs = [None] * dist.get_world_size()
        dist.all_gather_object(needs, [(n, len(t)) for _, _, n, t, _ in plan])
        if not any(needs):
            return
        filled = [x for x in needs if x]
        if any(x != filled[0] for x in filled):
            return                      # differing layouts: keep the per-micro-batch reduce-scatter
        from . import symm
        self._full_any = True
        region = symm.SymmetricRegion(symm.heap(), max(off, 4) * 4)
        self._full_region = region
        self._full_flat = region.tensor(off, torch.float32)
        self._full_flat.zero_()
        for p, o, n, team, me in plan:
            p.full_grad_view = self._full_flat[o:o + len(team) * n]
            self._full.append((p, o, n, team, me))

    # ------------------------------------------------- reduction overlapped with the backward pass
    def _setup_overlap(self, model, ordered):
        """Groups the unsharded accumulators by the model's blocks, so that a block's gradients can be
        reduced (and, without gradient clipping, applied) as soon as that block has finished the
        backward pass of the step's last micro-batch, while the blocks before it are still busy.
        Needs a model that reports the end of a block's backward pass (``add_block_backward_hook``,
        parameter names ``blocks.<i>.``) and the same grouping on every process."""
        import re
        hook = getattr(model, "add_block_backward_hook", None)
        if not self._full_any or os.environ.get("DISTDL_OVERLAP_GRADS", "1") == "0":
            return
        names = {id(p): n for n, p in ordered}
        for entry in self._full:
            mt = re.search(r"(?:^|\.)blocks\.(\d+)\.", names.get(id(entry[0]), ""))
            if mt is not None:
                self._by_block.setdefault(int(mt.group(1)), []).append(entry)
        # collective agreement: the barriers of the per-block reduction involve every process
        table = [None] * dist.get_world_size()
        dist.all_gather_object(table, (hook is not None, sorted((b, len(v)) for b, v in self._by_block.items())))
        filled = [t for t in table if t[1]]
        if not all(t[0] for t in table) or any(t[1] != filled[0][1] for t in filled):
            self._by_block = {}
            return
        self._all_blocks = [b for b, _ in filled[0][1]] if filled else []
        hook(self._on_block_backward_done)

    def begin_last_micro_batch(self):
        """The next backward pass is the last one before :meth:`step`: from now on a block's
        accumulated gradients are final as soon as its backward pass ends.  (``Trainer`` calls
        this; without the call everything is reduced inside :meth:`step`.)"""
        if self._by_block or getattr(self, "_all_blocks", None):
            self._armed = True
            self._block_done = set()
            self._updated_ranges = []

    def _on_block_backward_done(self, block):
        if not self._armed or block in self._block_done or block not in getattr(self, "_all_blocks", ()):
            return
        import ctypes
        from . import collectives
        self._block_done.add(block)
        # every process of the job has finished this block's backward pass: the peers' accumulators
        # of the block are complete, and nobody reads the block's parameter shards any more
        collectives.barrier(list(range(dist.get_world_size())))
        lib = _native.lib()
        reg = self._full_region
        stream = stream_ptr()
        fused = not self.max_grad_norm
        b1, b2 = self.betas
        for p, o, n, team, me in self._by_block.get(block, ()):
            srcs = (ctypes.c_void_p * len(team))(*[reg.ptrs[r] + 4 * (o + me * n) for r in team])
            g = p.main_grad_view
            _native.launch_count += 1
            if fused:
                lo = (g.data_ptr() - self.grad.data_ptr()) // 4
                wd = self.weight_decay if lo < self.groups[0][1] else 0.0
                _native.check(lib.dd_grad_rs_adamw(
                    len(team), srcs, g.data_ptr(), self.master[lo:lo + n].data_ptr(), self.exp_avg[lo:lo + n].data_ptr(),
                    self.exp_avg_sq[lo:lo + n].data_ptr(), self.param_flat[lo:lo + n].data_ptr(), n, self.lr, b1, b2,
                    self.eps, wd, self.step_count + 1, None, 1.0, stream), "dd_grad_rs_adamw")
                self._updated_ranges.append((lo, n))
            else:
                _native.check(lib.dd_rs_pull_f32(len(team), srcs, g.data_ptr(), n, 1.0, stream), "dd_rs_pull_f32")

    def _reduce_full_grads(self):
        if not self._full_any:
            return
        import ctypes
        from . import collectives
        from .. import _native
        everyone = list(range(dist.get_world_size()))
        collectives.barrier(everyone)                  # all accumulators of this step are complete
        lib = _native.lib()
        reg = self._full_region
        stream = stream_ptr()
        done = set()
        if self._armed:
            for b in self._block_done:
                done.update(id(e[0]) for e in self._by_block.get(b, ()))
        for p, o, n, team, me in self._full:
            if id(p) in done:
                continue                               # reduced while the backward pass was still running
            srcs = (ctypes.c_void_p * len(team))(*[reg.ptrs[r] + 4 * (o + me * n) for r in team])
            _native.launch_count += 1
            _native.check(lib.dd_rs_pull_f32(len(team), srcs, p.main_grad_view.data_ptr(), n, 1.0, stream),
                          "dd_rs_pull_f32")
        collectives.barrier(everyone)                  # nobody reads my accumulators any more
        if self._full:
            self._full_flat.zero_()

    def reduce_gradients(self):
        """Brings every gradient of this step into the sharded fp32 accumulator: flushes the
        parameters that the model keeps gathered and reduce-scatters the unsharded
        accumulators.  ``step()`` calls it; collective over all processes."""
        if self._release is not None:
            self._release()
        self._reduce_full_grads()

    def _publish(self):
        """After the parameters changed: no process may read a peer's shard in place
        before every process has finished writing its own."""
        if self._symmetric:
            from . import collectives
            collectives.barrier(list(range(dist.get_world_size())))

    def _quiesce(self):
        """Before the parameters change: every process has finished reading."""
        if self._symmetric:
            from . import collectives
            collectives.barrier(list(range(dist.get_world_size())))

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
        self.reduce_gradients()
        if self.total == 0:
            # nothing to update here, but the other processes' collective steps still need this one
            multi = dist.is_initialized() and dist.get_world_size() > 1
            if self.max_grad_norm and multi:
                dist.all_reduce(torch.zeros(1, device="cuda" if torch.cuda.is_available() else "cpu"))
            elif multi:
                self._quiesce()
            if multi:
                self._publish()
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
        if not self.max_grad_norm:
            self._quiesce()           # (the all-reduce of the gradient norm already orders the processes)
        for start, length, wd in self.groups:
            for lo, n in self._remaining(start, length):
                sl = slice(lo, lo + n)
                ops.adamw_step_(self.master[sl], self.exp_avg[sl], self.exp_avg_sq[sl], self.grad[sl],
                                self.param_flat[sl], lr=self.lr, beta1=b1, beta2=b2, eps=self.eps, weight_decay=wd,
                                step=self.step_count, grad_scale_tensor=clip_ptr, grad_scale=grad_scale,
                                zero_grad=True)
        self._armed = False
        self._updated_ranges = []
        self._publish()

    def _remaining(self, start, length):
        """The parts of ``[start, start + length)`` that the per-block fused updates of this step
        have not already taken care of, as (offset, length) runs."""
        if length <= 0:
            return []
        taken = sorted((lo, n) for lo, n in getattr(self, "_updated_ranges", ()) if lo < start + length and lo + n > start)
        out, at = [], start
        for lo, n in taken:
            if lo > at:
                out.append((at, lo - at))
            at = max(at, lo + n)
        if at < start + length:
            out.append((at, start + length - at))
        return out

    def zero_grad(self):
        if self.total:
            self.grad.zero_()
            if getattr(self, "_full", None):
                self._full_flat.zero_()

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
            self._quiesce()
            self.param_flat.copy_(self.master)
            self._publish()


    def sync_master_from_params(self, reset_moments: bool = True):
        """After the model's parameters were overwritten in place (``model.load_state_dict`` of a
        checkpoint written on another worker grid): takes the fp32 master weights from the parameters
        and, by default, clears the moments and the step count (they belong to the old sharding)."""
        if self.total:
            self._quiesce()
            self.master.copy_(self.param_flat)
            if reset_moments:
                self.exp_avg.zero_()
                self.exp_avg_sq.zero_()
            self._publish()
        if reset_moments:
            self.step_count = 0


def cosine_lr(step, base_lr, warmup, total, min_ratio=0.1):
    if step < warmup:
        return base_lr * (step + 1) / max(1, warmup)
    t = min(1.0, (step - warmup) / max(1, total - warmup))
    return base_lr * (min_ratio + (1 - min_ratio) * 0.5 * (1 + math.cos(math.pi * t)))

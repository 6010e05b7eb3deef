"""Decoder-only transformer assembled from the distributed layers.

One class covers the three model families of the benchmark configurations:

* Llama-style: RMSNorm, rotary embedding, grouped-query attention, SwiGLU, no biases;
* GPT-2-style: LayerNorm, learned positions, multi-head attention, GELU, biases;
* Mixtral-style: Llama attention with a top-k routed mixture-of-experts FFN.

Parallel layout (``D`` data-parallel x ``M`` tensor-parallel workers):
activations between blocks are ``[batch / D, seq / M, d]`` (sequence
parallel); QKV and the first FFN GEMM are column-parallel layers that
all-gather the sequence, the output projection and second FFN GEMM are
row-parallel layers that reduce-scatter it back.  With ``zero=True`` every
weight is additionally sharded over the ``D`` workers (ZeRO-3 / FSDP) and
gathered on use.  Token embedding, final norm and the LM head work on the
sequence-sharded tokens as pure data parallelism over all ``D * M`` workers with
their weights ZeRO-sharded over all of them, so that the loss needs no
tensor-parallel communication.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass

import numpy as np
import torch
import torch.utils.checkpoint

from .. import nn as dnn
from .. import ops
from ..utilities import recompute
from ..utilities.slicing import compute_start_index, compute_subshape


@dataclass
class DecoderConfig:
    vocab_size: int = 128256
    d_model: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn_dim: int = 14336
    max_seq: int = 4096
    norm: str = "rms"            # "rms" | "layer"
    activation: str = "swiglu"   # "swiglu" | "gelu"
    rope: bool = True
    rope_theta: float = 500000.0
    bias: bool = False
    eps: float = 1e-5
    n_experts: int = 0           # > 0: mixture-of-experts FFN
    top_k: int = 2
    capacity_factor: float = 1.25
    dtype: torch.dtype = torch.bfloat16
    checkpoint_blocks: bool = True    # False: never recompute a block (the same as activation_policy="none")
    activation_policy: str = "auto"   # which blocks keep their activations for the backward pass:
                                      # "auto"  as many (counted from the last block) as the free device memory
                                      #         holds, the others recompute their forward pass in backward;
                                      # "full"  every block recomputes; "none" every block keeps;
                                      # an integer (or a string of digits): that many blocks keep.
                                      # A block that keeps stores the outputs of its GEMMs and of attention;
                                      # norm outputs and the activation function's output are rebuilt
    zero: bool = True
    keep_gathered: bool = False  # gather ZeRO shards once per optimizer step, reduce-scatter gradients once
    keep_root_gathered: bool = True   # the same for the embedding, final norm and head only (each is used
                                      # once per pass, so re-sharding them between micro-batches buys nothing)
    keep_norms_gathered: bool = True  # and for the norm weights of the blocks (a few KB each)
    prefetch: bool = True             # gather the next block's ZeRO weights while the current block computes
    init_std: float = 0.02
    cp_mode: str = "ring"             # context-parallel attention: "ring" (K / V blocks travel), "zigzag" (the
                                      # ring on the load-balanced layout: worker r holds chunks r and 2 cp - 1 - r
                                      # of every sequence) or "a2a" (head <-> sequence all-to-all; the local
                                      # head counts must divide by cp)
    collect_state: bool = False       # state_dict() / load_state_dict() in the serial layout on the first worker:
                                      # a checkpoint that loads on any worker grid

    @property
    def head_dim(self):
        return self.d_model // self.n_heads

    def padded_vocab(self, multiple=128):
        return (self.vocab_size + multiple - 1) // multiple * multiple

    def num_parameters(self):
        d, f, L = self.d_model, self.ffn_dim, self.n_layers
        hd = self.head_dim
        attn = d * (self.n_heads + 2 * self.n_kv_heads) * hd + self.n_heads * hd * d
        ffn = (3 if self.activation == "swiglu" else 2) * d * f
        if self.n_experts:
            ffn = ffn * self.n_experts + d * self.n_experts
        emb = 2 * self.vocab_size * d + (0 if self.rope else self.max_seq * d)
        return L * (attn + ffn + 2 * d) + emb + d

    def train_flops_per_token(self, seq: int = None):
        """Model FLOPs of one training token (forward + backward, no recomputation): 6 per weight
        that takes part in a matrix product (of the experts only the ``top_k`` that a token
        visits; the embedding lookup is not a product, the head is) plus causal attention."""
        seq = self.max_seq if seq is None else seq
        d, f, L, hd = self.d_model, self.ffn_dim, self.n_layers, self.head_dim
        attn = d * (self.n_heads + 2 * self.n_kv_heads) * hd + self.n_heads * hd * d
        ffn = (3 if self.activation == "swiglu" else 2) * d * f
        if self.n_experts:
            ffn = ffn * self.top_k + d * self.n_experts
        weights = L * (attn + ffn) + self.vocab_size * d
        # scores and context: 2 products of seq x head_dim per head and token, half of them masked
        attention = L * 2 * 2 * seq * self.n_heads * hd * 0.5
        return 6.0 * weights + 3.0 * attention


class ParallelLayout:
    """The partitions a decoder needs, derived from a ``[D, C, M]`` worker grid: ``D`` data-parallel
    replicas, ``C`` context-parallel workers that each hold one block of every sequence, ``M``
    tensor-parallel workers.  To every layer but attention a context-parallel worker is one more
    data-parallel worker (its "batch" is a block of the sequence), so parameters, gradients and
    optimizer state are ZeRO-sharded over ``D * C`` workers and only attention (ring over ``C``)
    and the token positions know about ``C``."""

    def __init__(self, dp: int, tp: int, P_world=None, cp: int = 1):
        from .. import backends
        be = backends.backend
        P_world = P_world if P_world is not None else be.Partition()
        if dp * cp * tp != P_world.size:
            raise ValueError(f"dp*cp*tp = {dp * cp * tp} does not match the {P_world.size} workers")
        base = P_world.create_partition_inclusive(range(P_world.size))
        self.dp, self.tp, self.cp = dp, tp, cp
        rows = dp * cp                                 # workers that differ in the data they see
        self.shard = rows
        self.P_world = P_world
        self.P_grid = base.create_cartesian_topology_partition([rows, tp])
        self.P_feat = base.create_cartesian_topology_partition([rows, 1, tp])
        self.P_seq = base.create_cartesian_topology_partition([rows, tp, 1])
        self.P_flat = base.create_cartesian_topology_partition([rows * tp, 1, 1])
        self.P_flat2 = base.create_cartesian_topology_partition([rows * tp, 1])
        row = int(self.P_grid.index[0])
        self.dp_index, self.cp_index = row // cp, row % cp
        self.tp_index = int(self.P_grid.index[1])
        # [data, sequence block, heads, 1]: the ring of a worker = same data and head shard
        self.P_ring = base.create_cartesian_topology_partition([dp, cp, tp, 1]) if cp > 1 else None


def _norm(cfg, P, zero, keep=None):
    keep = (cfg.keep_gathered or cfg.keep_norms_gathered) if keep is None else keep
    if cfg.norm == "rms":
        return dnn.DistributedRMSNormZero(P, cfg.d_model, eps=cfg.eps, dtype=cfg.dtype,
                                          auto_clear_buffer=not keep, collect_state=cfg.collect_state)
    if zero:
        return dnn.DistributedLayerNormZero(P, cfg.d_model, eps=cfg.eps, dtype=cfg.dtype,
                                            auto_clear_buffer=not keep, collect_state=cfg.collect_state)
    return dnn.DistributedLayerNorm(P, cfg.d_model, eps=cfg.eps, dtype=cfg.dtype, collect_state=cfg.collect_state)


def _col(cfg, layout, fin, fout, **kw):
    cls = dnn.DistributedLinearAllGatherZero if cfg.zero else dnn.DistributedLinearAllGather
    if cfg.zero:
        kw["auto_clear_buffer"] = not cfg.keep_gathered
    return cls(layout.P_feat, fin, fout, bias=cfg.bias, dtype=cfg.dtype, P_x=layout.P_seq,
               collect_state=cfg.collect_state, **kw)


def _row(cfg, layout, fin, fout, **kw):
    cls = dnn.DistributedLinearReduceScatterZero if cfg.zero else dnn.DistributedLinearReduceScatter
    if cfg.zero:
        kw["auto_clear_buffer"] = not cfg.keep_gathered
    return cls(layout.P_feat, fin, fout, bias=cfg.bias, dtype=cfg.dtype, P_y=layout.P_seq,
               collect_state=cfg.collect_state, **kw)


class Attention(torch.nn.Module):
    def __init__(self, cfg: DecoderConfig, layout: ParallelLayout):
        super().__init__()
        self.cfg, self.layout = cfg, layout
        hd = cfg.head_dim
        self.hq = int(compute_subshape(layout.tp, layout.tp_index, [cfg.n_heads])[0])
        self.hkv = int(compute_subshape(layout.tp, layout.tp_index, [cfg.n_kv_heads])[0])
        self.qkv = _col(cfg, layout, cfg.d_model, (cfg.n_heads + 2 * cfg.n_kv_heads) * hd, num_heads=cfg.n_heads,
                        num_heads_kv=cfg.n_kv_heads)
        self.out = _row(cfg, layout, cfg.n_heads * hd, cfg.d_model, num_heads=cfg.n_heads)
        self.ring = None
        if layout.cp > 1:
            if cfg.cp_mode == "a2a":
                self.ring = dnn.DistributedSelfAttention(layout.P_ring, causal=True)
            else:
                self.ring = dnn.DistributedRingAttention(layout.P_ring, causal=True, zigzag=cfg.cp_mode == "zigzag")

    def forward(self, x, remake=None):
        """``remake``: a function that rebuilds ``x`` (the norm's output), so that the projection
        need not store it for its backward pass."""
        cfg = self.cfg
        with recompute.saved_as_recipe(x, remake):
            qkv = self.qkv(x)                                 # [b, s, (hq + 2 hkv) * hd]
        del x
        b, s = qkv.shape[0], qkv.shape[1]
        lay3 = (b * s, self.hq + 2 * self.hkv, cfg.head_dim)
        if self.ring is None:
            if cfg.rope:
                qkv = ops.rope_(qkv, s, self.hq + self.hkv, cfg.rope_theta, layout=lay3)
            o = ops.attention_packed(qkv.reshape(lay3), self.hq, self.hkv, b, s, causal=True)
        else:
            # context parallel: s is this worker's block of the sequence; positions are global
            if cfg.rope and cfg.cp_mode == "zigzag":
                qkv = ops.rope_(qkv, s, self.hq + self.hkv, cfg.rope_theta, layout=lay3,
                                ranges=zigzag_ranges(self.layout.cp, self.layout.cp_index, s * self.layout.cp))
            elif cfg.rope:
                qkv = ops.rope_(qkv, s, self.hq + self.hkv, cfg.rope_theta, offset=self.layout.cp_index * s,
                                layout=lay3)
            t = qkv.reshape(b, s, self.hq + 2 * self.hkv, cfg.head_dim)
            q, k, v = t.split([self.hq, self.hkv, self.hkv], dim=2)
            o = self.ring(q.contiguous(), k.contiguous(), v.contiguous())
        return self.out(o.reshape(b, s, self.hq * cfg.head_dim))


class MLP(torch.nn.Module):
    def __init__(self, cfg: DecoderConfig, layout: ParallelLayout):
        super().__init__()
        self.cfg = cfg
        if cfg.activation == "swiglu":
            self.up = _col(cfg, layout, cfg.d_model, 2 * cfg.ffn_dim, geglu=True)
        else:
            self.up = _col(cfg, layout, cfg.d_model, cfg.ffn_dim)
        self.down = _row(cfg, layout, cfg.ffn_dim, cfg.d_model)

    def forward(self, x, remake=None):
        act = ops.swiglu if self.cfg.activation == "swiglu" else ops.gelu
        with recompute.saved_as_recipe(x, remake):
            h = self.up(x)
        del x
        a = act(h)
        # the second GEMM saves its input: rebuilt from h, which the activation's backward keeps anyway
        with recompute.saved_as_recipe(a, (lambda: act(h)) if recompute.rebuilds_activation_output() else None):
            return self.down(a)


class Block(torch.nn.Module):
    def __init__(self, cfg: DecoderConfig, layout: ParallelLayout):
        super().__init__()
        self.norm1 = _norm(cfg, layout.P_seq, cfg.zero)
        self.attn = Attention(cfg, layout)
        self.norm2 = _norm(cfg, layout.P_seq, cfg.zero)
        if cfg.n_experts:
            from .moe import MoEFeedForward
            self.mlp = MoEFeedForward(cfg, layout)
        else:
            self.mlp = MLP(cfg, layout)

    def forward(self, x, delta=None):
        """``x``: the residual stream, ``delta``: what the block before this one still has to add to
        it (its feed-forward output), or None.  Returns the pair in the same form: the stream after
        the attention branch was added, and this block's feed-forward output.  Every residual add
        thereby runs inside the norm kernel that follows it."""
        keep = recompute.rebuilds_norm_outputs()   # this block keeps its activations: norm outputs are rebuilt in backward
        if delta is None:
            n1 = self.norm1(x)
        else:
            x, n1 = _add_norm(self.norm1, x, delta)
        a = self.attn(n1, remake=(lambda x=x: self.norm1(x)) if keep else None)
        del n1
        x, n2 = _add_norm(self.norm2, x, a)
        del a
        if isinstance(self.mlp, MLP):
            return x, self.mlp(n2, remake=(lambda x=x: self.norm2(x)) if keep else None)
        return x, self.mlp(n2)

    def kept_bytes(self, cfg, layout, b, s):
        """(bytes this block stores from forward to backward for a micro-batch of ``b`` sequences of
        ``s`` tokens when it keeps its activations, bytes it needs for a moment while its backward or
        its recomputation runs)."""
        e = torch.empty((), dtype=cfg.dtype).element_size()
        tp = layout.tp
        d, hd = cfg.d_model, cfg.head_dim
        tok, tok_loc = b * s, b * s // tp
        hq, hkv = -(-cfg.n_heads // tp), -(-cfg.n_kv_heads // tp)
        x = tok_loc * d * e
        gathered = tok * d * e if tp > 1 else 0              # the fused all-gather GEMM keeps the gathered input
        qkv = tok * (hq + 2 * hkv) * hd * e
        o = tok * hq * hd * e + tok * hq * 4
        ffn = cfg.ffn_dim * (2 if cfg.activation == "swiglu" else 1)
        h = tok * (-(-ffn // tp)) * e
        if cfg.n_experts:
            h = int(h * cfg.top_k * cfg.capacity_factor * 1.5) + 4 * tok * d * e
        kept = 2 * x + 2 * gathered + qkv + o + h
        import os
        if os.environ.get("DISTDL_FORCE_TORCH", "0") == "1":
            # the library operators keep more: the rotary embedding is not in place (a second copy of the
            # projection), silu(gate) and its product are separate tensors, attention keeps fp32 statistics
            kept += 2 * qkv + h + 2 * x
        moment = 2 * h + 2 * qkv + 6 * tok * d * e
        # what storing the cheap outputs as well would add: the activation function's output, and
        # (where the projections save their input itself, i.e. without tensor parallelism) both norm outputs
        self.activation_out_bytes = h // 2 if cfg.activation == "swiglu" else h
        self.norm_out_bytes = 2 * x if tp == 1 else 0
        return kept, moment

    def prefetch(self):
        """Starts gathering the ZeRO weight shards of this block's linear layers (a no-op for
        layers whose weights are already gathered or that are not ZeRO layers)."""
        for m in (self.attn.qkv, self.attn.out, getattr(self.mlp, "up", None), getattr(self.mlp, "down", None)):
            fn = getattr(m, "prefetch_weights", None)
            if fn is not None:
                fn()


def _add_norm(norm, x, delta):
    """``(x + delta, norm(x + delta))``, fused where the norm layer can take a residual."""
    if hasattr(norm, "_gathered"):
        return norm(x, residual=delta)
    s = x + delta
    return s, norm(s)


def zigzag_ranges(cp: int, cp_index: int, seq: int):
    """The two position ranges ``((start, length), (start, length))`` that context-parallel worker
    ``cp_index`` holds of a sequence of ``seq`` tokens in the load-balanced layout."""
    if seq % (2 * cp):
        raise ValueError(f"sequence length {seq} must divide by twice the context-parallel size {cp}")
    c = seq // (2 * cp)
    return (cp_index * c, c), ((2 * cp - 1 - cp_index) * c, c)


def stage_layers(n_layers: int, stage: int, n_stages: int):
    """Half-open range of the blocks that pipeline stage ``stage`` of ``n_stages`` owns (balanced:
    the first stages get the extra blocks)."""
    lo = int(compute_start_index(n_stages, stage, [n_layers])[0])
    return lo, lo + int(compute_subshape(n_stages, stage, [n_layers])[0])


class Decoder(torch.nn.Module):
    """``forward(tokens [b_local, seq]) -> hidden [b_local, seq / M, d]``;
    ``loss(tokens, targets)`` runs the LM head and the fused cross-entropy.

    ``stage=(i, n)`` builds pipeline stage ``i`` of ``n`` only: its share of the blocks, the
    embedding on the first stage, the final norm and the head on the last.  ``forward`` of a
    later stage takes the hidden state of the stage before it instead of token ids; ``layout`` then
    describes the workers of THIS stage (``ParallelLayout(..., P_world=<the stage's partition>)``)."""

    def __init__(self, cfg: DecoderConfig, layout: ParallelLayout, stage=(0, 1)):
        super().__init__()
        self.cfg, self.layout = cfg, layout
        self.stage_index, self.n_stages = int(stage[0]), int(stage[1])
        self.first_stage, self.last_stage = self.stage_index == 0, self.stage_index == self.n_stages - 1
        V = cfg.padded_vocab()
        self.padded_vocab = V
        keep_root = cfg.keep_gathered or cfg.keep_root_gathered
        if self.first_stage:
            self.embed = dnn.DistributedEmbeddingZero(layout.P_flat2, V, cfg.d_model, dtype=cfg.dtype,
                                                      auto_clear_buffer=not keep_root,
                                                      collect_state=cfg.collect_state)
            if not cfg.rope:
                self.pos_embed = dnn.DistributedEmbeddingZero(layout.P_flat2, cfg.max_seq, cfg.d_model,
                                                              dtype=cfg.dtype, auto_clear_buffer=not keep_root,
                                                              collect_state=cfg.collect_state)
        lo, hi = stage_layers(cfg.n_layers, self.stage_index, self.n_stages)
        self.layer_range = (lo, hi)
        self.blocks = torch.nn.ModuleList(Block(cfg, layout) for _ in range(hi - lo))
        self._block_backward_hooks = []
        if self.last_stage:
            self.final_norm = _norm(cfg, layout.P_flat, True, keep=keep_root)
            self.head = dnn.DistributedLinearAllGatherZero(layout.P_flat, cfg.d_model, V, bias=False, dtype=cfg.dtype,
                                                           auto_clear_buffer=not keep_root,
                                                           collect_state=cfg.collect_state)
        self.reset_parameters()

    def reset_parameters(self):
        cfg = self.cfg
        std = cfg.init_std
        with torch.no_grad():
            for name, p in self.named_parameters():
                if p.numel() == 0:
                    continue
                if name.endswith("bias"):
                    p.zero_()
                elif "norm" in name:
                    if name.endswith("weight"):
                        p.fill_(1.0)
                elif name.endswith("weight"):
                    s = std / math.sqrt(2 * cfg.n_layers) if (".out." in name or ".down." in name) else std
                    p.normal_(0.0, s)

    def _backward_prefetch(self, i, done=None):
        block = self.blocks[i] if i >= 0 else None

        def hook(_grad):
            if done is not None:
                for fn in self._block_backward_hooks:
                    fn(done)
            if block is not None:
                # (with gradient tracking on: where weight gradients travel through autograd, a
                # recomputed block must see the gather as part of its graph)
                with torch.enable_grad():
                    block.prefetch()
        return hook

    def add_block_backward_hook(self, fn):
        """``fn(i)`` is called during every backward pass as soon as block ``i`` (index within this
        stage) has finished its backward pass, i.e. when all its parameter gradients of this
        micro-batch are complete (in order ``n - 1, ..., 0``).  An optimizer uses it to reduce and
        apply a block's gradients while the blocks before it are still in their backward pass."""
        self._block_backward_hooks.append(fn)

    def _blocks_that_keep(self, tokens):
        """How many blocks (counted from the last) keep their activations for the backward pass; the
        others recompute their forward pass.  Decided once per input shape from
        ``cfg.activation_policy``; with "auto", from the device memory that is free at this moment (the
        optimizer's state is allocated by then) and agreed over the decoder's workers (the smallest answer
        wins), because a recomputed block repeats its collective kernels and its tensor-parallel
        peers must do the same."""
        cfg = self.cfg
        n = len(self.blocks)
        key = tuple(tokens.shape)
        plan = getattr(self, "_keep_plan", None)
        if plan is not None and plan["shape"] == key:
            return plan["keep"]
        policy = str(cfg.activation_policy) if cfg.checkpoint_blocks else "none"
        b = int(tokens.shape[0])
        s = int(tokens.shape[1]) // (self.layout.cp if self.first_stage else 1)
        if not self.first_stage:
            s *= self.layout.tp                       # a later stage is handed the sequence-parallel shard
        kept, moment = self.blocks[0].kept_bytes(cfg, self.layout, b, s) if n else (0, 0)
        plan = {"shape": key, "policy": policy, "bytes_per_kept_block": kept, "blocks": n}
        if policy == "full":
            keep = 0
        elif policy == "none" or n == 0:
            keep = n
        elif policy.isdigit():
            keep = min(n, int(policy))
        elif not tokens.is_cuda:
            keep = n
        else:
            free, _total = torch.cuda.mem_get_info()
            free += torch.cuda.memory_reserved() - torch.cuda.memory_allocated()
            rows = b * s // self.layout.tp
            head = int(2.5 * rows * self.padded_vocab * 2) if self.last_stage else 0
            if os.environ.get("DISTDL_FORCE_TORCH", "0") == "1":
                head = int(3.2 * head)         # the library loss keeps fp32 logits, their log-softmax and its gradient
            slack = 4 << 30
            budget = free - head - moment - kept - slack
            keep = max(0, min(n, int(budget // max(kept, 1))))
            plan["free_bytes"] = int(free)
            # memory to spare after every block keeps: store cheap outputs too instead of rebuilding them,
            # the activation function's output first (rebuilding it moves three times its size, a norm
            # output twice its size)
            left = budget - n * kept - (6 << 30) if keep == n else -1
            act_b, norm_b = (int(getattr(self.blocks[0], a, 0)) for a in ("activation_out_bytes", "norm_out_bytes"))
            spare_act = int(left >= n * act_b)
            left -= n * act_b if spare_act else 0
            spare_norm = int(left >= n * norm_b)
            # agreed among the workers of this decoder (of this pipeline stage) through the control plane
            agreed = self.layout.P_grid.allreduce_data(np.asarray([keep, spare_act, spare_norm], dtype=np.int64),
                                                       op="min")
            keep = int(agreed[0])
            plan["stores_activation_output"] = bool(agreed[1]) and keep == n
            plan["stores_norm_outputs"] = bool(agreed[2]) and keep == n
        plan["keep"] = keep
        self._keep_plan = plan
        return keep

    @property
    def activation_plan(self):
        """The last decision of the activation planner: ``{"keep": blocks that keep their
        activations, "blocks": all blocks, "bytes_per_kept_block": ..., "policy": ...}`` (None before
        the first training forward pass)."""
        return getattr(self, "_keep_plan", None)

    def release_gathered(self):
        """With ``keep_gathered``: reduce-scatters the gradients accumulated on the
        gathered parameters into the shards and drops the gathered copies.  Call
        once per optimizer step, after the last micro-batch's backward."""
        for m in self.modules():
            clear = getattr(m, "clear_weight_buffer", None)
            if clear is not None:
                clear()

    def _local_tokens(self, tokens):
        """This worker's part of the token ids ``[b_local, seq]`` (the same on all context- and
        tensor-parallel workers of a data-parallel replica): its context-parallel block of the
        sequence, and of that its sequence-parallel shard.  Returns (ids, global start position), or
        (ids, tensor of global positions) in the zigzag layout, where the ids are not contiguous."""
        lay = self.layout
        s = tokens.shape[1]
        base = 0
        if lay.cp > 1 and self.cfg.cp_mode == "zigzag":
            (a0, c), (a1, _) = zigzag_ranges(lay.cp, lay.cp_index, s)
            pos = torch.cat([torch.arange(a0, a0 + c), torch.arange(a1, a1 + c)])
            lo = int(compute_start_index(lay.tp, lay.tp_index, [2 * c])[0])
            n = int(compute_subshape(lay.tp, lay.tp_index, [2 * c])[0])
            pos = pos[lo:lo + n].to(tokens.device)
            return tokens.index_select(1, pos), pos
        if lay.cp > 1:
            if s % lay.cp:
                raise ValueError(f"sequence length {s} must divide by the context-parallel size {lay.cp}")
            s //= lay.cp
            base = lay.cp_index * s
        lo = base + int(compute_start_index(lay.tp, lay.tp_index, [s])[0])
        n = int(compute_subshape(lay.tp, lay.tp_index, [s])[0])
        return tokens[:, lo:lo + n], lo

    def forward(self, tokens):
        cfg = self.cfg
        if self.first_stage:
            # every worker sees the shape of the token block change, but not every worker's shard changes
            # with it: the layers' collective set-up has to run again on all of them
            shape = tuple(tokens.shape)
            if getattr(self, "_seen_shape", shape) != shape:
                dnn.reset_setup(self)
            self._seen_shape = shape
            local, lo = self._local_tokens(tokens)
            x = self.embed(local)
            if not cfg.rope:
                pos = lo if torch.is_tensor(lo) else torch.arange(lo, lo + local.shape[1], device=tokens.device)
                x = x + self.pos_embed(pos.unsqueeze(0).expand_as(local))
        else:
            x = tokens                                 # the hidden state handed over by the stage before
        n = len(self.blocks)
        n_keep = self._blocks_that_keep(tokens) if (self.training and torch.is_grad_enabled()) else n
        pre = cfg.prefetch and cfg.zero and not cfg.keep_gathered

        def run(x, delta, i):
            return self.blocks[i](x, delta)

        notify = bool(self._block_backward_hooks) and self.training and torch.is_grad_enabled()
        if notify and n and x.requires_grad:
            x.register_hook(self._backward_prefetch(-1, done=0))     # the input of block 0
        delta = None
        for i in range(n):
            if pre and i + 1 < n:
                self.blocks[i + 1].prefetch()
            if i < n - n_keep:
                x, delta = torch.utils.checkpoint.checkpoint(run, x, delta, i, use_reentrant=False)
            else:
                plan = getattr(self, "_keep_plan", None) or {}
                with recompute.enabled(norms=not plan.get("stores_norm_outputs", False),
                                       activation=not plan.get("stores_activation_output", False)):
                    x, delta = self.blocks[i](x, delta)
            if delta.requires_grad and ((pre and i > 0) or (notify and i + 1 < n)):
                # the gradient of block i's feed-forward output is ready when the backward pass of block
                # i + 1 is complete and that of block i begins: tell the listeners, and start gathering the
                # weights of block i - 1
                delta.register_hook(self._backward_prefetch(i - 1 if pre else -1,
                                                            done=i + 1 if notify and i + 1 < n else None))
        if pre and n and self.training and torch.is_grad_enabled():
            self.blocks[n - 1].prefetch()          # the first block of the backward pass
        if not self.last_stage:
            return x if delta is None else x + delta
        if delta is None:
            return self.final_norm(x)
        return _add_norm(self.final_norm, x, delta)[1]

    def loss(self, tokens, targets, scale=None, unit_grad=False):
        """Sum of this worker's token losses times ``scale`` (default: 1 / local
        tokens); ``targets`` has the same [b_local, seq] shape as ``tokens``.

        ``unit_grad=True`` is a promise that the returned loss is back-propagated as it is
        (``loss.backward()`` with gradient 1; fold any weighting into ``scale``): the fused
        cross-entropy has already written ``scale * d loss / d logits`` over the logits, and the
        backward pass then hands that buffer on without a multiplication.  With the default the
        incoming gradient is applied, so ``(loss * k).backward()`` is correct as well."""
        return self.loss_from_hidden(self.forward(tokens), targets, scale, unit_grad)

    @torch.no_grad()
    def generate(self, tokens, n_new: int):
        """Greedy continuation of ``tokens [b_local, seq]`` (the same on all workers of a data-parallel
        replica) by ``n_new`` tokens; returns ``[b_local, seq + n_new]`` on every worker.  A reference
        implementation for checking a trained model: every step recomputes the whole prefix (there is no
        key / value cache), the worker that holds the last position picks the token and the replica's
        workers agree on it through the control plane.  Contiguous layouts only (not ``cp_mode="zigzag"``)."""
        if self.n_stages != 1:
            raise ValueError("generate() runs on an unpipelined decoder")
        if self.layout.cp > 1 and self.cfg.cp_mode == "zigzag":
            raise ValueError("generate() needs a contiguous sequence layout")
        lay = self.layout
        was_training = self.training
        self.eval()
        # the workers that see the same sequences: one row of the [dp, cp * tp] grid
        base = lay.P_grid.create_partition_inclusive(range(lay.P_grid.size))
        replica = base.create_cartesian_topology_partition([lay.dp, lay.cp * lay.tp]).create_allreduction_partition((1,))
        for _ in range(n_new):
            s = tokens.shape[1]
            pad = (-s) % lay.cp                          # context parallelism wants equal blocks
            inp = torch.nn.functional.pad(tokens, (0, pad)) if pad else tokens
            dnn.reset_setup(self)                        # the length grows: not every worker's shard does
            h = self.forward(inp)
            local, lo = self._local_tokens(inp)
            pick = np.zeros(tokens.shape[0], dtype=np.int64)
            if lo <= s - 1 < lo + local.shape[1]:        # this worker holds the last real position
                logits = self.head(h[:, s - 1 - lo:s - lo])
                pick = logits[:, 0, :cfg_vocab(self.cfg)].float().argmax(-1).cpu().numpy().astype(np.int64)
            else:
                self.head(h[:, :1])                      # the head's gathers are collective: take part
            pick = replica.allreduce_data(pick)          # zeros from everybody but the owner
            tokens = torch.cat([tokens, torch.as_tensor(pick, device=tokens.device).unsqueeze(1)], dim=1)
        self.release_gathered()
        self.train(was_training)
        return tokens

    def loss_from_hidden(self, h, targets, scale=None, unit_grad=False):
        """The head and the cross-entropy on the output ``h`` of :meth:`forward` (last stage);
        ``unit_grad`` as in :meth:`loss`."""
        tl, _ = self._local_tokens(targets)
        logits = self.head(h)
        rows = logits.shape[0] * logits.shape[1]
        logits2 = logits.reshape(rows, logits.shape[-1])
        return ops.cross_entropy_(logits2, tl.reshape(-1), vocab=cfg_vocab(self.cfg), scale=scale,
                                  unit_grad=unit_grad)


def cfg_vocab(cfg):
    return cfg.vocab_size

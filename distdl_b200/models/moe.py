"""Mixture-of-experts feed-forward block with expert parallelism.

Top-k softmax router -> slot assignment with a capacity limit -> permuted
scatter into per-expert buffers -> all-to-all over the expert-parallel team
(device kernel over peer memory on the native backend) -> grouped SwiGLU expert
GEMMs on the tcgen05 kernel -> all-to-all back -> weighted combine.  Experts are
split evenly over the workers of the data-parallel dimension; the router is a
ZeRO-sharded linear layer.  The reference has the expert GEMMs only
(``src/distdl/nn/linear_ag_expert.py``, ``linear_rs_expert.py``); routing,
dispatch and combine are new.
"""
from __future__ import annotations

import math
import os

import torch
import torch.distributed as dist

from .. import nn as dnn
from .. import ops
from ..ops import moe as moe_ops
from ..ops.gemm import gemm


class _BatchedLinearFn(torch.autograd.Function):
    """y[e] = x[e] @ w[e].T for bf16 CUDA tensors, all three GEMMs on the native kernel."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return gemm(x, w)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = gemm(dy, w.transpose(1, 2))
        dw = gemm(dy.transpose(1, 2), x.transpose(1, 2))
        return dx, dw


def batched_linear(x, w):
    """x [E, rows, in], w [E, out, in] -> [E, rows, out]."""
    if x.is_cuda and x.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and w.shape[2] % 8 == 0 and x.shape[1] % 8 == 0:
        return _BatchedLinearFn.apply(x.contiguous(), w)
    return torch.einsum("ecm,enm->ecn", x, w)


class _AllToAllFn(torch.autograd.Function):
    """Equal-block all-to-all over a team; its adjoint is the same exchange."""

    @staticmethod
    def forward(ctx, x, ranks):
        ctx.ranks = ranks
        return _all_to_all(x, ranks)

    @staticmethod
    def backward(ctx, g):
        return _all_to_all(g.contiguous(), ctx.ranks), None


def _all_to_all(x, ranks):
    if len(ranks) == 1:
        return x
    from .. import backends
    if x.is_cuda and getattr(backends.backend, "name", "") == "native_cupy":
        from ..parallel import collectives
        return collectives.all_to_all(x, ranks)
    out = torch.empty_like(x)
    if x.is_cuda:
        from ..backends.common.transport import GroupTransport
        dist.all_to_all_single(out, x.contiguous(), group=GroupTransport().subgroup(ranks))
        return out
    from ..backends.common.transport import control_transport
    t = control_transport()
    me = dist.get_rank()
    sends = [(r, x[i]) for i, r in enumerate(ranks) if r != me]
    recvs = [(r, tuple(x[i].shape), x.dtype) for i, r in enumerate(ranks) if r != me]
    got = iter(t.exchange(sends, recvs))
    for i, r in enumerate(ranks):
        out[i] = x[i] if r == me else next(got)
    return out


class MoEFeedForward(torch.nn.Module):
    def __init__(self, cfg, layout):
        super().__init__()
        self.cfg, self.layout = cfg, layout
        E, d, F = cfg.n_experts, cfg.d_model, cfg.ffn_dim
        if layout.tp != 1:
            raise ValueError("the expert-parallel block expects tensor-parallel size 1")
        self.ep = layout.shard          # data- and context-parallel workers alike hold tokens to route
        if E % self.ep:
            raise ValueError("experts must divide evenly over the expert-parallel workers")
        self.e_local = E // self.ep
        self.ep_ranks = tuple(layout.P_grid.ranks)
        collect = bool(getattr(cfg, "collect_state", False))
        self.router = dnn.DistributedLinearAllGatherZero(layout.P_flat, d, max(E, 8), bias=False, dtype=cfg.dtype,
                                                         auto_clear_buffer=not cfg.keep_gathered,
                                                         collect_state=collect)
        dev = layout.P_flat.device
        self.w_up = torch.nn.Parameter(torch.empty(self.e_local, 2 * F, d, dtype=cfg.dtype, device=dev))
        self.w_down = torch.nn.Parameter(torch.empty(self.e_local, d, F, dtype=cfg.dtype, device=dev))
        with torch.no_grad():
            self.w_up.normal_(0.0, cfg.init_std)
            self.w_down.normal_(0.0, cfg.init_std / math.sqrt(2 * cfg.n_layers))
        self.aux_loss = None
        self.last_dropped = None
        self.collect_state = collect
        if collect:
            # serial layout: all experts along dimension 0, on the first worker only
            from ..nn._linear_common import root_partition
            self.P_ep = layout.P_flat                                  # [ep, 1, 1]: experts over the workers
            self.P_root = root_partition(self.P_ep)
            # one pair per tensor: a module re-runs its (collective) set-up when its input structure
            # changes, and the workers that feed zero-volume tensors would not notice the change
            self.gather_experts = torch.nn.ModuleDict(
                {n: dnn.Repartition(self.P_ep, self.P_root, preserve_batch=False) for n in ("w_up", "w_down")})
            self.scatter_experts = torch.nn.ModuleDict(
                {n: dnn.Repartition(self.P_root, self.P_ep, preserve_batch=False) for n in ("w_up", "w_down")})
            self._register_state_dict_hook(self._gather_state_dict)
            self._register_load_state_dict_pre_hook(self._scatter_state_dict)

    def _gather_state_dict(self, module, destination, prefix, *args):
        for name in ("w_up", "w_down"):
            full = self.gather_experts[name](destination.pop(prefix + name).detach())
            if self.P_root.active:
                destination[prefix + name] = full
        return destination

    def _scatter_state_dict(self, destination, prefix, *args):
        from ..utilities.torch import zero_volume_tensor
        for name in ("w_up", "w_down"):
            p = getattr(self, name)
            full = destination.pop(prefix + name, None)
            full = full.to(p.device) if self.P_root.active else zero_volume_tensor(device=p.device, dtype=p.dtype)
            destination[prefix + name] = self.scatter_experts[name](full)
        return destination

    def forward(self, x):
        cfg = self.cfg
        E, k = cfg.n_experts, cfg.top_k
        b, s, d = x.shape
        T = b * s
        xt = x.reshape(T, d)
        logits = self.router(x).reshape(T, -1)
        C = int(math.ceil(cfg.capacity_factor * T * k / E / 8.0) * 8)
        # softmax, top-k, renormalisation, slot assignment and the probability sums: one kernel
        topw, prob_sum, ids, slot, counts = moe_ops.route(logits, E, k, C)
        # load-balancing auxiliary loss (fraction routed x mean router probability)
        frac = counts.float() / float(T * k)
        self.aux_loss = E * (frac.detach() * (prob_sum / float(T))).sum()
        self.last_dropped = (slot < 0).sum()
        P, El = self.ep, self.e_local
        peer = None
        if xt.is_cuda and P > 1 and os.environ.get("DISTDL_MOE_PEER", "1") != "0":
            from ..parallel import moe_peer
            if moe_peer.usable(xt, self.ep_ranks, El, C):
                peer = moe_peer
        if peer is not None:
            # dispatch and combine over peer memory: permutation + all-to-all in one kernel each
            h = peer.dispatch(xt, ids, slot, self.ep_ranks, El, C, k)             # [El, P*C, d]
            h = batched_linear(h, self.w_up)
            h = ops.swiglu(h)
            h = batched_linear(h, self.w_down)
            y = peer.combine(h, topw, ids, slot, self.ep_ranks, T, k, C)
            return y.reshape(b, s, d).to(x.dtype)
        send = moe_ops.dispatch(xt, ids, slot, E, C, k)                       # [E, C, d]
        recv = _AllToAllFn.apply(send.reshape(P, El * C, d), self.ep_ranks)   # [P(src), El*C, d]
        h = recv.reshape(P, El, C, d).transpose(0, 1).reshape(El, P * C, d)
        h = batched_linear(h, self.w_up)
        h = ops.swiglu(h)
        h = batched_linear(h, self.w_down)                                    # [El, P*C, d]
        back = h.reshape(El, P, C, d).transpose(0, 1).reshape(P, El * C, d)
        back = _AllToAllFn.apply(back.contiguous(), self.ep_ranks).reshape(E, C, d)
        y = moe_ops.combine(back, topw, ids, slot, T, k)
        return y.reshape(b, s, d).to(x.dtype)

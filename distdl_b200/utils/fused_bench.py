"""Roofline table of the fused compute + collective paths (run under torchrun, one rank per GPU):

    torchrun --nnodes=1 --nproc-per-node N -m distdl_b200.utils.fused_bench [--md FILE]

Each path is timed on the device (CUDA events on the launching stream, warm-up, a buffer larger than
L2 written between timed launches, maximum over ranks) at the shapes of the Llama-3-8B configuration
(d = 4096, FFN 14336, 4 sequences of 4096 tokens per micro-batch).  The roofline time of a path is
the slower of its FLOPs at the measured sustained cuBLAS bf16 rate and its bytes that must cross
NVLink into (or out of) one GPU at the measured peer-copy bandwidth; the table gives roofline time /
measured time.

  K1  all-gather -> GEMM          sequence shards gathered inside the QKV / FFN-up GEMM
  K2  GEMM -> reduce-scatter      partial products leave through the GEMM epilogue, fold inside
  K3  ZeRO parameter gather       peers' weight shards read in place (copy engines), no staging
  K4  ZeRO gradient step          peers' fp32 accumulators read in place + AdamW in one kernel
  K5  split-norm statistics       statistics exchange inside the RMSNorm kernel
  K6  MoE dispatch / combine      token rows written to / read from the expert owners' memory
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0           # measured peer-copy bandwidth per direction and GPU on this pool


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                        "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            d = json.load(fh)
            return float(d["bf16_tflops_sustained"]), float(d["hbm_gbs"]), "measured"
    except (OSError, ValueError, KeyError):
        return 1400.0, 6650.0, "fallback"


_flush = None


def _time(fn, iters=6, warmup=3):
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        _flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    t = torch.tensor([total / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--md", default=None)
    args = ap.parse_args()
    import distdl_b200
    from distdl_b200 import _native
    from distdl_b200.backends.common import world as dworld
    dworld.init_process_group_from_env()
    distdl_b200.config.set_backend("native", "cupy")
    distdl_b200.backends.backend.Partition()
    from distdl_b200.parallel import collectives, fused, moe_peer, split_norm, symm
    from distdl_b200.ops import moe as moe_ops
    rank, P = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    ranks = tuple(range(P))
    peak, hbm, kind = _peaks()
    rows = []

    def add(name, what, flops, nvlink_bytes, ms, hbm_bytes=0.0):
        t_c = flops / (peak * 1e12) * 1e3
        t_n = nvlink_bytes / (NVLINK_GBS * 1e9) * 1e3
        t_h = hbm_bytes / (hbm * 1e9) * 1e3
        roof = max(t_c, t_n, t_h)
        bound = "compute" if roof == t_c else ("NVLink" if roof == t_n else "HBM")
        rows.append({"path": name, "what": what, "tflop": flops / 1e12, "nvlink_mb": nvlink_bytes / 1e6,
                     "ms": ms, "roofline_ms": roof, "bound": bound, "fraction": roof / ms})

    b, S, d, F = 4, 4096, 4096, 14336
    s_local = S // P
    torch.manual_seed(1)
    # K1: FFN-up projection, this GPU's share of the columns (gate | up = 2 F / P)
    x = torch.randn(b, s_local, d, device=dev).to(torch.bfloat16)
    w = (torch.randn(2 * F // P, d, device=dev) * 0.02).to(torch.bfloat16)
    ms = _time(lambda: fused.ag_gemm(x, w, None, ranks))
    add("K1 all-gather -> GEMM", f"[{b}x{S},{d}] x [{d},{2 * F // P}], TP={P}", 2.0 * b * S * d * (2 * F // P),
        (P - 1) * x.numel() * 2, ms)
    # K2: FFN-down projection, this GPU's share of the inner dimension
    h = torch.randn(b * S, F // P, device=dev).to(torch.bfloat16)
    w2 = (torch.randn(d, F // P, device=dev) * 0.02).to(torch.bfloat16)
    ms = _time(lambda: fused.gemm_rs(h, w2, None, ranks, b, s_local))
    add("K2 GEMM -> reduce-scatter", f"[{b}x{S},{F // P}] x [{F // P},{d}], TP={P}", 2.0 * b * S * d * (F // P),
        (P - 1) * b * s_local * d * 2, ms)
    # K3: ZeRO gather of the FFN-up weight (shards in a peer-mapped buffer, read in place)
    n_shard = d * (2 * F // 2) // P // 8 * 8
    region = symm.SymmetricRegion(symm.heap(), n_shard * 2)
    symm.register_param_region(region)
    shard = region.tensor(n_shard, torch.bfloat16)
    shard.normal_()
    dist.barrier()
    ms = _time(lambda: collectives.gather_in_place(shard, ranks))
    add("K3 ZeRO parameter gather", f"weight of {n_shard * P / 1e6:.0f} M elements over {P} shards", 0.0,
        (P - 1) * n_shard * 2, ms)
    # K4: ZeRO gradient step: peers' accumulators read in place + AdamW
    n = n_shard
    acc_region = symm.SymmetricRegion(symm.heap(), P * n * 4)
    acc = acc_region.tensor(P * n, torch.float32)
    acc.normal_()
    master, m1, m2, g = (torch.zeros(n, device=dev) for _ in range(4))
    pbf = torch.zeros(n, device=dev, dtype=torch.bfloat16)
    srcs = (ctypes.c_void_p * P)(*[acc_region.ptrs[r] + 4 * rank * n for r in ranks])
    from distdl_b200.ops._util import stream_ptr
    dist.barrier()

    def grad_step():
        _native.check(_native.lib().dd_grad_rs_adamw(P, srcs, g.data_ptr(), master.data_ptr(), m1.data_ptr(),
                                                     m2.data_ptr(), pbf.data_ptr(), n, 1e-4, 0.9, 0.95, 1e-8, 0.1, 1,
                                                     None, 1.0, stream_ptr()), "dd_grad_rs_adamw")
    ms = _time(grad_step)
    # (local traffic of the update itself: master, both moments and the shard gradient read and written,
    # the bf16 copy written, this GPU's own accumulator slice read)
    add("K4 gradient reduce + AdamW", f"shard of {n / 1e6:.0f} M elements, {P} accumulators", 0.0,
        (P - 1) * n * 4, ms, hbm_bytes=n * (4 * 8 + 2 + 4))
    # K5: RMSNorm over features split across the team
    xs = torch.randn(b * S // 4, d // P, device=dev).to(torch.bfloat16)
    wn = torch.ones(d // P, device=dev, dtype=torch.bfloat16)
    if split_norm.usable(xs, wn, None, ranks):
        ms = _time(lambda: split_norm.split_norm(xs, wn, None, 1e-5, ranks, d, rms=True))
        add("K5 split-norm statistics", f"[{xs.shape[0]},{d}] over {P} feature shards", 0.0,
            (P - 1) * xs.shape[0] * 8, ms, hbm_bytes=2 * xs.numel() * 2)
    # K6: expert-parallel dispatch and combine (top-2 of P experts, one expert per GPU)
    T, k, E = b * S, 2, P
    C = int(-(-1.25 * T * k / E // 8) * 8)
    xt = torch.randn(T, d, device=dev).to(torch.bfloat16)
    logits = torch.randn(T, max(E, 8), device=dev).to(torch.bfloat16)
    topw, _ps, ids, slot, _cnt = moe_ops.route(logits, E, k, C)
    if moe_peer.usable(xt, ranks, 1, C):
        ms = _time(lambda: moe_peer.dispatch(xt, ids, slot, ranks, 1, C, k))
        add("K6 MoE dispatch", f"{T} tokens, top-{k} of {E} experts", 0.0, T * k * d * 2 * (P - 1) / P, ms)
        buf = moe_peer.dispatch(xt, ids, slot, ranks, 1, C, k)
        ms = _time(lambda: moe_peer.combine(buf, topw, ids, slot, ranks, T, k, C))
        add("K6 MoE combine", f"{T} tokens, top-{k} of {E} experts", 0.0, T * k * d * 2 * (P - 1) / P, ms)
    if rank == 0:
        lines = [f"# Fused paths on {P} GPUs: achieved fraction of the roofline",
                 "",
                 f"Command: `torchrun --nnodes=1 --nproc-per-node {P} -m distdl_b200.utils.fused_bench --md FILE`.",
                 f"Roofline = max(FLOPs / {peak:.0f} TFLOP/s ({kind} sustained cuBLAS bf16), NVLink bytes per GPU / "
                 f"{NVLINK_GBS:.0f} GB/s, local bytes / {hbm:.0f} GB/s ({kind} copy bandwidth)); device time by CUDA "
                 "events around ONE call (so a path of a few tens of microseconds shows the launch latency of the "
                 "host, about 0.1 ms, not the kernel), L2 flushed between launches, max over ranks.",
                 "",
                 "| path | case | TFLOP | NVLink MB / GPU | device ms | roofline ms | bound | fraction |",
                 "|---|---|---|---|---|---|---|---|"]
        for r in rows:
            lines.append(f"| {r['path']} | {r['what']} | {r['tflop']:.2f} | {r['nvlink_mb']:.1f} | {r['ms']:.3f} | "
                         f"{r['roofline_ms']:.3f} | {r['bound']} | {r['fraction']:.2f} |")
        text = "\n".join(lines) + "\n"
        print(text)
        if args.md:
            with open(args.md, "w") as fh:
                fh.write(text)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

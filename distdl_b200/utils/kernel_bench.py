"""Times the hand-written kernels in isolation and prints achieved TFLOP/s or
GB/s beside the measured peaks of the machine (``MEASURED_PEAKS.json`` at the
repository root when present).

    python -m distdl_b200.utils.kernel_bench [--gemm] [--elementwise] [--attention]

Timing follows the usual hygiene: warm-up, CUDA events on the launching
stream, and an L2 flush (a write larger than L2) between timed launches.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


_flush = None


def time_op(fn, iters=10, warmup=3, flush=True):
    """Median device time of ``fn()`` in milliseconds."""
    global _flush
    if flush and _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            _flush.zero_()
        s = torch.cuda.Event(enable_timing=True)
        e = torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def bench_gemm(rows):
    from distdl_b200.ops import gemm
    hbm, tf, kind = _peaks()
    shapes = [(8192, 8192, 8192), (4096, 6144, 4096), (4096, 4096, 4096), (4096, 28672, 4096), (4096, 4096, 14336),
              (8192, 128256, 4096), (32768, 1600, 6400)]
    for (M, N, K) in shapes:
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        for name, fn in (("tcgen05 NT", lambda: gemm(a, b, out=out)),
                         ("cuBLAS  NT", lambda: torch.matmul(a, b.t(), out=out))):
            ms = time_op(fn)
            tfl = 2.0 * M * N * K / ms / 1e9
            rows.append(f"gemm {name} {M}x{N}x{K}: {ms:.3f} ms  {tfl:.1f} TFLOP/s  ({tfl / tf:.2f} of {kind} {tf:.0f})")
        # gradient layouts
        dy = out
        dx = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
        ms = time_op(lambda: gemm(dy, b.t(), out=dx))
        rows.append(f"gemm tcgen05 NN(dgrad) {M}x{K}x{N}: {ms:.3f} ms  {2.0 * M * N * K / ms / 1e9:.1f} TFLOP/s")
        dw = torch.empty(N, K, device="cuda", dtype=torch.float32)
        ms = time_op(lambda: gemm(dy.t(), a.t(), out=dw))
        rows.append(f"gemm tcgen05 TN(wgrad,f32 out) {N}x{K}x{M}: {ms:.3f} ms  {2.0 * M * N * K / ms / 1e9:.1f} TFLOP/s")
        del a, b, out, dx, dw


def bench_elementwise(rows):
    from distdl_b200 import ops
    hbm, tf, kind = _peaks()
    T, d = 32768, 4096
    x = torch.randn(T, d, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(d, device="cuda", dtype=torch.bfloat16)
    ms = time_op(lambda: ops.rms_norm(x, w))
    gbs = 2 * x.numel() * 2 / ms / 1e6
    rows.append(f"rms_norm fwd {T}x{d}: {ms:.3f} ms {gbs:.0f} GB/s ({gbs / hbm:.2f} of {kind} {hbm:.0f})")
    xg = x.clone().requires_grad_()
    wg = w.clone().requires_grad_()
    y = ops.rms_norm(xg, wg)
    dy = torch.randn_like(y)
    ms = time_op(lambda: torch.autograd.grad(y, (xg, wg), dy, retain_graph=True))
    gbs = 3 * x.numel() * 2 / ms / 1e6
    rows.append(f"rms_norm bwd {T}x{d}: {ms:.3f} ms {gbs:.0f} GB/s ({gbs / hbm:.2f} of {kind} {hbm:.0f})")
    r = torch.randn_like(x)
    ms = time_op(lambda: ops.add_rms_norm(x, r, w))
    gbs = 4 * x.numel() * 2 / ms / 1e6
    rows.append(f"add + rms_norm fwd {T}x{d}: {ms:.3f} ms {gbs:.0f} GB/s ({gbs / hbm:.2f} of {kind} {hbm:.0f})")
    del xg, wg, y, dy, r
    gu = torch.randn(T, 2 * 7168, device="cuda", dtype=torch.bfloat16)
    ms = time_op(lambda: ops.swiglu(gu))
    gbs = (gu.numel() * 2 * 1.5) / ms / 1e6
    rows.append(f"swiglu fwd {T}x{2 * 7168}: {ms:.3f} ms {gbs:.0f} GB/s ({gbs / hbm:.2f} of {kind})")
    n = 256 * 1024 * 1024
    p = torch.zeros(n, device="cuda"); m = torch.zeros(n, device="cuda"); v = torch.zeros(n, device="cuda")
    g = torch.zeros(n, device="cuda"); pb = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    ms = time_op(lambda: ops.adamw_step_(p, m, v, g, pb, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                                         step=1), flush=False)
    gbs = n * (4 * 4 + 4 * 4 + 2) / ms / 1e6
    rows.append(f"adamw {n} params: {ms:.3f} ms {gbs:.0f} GB/s ({gbs / hbm:.2f} of {kind})")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gemm", action="store_true")
    ap.add_argument("--elementwise", action="store_true")
    ap.add_argument("--attention", action="store_true")
    args = ap.parse_args()
    every = not (args.gemm or args.elementwise or args.attention)
    rows = []
    if args.gemm or every:
        bench_gemm(rows)
    if args.elementwise or every:
        bench_elementwise(rows)
    if args.attention or every:
        try:
            from distdl_b200.utils.kernel_bench_attention import bench_attention
            bench_attention(rows, time_op)
        except ImportError:
            pass
    print("\n".join(rows))


if __name__ == "__main__":
    main()

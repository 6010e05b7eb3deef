"""Runs a few launches of ONE hand-written kernel on a small case, for use
under a profiler:

    python -m distdl_b200.utils.profile_case gemm|gemm_wgrad|ag_gemm|gemm_rs|attn_fwd|attn_bwd|rmsnorm|rmsnorm_bwd|
        add_rmsnorm|router|adamw|xent [launches]

Inputs are larger than the 126 MB L2 where that matters for the DRAM figures
but stay well under a few GB.
"""
import sys

import torch


def main():
    what = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    n = int(sys.argv[2]) if len(sys.argv) > 2 else 3
    from distdl_b200 import ops
    dev = "cuda"
    if what == "gemm":
        a = torch.randn(8192, 4096, device=dev, dtype=torch.bfloat16)
        b = torch.randn(14336, 4096, device=dev, dtype=torch.bfloat16)
        out = torch.empty(8192, 14336, device=dev, dtype=torch.bfloat16)
        fn = lambda: ops.gemm(a, b, out=out)  # noqa: E731
    elif what == "gemm_wgrad":
        dy = torch.randn(8192, 14336, device=dev, dtype=torch.bfloat16)
        x = torch.randn(8192, 4096, device=dev, dtype=torch.bfloat16)
        out = torch.zeros(14336, 4096, device=dev, dtype=torch.float32)
        fn = lambda: ops.gemm(dy.t(), x.t(), out=out, accumulate=True)  # noqa: E731
    elif what in ("ag_gemm", "gemm_rs"):
        # The fused tensor-parallel kernels on a team of ONE process: the same kernels (comm
        # warps, ready words, owner-ordered tiles, TMA-store epilogue) with every "peer" being
        # this GPU, so that a profiler can be attached (it must never wrap a multi-rank job).
        import os

        import torch.distributed as dist

        import distdl_b200
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29655")
        dist.init_process_group("nccl", rank=0, world_size=1)
        distdl_b200.config.set_backend("native", "cupy")
        distdl_b200.backends.backend.Partition()                 # creates the symmetric heap
        from distdl_b200.parallel import fused
        if what == "ag_gemm":
            x = torch.randn(2, 4096, 4096, device=dev, dtype=torch.bfloat16)
            w = torch.randn(14336, 4096, device=dev, dtype=torch.bfloat16)
            fn = lambda: fused.ag_gemm(x, w, None, (0,))  # noqa: E731
        else:
            x = torch.randn(8192, 7168, device=dev, dtype=torch.bfloat16)
            w = torch.randn(4096, 7168, device=dev, dtype=torch.bfloat16)
            fn = lambda: fused.gemm_rs(x, w, None, (0,), 2, 4096)  # noqa: E731
    elif what in ("attn_fwd", "attn_bwd"):
        batch, seq, Hq, Hkv, D = 2, 4096, 32, 8, 128
        qkv = torch.randn(batch * seq, Hq + 2 * Hkv, D, device=dev, dtype=torch.bfloat16)
        q, k, v = qkv[:, :Hq], qkv[:, Hq:Hq + Hkv], qkv[:, Hq + Hkv:]
        if what == "attn_fwd":
            fn = lambda: ops.attention_forward(q, k, v, batch, seq, True)  # noqa: E731
        else:
            o, lse = ops.attention_forward(q, k, v, batch, seq, True)
            do = torch.randn_like(o)
            fn = lambda: ops.attention_backward(do, q, k, v, o, lse, batch, seq, True)  # noqa: E731
    elif what == "rmsnorm":
        x = torch.randn(32768, 4096, device=dev, dtype=torch.bfloat16)
        w = torch.ones(4096, device=dev, dtype=torch.bfloat16)
        fn = lambda: ops.rms_norm(x, w)  # noqa: E731
    elif what == "rmsnorm_bwd":
        x = torch.randn(32768, 4096, device=dev, dtype=torch.bfloat16, requires_grad=True)
        w = torch.ones(4096, device=dev, dtype=torch.bfloat16, requires_grad=True)
        y = ops.rms_norm(x, w)
        dy = torch.randn_like(y)
        fn = lambda: torch.autograd.grad(y, (x, w), dy, retain_graph=True)  # noqa: E731
    elif what == "add_rmsnorm":
        x = torch.randn(32768, 4096, device=dev, dtype=torch.bfloat16)
        r = torch.randn_like(x)
        w = torch.ones(4096, device=dev, dtype=torch.bfloat16)
        fn = lambda: ops.add_rms_norm(x, r, w)  # noqa: E731
    elif what == "router":
        from distdl_b200.ops import moe
        logits = torch.randn(1 << 20, 8, device=dev, dtype=torch.bfloat16)
        fn = lambda: moe.route(logits, 8, 2, 1 << 19)  # noqa: E731
    elif what == "adamw":
        m = 64 * 1024 * 1024
        p, a, b, g = (torch.zeros(m, device=dev) for _ in range(4))
        pb = torch.zeros(m, device=dev, dtype=torch.bfloat16)
        fn = lambda: ops.adamw_step_(p, a, b, g, pb, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8,  # noqa: E731
                                     weight_decay=0.1, step=1)
    elif what == "xent":
        logits = torch.randn(4096, 128256, device=dev, dtype=torch.bfloat16)
        tgt = torch.randint(0, 128256, (4096,), device=dev)
        fn = lambda: ops.cross_entropy_(logits, tgt, unit_grad=True)  # noqa: E731
    else:
        raise SystemExit(f"unknown case {what}")
    for _ in range(n):
        fn()
    torch.cuda.synchronize()
    print(f"{what}: {n} launches done")


if __name__ == "__main__":
    main()

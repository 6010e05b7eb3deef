"""Primitive sweep (run under torchrun, one rank per GPU):

    torchrun --nnodes=1 --nproc-per-node N -m distdl_b200.utils.primitive_bench [--max-bytes B]

AllSumReduce, AllGather, ReduceScatter, Broadcast, SumReduce and Repartition (an
[n, n] tensor from a row partition to a column partition) in bf16 for message sizes
4 KB ... 1 GB in powers of 4, values ~ U(-1, 1), seed 1; plus HaloExchange of an fp32
[8, 64, 512, 512] tensor with width-1 halos on a 2 x (N/2) spatial partition.
Each op is timed on the device (CUDA events, warm-up, max over ranks) for the
native backend (this library's kernels over peer memory) and for the NCCL
backend (library collectives); bus bandwidth uses the usual factors
(all-reduce 2(P-1)/P, others (P-1)/P of the full message).  ``--multimem`` runs the
native all-reduce through the NVLink multicast region (``multimem.ld_reduce`` /
``multimem.st``); ``--md FILE`` writes the table as a markdown summary.
"""
from __future__ import annotations

import argparse
import json
import math

import torch
import torch.distributed as dist


def _time(fn, iters=5, warmup=2):
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--json", default=None)
    ap.add_argument("--md", default=None, help="write a markdown summary (native vs NCCL per op and size)")
    ap.add_argument("--multimem", action="store_true", help="native all-reduce through the NVLink multicast region")
    ap.add_argument("--ops", default="", help="comma-separated subset of the op names (default: all)")
    ap.add_argument("--backends", default="native,nccl")
    args = ap.parse_args()
    import distdl_b200
    from distdl_b200.backends.common import world as dworld
    dworld.init_process_group_from_env()
    rank, P = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    rows = []
    only = set(filter(None, args.ops.split(",")))
    want = lambda name: not only or name in only
    sizes = []
    b = 4096
    while b <= args.max_bytes:
        sizes.append(b)
        b *= 4
    for backend in args.backends.split(","):
        distdl_b200.config.set_backend(backend, "cupy")
        from distdl_b200.nn import (AllGather, AllSumReduce, Broadcast, HaloExchange, ReduceScatter, Repartition,
                                    SumReduce)
        if backend == "native" and args.multimem:
            from distdl_b200.parallel import symm
            symm.heap()
            symm.enable_multicast(min(2 * args.max_bytes, 1 << 30) + (4 << 20))
        failure = None
        try:
            P_world = distdl_b200.backends.backend.Partition()
            P_flat = P_world.create_cartesian_topology_partition([P])
            P_rows = P_world.create_cartesian_topology_partition([P, 1])
            P_cols = P_world.create_cartesian_topology_partition([1, P])
            for nbytes in sizes:
                n = nbytes // 2
                torch.manual_seed(1)
                x = (torch.rand(n, device=dev) * 2 - 1).to(torch.bfloat16)
                ar, ag, rs = AllSumReduce(P_flat, axes_reduce=(0,)), AllGather(P_flat, axes_all_gather=(0,)), \
                    ReduceScatter(P_flat, axes_reduce_scatter=(0,))
                shard = x[: max(8, n // P // 8 * 8)]
                full = x[: shard.numel() * P]
                for name, fn, factor, msg in (
                        ("all_sum_reduce", lambda: ar(x), 2 * (P - 1) / P, nbytes),
                        ("all_gather", lambda: ag(shard), (P - 1) / P, shard.numel() * 2 * P),
                        ("reduce_scatter", lambda: rs(full), (P - 1) / P, full.numel() * 2)):
                    if not want(name):
                        continue
                    ms = _time(fn)
                    rows.append({"op": name, "backend": backend, "bytes": msg, "ms": ms,
                                 "busbw_GBs": msg * factor / ms / 1e6})
                P_one = P_world.create_partition_inclusive([0]).create_cartesian_topology_partition([1])
                bc, sr = Broadcast(P_one, P_flat, preserve_batch=False), SumReduce(P_flat, P_one, preserve_batch=False)
                src = x if rank == 0 else x[:0]
                for name, fn, msg in (("broadcast", lambda: bc(src), nbytes), ("sum_reduce", lambda: sr(x), nbytes)):
                    if not want(name):
                        continue
                    ms = _time(fn)
                    rows.append({"op": name, "backend": backend, "bytes": msg, "ms": ms, "busbw_GBs": msg / ms / 1e6})
                side = int(math.sqrt(n)) // (8 * P) * (8 * P)
                if side >= 8 * P and want("repartition_row_to_col"):
                    m = torch.rand(side // P, side, device=dev).to(torch.bfloat16)
                    rp = Repartition(P_rows, P_cols)
                    ms = _time(lambda: rp(m))
                    msg = side * side * 2
                    rows.append({"op": "repartition_row_to_col", "backend": backend, "bytes": msg, "ms": ms,
                                 "busbw_GBs": msg / P * (P - 1) / P / ms / 1e6})
            if P >= 2 and want("halo_exchange"):
                py = 2 if P % 2 == 0 and P > 2 else 1
                px = P // py
                P_sp = P_world.create_cartesian_topology_partition([1, 1, py, px])
                halo = [[0, 0], [0, 0], [int(P_sp.index[2] > 0), int(P_sp.index[2] < py - 1)],
                        [int(P_sp.index[3] > 0), int(P_sp.index[3] < px - 1)]]
                H, Wd = 512 // py, 512 // px
                xt = torch.rand(8, 64, H + halo[2][0] + halo[2][1], Wd + halo[3][0] + halo[3][1], device=dev)
                he = HaloExchange(P_sp, halo, halo, halo)
                ms = _time(lambda: he(xt))
                rows.append({"op": f"halo_exchange_8x64x512x512_on_{py}x{px}", "backend": backend,
                             "bytes": xt.numel() * 4, "ms": ms, "busbw_GBs": None})
        except Exception as exc:      # noqa: BLE001  (raised again once no memory is bound to the multicast object)
            failure = exc
        if backend == "native" and args.multimem:
            symm.disable_multicast()
        if failure is not None:
            raise failure
    if rank == 0 and args.md:
        ops = []
        for r in rows:
            if r["op"] not in ops:
                ops.append(r["op"])
        with open(args.md, "w") as fh:
            fh.write(f"# Primitive sweep on {P} GPUs (bf16; device-timed, max over ranks)\n\n")
            fh.write("Command: `torchrun --nnodes=1 --nproc-per-node " + str(P) + " -m distdl_b200.utils.primitive_bench"
                     + (" --multimem" if args.multimem else "") + f" --max-bytes {args.max_bytes}"
                     + (f" --ops {args.ops}" if args.ops else "") + " --md FILE`\n\n")
            fh.write("| op | bytes | native ms | NCCL ms | native GB/s | NCCL GB/s |\n|---|---|---|---|---|---|\n")
            for op in ops:
                sizes_seen = sorted({r["bytes"] for r in rows if r["op"] == op})
                for nb in sizes_seen:
                    nat = next((r for r in rows if r["op"] == op and r["bytes"] == nb and r["backend"] == "native"), None)
                    lib = next((r for r in rows if r["op"] == op and r["bytes"] == nb and r["backend"] == "nccl"), None)
                    f = lambda r, k: "-" if r is None or r[k] is None else (f"{r[k]:.4f}" if k == "ms" else f"{r[k]:.0f}")
                    fh.write(f"| {op} | {nb} | {f(nat, 'ms')} | {f(lib, 'ms')} | {f(nat, 'busbw_GBs')} | "
                             f"{f(lib, 'busbw_GBs')} |\n")
    if rank == 0:
        for r in rows:
            bw = "" if r["busbw_GBs"] is None else f"{r['busbw_GBs']:.1f} GB/s"
            print(f"{r['op']:<40} {r['backend']:<7} {r['bytes']:>12} B  {r['ms']:.4f} ms  {bw}")
        if args.json:
            with open(args.json, "w") as fh:
                json.dump(rows, fh)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

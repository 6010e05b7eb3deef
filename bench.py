#!/usr/bin/env python
"""Headline benchmark: training tokens/s of the Llama-3-8B-shape decoder
(32 layers, d=4096, 32 heads / 8 KV heads, SwiGLU 14336, RMSNorm, RoPE, vocab
128256), bf16 parameters with fp32 master weights and AdamW, tensor-parallel
x ZeRO-3/FSDP on one node.

    python bench.py --gpus N --steps K --warmup W
    torchrun --nnodes=1 --nproc-per-node N ... bench.py --gpus N --steps K --warmup W

Weak scaling: 8 sequences of 4096 tokens per GPU and step (64 x 4096 at N=8,
the configuration named by the baseline).  Layout: N=1 -> no parallelism,
N=2 -> TP=2, N=4 -> TP=2 x FSDP=2, N=8 -> TP=2 x FSDP=4.  Prints one JSON line
on rank 0.  `value` is device-timed with the token blocks already on the
device; `e2e` goes through `Trainer.step()` with, every step, the host->device
copy of the step's tokens from pinned memory and a device->host read of the loss.
"""
import argparse
import json
import os
import subprocess
import sys
import threading

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "train tokens/sec (8B TP+FSDP, max over ranks)"


def reference_arm(args):
    """The reference (microsoft/distdl) cannot be built or imported offline in
    this image: report that and exit 0."""
    why = None
    ref = os.path.join(ROOT, "baseline", "_ref")
    if os.path.isdir(os.path.join(ref, "distdl")):
        sys.path.insert(0, ref)
        import tempfile
        here = os.getcwd()
        try:
            # the reference's logger opens ./distdl.log when it is imported: not in this tree
            os.chdir(tempfile.mkdtemp(prefix="distdl_ref_"))
            import distdl  # noqa: F401
        except Exception as e:  # pragma: no cover
            why = f"import distdl failed: {type(e).__name__}: {e}"
        else:
            why = ("reference imports but has no attention/optimizer/trainer code and needs mpirun to launch; "
                   "no stock code path produces this metric")
    else:
        why = ("offline install failed: its C++ extension does not link here and mpi4py, cupy, pytorch-pfn-extras "
               "and mpirun are absent, so `import distdl` cannot succeed")
    if os.path.isdir(os.path.join(ref, "distdl")):
        os.chdir(here)
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


class ClockSampler:
    """Samples SM clocks and throttle reasons of this process's GPU with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.rows = []
        self._stop = threading.Event()
        self._t = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                if out.returncode == 0 and out.stdout.strip():
                    self.rows.append([c.strip() for c in out.stdout.strip().splitlines()[0].split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = sorted(float(r[0]) for r in self.rows if r[0].replace(".", "", 1).isdigit())
        mx = max((float(r[1]) for r in self.rows if r[1].replace(".", "", 1).isdigit()), default=None)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 4 + i and r[4 + i].lower().startswith("active")
                                                         for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": reasons,
                "samples": len(self.rows)}


def layout_for(n):
    return {1: (1, 1), 2: (1, 2), 4: (2, 2), 8: (4, 2)}[n]


def model_flops_report(cfg, seq, tokens_per_s, gpus):
    """Model FLOPs per token (forward + backward, recomputation not counted) turned into TFLOP/s per
    GPU, and its fraction of the measured sustained cuBLAS bf16 rate when that file is present."""
    per_token = cfg.train_flops_per_token(seq)
    tflops = tokens_per_s * per_token / max(1, gpus) / 1e12
    out = {"gflop_per_token": per_token / 1e9, "tflops_per_gpu": tflops}
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as fh:
                peak = float(json.load(fh)["bf16_tflops_sustained"])
            out["fraction_of_measured_sustained_bf16"] = tflops / peak
        except (OSError, ValueError, KeyError):
            pass
    return out


def activation_report(model):
    plan = model.activation_plan or {}
    keep, n = plan.get("keep", 0), plan.get("blocks", 0)
    per = plan.get("bytes_per_kept_block", 0)
    return (f"policy {plan.get('policy')}: {keep} of {n} blocks keep the outputs of their GEMMs and of attention "
            f"(with its log-sum-exp) for the backward pass, {per / 1e9:.2f} GB per block and micro-batch, "
            f"{keep * per / 1e9:.1f} GB per GPU; in those blocks " +
            ("nothing is recomputed (memory to spare: norm and activation outputs are stored as well)"
             if plan.get("stores_activation_output") and plan.get("stores_norm_outputs") else
             "only norm outputs are recomputed (the activation function's output is stored as well)"
             if plan.get("stores_activation_output") else
             "only norm outputs and the activation function's output are recomputed") +
            f" and the ZeRO weight shards are gathered again; the other {n - keep} blocks recompute their forward pass")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "nccl_cublas"],
                    help="nccl_cublas: the same model on library kernels only (cuBLAS GEMMs, library attention, "
                         "ATen elementwise, NCCL collectives, no fusion): the restated reference op sequence")
    ap.add_argument("--model", default="llama3_8b", choices=["llama3_8b", "llama_tiny", "gpt2_xl", "mixtral_8x7b"])
    ap.add_argument("--seqs-per-gpu", type=int, default=8)
    ap.add_argument("--micro-batch", type=int, default=0, help="sequences per forward/backward (0 = auto)")
    ap.add_argument("--tp", type=int, default=0, help="tensor-parallel size (0 = the layout named by the baseline)")
    ap.add_argument("--cp", type=int, default=1,
                    help="context-parallel size: every sequence is split into this many blocks (ring attention)")
    ap.add_argument("--keep-gathered", action="store_true",
                    help="gather the ZeRO shards once per optimizer step and reduce-scatter the gradients once "
                         "(ZeRO-1 behaviour within a step; not the named ZeRO-3 configuration)")
    ap.add_argument("--profile", action="store_true",
                    help="diagnosis only: after the timed runs, trace ONE step with torch.profiler on rank 0 and "
                         "print the kernels by total device time (numbers under a profiler are never bench values)")
    ap.add_argument("--activation-policy", default="auto",
                    help="auto: as many blocks as the free device memory holds keep their activations for the "
                         "backward pass, the others recompute; full: every block recomputes; none: every block keeps; "
                         "an integer: that many blocks keep")
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (invalid as a result)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.impl == "nccl_cublas":
        os.environ["DISTDL_FORCE_TORCH"] = "1"
        os.environ["DISTDL_FUSED"] = "0"

    # NCCL only carries two scalars per step here (gradient norm, loss) and the rendezvous;
    # in-switch reduction buys nothing for them, and plain peer transfers keep the GPUs of a
    # rank that exits early out of multicast groups
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            # re-launch under torchrun, one rank per GPU
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", str(29500 + os.getpid() % 2000), __file__] + sys.argv[1:]
            return subprocess.call(cmd)
        raise SystemExit(f"WORLD_SIZE={world} but --gpus {args.gpus}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")

    import distdl_b200
    from distdl_b200 import _native
    from distdl_b200.backends.common import world as dworld
    if world > 1:
        dworld.init_process_group_from_env()
    rank = dist.get_rank() if world > 1 else 0
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    distdl_b200.config.set_backend("nccl" if args.impl == "nccl_cublas" else "native", "cupy")
    from distdl_b200 import models
    from distdl_b200.parallel import SyntheticTokens, Trainer

    cfg = getattr(models, args.model)()
    if args.layers:
        cfg.n_layers = args.layers
    cfg.keep_gathered = bool(args.keep_gathered)
    cfg.activation_policy = args.activation_policy
    dp, tp = layout_for(args.gpus)
    if args.tp:
        tp, dp = args.tp, args.gpus // args.tp
    if cfg.n_experts:
        dp, tp = args.gpus, 1                      # expert parallel over all GPUs
    cp = max(1, args.cp)
    if dp % cp:
        raise SystemExit(f"--cp {cp} does not divide the {dp} data-parallel workers")
    dp //= cp
    seq = cfg.max_seq
    global_batch = args.seqs_per_gpu * args.gpus
    local_batch = global_batch // dp
    # sequences per forward/backward: the 8B model is sized by memory and by the staging regions of
    # the fused kernels; a model of a few billion parameters is launch-bound at small micro-batches
    # (GPT-2-XL on 2 GPUs: 17.8k / 67.1k / 87.2k tokens/s at 2 / 8 / 16 sequences)
    if args.micro_batch:
        micro = args.micro_batch
    elif cfg.num_parameters() < 3e9:
        micro = min(local_batch, 16)
    else:
        # 1 GPU holds 144 GB of parameters, gradients and optimizer state: with 2 sequences per pass all 32
        # blocks keep their activations for the backward pass, with 4 only some do
        micro = {1: 2, 2: 2}.get(args.gpus, 4)
    torch.manual_seed(1234 + rank)
    layout = models.ParallelLayout(dp, tp, cp=cp)
    model = models.Decoder(cfg, layout)
    trainer = Trainer(model, global_tokens_per_step=global_batch * seq, micro_batch=micro, lr=3e-4,
                      warmup_steps=10, total_steps=1000)
    # device-timed arm: one distinct block per step, staged before the clock starts
    pre = SyntheticTokens(local_batch, seq, cfg.vocab_size, dp_index=layout.dp_index, seed=1,
                          n_buffers=args.warmup + args.steps)
    dev_blocks = [b.cuda() for b in pre.blocks]
    data = SyntheticTokens(local_batch, seq, cfg.vocab_size, dp_index=layout.dp_index, seed=0)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        l0 = _native.launch_count
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for i in range(steps):
            fn(i)
        e.record()
        barrier()
        ms = torch.tensor([s.elapsed_time(e)], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item(), _native.launch_count - l0

    for i in range(args.warmup):
        trainer.step_device(dev_blocks[i])
        # a bounded device-side wait that ran out leaves every later kernel waiting too:
        # stop at once instead of running into the caller's time limit
        st = _native.read_status()
        if st[0]:
            sys.stderr.write(f"[bench] rank {rank}: device status {st} after warm-up step {i}; aborting\n")
            sys.stderr.flush()
            os._exit(3)
    with ClockSampler(local_rank) as clocks:
        ms_dev, launches = timed(lambda i: trainer.step_device(dev_blocks[args.warmup + i]), args.steps)
    losses = []
    ms_e2e, _ = timed(lambda i: losses.append(trainer.step(data.next()).item()), args.steps)
    status = _native.read_status()
    if args.profile:
        from torch.profiler import ProfilerActivity, profile
        barrier()
        _native.read_wait_ns()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            trainer.step_device(dev_blocks[0])
            torch.cuda.synchronize()
        waits = _native.read_wait_ns()
        if rank == 0:
            for kind, ns in waits.items():
                if ns:
                    sys.stderr.write(f"[profile] cross-GPU wait (block 0's designated threads) {ns / 1e6:9.2f} ms  {kind}\n")
            rows = sorted(prof.key_averages(), key=lambda e: -e.device_time_total)[:28]
            total = sum(e.device_time_total for e in prof.key_averages())
            sys.stderr.write(f"[profile] total device time of one step: {total / 1e3:.1f} ms\n")
            for e in rows:
                sys.stderr.write(f"[profile] {e.device_time_total / 1e3:9.2f} ms  x{e.count:<6d} {e.key[:110]}\n")

    tokens_per_step = global_batch * seq
    value = tokens_per_step * args.steps / (ms_dev / 1e3)
    e2e = tokens_per_step * args.steps / (ms_e2e / 1e3)
    if rank == 0:
        out = {
            "metric": METRIC, "impl": args.impl, "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_dev / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform token ids, random-init weights",
            "config": {"model": f"{args.model} ({cfg.num_parameters() / 1e9:.2f}B params)", "global_batch": global_batch,
                       "seq_len": seq,
                       "parallelism": (f"ep{dp} (experts) + fsdp{dp} (attention, router, embedding)" if cfg.n_experts
                                       else f"tp{tp} x fsdp{dp}" if cp == 1 else
                                       f"tp{tp} x cp{cp} x dp{dp} (ZeRO over {dp * cp} workers, ring attention)"),
                       "micro_batch": micro,
                       "zero": ("not used (parameters live on their tensor-parallel owners)" if not cfg.zero else
                                "gathered once per step (--keep-gathered)" if args.keep_gathered else
                                "ZeRO-3 parameters and optimizer state: block weight matrices re-gathered at every "
                                "use (forward and backward); their gradients " +
                                ("accumulate unsharded in fp32 and are reduce-scattered once per step"
                                 if os.environ.get("DISTDL_FULL_GRADS", "1") != "0" else
                                 "are reduce-scattered after every layer and micro-batch (DISTDL_FULL_GRADS=0)") +
                                "; norm weights, embedding and head gathered once per step"),
                       "optimizer": "AdamW fp32 master + moments, grad clip 1.0",
                       "activation_checkpointing": activation_report(model),
                       "l2": "inputs larger than L2: every step streams the model's weights, gradients and optimizer state "
                             f"({cfg.num_parameters() * 16 / max(1, args.gpus) / 1e9:.0f} GB per GPU) through the 126 MB L2; no explicit flush"},
            "clocks": clocks.summary(),
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": data.bytes_per_block, "d2h_bytes_per_step": 4},
            "gpu_launches": launches, "final_loss": losses[-1] if losses else None, "device_status": status[0],
            "model_flops": model_flops_report(cfg, seq, value, args.gpus),
        }
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""Pipeline parallelism: every process owns one stage of an MLP; six micro-batches run
through the one-forward-one-backward schedule.

    torchrun --nproc-per-node 3 --master-addr 127.0.0.1 examples/basics/ex_pipeline.py
"""
import torch
import torch.distributed as dist
import os, sys
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))  # noqa: E402
from common import say, start

P_world, rank = start()
from distdl_b200.parallel import PipelineStage, run_1f1b  # noqa: E402

world = dist.get_world_size()
torch.manual_seed(rank)
layer = torch.nn.Sequential(torch.nn.Linear(32, 32), torch.nn.GELU())
stage = PipelineStage(layer, list(range(world)), act_shape=(8, 32))
torch.manual_seed(100)
xs = [torch.randn(8, 32) for _ in range(6)]
ts = [torch.randn(8, 32) for _ in range(6)]
loss = run_1f1b(stage, xs if stage.first else None, ts if stage.last else None,
                lambda y, t: ((y - t) ** 2).mean(), n_micro=6)
gnorm = sum(float(p.grad.norm()) for p in layer.parameters())
say(P_world, f"stage {stage.index}", "loss" if stage.last else "", float(loss) if stage.last else "", "|grad|", gnorm)

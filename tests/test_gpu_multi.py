"""Multi-GPU tests (skipped with fewer than 2 devices): child processes, one
rank per GPU, NVLS off in NCCL, plain peer loads in this library's kernels."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(what, nproc):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(29400 + os.getpid() % 500),
           os.path.join(HERE, "multi_gpu_worker.py"), what]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    if res.returncode != 0:
        # the ranks' own tracebacks come before the launcher's summary: show their last frames and errors
        lines = (res.stdout + "\n" + res.stderr).splitlines()
        keep = [ln for ln in lines if "multi_gpu_" in ln or "Error" in ln or "assert" in ln or "distdl_b200" in ln]
        raise AssertionError("\n".join(keep[:60]) + "\n...\n" + res.stderr[-1500:])
    assert "OK" in res.stdout


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_native_collectives_match_nccl():
    _run("collectives", min(_ngpu(), 8))


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_primitives_on_native_backend():
    _run("primitives", min(_ngpu(), 8))


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_fused_ag_gemm_and_gemm_rs():
    _run("fused", min(_ngpu(), 8))


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_blocks_that_keep_activations_train_like_blocks_that_recompute():
    _run("activation_policies", min(_ngpu(), 8))


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_context_parallel_decoder_on_gpus():
    _run("context_decoder", 2 if _ngpu() < 4 else 4)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_pipelined_decoder_on_gpus():
    _run("pipeline", 2 if _ngpu() < 4 else 4)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_halo_exchange_and_repartition_in_one_kernel():
    _run("box", min(_ngpu(), 8))


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_all_reduce_through_the_multicast_region():
    _run("multimem", min(_ngpu(), 8))

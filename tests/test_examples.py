"""A few of the examples run end to end on CPU ranks (one per family), so that they keep
working with the library."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("script,nproc", [("examples/primitives/ex_repartition.py", 4),
                                          ("examples/basics/ex_linear_tp_sp.py", 4),
                                          ("examples/basics/ex_pipeline.py", 3),
                                          ("examples/basics/ex_layernorm_split.py", 3),
                                          ("examples/basics/ex_conv_transpose.py", 4),
                                          ("examples/basics/ex_expert.py", 4),
                                          ("examples/basics/ex_linear_zero.py", 4),
                                          ("examples/basics/train_decoder.py --cp 2", 4),
                                          ("examples/basics/ex_pipelined_decoder.py", 4),
                                          ("examples/basics/ex_window_attention.py", 4),
                                          ("examples/basics/ex_moe_decoder.py", 4)])
def test_example_runs(script, nproc):
    script, *extra = script.split()
    port = 29600 + (os.getpid() + hash(script)) % 300
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, script)] + extra
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=240, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]

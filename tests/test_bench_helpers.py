"""bench.py helpers that need no GPU: the layouts named by the benchmark configuration, the
summary of sampled clocks, and the reference arm's answer."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_layouts_named_by_the_configuration():
    b = _bench()
    assert b.layout_for(1) == (1, 1) and b.layout_for(2) == (1, 2)
    assert b.layout_for(4) == (2, 2) and b.layout_for(8) == (4, 2)          # TP=2 x FSDP=4 on 8 GPUs


def test_clock_summary_median_and_reasons():
    b = _bench()
    s = b.ClockSampler(0)
    assert s.summary()["reasons"] == ["unsampled"]
    s.rows = [["1300", "1965", "990.1", "0x4", "Not Active", "Not Active", "Not Active", "Active"],
              ["1400", "1965", "1001.0", "0x4", "Not Active", "Not Active", "Not Active", "Active"],
              ["1900", "1965", "400.0", "0x0", "Not Active", "Not Active", "Not Active", "Not Active"]]
    out = s.summary()
    assert out["sm_mhz"] == 1400.0 and out["sm_max_mhz"] == 1965.0 and out["reasons"] == ["sw_power_cap"]
    assert out["samples"] == 3


def test_reference_arm_reports_unavailable_and_exits_zero():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1",
                          "--steps", "2", "--warmup", "3"], capture_output=True, text=True, timeout=120)
    assert res.returncode == 0
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line


def test_model_flops_report():
    from distdl_b200 import models
    b = _bench()
    cfg = models.llama3_8b()
    r = b.model_flops_report(cfg, 4096, 8 * 16000.0, 8)
    assert abs(r["tflops_per_gpu"] - 16000.0 * r["gflop_per_token"] / 1e3) < 1e-6
    assert 700 < r["tflops_per_gpu"] < 850
    if "fraction_of_measured_sustained_bf16" in r:
        assert 0.3 < r["fraction_of_measured_sustained_bf16"] < 1.0


def test_exchange_split_is_decided_alike_at_both_ends_of_a_pair():
    """Three members, one oversize message (0 -> 1) and one pair with two messages (2 -> 0):
    each member marks exactly those for the library path, whichever end it is, and keeps
    every other message in the kernel, so no member ever waits for a kernel message that
    its partner sent another way."""
    import torch
    from distdl_b200.parallel.collectives import exchange_split
    staging = 3 * 1024                      # slot = 1024 bytes per member
    big, small = torch.zeros(2000, dtype=torch.uint8), torch.zeros(100, dtype=torch.uint8)
    msgs = {(0, 1): [big], (1, 0): [small], (1, 2): [small], (2, 1): [small], (2, 0): [small, small], (0, 2): [small]}
    marks = {}
    for me in range(3):
        sends = [(dst, t) for (src, dst), ts in msgs.items() if src == me for t in ts]
        recvs = [(src, tuple(t.shape), t.dtype) for (src, dst), ts in msgs.items() if dst == me for t in ts]
        ok_s, ok_r = exchange_split(3, staging, sends, recvs)
        for (dst, _), ok in zip(sends, ok_s):
            marks.setdefault((me, dst), []).append(("s", ok))
        for (src, _, _), ok in zip(recvs, ok_r):
            marks.setdefault((src, me), []).append(("r", ok))
    for pair, seen in marks.items():
        native = {ok for _, ok in seen}
        assert len(native) == 1, (pair, seen)                       # both ends agree
        assert native.pop() == (pair not in ((0, 1), (2, 0))), pair


def test_reduce_scatter_staging_sees_adjacent_slices_as_one_tensor():
    """Slices of one contiguous tensor are staged with a single copy; separate tensors one by one."""
    import torch

    from distdl_b200.parallel import collectives as C
    x = torch.arange(24.).view(4, 6)
    rows = [x[i].contiguous().view(-1) for i in range(4)]
    one = C._as_one(rows)
    assert isinstance(one, torch.Tensor) and one.shape == (4, 6) and torch.equal(one, x)
    apart = [torch.randn(6) for _ in range(4)]
    assert isinstance(C._as_one(apart), list)
    for src in (one, apart):
        stage = torch.zeros(4, 8)
        C._stage_rows(stage, src, 2, 3)
        want = torch.stack([r[2:5] for r in (rows if src is one else apart)])
        assert torch.equal(stage[:, :3], want) and not stage[:, 3:].any()

"""Failure detection without faulting a GPU.

Host side (CPU ranks): a rank that raises, and a rank that never joins a
collective, are reported to the caller within the time limit instead of hanging
the job.  Device side: a bounded wait that runs out (a flag that nothing ever
sets) ends the kernel normally, records a status the host can read, and leaves
the CUDA context usable.
"""
import time

import pytest
import torch

from dist_harness import run_ranks


def body_rank_raises(rank, world):
    if rank == 1:
        raise RuntimeError("injected failure on rank 1")
    return True


def test_rank_that_raises_is_reported():
    with pytest.raises(AssertionError, match="injected failure on rank 1"):
        run_ranks("test_failure_detection", "body_rank_raises", 2, timeout=60)


def body_rank_never_joins(rank, world):
    """Rank 1 skips the collective: rank 0's bounded receive must raise, not hang."""
    import distdl_b200
    from distdl_b200.nn import AllSumReduce
    if rank == 1:
        time.sleep(3)
        return "skipped"
    P = distdl_b200.backends.backend.Partition().create_cartesian_topology_partition([world])
    try:
        AllSumReduce(P, axes_reduce=(0,))(torch.ones(4))
    except RuntimeError as e:
        return f"detected: {type(e).__name__}"
    return "no error"


def test_rank_that_never_joins_times_out():
    # a pool of its own whose gloo process group has a 10 s limit; it is torn down afterwards
    try:
        out = run_ranks("test_failure_detection", "body_rank_never_joins", 2, timeout=150,
                        env={"DIST_HARNESS_TIMEOUT_S": "10"})
    except AssertionError as e:
        # the harness's own closing barrier can be what notices the broken world first
        assert any(k in str(e) for k in ("Timed out", "timeout", "detected", "Connection closed")), str(e)[-400:]
        return
    assert out[0].startswith("detected"), out


@pytest.mark.gpu
def test_device_wait_that_runs_out_reports_status_and_context_survives():
    import ctypes

    from distdl_b200 import _native
    lib = _native.lib()
    vp, ci = ctypes.c_void_p, ctypes.c_int
    lib.dd_symm_alloc.argtypes = [ctypes.c_size_t, ctypes.POINTER(vp)]
    lib.dd_team_barrier.argtypes = [ci, ci, ci, ctypes.POINTER(vp), ctypes.POINTER(vp), ctypes.POINTER(ci),
                                    ctypes.POINTER(ctypes.c_uint), ctypes.POINTER(ci), vp]
    pad, buf = vp(), vp()
    assert lib.dd_symm_alloc(64 * 1024, ctypes.byref(pad)) == 0
    assert lib.dd_symm_alloc(4096, ctypes.byref(buf)) == 0
    _native.read_status()                               # clear
    # a "team" of two whose second member does not exist: its flag is never raised
    bufs = (vp * 2)(buf.value, buf.value)
    pads = (vp * 2)(pad.value, pad.value)
    writers = (ci * 2)(0, 1)
    expect = (ctypes.c_uint * 2)(1, 1)
    steps = ci(0)
    t0 = time.time()
    assert lib.dd_team_barrier(2, 0, 0, bufs, pads, writers, expect, ctypes.byref(steps),
                               torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    dt = time.time() - t0
    code, where, expected, seen = _native.read_status()
    assert code == 1005 and where == 100 and expected == 1 and seen == 0, (code, where, expected, seen)
    assert 1.0 < dt < 20.0, dt
    # the context is alive: an ordinary kernel still runs and the status is clear again
    x = torch.ones(1024, device="cuda")
    assert float((x * 2).sum()) == 2048.0
    assert _native.read_status()[0] == 0
    # the host-side health check turns the same event into an exception (and a clean record)
    from distdl_b200.parallel import symm
    symm.check_health()                                  # nothing pending: returns
    expect2 = (ctypes.c_uint * 2)(2, 2)
    assert lib.dd_team_barrier(2, 0, 0, bufs, pads, writers, expect2, ctypes.byref(steps),
                               torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()                             # that wait has run out: the record is set
    # while the record is set, later waits give up at once instead of spending the limit again
    t1 = time.time()
    expect3 = (ctypes.c_uint * 2)(3, 3)
    assert lib.dd_team_barrier(2, 0, 0, bufs, pads, writers, expect3, ctypes.byref(steps),
                               torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert time.time() - t1 < 1.0
    with pytest.raises(symm.DeviceTimeout):
        symm.check_health()
    symm.check_health()
    lib.dd_symm_free.argtypes = [vp]
    lib.dd_symm_free(pad)
    lib.dd_symm_free(buf)


def body_heartbeat(rank, world):
    """Three ranks beat into the rendezvous store.  Rank 2 falls silent (a stalled process), then
    rank 1 leaves in an orderly way; the remaining ranks learn of both on the host, by name, within
    the limit, and no collective is involved."""
    from distdl_b200.parallel import Heartbeat, RankFailure
    hb = Heartbeat(interval=0.1, limit=1.0, prefix="test/hb").start()
    hb.wait_for_all(timeout=30)
    time.sleep(0.5)
    hb.check()                                   # everybody alive
    seen = {}

    def poll(expect_ranks, seconds):
        end = time.monotonic() + seconds
        while time.monotonic() < end:
            try:
                hb.check()
            except RankFailure as e:
                if set(expect_ranks) <= set(e.ranks):
                    return e
            time.sleep(0.1)
        return None
    if rank == 2:
        hb.stop()                                # no goodbye: looks like a hang
        time.sleep(4.0)
        return "silent"
    t0 = time.monotonic()
    e = poll([2], 6.0)
    assert e is not None and 2 in e.ranks and 2 not in e.left, e
    seen["silent_after"] = time.monotonic() - t0
    assert "no heartbeat from rank(s) [2]" in str(e)
    if rank == 1:
        hb.leave()
        return seen
    e = poll([1, 2], 6.0)
    assert e is not None and e.left == (1,) and set(e.ranks) == {1, 2}, e
    assert "left the job" in str(e)
    hb.stop()
    return seen


def test_heartbeat_names_silent_and_departed_ranks():
    out = run_ranks("test_failure_detection", "body_heartbeat", 3, timeout=120)
    assert out[2] == "silent" and 0.5 < out[0]["silent_after"] < 6.0, out


def test_watchdog_fires_only_when_the_block_overruns():
    from distdl_b200.parallel import Watchdog
    fired = []
    with Watchdog(5.0, "quick block", on_expire=lambda w, s: fired.append(w), exit_code=None) as w:
        time.sleep(0.05)
    assert not w.expired and not fired
    with Watchdog(0.1, "slow block", on_expire=lambda w, s: fired.append(w), exit_code=None, dump_stacks=False) as w:
        time.sleep(0.5)
    assert w.expired and fired == ["slow block"]


def test_watchdog_ends_a_stuck_process_with_its_exit_code():
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = ("import time\nfrom distdl_b200.parallel.health import Watchdog\n"
            "with Watchdog(0.3, 'stuck rendezvous'):\n    time.sleep(60)\n")
    t0 = time.monotonic()
    res = subprocess.run([sys.executable, "-c", code], cwd=root, capture_output=True, text=True, timeout=120,
                         env=dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=root))
    assert res.returncode == 87, (res.returncode, res.stderr[-500:])
    assert "stuck rendezvous" in res.stderr and time.monotonic() - t0 < 60


def body_trainer_heartbeat(rank, world):
    """The trainer checks the heartbeat before every step: after rank 1 has gone silent, rank 0's next
    step raises RankFailure on the host instead of entering a collective that nobody answers."""
    from distdl_b200 import models
    from distdl_b200.parallel import Heartbeat, RankFailure, SyntheticTokens, Trainer
    torch.manual_seed(0)
    cfg = models.llama_tiny(dtype=torch.float32, max_seq=16, vocab_size=64, d_model=32, ffn_dim=64)
    cfg.n_layers, cfg.n_heads, cfg.n_kv_heads = 1, 2, 2
    layout = models.ParallelLayout(2, 1)
    hb = Heartbeat(interval=0.1, limit=1.0, prefix="test/hb_trainer").start()
    hb.wait_for_all(timeout=30)
    trainer = Trainer(models.Decoder(cfg, layout), global_tokens_per_step=2 * 16, micro_batch=1, warmup_steps=0,
                      heartbeat=hb)
    block = SyntheticTokens(1, 16, cfg.vocab_size, dp_index=layout.dp_index).next()
    trainer.step(block)                          # both ranks alive: a normal step
    if rank == 1:
        hb.stop()
        time.sleep(3.0)
        return "silent"
    time.sleep(2.0)
    try:
        trainer.step(block)
    except RankFailure as e:
        return f"detected {e.ranks}"
    return "not detected"


def test_trainer_step_raises_when_a_peer_stopped_beating():
    out = run_ranks("test_failure_detection", "body_trainer_heartbeat", 2, timeout=180)
    assert out == ["detected (1,)", "silent"], out


# ------------------------------------------------ the flag protocol, modelled on the host
def test_flag_protocol_overlapping_teams_and_counter_wrap():
    """Counters are per pair of ranks and only grow: launches on overlapping teams stay in step
    without any reset, also across the wrap of the 32-bit counters."""
    from distdl_b200.parallel import protocol_model as pm
    assert pm.signed_distance(3, 0xFFFFFFFE) == 5 and pm.signed_distance(0xFFFFFFFE, 3) == -5
    teams = [[0, 1, 2, 3], [0, 1], [2, 3], [0, 2], [1, 3], [1, 2], [3, 0, 1]]
    for start in (0, (1 << 32) - 7):
        world = pm.World(4, ctas=2, start=start, spin_limit_s=20.0)

        def rank_program(me):
            seen = []
            for it in range(12):
                for team in teams:
                    if me in team:
                        got = world.all_gather(me, team, (me, it, tuple(team)))
                        assert got == [(peer, it, tuple(team)) for peer in team], (me, it, team, got)
                        seen.append(len(got))
            return sum(seen)
        out = pm.run_ranks(world, rank_program)
        assert all(world.status[r].code == 0 for r in range(4)) and out[0] > 0
        # 12 rounds x 2 steps per launch, counted per pair: ranks 0 and 1 share three of the teams
        assert world.steps_done[0][1] - start == 12 * 2 * 3
        assert world.pad[0][0][1] == (start + 12 * 2 * 3) & 0xFFFFFFFF


def test_flag_protocol_withheld_signal_times_out_and_fails_fast():
    """A peer whose signals never arrive: the bounded wait records (1005, 100 + step, expected, seen),
    the launch returns without a result, and every later wait of that rank gives up at once."""
    from distdl_b200.parallel import protocol_model as pm
    world = pm.World(2, ctas=1, spin_limit_s=0.3)
    world.withheld.add((1, 0))                     # rank 1's signals to rank 0 are lost

    def rank_program(me):
        t0 = time.monotonic()
        first = world.all_gather(me, [0, 1], me)
        t1 = time.monotonic()
        second = world.all_gather(me, [0, 1], me)
        return first, second, t1 - t0, time.monotonic() - t1
    (a1, a2, ta1, ta2), (b1, b2, _, _) = pm.run_ranks(world, rank_program)
    assert a1 is None and a2 is None
    code, where, expected, seen = world.status[0].read()
    assert (code, where, expected, seen) == (pm.TIMEOUT_CODE, 100, 1, 0)
    assert ta1 >= 0.3 and ta2 < 0.2                # the second launch does not wait again
    # rank 1 got rank 0's first signal and read a result; after that its counters are out of step with
    # rank 0's (whose second launch signals again while giving up at once), so one of its later waits runs
    # out as well: a failure on one rank surfaces on its peers, which is why the heap is then poisoned
    assert b1 == [0, 1] and b2 is None
    assert world.status[1].code == pm.TIMEOUT_CODE and world.status[1].where in (100, 101)


def test_push_collectives_keep_every_launch_apart():
    """The reduce-scatter that pushes slices into the owners' staging buffers and the two-rank
    all-reduce that pushes its sums: many launches in a row with ranks running ahead of each other at
    random; every launch must see its own data only (a missing barrier would let a fast rank's next
    launch overwrite a slice that its owner has not summed yet: with the first barrier taken out of
    the model, about half of these launches return wrong sums), mixed with all-gathers on the same
    counters."""
    import random

    from distdl_b200.parallel import protocol_model as pm
    n, launches, length = 4, 60, 6
    world = pm.World(n, ctas=2, spin_limit_s=30.0)
    team = list(range(n))

    def rank_program(me):
        rng = random.Random(me)

        def jitter():
            if rng.random() < 0.3:
                time.sleep(rng.random() * 0.002)
        for it in range(launches):
            rows = [[1000 * it + 10 * me + j + v for v in range(length)] for j in range(n)]
            got = world.reduce_scatter_push(me, team, rows, jitter)
            want = [sum(1000 * it + 10 * r + me + v for r in range(n)) for v in range(length)]
            assert got == want, (me, it, got, want)
            if it % 7 == 0:
                assert world.all_gather(me, team, (me, it)) == [(r, it) for r in team]
        return True
    assert all(pm.run_ranks(world, rank_program))
    assert all(world.status[r].code == 0 for r in range(n))
    # the two-rank all-reduce, odd length (unequal halves), on a sub-team while the others idle
    world = pm.World(n, ctas=2, spin_limit_s=30.0)
    pair = [2, 1]

    def pair_program(me):
        if me not in pair:
            return True
        rng = random.Random(7 + me)

        def jitter():
            if rng.random() < 0.3:
                time.sleep(rng.random() * 0.002)
        for it in range(launches):
            value = [100 * it + me + 3 * v for v in range(7)]
            got = world.all_reduce_push(me, pair, value, jitter)
            want = [200 * it + pair[0] + pair[1] + 6 * v for v in range(7)]
            assert got == want, (me, it, got, want)
        return True
    assert all(pm.run_ranks(world, pair_program))
    assert world.steps_done[1][2] == 2 * launches and world.steps_done[0][1] == 0

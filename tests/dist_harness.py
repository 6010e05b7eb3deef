"""Runs test bodies on several CPU ranks (gloo, 127.0.0.1) in child processes.

The reference runs its suite under ``mpirun`` with oversubscribed ranks
(``tox.ini:33-37``); here a pool of worker processes per world size is started
on first use and reused by every multi-rank test of the session, so the whole
suite runs under a plain ``pytest``.  A rank that raises reports its traceback
to the parent; after any failure or timeout the pool is torn down (the ranks
may be out of step) and the next test gets a fresh one.
"""
import atexit
import multiprocessing as mp
import os
import queue as queue_mod
import socket
import traceback

_pools = {}


def _free_port():
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world_size, port, jobs, results, env):
    try:
        os.environ.update(env)
        os.environ["RANK"] = str(rank)
        os.environ["WORLD_SIZE"] = str(world_size)
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ.setdefault("OMP_NUM_THREADS", "1")
        import datetime
        import importlib

        import torch
        import torch.distributed as dist
        torch.set_num_threads(1)
        dist.init_process_group("gloo", rank=rank, world_size=world_size,
                                timeout=datetime.timedelta(seconds=float(os.environ.get("DIST_HARNESS_TIMEOUT_S", 60))))
        import distdl_b200
        distdl_b200.config.set_backend("mpi", "numpy")
        results.put((rank, "ready", None))
    except BaseException:
        results.put((rank, "error", traceback.format_exc()))
        return
    while True:
        job = jobs.get()
        if job is None:
            break
        module, fn_name, args = job
        try:
            mod = importlib.import_module(module)
            out = getattr(mod, fn_name)(rank, world_size, *args)
            dist.barrier()
            results.put((rank, "ok", out))
        except BaseException:
            results.put((rank, "error", traceback.format_exc()))
    try:
        dist.destroy_process_group()
    except BaseException:
        pass


class _Pool:
    def __init__(self, world_size, env):
        ctx = mp.get_context("spawn")
        self.world_size = world_size
        self.env_key = tuple(sorted(env.items()))
        self.results = ctx.Queue()
        self.jobs = [ctx.Queue() for _ in range(world_size)]
        port = _free_port()
        self.procs = [ctx.Process(target=_worker, args=(r, world_size, port, self.jobs[r], self.results, env),
                                  daemon=True) for r in range(world_size)]
        for p in self.procs:
            p.start()
        self._collect("ready", 240)

    def _collect(self, want, timeout):
        out = {}
        for _ in range(self.world_size):
            try:
                rank, status, payload = self.results.get(timeout=timeout)
            except queue_mod.Empty:
                self.kill()
                raise AssertionError(f"timeout after {timeout}s waiting for ranks (got {sorted(out)})")
            if status == "error":
                self.kill()
                raise AssertionError(f"rank {rank} failed:\n{payload}")
            out[rank] = payload
        return [out[r] for r in range(self.world_size)]

    def run(self, module, fn_name, args, timeout):
        for q in self.jobs:
            q.put((module, fn_name, tuple(args)))
        return self._collect("ok", timeout)

    def kill(self):
        for p in self.procs:
            if p.is_alive():
                p.terminate()
        for p in self.procs:
            p.join(timeout=5)
        _pools.pop((self.world_size, self.env_key), None)

    def close(self):
        for q in self.jobs:
            q.put(None)
        for p in self.procs:
            p.join(timeout=5)
            if p.is_alive():
                p.terminate()


def run_ranks(module, fn_name, world_size, args=(), timeout=120, env=None):
    """Runs ``module.fn_name(rank, world_size, *args)`` on ``world_size`` ranks.
    Returns the per-rank results; raises AssertionError when a rank fails."""
    env = env or {}
    key = (world_size, tuple(sorted(env.items())))
    pool = _pools.get(key)
    if pool is None:
        pool = _Pool(world_size, env)
        _pools[key] = pool
    return pool.run(module, fn_name, args, timeout)


@atexit.register
def _shutdown():
    for pool in list(_pools.values()):
        pool.close()
    _pools.clear()

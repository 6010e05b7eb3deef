"""Host-side failure detection: a heartbeat between the ranks of a job and a wall-clock watchdog
around steps that can block.

The reference has neither (a rank that dies or stalls hangs every other rank in its next MPI /
NCCL call).  Here the ranks learn about a missing peer ON THE HOST, before they launch the next
kernel or collective that would wait for it:

* :class:`Heartbeat` -- every rank writes a counter to the job's key-value store (the
  ``torch.distributed`` rendezvous store) from a daemon thread; :meth:`Heartbeat.check` reads the
  others' entries and raises :class:`RankFailure` naming the ranks whose entry has not moved for
  longer than the limit, or that announced their departure with :meth:`Heartbeat.leave`.  Nothing
  on a GPU is involved, so a test can make a rank fall silent without touching a device.
* :class:`Watchdog` -- a context manager with a wall-clock limit for steps that may block forever
  (creating communicators, the first collective of a new team, loading a checkpoint from shared
  storage).  When the limit passes it dumps all Python stacks, runs ``on_expire`` and, by default,
  ends the process with exit code 87 so that the launcher sees a failed rank instead of a silent
  job; the other ranks then find it through their heartbeat or the process-group time-out.

The device-side half of failure detection (bounded waits inside the kernels, the status record
and ``symm.check_health``) lives in :mod:`distdl_b200.parallel.symm`.
"""
from __future__ import annotations

import faulthandler
import os
import sys
import threading
import time

import torch.distributed as dist


class RankFailure(RuntimeError):
    """Some ranks stopped answering.  ``ranks`` lists them, ``left`` those that said goodbye."""

    def __init__(self, ranks, left=()):
        self.ranks, self.left = tuple(ranks), tuple(left)
        parts = []
        silent = [r for r in self.ranks if r not in self.left]
        if silent:
            parts.append(f"no heartbeat from rank(s) {silent}")
        if self.left:
            parts.append(f"rank(s) {list(self.left)} left the job")
        super().__init__("; ".join(parts))


def _default_store():
    from torch.distributed import distributed_c10d
    return distributed_c10d._get_default_store()


class Heartbeat:
    """``Heartbeat(interval=1.0, limit=10.0).start()`` on every rank; ``check()`` where a missing
    peer would otherwise hang this rank (the trainer calls it before every step).

    ``store`` defaults to the rendezvous store of the default process group; ``rank`` / ``world``
    to its rank and size.  The beat is a counter, not a timestamp, so the ranks' clocks need not
    agree: a peer is stale when its counter has not changed for ``limit`` seconds of THIS rank's
    monotonic clock."""

    def __init__(self, interval: float = 1.0, limit: float = 10.0, store=None, rank: int = None, world: int = None,
                 prefix: str = "distdl/heartbeat"):
        self.interval, self.limit = float(interval), float(limit)
        self.store = store if store is not None else _default_store()
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.prefix = prefix
        self._count = 0
        self._stop = threading.Event()
        self._thread = None
        self._seen = {}            # rank -> (last counter value, monotonic time it changed)
        self._left = set()
        self._lock = threading.Lock()

    def _key(self, rank):
        return f"{self.prefix}/{rank}"

    def beat(self):
        self._count += 1
        self.store.set(self._key(self.rank), str(self._count))

    def start(self):
        self.beat()
        if self._thread is None:
            def run():
                while not self._stop.wait(self.interval):
                    try:
                        self.beat()
                        self._observe()        # so that staleness is measured between checks too
                    except Exception:          # the store went away with rank 0: nothing left to tell
                        return
            self._thread = threading.Thread(target=run, name="distdl-heartbeat", daemon=True)
            self._thread.start()
        now = time.monotonic()
        with self._lock:
            for r in range(self.world):
                self._seen.setdefault(r, (None, now))
        return self

    def stop(self):
        """Stops beating WITHOUT saying goodbye (what a stalled or dead rank looks like)."""
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)
            self._thread = None

    def leave(self):
        """Announces an orderly departure, then stops beating.  Call between steps, with none of
        this rank's kernels or collectives in flight."""
        self.store.set(self._key(self.rank) + "/left", "1")
        self.stop()

    def _read(self, key):
        # a plain get() blocks until the key exists: ask first
        try:
            if not self.store.check([key]):
                return None
            return self.store.get(key).decode()
        except Exception:
            return None

    def _observe(self):
        """Reads the peers' entries and notes when each counter last moved."""
        now = time.monotonic()
        with self._lock:
            for r in range(self.world):
                if r == self.rank or r in self._left:
                    continue
                if self._read(self._key(r) + "/left") is not None:
                    self._left.add(r)
                    continue
                value = self._read(self._key(r))
                last, _ = self._seen.get(r, (None, now))
                if value is not None and value != last:
                    self._seen[r] = (value, now)
                else:
                    self._seen.setdefault(r, (None, now))

    def stale(self):
        """(silent ranks, ranks that left).  Never blocks longer than the store round trips."""
        self._observe()
        now = time.monotonic()
        with self._lock:
            left = sorted(self._left)
            silent = [r for r, (_, since) in sorted(self._seen.items())
                      if r != self.rank and r not in self._left and now - since > self.limit]
        return silent, left

    def check(self):
        silent, left = self.stale()
        if silent or left:
            raise RankFailure(sorted(silent + left), left)

    def wait_for_all(self, timeout: float = 60.0):
        """Blocks until every rank has beaten at least once (start-up), or raises RankFailure."""
        end = time.monotonic() + timeout
        missing = list(range(self.world))
        while time.monotonic() < end:
            missing = [r for r in range(self.world) if r != self.rank and self._read(self._key(r)) is None]
            if not missing:
                now = time.monotonic()
                values = {r: self._read(self._key(r)) for r in range(self.world)}
                with self._lock:
                    for r, v in values.items():
                        self._seen[r] = (v, now)
                return
            time.sleep(min(0.05, self.interval))
        raise RankFailure(missing)


class Watchdog:
    """``with Watchdog(120, "creating the tensor-parallel teams"): ...`` -- if the block is still
    running after the limit: all Python stacks go to stderr, ``on_expire(what, limit)`` runs, and
    (unless ``exit_code`` is None) the process ends with ``exit_code``.  Finishing in time cancels
    it.  ``expired`` tells afterwards whether the limit was hit (for ``exit_code=None``)."""

    def __init__(self, limit_s: float, what: str = "", on_expire=None, exit_code=87, dump_stacks: bool = True):
        self.limit, self.what, self.on_expire = float(limit_s), what, on_expire
        self.exit_code, self.dump_stacks = exit_code, dump_stacks
        self.expired = False
        self._timer = None

    def _fire(self):
        self.expired = True
        sys.stderr.write(f"[distdl watchdog] '{self.what}' still running after {self.limit:.1f} s\n")
        if self.dump_stacks:
            try:
                faulthandler.dump_traceback(file=sys.stderr, all_threads=True)
            except Exception:
                pass
        if self.on_expire is not None:
            try:
                self.on_expire(self.what, self.limit)
            except Exception as e:               # the hook must not keep the process alive
                sys.stderr.write(f"[distdl watchdog] on_expire raised {e!r}\n")
        sys.stderr.flush()
        if self.exit_code is not None:
            os._exit(self.exit_code)

    def __enter__(self):
        self._timer = threading.Timer(self.limit, self._fire)
        self._timer.daemon = True
        self._timer.start()
        return self

    def __exit__(self, *exc):
        self._timer.cancel()
        return False

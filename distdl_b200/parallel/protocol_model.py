"""A host model of the flag protocol that the device collectives use, for tests without a GPU.

The kernels in ``csrc/collectives.cu`` synchronise the members of a team through one signal pad
per GPU: 32-bit counters that only grow, one per (CTA, writing rank).  Barrier number ``step`` of a
launch on a team is

    for every peer i:  pad[i][cta][me] += 1                       (a release store into i's memory)
    for every peer i:  wait until pad[me][cta][i] - (expect[i] + step) >= 0 as a SIGNED 32-bit number

where ``expect[i]`` = 1 + the number of barrier steps this rank has completed with peer ``i`` in all
earlier launches (kept on the host, ``SymmetricHeap.steps_done``).  Counters therefore never need
resetting, teams may overlap (the count is per pair of ranks), and the comparison survives the wrap
of the counter after 2^32 signals.  Every wait is bounded: when it runs out, the waiter records
``(code 1005, where = 100 + step, expected, seen)`` in a status record, and from then on every wait
of that rank gives up at once, because its counters are out of step with its peers'.

This module restates exactly that in Python, with one thread per rank, so that the bookkeeping
(overlapping teams, wrap-around, a signal that never comes) can be exercised on any machine:
``tests/test_failure_detection.py`` and ``tests/test_utilities.py`` use it.  It is a model for
tests and documentation, not a transport.
"""
from __future__ import annotations

import threading
import time

TIMEOUT_CODE = 1005
MASK = 0xFFFFFFFF


def signed_distance(seen: int, want: int) -> int:
    """``(int32_t)(seen - want)`` of the device code."""
    d = (seen - want) & MASK
    return d - (1 << 32) if d & 0x80000000 else d


class Status:
    """The per-device status record: first failure wins, later waits fail fast."""

    def __init__(self):
        self.code, self.where, self.expected, self.seen = 0, 0, 0, 0

    def report(self, where, expected, seen):
        if self.code == 0:
            self.code, self.where, self.expected, self.seen = TIMEOUT_CODE, where, expected, seen

    def read(self):
        return self.code, self.where, self.expected, self.seen


class World:
    """Signal pads and staging buffers of ``n`` ranks (shared by the rank threads), plus what every
    rank's host keeps: ``steps_done[rank][peer]``.  ``start`` presets all pair counters (pads and
    host counts alike), e.g. just below 2^32 to cross the wrap."""

    def __init__(self, n: int, ctas: int = 2, start: int = 0, spin_limit_s: float = 0.5):
        self.n, self.ctas, self.spin_limit = n, ctas, spin_limit_s
        self.pad = [[[start & MASK for _ in range(n)] for _ in range(ctas)] for _ in range(n)]
        self.steps_done = [[start for _ in range(n)] for _ in range(n)]
        self.staging = [None] * n
        self.status = [Status() for _ in range(n)]
        self._lock = threading.Lock()          # stands in for the atomicity of a 32-bit store / add
        self.withheld = set()                  # (from_rank, to_rank): signals a test wants dropped

    # ---- device side -------------------------------------------------------------------
    def _signal(self, me, peer, cta):
        if (me, peer) in self.withheld:
            return
        with self._lock:
            self.pad[peer][cta][me] = (self.pad[peer][cta][me] + 1) & MASK

    def _wait(self, me, peer, cta, want, step):
        st = self.status[me]
        t0 = time.monotonic()
        while True:
            seen = self.pad[me][cta][peer]
            if signed_distance(seen, want) >= 0:
                return True
            if st.code != 0:                   # an earlier wait ran out: do not wait again
                return False
            if time.monotonic() - t0 > self.spin_limit:
                st.report(100 + step, want, seen)
                return False
            time.sleep(0)

    def barrier(self, me, team, expect, step):
        """All CTAs of rank ``me``: signal every peer, then wait for every peer."""
        ok = True
        for cta in range(self.ctas):
            for peer in team:
                if peer != me:
                    self._signal(me, peer, cta)
            for i, peer in enumerate(team):
                if peer != me:
                    ok &= self._wait(me, peer, cta, (expect[i] + step) & MASK, step)
        return ok

    # ---- host side ---------------------------------------------------------------------
    def team_args(self, me, team):
        return [(self.steps_done[me][peer] + 1) & MASK for peer in team]

    def advance(self, me, team, steps):
        for peer in team:
            if peer != me:
                self.steps_done[me][peer] += steps

    def all_gather(self, me, team, value):
        """One launch of the all-gather kernel on ``team``: stage, barrier 0 (everybody staged),
        read the peers' staging buffers, barrier 1 (everybody done reading, the buffers may be
        reused).  Returns the gathered list, or None after a time-out."""
        self.staging[me] = value
        expect = self.team_args(me, team)
        out = None
        if self.barrier(me, team, expect, 0):
            out = [self.staging[peer] for peer in team]
            self.barrier(me, team, expect, 1)
        self.advance(me, team, 2)              # the host counts the launch's steps either way
        return out


    # ---- the push forms (csrc/collectives.cu: reducescatter_push_kernel, allreduce_kernel in teams of two) ----
    def reduce_scatter_push(self, me, team, rows, jitter=None):
        """One launch of the reduce-scatter that needs no staging copy.  ``rows[i]`` is this rank's
        slice (a list of numbers) for member ``i``.  Barrier 0: the members are done with their staging
        buffers (a fast rank must not push the next launch's slices into a buffer that its owner is
        still summing).  Then slice ``j`` goes straight into slot ``[me]`` of member ``j``'s staging
        buffer; barrier 1: everything for this rank has arrived; the sum is formed from local memory in
        member order.  Returns this rank's summed slice, or None after a time-out."""
        idx, n = team.index(me), len(team)
        expect = self.team_args(me, team)
        out = None
        if self.barrier(me, team, expect, 0):
            for k in range(1, n):
                j = (idx + k) % n
                if jitter:
                    jitter()
                if not isinstance(self.staging[team[j]], dict):
                    self.staging[team[j]] = {}
                self.staging[team[j]][("slot", idx)] = list(rows[j])
            if self.barrier(me, team, expect, 1):
                mine = self.staging[me] if isinstance(self.staging[me], dict) else {}
                parts = [rows[idx] if i == idx else mine[("slot", i)] for i in range(n)]
                if jitter:
                    jitter()
                out = [sum(vals) for vals in zip(*parts)]
        self.advance(me, team, 2)
        return out

    def all_reduce_push(self, me, team, value, jitter=None):
        """One launch of the two-shot all-reduce of a team of two.  The input is staged in this rank's
        buffer; barrier 0; this rank sums ITS half of the vector from both buffers and writes the sums
        into its output and, in place, into the other rank's staging buffer (that half of the other
        rank's input has just been read by the one reader it has); barrier 1; the other half of the
        result is now in this rank's own staging buffer.  No third barrier: after barrier 1 nobody
        touches the other rank's buffer any more."""
        assert len(team) == 2
        idx = team.index(me)
        other = team[1 - idx]
        self.staging[me] = list(value)
        expect = self.team_args(me, team)
        n = len(value)
        half = (n + 1) // 2
        lo, hi = (0, half) if idx == 0 else (half, n)
        out = None
        if self.barrier(me, team, expect, 0):
            out = [None] * n
            for v in range(lo, hi):
                s = self.staging[team[0]][v] + self.staging[team[1]][v]
                if jitter:
                    jitter()
                self.staging[other][v] = s
                out[v] = s
            if self.barrier(me, team, expect, 1):
                for v in list(range(0, lo)) + list(range(hi, n)):
                    out[v] = self.staging[me][v]
            else:
                out = None
        self.advance(me, team, 2)
        return out


def run_ranks(world: World, fn):
    """Runs ``fn(rank)`` on one thread per rank; returns the results (exceptions re-raised)."""
    results, errors = [None] * world.n, []

    def work(r):
        try:
            results[r] = fn(r)
        except BaseException as e:             # noqa: BLE001 - handed to the caller
            errors.append(e)
    threads = [threading.Thread(target=work, args=(r,)) for r in range(world.n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]
    return results

"""A host model of the pipelines inside the attention kernels (``csrc/attention_bwd2_impl.cuh`` and the
two-tile forward kernel ``csrc/attention_fwd2_impl.cuh``), for tests without a GPU.

The kernels are warp-specialised: one thread issues TMA loads, one thread issues tensor-core products
(which execute in issue order and signal completion through ``tcgen05.commit``), sixteen warps do the
softmax arithmetic; they hand tiles to each other through mbarriers whose phases are waited for by
parity.  What can go wrong in such a design is not arithmetic but scheduling: a barrier that is waited
for with the wrong parity, a tile that is overwritten before its last reader is through, a cycle of
waits.  This module restates the kernels' schedules with the same barriers, the same parities and
the same issue order, one Python thread per role, tiles as small NumPy arrays, and random delays in
every role, so that

* every run must terminate (each wait is bounded, as on the device), and
* the gradients must equal the directly computed ones, which they only do if no tile was overwritten
  early or read late.

``tests/test_attention_model.py`` runs it over short and long sweeps, grouped-query heads, causal and
full attention.  It is a model for tests and documentation, not an implementation.
"""
from __future__ import annotations

import queue
import random
import threading
import time

import numpy as np

WAIT_LIMIT_S = 20.0


class PipelineStuck(RuntimeError):
    """A bounded wait of the model ran out."""


class MBarrier:
    """``mbarrier`` with an arrival count: the phase flips when ``count`` arrivals have come in, and
    ``wait(parity)`` returns once the phase of that parity has completed (so a fresh barrier lets
    ``wait(1)`` through at once, the idiom for "empty" barriers)."""

    def __init__(self, count: int, name: str):
        self.count, self.pending, self.phase, self.name = count, count, 0, name
        self._cv = threading.Condition()

    def arrive(self):
        with self._cv:
            self.pending -= 1
            if self.pending == 0:
                self.pending = self.count
                self.phase ^= 1
                self._cv.notify_all()

    def wait(self, parity: int):
        deadline = time.monotonic() + WAIT_LIMIT_S
        with self._cv:
            while self.phase == parity:
                left = deadline - time.monotonic()
                if left <= 0:
                    raise PipelineStuck(f"wait on {self.name} (parity {parity}) ran out")
                self._cv.wait(left)


class TensorPipe:
    """The tensor cores of one SM: products execute in the order they were issued; a commit arrives on
    its barrier when everything issued before it has finished."""

    def __init__(self, rng):
        self._q = queue.Queue()
        self._rng = rng
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def _run(self):
        while True:
            item = self._q.get()
            if item is None:
                return
            if self._rng.random() < 0.3:
                time.sleep(self._rng.random() * 0.001)
            item()

    def issue(self, fn):
        self._q.put(fn)

    def commit(self, bar: MBarrier):
        self._q.put(bar.arrive)

    def close(self):
        self._q.put(None)
        self._t.join()


def _jitter(rng):
    if rng.random() < 0.3:
        time.sleep(rng.random() * 0.001)


def _run_roles(roles):
    errors = []

    def guard(fn):
        def run():
            try:
                fn()
            except BaseException as e:      # noqa: BLE001 - handed to the caller
                errors.append(e)
        return run
    threads = [threading.Thread(target=guard(fn)) for fn in roles]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]


def dkdv_tile(Q, dO, K, V, lse2, delta, scale, causal_diag_at=None, softmax_warps=4, seed=0, slow_warp=None):
    """The dK / dV kernel for ONE key tile: ``Q``, ``dO`` are lists with one ``[BT, D]`` array per
    iteration of the sweep (query tile x head of the group), ``lse2`` / ``delta`` lists of ``[BT]``
    statistics, ``K`` / ``V`` ``[BT, D]``.  ``causal_diag_at``: iterations whose query tile is the key
    tile itself (the causal mask applies there).  Returns ``(dK, dV)`` as the kernel would store them.
    Here single barriers for "P written" and "dS written" suffice: dP of the next iteration is issued
    only after dS of this one, so no softmax warp can be a whole iteration ahead of another
    (``slow_warp`` delays one of them to show it)."""
    iters, (BT, D) = len(Q), K.shape
    W = softmax_warps
    cols = BT // W
    diag = set(causal_diag_at or ())
    c = scale * 1.4426950408889634
    bar = {n: MBarrier(1, n) for n in ("kv_full", "s_full", "dp_full", "acc_done")}
    for n in ("q_full", "q_empty", "do_full", "do_empty"):
        bar[n] = [MBarrier(1, f"{n}[{s}]") for s in range(2)]
    bar["p_full"], bar["ds_full"] = MBarrier(W, "p_full"), MBarrier(W, "ds_full")
    smem = {"K": None, "V": None, "Q": [None, None], "dO": [None, None], "stats": [None, None]}
    tmem = {"S": np.zeros((BT, BT)), "dP": np.zeros((BT, BT)), "dV": np.zeros((BT, D)), "dK": np.zeros((BT, D))}
    pipe = TensorPipe(random.Random(seed))

    def tma():
        rng = random.Random(seed + 1)
        smem["K"], smem["V"] = K.copy(), V.copy()
        bar["kv_full"].arrive()
        for it in range(iters):
            st, ph = it & 1, (it >> 1) & 1
            bar["q_empty"][st].wait(ph ^ 1)
            _jitter(rng)
            smem["Q"][st], smem["stats"][st] = Q[it].copy(), (lse2[it].copy(), delta[it].copy())
            bar["q_full"][st].arrive()
            bar["do_empty"][st].wait(ph ^ 1)
            _jitter(rng)
            smem["dO"][st] = dO[it].copy()
            bar["do_full"][st].arrive()

    def mma():
        rng = random.Random(seed + 2)

        def s_t(st):            # S^T = K Q^T
            return lambda: tmem["S"].__setitem__(slice(None), smem["K"] @ smem["Q"][st].T)

        def dp_t(st):           # dP^T = V dO^T
            return lambda: tmem["dP"].__setitem__(slice(None), smem["V"] @ smem["dO"][st].T)

        def acc(name, a, b_name, st, first):      # dV (+)= P^T dO,  dK (+)= dS^T Q  (A operand from tensor memory)
            def fn():
                prod = tmem[a] @ smem[b_name][st]
                tmem[name][:] = prod if first else tmem[name] + prod
            return fn
        bar["kv_full"].wait(0)
        bar["q_full"][0].wait(0)
        pipe.issue(s_t(0))
        pipe.commit(bar["s_full"])
        bar["do_full"][0].wait(0)
        pipe.issue(dp_t(0))
        pipe.commit(bar["dp_full"])
        for it in range(iters):
            st, nst, nph, more = it & 1, (it & 1) ^ 1, ((it + 1) >> 1) & 1, it + 1 < iters
            bar["p_full"].wait(it & 1)
            _jitter(rng)
            pipe.issue(acc("dV", "S", "dO", st, it == 0))
            pipe.commit(bar["do_empty"][st])
            if more:
                bar["q_full"][nst].wait(nph)
                pipe.issue(s_t(nst))
                pipe.commit(bar["s_full"])
            bar["ds_full"].wait(it & 1)
            _jitter(rng)
            pipe.issue(acc("dK", "dP", "Q", st, it == 0))
            pipe.commit(bar["q_empty"][st])
            if more:
                bar["do_full"][nst].wait(nph)
                pipe.issue(dp_t(nst))
                pipe.commit(bar["dp_full"])
        pipe.commit(bar["acc_done"])

    def softmax(w):
        def run():
            rng = random.Random(seed + 10 + w)
            mine = slice(w * cols, (w + 1) * cols)              # this warp's query columns
            rows = np.arange(BT)[:, None]
            for it in range(iters):
                st = it & 1
                bar["q_full"][st].wait((it >> 1) & 1)           # the statistics came with the Q tile
                bar["s_full"].wait(it & 1)
                _jitter(rng)
                l2, dl = smem["stats"][st]
                p = np.exp2(tmem["S"][:, mine] * c - l2[None, mine])
                if it in diag:
                    p = np.where(np.arange(w * cols, (w + 1) * cols)[None, :] < rows, 0.0, p)
                tmem["S"][:, mine] = p                          # P^T over S^T, this warp's columns only
                bar["p_full"].arrive()
                bar["dp_full"].wait(it & 1)
                _jitter(rng)
                if w == slow_warp:
                    time.sleep(0.01)                            # a warp that lags behind the others
                tmem["dP"][:, mine] = p * (tmem["dP"][:, mine] - dl[None, mine])
                bar["ds_full"].arrive()
            bar["acc_done"].wait(0)
        return run

    try:
        _run_roles([tma, mma] + [softmax(w) for w in range(W)])
    finally:
        pipe.close()
    return tmem["dK"] * scale, tmem["dV"].copy()


def dq_tile(Q, dO, K, V, lse2, delta, scale, causal_diag_at=None, softmax_warps=4, seed=0, ds_full_buffers=2,
            slow_warp=None):
    """The dQ kernel for ONE query tile: ``K``, ``V`` are lists with one ``[BT, D]`` array per key tile
    of the sweep, ``Q`` / ``dO`` ``[BT, D]``, ``lse2`` / ``delta`` ``[BT]``.  Returns ``dQ``.
    ``slow_warp`` delays one softmax warp before every dS write (the others may then run an iteration
    ahead of it); ``ds_full_buffers=1`` restates the schedule with a single "dS written" barrier."""
    nblocks, (BT, D) = len(K), Q.shape
    W = softmax_warps
    cols = BT // W
    diag = causal_diag_at
    c = scale * 1.4426950408889634
    KS, VS = 3, 2
    bar = {n: MBarrier(1, n) for n in ("qdo_full", "s_full", "acc_done")}
    bar["k_full"] = [MBarrier(1, f"k_full[{s}]") for s in range(KS)]
    bar["k_empty"] = [MBarrier(1, f"k_empty[{s}]") for s in range(KS)]
    bar["v_full"] = [MBarrier(1, f"v_full[{s}]") for s in range(VS)]
    bar["v_empty"] = [MBarrier(1, f"v_empty[{s}]") for s in range(VS)]
    bar["dp_full"] = [MBarrier(1, f"dp_full[{s}]") for s in range(2)]
    bar["p_done"] = MBarrier(W, "p_done")
    # one per dP buffer: a warp that runs an iteration ahead arrives for the OTHER buffer and cannot
    # complete the phase that a slower warp has not arrived for yet (ds_full_buffers=1 models the single
    # barrier, with which exactly that happens)
    bar["ds_full"] = [MBarrier(W, f"ds_full[{s}]") for s in range(ds_full_buffers)]
    smem = {"Q": None, "dO": None, "K": [None] * KS, "V": [None] * VS}
    tmem = {"S": np.zeros((BT, BT)), "dP": [np.zeros((BT, BT)), np.zeros((BT, BT))], "dQ": np.zeros((BT, D))}
    pipe = TensorPipe(random.Random(seed))

    def tma():
        rng = random.Random(seed + 1)
        smem["Q"], smem["dO"] = Q.copy(), dO.copy()
        bar["qdo_full"].arrive()
        for jj in range(nblocks):
            ks, vs = jj % KS, jj % VS
            bar["k_empty"][ks].wait(((jj // KS) & 1) ^ 1)
            _jitter(rng)
            smem["K"][ks] = K[jj].copy()
            bar["k_full"][ks].arrive()
            bar["v_empty"][vs].wait(((jj // VS) & 1) ^ 1)
            _jitter(rng)
            smem["V"][vs] = V[jj].copy()
            bar["v_full"][vs].arrive()

    def mma():
        rng = random.Random(seed + 2)

        def issue_s_dp(jj):
            ks, vs, b = jj % KS, jj % VS, jj & 1
            bar["k_full"][ks].wait((jj // KS) & 1)
            pipe.issue(lambda: tmem["S"].__setitem__(slice(None), smem["Q"] @ smem["K"][ks].T))
            pipe.commit(bar["s_full"])
            bar["v_full"][vs].wait((jj // VS) & 1)
            pipe.issue(lambda: tmem["dP"][b].__setitem__(slice(None), smem["dO"] @ smem["V"][vs].T))
            pipe.commit(bar["dp_full"][b])
            pipe.commit(bar["v_empty"][vs])
        bar["qdo_full"].wait(0)
        issue_s_dp(0)
        for jj in range(nblocks):
            bar["p_done"].wait(jj & 1)                          # S(jj) is in the softmax threads' registers
            _jitter(rng)
            if jj + 1 < nblocks:
                issue_s_dp(jj + 1)
            nb = len(bar["ds_full"])
            bar["ds_full"][jj % nb].wait((jj // nb) & 1)
            _jitter(rng)
            ks, b, first = jj % KS, jj & 1, jj == 0

            def dq(ks=ks, b=b, first=first):                    # dQ (+)= dS K  (A operand from tensor memory)
                prod = tmem["dP"][b] @ smem["K"][ks]
                tmem["dQ"][:] = prod if first else tmem["dQ"] + prod
            pipe.issue(dq)
            pipe.commit(bar["k_empty"][ks])
        pipe.commit(bar["acc_done"])

    def softmax(w):
        def run():
            rng = random.Random(seed + 10 + w)
            mine = slice(w * cols, (w + 1) * cols)              # this warp's key columns
            rows = np.arange(BT)[:, None]
            for jj in range(nblocks):
                bar["s_full"].wait(jj & 1)
                _jitter(rng)
                s = tmem["S"][:, mine].copy()                   # tcgen05.ld: into registers
                bar["p_done"].arrive()
                p = np.exp2(s * c - lse2[:, None])
                if diag is not None and jj == diag:
                    p = np.where(np.arange(w * cols, (w + 1) * cols)[None, :] > rows, 0.0, p)
                bar["dp_full"][jj & 1].wait((jj >> 1) & 1)
                _jitter(rng)
                if w == slow_warp:
                    time.sleep(0.01)                            # a warp that lags by more than an iteration
                buf = tmem["dP"][jj & 1]
                buf[:, mine] = p * (buf[:, mine] - delta[:, None])
                bar["ds_full"][jj % len(bar["ds_full"])].arrive()
            bar["acc_done"].wait(0)
        return run

    try:
        _run_roles([tma, mma] + [softmax(w) for w in range(W)])
    finally:
        pipe.close()
    return tmem["dQ"] * scale


def fwd_pair(Q, K, V, n, scale, diag=(None, None), row_warps=4, seed=0, grow_threshold=8.0, slow_warp=None):
    """The two-tile forward kernel for ONE pair of query tiles: ``Q`` = two ``[BQ, D]`` tiles, ``K`` /
    ``V`` = lists of ``[BKV, D]`` blocks, ``n = (n0, n1)`` blocks seen by tile 0 / tile 1 (``n1 >= n0``),
    ``diag[t]`` = the block on which tile ``t`` applies the causal mask.  Scores, probabilities and the
    output accumulators live in "tensor memory"; the output is rescaled lazily (only when a row's
    running maximum has grown by more than ``grow_threshold`` in base-2 exponent units).  Returns
    ``(O, lse)`` with ``O`` = ``[2, BQ, D]`` and ``lse`` = ``[2, BQ]`` (natural logarithm)."""
    n0, n1 = n
    BQ, D = Q[0].shape
    BKV = K[0].shape[0]
    rows_per = BQ // row_warps
    c = scale * 1.4426950408889634
    ST = 2
    bar = {"q_full": MBarrier(1, "q_full")}
    for name in ("k_full", "k_empty", "v_full", "v_empty"):
        bar[name] = [MBarrier(1, f"{name}[{s}]") for s in range(ST)]
    bar["s_full"] = [MBarrier(1, f"s_full[{t}]") for t in range(2)]
    bar["p_full"] = [MBarrier(row_warps, f"p_full[{t}]") for t in range(2)]
    bar["pv_done"] = [MBarrier(1, f"pv_done[{t}]") for t in range(2)]
    smem = {"Q": [None, None], "K": [None] * ST, "V": [None] * ST}
    tmem = {"S": [np.zeros((BQ, BKV)), np.zeros((BQ, BKV))], "O": [np.zeros((BQ, D)), np.zeros((BQ, D))]}
    out, lse = np.zeros((2, BQ, D)), np.zeros((2, BQ))
    pipe = TensorPipe(random.Random(seed))

    def tma():
        rng = random.Random(seed + 1)
        smem["Q"] = [Q[0].copy(), Q[1].copy()]
        bar["q_full"].arrive()
        for j in range(n1):
            st, ph = j % ST, (j // ST) & 1
            bar["k_empty"][st].wait(ph ^ 1)
            _jitter(rng)
            smem["K"][st] = K[j].copy()
            bar["k_full"][st].arrive()
            bar["v_empty"][st].wait(ph ^ 1)
            _jitter(rng)
            smem["V"][st] = V[j].copy()
            bar["v_full"][st].arrive()

    def mma():
        rng = random.Random(seed + 2)

        def issue_s(t, j):
            st = j % ST
            pipe.issue(lambda: tmem["S"][t].__setitem__(slice(None), smem["Q"][t] @ smem["K"][st].T))
            pipe.commit(bar["s_full"][t])

        def issue_pv(t, j):
            st = j % ST

            def fn():
                prod = tmem["S"][t] @ smem["V"][st]             # P from tensor memory
                tmem["O"][t][:] = prod if j == 0 else tmem["O"][t] + prod
            pipe.issue(fn)
            pipe.commit(bar["pv_done"][t])
        bar["q_full"].wait(0)
        bar["k_full"][0].wait(0)
        issue_s(0, 0)
        issue_s(1, 0)
        for j in range(n1):
            st, ph = j % ST, (j // ST) & 1
            stn, phn = (j + 1) % ST, ((j + 1) // ST) & 1
            bar["v_full"][st].wait(ph)
            k_next_ready = False
            for t in range(2):
                nt = n0 if t == 0 else n1
                if j >= nt:
                    continue
                bar["p_full"][t].wait(j & 1)
                _jitter(rng)
                issue_pv(t, j)
                if j + 1 < nt:
                    if not k_next_ready:
                        bar["k_full"][stn].wait(phn)
                        k_next_ready = True
                    issue_s(t, j + 1)
            pipe.commit(bar["v_empty"][st])
            pipe.commit(bar["k_empty"][st])

    def softmax(t, w):
        def run():
            rng = random.Random(seed + 10 + 4 * t + w)
            mine = slice(w * rows_per, (w + 1) * rows_per)
            rows = np.arange(w * rows_per, (w + 1) * rows_per)[:, None]
            nt = n0 if t == 0 else n1
            m_ref = np.full(rows_per, -np.inf)
            l = np.zeros(rows_per)
            for j in range(nt):
                bar["s_full"][t].wait(j & 1)
                _jitter(rng)
                s = tmem["S"][t][mine].copy()
                if diag[t] is not None and j == diag[t]:
                    s = np.where(np.arange(BKV)[None, :] > rows, -np.inf, s)
                mx = np.maximum(m_ref, s.max(axis=1))
                grow = (mx - m_ref) * c > grow_threshold if j > 0 else np.zeros(rows_per, dtype=bool)
                if j == 0:
                    m_ref = mx
                if grow.any():
                    alpha = np.where(grow, np.exp2((m_ref - mx) * c), 1.0)
                    m_ref = np.where(grow, mx, m_ref)
                    l = l * alpha
                    bar["pv_done"][t].wait((j - 1) & 1)          # O_t is complete up to block j - 1
                    _jitter(rng)
                    tmem["O"][t][mine] *= alpha[:, None]
                p = np.exp2(s * c - (m_ref * c)[:, None])
                l = l + p.sum(axis=1)
                if (t, w) == slow_warp:
                    time.sleep(0.01)                             # a warp that lags behind the others
                tmem["S"][t][mine] = p                           # P over S, this warp's rows
                bar["p_full"][t].arrive()
            bar["pv_done"][t].wait((nt - 1) & 1)
            out[t, mine] = tmem["O"][t][mine] / l[:, None]
            lse[t, mine] = m_ref * scale + np.log(l)
        return run

    try:
        _run_roles([tma, mma] + [softmax(t, w) for t in range(2) for w in range(row_warps)])
    finally:
        pipe.close()
    return out, lse

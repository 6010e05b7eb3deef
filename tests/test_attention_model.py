"""The schedules of the attention backward kernels, run as a host model (one thread per role, the same
barriers, parities and issue order as ``csrc/attention_bwd2_impl.cuh``, random delays in every role):
every sweep length must terminate and give the directly computed gradients."""
import numpy as np
import pytest

from distdl_b200.ops import attention_model as model

BT, D = 8, 4
SCALE = 0.5
C = SCALE * 1.4426950408889634


def _tiles(rng, n):
    return [rng.standard_normal((BT, D)) for _ in range(n)]


def _p(q, k, l2, mask):
    p = np.exp2(q @ k.T * C - l2[:, None])
    return np.where(mask, 0.0, p) if mask is not None else p


UPPER = np.arange(BT)[None, :] > np.arange(BT)[:, None]          # key later than query


@pytest.mark.parametrize("iters,diag_at", [(1, (0,)), (2, (0,)), (3, ()), (4, (0, 2)), (7, (0,)), (12, ())])
def test_dkdv_schedule_terminates_and_matches(iters, diag_at):
    rng = np.random.default_rng(iters)
    Q, dO = _tiles(rng, iters), _tiles(rng, iters)
    K, V = _tiles(rng, 2)
    l2 = [rng.standard_normal(BT) + 2 for _ in range(iters)]
    dl = [rng.standard_normal(BT) for _ in range(iters)]
    dK = np.zeros((BT, D))
    dV = np.zeros((BT, D))
    for it in range(iters):
        p = _p(Q[it], K, l2[it], UPPER if it in diag_at else None)          # [query, key]
        ds = p * (dO[it] @ V.T - dl[it][:, None]) * SCALE
        dV += p.T @ dO[it]
        dK += ds.T @ Q[it]
    for seed in range(3):
        got_dk, got_dv = model.dkdv_tile(Q, dO, K, V, l2, dl, SCALE, causal_diag_at=diag_at, seed=seed)
        assert np.allclose(got_dv, dV, rtol=1e-10, atol=1e-10), (iters, seed)
        assert np.allclose(got_dk, dK, rtol=1e-10, atol=1e-10), (iters, seed)


@pytest.mark.parametrize("nblocks,causal", [(1, True), (2, True), (3, False), (4, True), (6, False), (9, True)])
def test_dq_schedule_terminates_and_matches(nblocks, causal):
    rng = np.random.default_rng(100 + nblocks)
    (Q, dO), K, V = _tiles(rng, 2), _tiles(rng, nblocks), _tiles(rng, nblocks)
    l2, dl = rng.standard_normal(BT) + 2, rng.standard_normal(BT)
    diag = nblocks - 1 if causal else None
    dQ = np.zeros((BT, D))
    for jj in range(nblocks):
        p = _p(Q, K[jj], l2, UPPER if jj == diag else None)
        ds = p * (dO @ V[jj].T - dl[:, None]) * SCALE
        dQ += ds @ K[jj]
    for seed in range(3):
        got = model.dq_tile(Q, dO, K, V, l2, dl, SCALE, causal_diag_at=diag, seed=seed)
        assert np.allclose(got, dQ, rtol=1e-10, atol=1e-10), (nblocks, seed)


def test_a_wrong_parity_is_caught():
    """The model has teeth: waiting for the Q tile of the NEXT iteration with the parity of this one
    (the mistake the per-stage phase arithmetic guards against) ends in a bounded wait that runs out."""
    rng = np.random.default_rng(5)
    iters = 4
    Q, dO = _tiles(rng, iters), _tiles(rng, iters)
    K, V = _tiles(rng, 2)
    l2 = [np.zeros(BT) for _ in range(iters)]
    dl = [np.zeros(BT) for _ in range(iters)]
    real_wait = model.MBarrier.wait

    def wrong(self, parity):
        return real_wait(self, parity ^ 1 if self.name == "q_full[1]" else parity)
    old_limit = model.WAIT_LIMIT_S
    model.MBarrier.wait, model.WAIT_LIMIT_S = wrong, 0.5
    try:
        with pytest.raises(model.PipelineStuck):
            model.dkdv_tile(Q, dO, K, V, l2, dl, SCALE)
    finally:
        model.MBarrier.wait, model.WAIT_LIMIT_S = real_wait, old_limit


def test_a_softmax_warp_that_lags_an_iteration_behind():
    """One softmax warp far behind the others.  The dK / dV schedule cannot let any warp run a whole
    iteration ahead (dP of the next iteration waits for dS of this one).  The dQ schedule can: S and
    dP of the next key tile are issued early, so a fast warp reaches its next "dS written" arrival
    while the slow one has not arrived for this tile; with one barrier per dP buffer that arrival
    belongs to the other buffer's phase, with a single barrier it completes the wrong phase and dQ of
    this tile is formed from a dS tile with columns missing."""
    rng = np.random.default_rng(9)
    n = 5
    Q, dO = _tiles(rng, n), _tiles(rng, n)
    K, V = _tiles(rng, 2)
    l2 = [rng.standard_normal(BT) + 2 for _ in range(n)]
    dl = [rng.standard_normal(BT) for _ in range(n)]
    dK, dV = np.zeros((BT, D)), np.zeros((BT, D))
    for it in range(n):
        p = _p(Q[it], K, l2[it], None)
        dV += p.T @ dO[it]
        dK += (p * (dO[it] @ V.T - dl[it][:, None]) * SCALE).T @ Q[it]
    got_dk, got_dv = model.dkdv_tile(Q, dO, K, V, l2, dl, SCALE, slow_warp=2)
    assert np.allclose(got_dk, dK) and np.allclose(got_dv, dV)
    (q, do), Ks, Vs = _tiles(rng, 2), _tiles(rng, n), _tiles(rng, n)
    dQ = sum((_p(q, Ks[j], l2[0], None) * (do @ Vs[j].T - dl[0][:, None]) * SCALE) @ Ks[j] for j in range(n))
    assert np.allclose(model.dq_tile(q, do, Ks, Vs, l2[0], dl[0], SCALE, slow_warp=1), dQ)
    assert not np.allclose(model.dq_tile(q, do, Ks, Vs, l2[0], dl[0], SCALE, slow_warp=1, ds_full_buffers=1), dQ)


@pytest.mark.parametrize("qp,causal", [(0, True), (1, True), (3, True), (0, False), (2, False)])
def test_forward_pair_schedule_terminates_and_matches(qp, causal):
    """The two-tile forward kernel: both tiles alternate on the tensor pipe, the causal tiles see
    different numbers of blocks (2 qp + 1 and 2 qp + 2), scores that grow from block to block force
    the lazy rescale of the output accumulator."""
    rng = np.random.default_rng(50 + qp)
    nkv = 2 * qp + 2 if causal else 5
    n = (2 * qp + 1, 2 * qp + 2) if causal else (nkv, nkv)
    diag = (2 * qp, 2 * qp + 1) if causal else (None, None)
    Q = _tiles(rng, 2)
    K = [rng.standard_normal((BT, D)) * (1 + 4 * j) for j in range(nkv)]        # later blocks score higher
    V = _tiles(rng, nkv)
    want_o, want_l = np.zeros((2, BT, D)), np.zeros((2, BT))
    for t in range(2):
        s = np.concatenate([Q[t] @ K[j].T for j in range(n[t])], axis=1) * SCALE
        if causal:
            cols = np.arange(n[t] * BT)[None, :]
            s = np.where(cols > (diag[t] * BT + np.arange(BT))[:, None], -np.inf, s)
        m = s.max(axis=1, keepdims=True)
        e = np.exp(s - m)
        want_o[t] = (e / e.sum(axis=1, keepdims=True)) @ np.concatenate(V[:n[t]], axis=0)
        want_l[t] = (m + np.log(e.sum(axis=1, keepdims=True)))[:, 0]
    for seed in range(3):
        o, lse = model.fwd_pair(Q, K, V, n, SCALE, diag=diag, seed=seed, grow_threshold=2.0)
        assert np.allclose(o, want_o, rtol=1e-9, atol=1e-9), (qp, causal, seed)
        assert np.allclose(lse, want_l, rtol=1e-9, atol=1e-9)
    # one softmax warp of tile 1 lagging: S of the next block is only issued after all four warps of a tile
    # have written their probabilities, so nobody can run ahead of it
    o, lse = model.fwd_pair(Q, K, V, n, SCALE, diag=diag, grow_threshold=2.0, slow_warp=(1, 2))
    assert np.allclose(o, want_o, rtol=1e-9, atol=1e-9) and np.allclose(lse, want_l, rtol=1e-9, atol=1e-9)

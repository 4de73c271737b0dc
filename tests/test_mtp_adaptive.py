"""Adaptive speculation depth (engine/mtp_adaptive.h): the tracker's state machine on synthetic
acceptance streams (CPU), and the adaptive loop on the device, where random-init weights accept
almost nothing: it must give up speculating and still emit exactly the plain-greedy tokens."""
from __future__ import annotations

import random

import pytest
import torch


def feed(tr, k, p1, p2, rounds, rng):
    """Rounds at depth k with per-candidate acceptance p1 (first) and p2 (second given first)."""
    changes = []
    for _ in range(rounds):
        if tr.k == 0:
            break
        kk = tr.k
        n = 1
        if kk >= 1 and rng.random() < p1:
            n = 2
            if kk >= 2 and rng.random() < p2:
                n = 3
        c = tr.note(kk, float(n))
        if c.fired:
            changes.append((c.from_k, c.to_k, c.seen))
    return changes


def test_no_acceptance_demotes_then_abandons(pkg):
    A = pkg.mtp_adaptive
    tr = A.DepthTracker(2)
    ch = feed(tr, 2, 0.0, 0.0, 200, random.Random(1))
    # 16 observed rounds at depth 2 (est 1 / 1.95 = 0.51 < 0.95), then 24 at depth 1 (1 / 1.81 = 0.55 < 0.90)
    assert ch == [(2, 1, A.MIN_OBSERVE_ROUNDS), (1, 0, A.MIN_OBSERVE_BEFORE_ABANDON)]
    assert tr.abandoned and tr.changes == 2 and tr.rounds == [0, 24, 16]
    assert tr.note(0, 1.0).fired is False                      # a plain step is counted, nothing else happens
    assert tr.rounds[0] == 1 and tr.k == 0


def test_good_acceptance_stays_at_depth_two(pkg):
    A = pkg.mtp_adaptive
    tr = A.DepthTracker(2, cost_k1=1.58, cost_k2=1.90)          # the reference's own cost constants
    # the reference's templated row: p1 = 0.729, p2 = 0.726 (0.529 joint): 2.26 tokens per 1.90 steps = 1.19,
    # three window-sigmas above the demotion line
    assert feed(tr, 2, 0.729, 0.726, 300, random.Random(2)) == []
    assert tr.k == 2 and A.DEMOTE_EST <= tr.est() < 1.45 and tr.seen == A.WINDOW_ROUNDS


def test_window_is_a_ratio_of_tallies_and_clears_on_change(pkg):
    A = pkg.mtp_adaptive
    tr = A.DepthTracker(2, cost_k1=1.58, cost_k2=1.90)          # the reference's own cost constants
    for _ in range(15):
        assert not tr.note(2, 3.0).fired                        # below min_observe: no decision yet
    assert abs(tr.est() - 45.0 / (15 * 1.90)) < 1e-12
    for _ in range(100):                                        # acceptance collapses: the window forgets the good start
        c = tr.note(2, 1.0)
        if c.fired:
            break
    assert c.fired and (c.from_k, c.to_k) == (2, 1) and c.est < A.DEMOTE_EST and c.seen == A.WINDOW_ROUNDS
    assert tr.seen == 0 and tr.est() == 0.0
    assert "k_start=2" in tr.config_line() and "cost_k1=1.58 cost_k2=1.90 re_promote=0" in tr.config_line()
    assert tr.describe(0).startswith("rounds_k2=") and "final_k=1" in tr.describe(0)


def test_depth_one_start_and_marginal_acceptance(pkg):
    A = pkg.mtp_adaptive
    tr = A.DepthTracker(1, cost_k1=1.58, cost_k2=1.90)
    # p1 = 0.75: 1.75 tokens per 1.58 steps = 1.11, four window-sigmas above the line: keeps speculating
    assert feed(tr, 1, 0.75, 0.0, 300, random.Random(3)) == [] and tr.k == 1
    tr2 = A.DepthTracker(1, cost_k1=1.58, cost_k2=1.90)
    # p1 = 0.03 (the reference's bad row): 1.03 / 1.58 = 0.65 < 0.90: abandons after 24 rounds
    assert feed(tr2, 1, 0.03, 0.0, 500, random.Random(4)) == [(1, 0, 24)]
    with pytest.raises(ValueError):
        A.DepthTracker(3)


@pytest.mark.gpu
@pytest.mark.parametrize("graphs", [False, True])
def test_adaptive_loop_gives_up_and_stays_lossless(pkg, weights, golden, graphs):
    pkg.build_lib.build()
    eng = pkg.Engine(weights, max_rows=256)
    lanes, budget = 3, 56
    base = torch.from_numpy(golden["mtp"]["prompt"]).int()
    gen = torch.Generator().manual_seed(23)
    ids = torch.stack([base] + [torch.randint(0, 248320, (16,), generator=gen).int() for _ in range(lanes - 1)]).cuda()
    # plain greedy (state with MTP buffers attached, so both runs use the same kernels)
    sp = eng.allocate_state(lanes, 256)
    mp = eng.mtp_allocate(sp, 8, depth=2)
    cur, _ = eng.prefill(sp, ids)
    plain = [cur.clone()]
    for _ in range(budget + 4):
        cur = eng.decode_step(sp, cur)
        plain.append(cur.clone())
    plain = torch.stack(plain).cpu()

    # capacities that only suffice if the host's bounds follow the true positions: 16 depth-2 and 24
    # depth-1 rounds would move the position bound by 96 and the draft-cache bound by 56
    ss = eng.allocate_state(lanes, 16 + budget + 24)
    m = eng.mtp_allocate(ss, 40, depth=2)
    t, h = eng.prefill(ss, ids, want_normed=True)
    out, tr, plain_steps = pkg.mtp_adaptive.speculate(eng, ss, m, t, h, budget, start_k=2, readback_every=8, graphs=graphs)
    for i in range(lanes):
        assert len(out[i]) >= budget + 1
        n = min(len(out[i]), plain.shape[0])
        assert out[i][:n] == plain[:n, i].tolist(), f"lane {i}"
    # random-init draft and target do not agree: 16 rounds at depth 2, 24 at depth 1, then plain steps
    assert tr.abandoned and tr.changes == 2 and plain_steps > 0
    assert tr.rounds[2] >= 16 and tr.rounds[1] >= 24
    assert eng.status() == 0
    for x in (m, mp, ss, sp):
        x.close()
    eng.close()

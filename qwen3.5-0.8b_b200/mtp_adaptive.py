"""Adaptive speculation depth: from what the rounds have accepted so far, run the next round at
depth 2, at depth 1, or stop speculating.

Mirrors the policy of the reference (engine/mtp_adaptive.h:1-47 for the rule, :80-87 for the
constants, `Tracker::note` for the state machine):

* the estimate is tokens emitted per step-equivalent over the last `window` rounds - a ratio of two
  tallies, where a round is billed the cost of ITS OWN depth in units of one plain decode step;
* at depth 2, once `min_observe` rounds are in the window, an estimate below `demote_est` demotes to
  depth 1; at depth 1, once `min_observe_abandon` rounds are in, an estimate below `abandon_est`
  abandons speculation for good (a plain step costs exactly one step, so below ~1 token per
  step-equivalent speculation is a tax); a change clears the window; nothing is ever re-promoted;
* the policy only changes GEOMETRY: every emitted token is still the target's own argmax or a
  candidate proved equal to it, so the output is the plain-greedy output at any depth.

The reference bills a round 1.58 (depth 1) / 1.90 (depth 2) plain steps, midpoints of bands it
measured on its own hardware (engine/mtp_adaptive.h:58-76).  Measured here on B200 at 16 lanes
(bench.py, configs[4]): 2.06 ms and 2.22 ms per round against a 1.14 ms plain step = 1.81 and 1.95,
which are this module's defaults; billing a round dearer than it is only demotes a little early
(later kernel work brought the rounds to 1.57 / 1.93 ms as replayed graphs, `engine.MtpRoundGraph`,
and the plain step to 1.11 ms; the call-by-call rounds this loop issues sit in between).

The reference feeds its tracker from the verdict words it reads back every round.  Rounds here are
chained on the device with no host round trip, so `speculate()` reads the emitted counts back once
per `readback_every` rounds and feeds the tracker those rounds one by one; a lane batch shares one
body shape, so a round's `emitted` is the mean over the lanes.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

ROUND_COST_STEPS_K1 = 1.81
ROUND_COST_STEPS_K2 = 1.95
WINDOW_ROUNDS = 32
MIN_OBSERVE_ROUNDS = 16
MIN_OBSERVE_BEFORE_ABANDON = 24
DEMOTE_EST = 0.95
ABANDON_EST = 0.90
PLAIN = 0


@dataclass
class Change:
    fired: bool = False
    from_k: int = 0
    to_k: int = 0
    est: float = 0.0
    seen: int = 0            # rounds in the window when the decision was taken


class DepthTracker:
    """Depth state machine 2 -> 1 -> plain (engine/mtp_adaptive.h `Tracker`)."""

    def __init__(self, start_k: int, cost_k1: float = ROUND_COST_STEPS_K1, cost_k2: float = ROUND_COST_STEPS_K2,
                 window: int = WINDOW_ROUNDS, min_observe: int = MIN_OBSERVE_ROUNDS,
                 min_observe_abandon: int = MIN_OBSERVE_BEFORE_ABANDON,
                 demote_est: float = DEMOTE_EST, abandon_est: float = ABANDON_EST):
        if start_k not in (0, 1, 2):
            raise ValueError("start depth must be 0, 1 or 2")
        self.k = start_k
        self.ceiling = start_k
        self.cost = {1: cost_k1, 2: cost_k2}
        self.window, self.min_observe, self.min_observe_abandon = window, min_observe, min_observe_abandon
        self.demote_est, self.abandon_est = demote_est, abandon_est
        self._emit = [0.0] * window
        self._cost = [0.0] * window
        self._head = 0
        self.seen = 0
        self.changes = 0
        self.rounds = [0, 0, 0]              # rounds fed to note(), by the depth they ran at
        self._all_emitted = 0.0
        self._all_cost = 0.0

    def round_cost_steps(self, k: int) -> float:
        return self.cost[2] if k >= 2 else self.cost[1]

    @property
    def abandoned(self) -> bool:
        return self.k == PLAIN

    def est(self) -> float:
        e, c = sum(self._emit[:self.seen]), sum(self._cost[:self.seen])
        return e / c if c > 0.0 else 0.0

    def note(self, k_round: int, emitted: float) -> Change:
        """Account one finished round that ran at depth `k_round` and emitted `emitted` tokens
        (per lane); returns the depth change it triggered, if any."""
        self.rounds[k_round if 0 <= k_round <= 2 else 0] += 1
        if self.k == PLAIN:
            return Change()
        cost = self.round_cost_steps(k_round)
        self._emit[self._head], self._cost[self._head] = emitted, cost
        self._head = (self._head + 1) % self.window
        self.seen = min(self.seen + 1, self.window)
        self._all_emitted += emitted
        self._all_cost += cost
        need = self.min_observe if self.k >= 2 else self.min_observe_abandon
        if self.seen < need:
            return Change()
        e = self.est()
        to = self.k
        if self.k >= 2 and e < self.demote_est:
            to = self.k - 1
        elif self.k == 1 and e < self.abandon_est:
            to = PLAIN
        if to == self.k:
            return Change()
        c = Change(True, self.k, to, e, self.seen)
        self.k = to
        self.changes += 1
        self._head = 0
        self.seen = 0
        return c

    def config_line(self) -> str:
        return (f"on=1 k_start={self.ceiling} floor=1 ceiling={self.ceiling} plain={PLAIN} window={self.window} "
                f"min_observe={self.min_observe} min_observe_abandon={self.min_observe_abandon} "
                f"demote_est={self.demote_est:.3f} abandon_est={self.abandon_est:.3f} "
                f"cost_k1={self.cost[1]:.2f} cost_k2={self.cost[2]:.2f} re_promote=0")

    def describe(self, plain_steps: int) -> str:
        e, c = sum(self._emit[:self.seen]), sum(self._cost[:self.seen])
        est_all = self._all_emitted / self._all_cost if self._all_cost > 0 else 0.0
        return (f"rounds_k2={self.rounds[2]} rounds_k1={self.rounds[1]} plain={plain_steps} changes={self.changes} "
                f"final_k={self.k} ceiling={self.ceiling} window_rounds={self.seen} window_emitted={e:.3f} "
                f"window_cost_steps={c:.3f} est={self.est():.3f} est_all={est_all:.3f}")


def speculate(engine, state, mtp, first_token, h_norm, budget: int, start_k: int = 2, readback_every: int = 8,
              tracker: DepthTracker | None = None, graphs: bool = False):
    """Greedy generation of at least `budget` tokens per lane after a prefill, with adaptive depth.

    `first_token` [lanes] and `h_norm` [lanes, 1024] are what `engine.prefill(..., want_normed=True)`
    returned.  Returns (tokens: list of per-lane lists, tracker, plain_steps).  Rounds are chained
    on the device; the emitted counts are read back every `readback_every` rounds.  The draft cache
    of `mtp` must hold one row per drafted token (depth x rounds), the state's context the prompt
    plus (depth + 1) x rounds.  With `graphs=True` the rounds between two readbacks are replays of one captured
    CUDA graph per depth (`engine.MtpRoundGraph` with a verdict ring of `readback_every` slots): same tokens,
    same decisions, nothing launched between the rounds.
    """
    if graphs:
        return _speculate_graphs(engine, state, mtp, first_token, h_norm, budget, start_k, readback_every, tracker)
    lanes = state.lanes
    tr = tracker or DepthTracker(start_k)
    out = [[int(x)] for x in first_token.tolist()]
    t, h = first_token, h_norm
    plain_steps = 0
    pending = []                                   # (k, emit, n_emit) of rounds not yet read back

    def flush():
        for k_round, emit, n_emit in pending:
            em, ne = emit.cpu(), n_emit.cpu()
            for i in range(lanes):
                out[i].extend(em[i, :int(ne[i])].tolist())
            tr.note(k_round, float(ne.float().mean()))
        if pending:
            # the copies above synchronised the stream anyway: let the host's capacity bounds follow the
            # positions the lanes really reached instead of growing by the maximum every round
            state.sync_bound()
            mtp.sync_bound()
        pending.clear()

    while min(len(o) for o in out) + len(pending) < budget + 1:
        k = tr.k
        if k == PLAIN:
            flush()
            if min(len(o) for o in out) >= budget + 1:
                break
            # every lane sits at its own position; a plain step consumes one token per lane
            t = engine.decode_step(state, t)
            for i, x in enumerate(t.tolist()):
                out[i].append(int(x))
            plain_steps += 1
            continue
        pos = (state.positions + 1).int()
        if k == 1:
            d = engine.mtp_draft(mtp, h, t, pos).reshape(lanes, 1).contiguous()
        else:
            d = engine.mtp_draft_k(mtp, h, t, pos, k)
        emit, n_emit, h = engine.mtp_verify_k(state, mtp, t, d)
        t = emit.gather(1, (n_emit - 1).long()[:, None])[:, 0].int().contiguous()
        pending.append((k, emit, n_emit))
        if len(pending) >= readback_every:
            flush()
    flush()
    return out, tr, plain_steps


def _speculate_graphs(engine, state, mtp, first_token, h_norm, budget, start_k, readback_every, tracker):
    from .engine import MtpRoundGraph

    lanes = state.lanes
    tr = tracker or DepthTracker(start_k)
    out = [[int(x)] for x in first_token.tolist()]
    t, h = first_token.clone(), h_norm.clone()
    plain_steps = 0
    by_depth = {}                                  # depth -> captured round
    cur = None                                     # the graph whose buffers hold the live token and row
    pending = 0

    def flush():
        nonlocal pending, t, h
        if cur is None or pending == 0:
            return
        em, ne = cur.last_rounds(pending)          # synchronises
        for r in range(pending):
            for i in range(lanes):
                out[i].extend(em[r, i, :int(ne[r, i])].tolist())
            tr.note(cur.depth, float(ne[r].float().mean()))
        state.sync_bound()
        mtp.sync_bound()
        t, h = cur.tok.clone(), cur.h.clone()
        pending = 0

    while min(len(o) for o in out) + pending < budget + 1:
        k = tr.k
        if k == PLAIN:
            flush()
            if min(len(o) for o in out) >= budget + 1:
                break
            t = engine.decode_step(state, t)
            for i, x in enumerate(t.tolist()):
                out[i].append(int(x))
            plain_steps += 1
            continue
        g = by_depth.get(k)
        if g is not cur or g is None:
            flush()                                # the depth only changes at a readback, so nothing is pending here
            if g is None:
                g = by_depth[k] = MtpRoundGraph(engine, state, mtp, depth=k, history=readback_every)
            g.tok.copy_(t)
            g.h.copy_(h)
            cur = g
        cur.replay()
        pending += 1
        if pending >= readback_every:
            flush()
    flush()
    return out, tr, plain_steps

"""The resident session protocol (feed / gen / reset / stats / quit), its stop rule, its
pending-token rule and its poisoning, as the reference's driver defines them
(engine/decode_run.cpp:1760-1795, 2436-2560; engine/decode_step.h:487-492).

CPU tests drive the protocol over a test double of the engine (a toy next-token rule with the
engine's call signatures); GPU tests run it on the real engine and check the transcript against
direct engine calls and across suspend / resume."""
from __future__ import annotations

import pytest
import torch


class ToyState:
    def __init__(self, cap):
        self.cap, self.hist = cap, []

    def reset(self):
        self.hist = []

    def close(self):
        pass


class ToyEngine:
    """next token = (7 * last + len(history)) % vocab; capacity errors like the engine's."""
    device = "cpu"
    vocab = 1000

    def __init__(self, pkg):
        self.pkg = pkg

    def allocate_state(self, lanes, cap):
        assert lanes == 1
        return ToyState(cap)

    def _next(self, st):
        return (7 * st.hist[-1] + len(st.hist)) % self.vocab

    def prefill(self, st, ids):
        toks = ids[0].tolist()
        if len(st.hist) + len(toks) > st.cap:
            raise self.pkg.Q35Error(3, "prompt beyond max_ctx")
        st.hist += toks
        return torch.tensor([self._next(st)], dtype=torch.int32), None

    def decode_step(self, st, tok):
        if len(st.hist) + 1 > st.cap:
            raise self.pkg.Q35Error(3, "position beyond max_ctx")
        st.hist.append(int(tok[0]))
        return torch.tensor([self._next(st)], dtype=torch.int32)


def run(sess, script):
    out = []
    sess.loop(script, out.append)
    return out


def test_protocol_transcript(pkg):
    eng = ToyEngine(pkg)
    s = pkg.session.Session(eng, cap=64, stop_token=999)
    out = run(s, ["", "gen 3", "feed 5 6 7", "stats", "gen 3", "gen 2", "feed 9", "gen 1", "reset", "stats", "quit", "feed 1"])
    assert out[0] == "READY cap=64"
    assert out[1] == "ERROR gen with no sampled token: feed this turn's prompt first"
    assert out[2] == "FED n=3 prefix_len=3"
    s0 = (7 * 7 + 3) % 1000
    assert out[3] == f"PREFIX p=3 sampled={s0} stopped=0"
    s1 = (7 * s0 + 4) % 1000
    s2 = (7 * s1 + 5) % 1000
    assert out[4:8] == [f"GEN {s0} 2", f"GEN {s1} 3", f"GEN {s2} 4", "END steps=3 stop=0 prefix_len=6"]
    # the budget was spent: the last token handed out was consumed, nothing is pending
    assert out[8] == "ERROR gen with no sampled token: feed this turn's prompt first"
    assert out[9] == "FED n=1 prefix_len=7"                      # only the caller's token
    t0 = (7 * 9 + 7) % 1000
    assert out[10:12] == [f"GEN {t0} 6", "END steps=1 stop=0 prefix_len=8"]
    assert out[12:] == ["RESET prefix_len=0", "PREFIX p=0 sampled=-1 stopped=0", "BYE"]


def test_stop_token_ends_the_turn_and_is_fed_first(pkg):
    eng = ToyEngine(pkg)
    first = (7 * 3 + 1) % 1000                                   # sampled after feeding [3]
    second = (7 * first + 2) % 1000
    s = pkg.session.Session(eng, cap=64, stop_token=second)
    out = run(s, ["feed 3", "gen 10", "stats", "feed 4", "quit"])
    assert out[1] == "FED n=1 prefix_len=1"
    assert out[2:5] == [f"GEN {first} 0", f"GEN {second} 1", "END steps=2 stop=1 prefix_len=2"]
    assert out[5] == f"PREFIX p=2 sampled={second} stopped=1"
    # the stop token was handed out but never consumed: the next feed consumes it before the caller's
    assert out[6] == "FED n=2 prefix_len=4"
    assert s.state.hist == [3, first, second, 4]


def test_errors_poison_until_reset(pkg):
    eng = ToyEngine(pkg)
    s = pkg.session.Session(eng, cap=4, stop_token=999)
    out = run(s, ["feed 1 2 3", "gen 5", "gen 1", "feed 1", "stats", "reset", "feed 1", "gen x", "feed 5000", "feed 1", "bye"])
    assert out[1] == "FED n=3 prefix_len=3"
    assert out[2].startswith("GEN ") and out[3].startswith("GEN ")      # positions 2 and 3; the step after overflows
    assert out[4].startswith("ERROR") and "max_ctx" in out[4]
    assert out[5] == out[6] == out[7] == "ERROR session is poisoned by the failed step: send reset before the next feed or gen"
    assert out[8] == "RESET prefix_len=0"
    assert out[9] == "FED n=1 prefix_len=1"
    assert out[10] == "ERROR gen needs a token count"
    assert out[11].startswith("ERROR") and "out of range" in out[11]
    assert out[12].startswith("ERROR session is poisoned")
    assert out[13] == "BYE"


@pytest.mark.gpu
def test_session_matches_direct_engine_calls_and_survives_suspend_resume(pkg, weights):
    pkg.build_lib.build()
    eng = pkg.Engine(weights, max_rows=64)
    g = torch.Generator().manual_seed(8)
    A = torch.randint(0, 248320, (12,), generator=g).tolist()
    B = torch.randint(0, 248320, (5,), generator=g).tolist()
    s = pkg.session.Session(eng, cap=64)
    out = run(s, ["feed " + " ".join(map(str, A)), "gen 5", "feed " + " ".join(map(str, B)), "gen 3"])
    gen = [tuple(map(int, l.split()[1:])) for l in out if l.startswith("GEN")]
    assert [p for _, p in gen] == [11, 12, 13, 14, 15, 21, 22, 23]
    assert out[-1] == "END steps=3 stop=0 prefix_len=25"

    # the same transcript through the engine's own calls
    st = eng.allocate_state(1, 64)
    cur, _ = eng.prefill(st, torch.tensor([A], dtype=torch.int32).cuda())
    direct = []
    for _ in range(5):
        direct.append(int(cur))
        cur = eng.decode_step(st, cur)
    cur, _ = eng.prefill(st, torch.tensor([B], dtype=torch.int32).cuda())
    for _ in range(3):
        direct.append(int(cur))
        cur = eng.decode_step(st, cur)
    assert [t for t, _ in gen] == direct
    a, b = s.state.export_lane(0, 64), st.export_lane(0, 64)
    assert a["prefix_len"] == b["prefix_len"] == 25
    assert torch.equal(a["gdn_state"], b["gdn_state"]) and torch.equal(a["kv_keys"], b["kv_keys"])

    # pre-empt after the feed, resume in a second session: the continuation is identical
    s1 = pkg.session.Session(eng, cap=64)
    run(s1, ["feed " + " ".join(map(str, A)), "gen 2"])
    blob = s1.suspend()
    s2 = pkg.session.Session(eng, cap=64)
    s2.resume(blob)
    assert s2.prefix_len == 14 and s2.stats() == s1.stats()
    o1 = run(s1, ["feed 77 78", "gen 4"])
    o2 = run(s2, ["feed 77 78", "gen 4"])
    assert o1 == o2 and o1[-1] == "END steps=4 stop=0 prefix_len=20"
    for x in (s, s1, s2):
        x.close()
    st.close()
    eng.close()

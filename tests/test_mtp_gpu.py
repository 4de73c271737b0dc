"""MTP draft / verify rounds through the C-ABI.

On random-init weights the draft almost never agrees with the target (accept rate ~ 0), so, as in
the reference's own G8a gate (speccheck/gates/run_mtp.py:121-148), the binding checks are:
the speculative loop emits exactly the tokens of plain greedy decoding, the state after the
rounds is bit-identical to a sequential replay, and both the accept and the reject branch leave
positions, draft-cache length and GDN state where a sequential run has them.  The accept branch
is exercised by handing the verifier the true next token as the candidate.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import q35_oracle as O

from conftest import rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def eng(pkg, weights):
    pkg.build_lib.build()
    e = pkg.Engine(weights, max_rows=256)
    yield e
    e.close()


def bf(a):
    return torch.from_numpy(np.asarray(a)).to(torch.bfloat16)


_W = {}


def eng_fc_weight(eng):
    return _W.get("mtp.fc.weight")


def eng_norm(eng, name):
    return _W["mtp." + name + ".weight"]


@pytest.fixture(scope="module", autouse=True)
def _mtp_weights(weights):
    for k, v in weights.items():
        if k.startswith("mtp."):
            _W[k] = v
    yield
    _W.clear()


def prompts(golden, lanes):
    base = torch.from_numpy(golden["mtp"]["prompt"]).int()
    gen = torch.Generator().manual_seed(17)
    rows = [base] + [torch.randint(0, 248320, (16,), generator=gen).int() for _ in range(lanes - 1)]
    return torch.stack(rows).cuda()


def test_draft_matches_reference(eng, golden):
    """One draft call on the reference's own (h, y_next, pos): same proposal id, and the block's taps
    (speccheck/mtp.py:57-83) within the stage tolerance: u = fc([N(E[y]) | N(h)]) - a swapped operand
    order shows here at once -, the final-norm row x_d, and the sub-sampled logits."""
    g = golden["mtp"]
    st = eng.allocate_state(1, 64)
    m = eng.mtp_allocate(st, 64)
    h, y = bf(g["draft_h"]).cuda(), torch.tensor(g["draft_y"], dtype=torch.int32).cuda()
    pos = torch.tensor(g["draft_pos"], dtype=torch.int32).cuda()
    prop, u, xd, lg = eng.mtp_draft_taps(m, h, y, pos, want_logits=True)
    assert int(prop[0]) == int(g["draft_id"][0])
    e_u = rel_l2(u.float().cpu(), g["draft_u"])
    e_x = rel_l2(xd.float().cpu(), g["draft_xd"])
    e_l = rel_l2(lg.cpu()[:, ::97], g["draft_logits_sub"])
    assert e_u <= 1e-2 and e_x <= 1e-2 and e_l <= 1e-2, (e_u, e_x, e_l)
    # the wrong operand order [N(h) | N(E[y])] is far outside that band: the check bites
    swapped_u = None
    fc = eng_fc_weight(eng)
    if fc is not None:
        ne = O.norm_zc(eng.embed[int(y[0])].cpu()[None], eng_norm(eng, "pre_fc_norm_embedding"))
        nh = O.norm_zc(h.cpu(), eng_norm(eng, "pre_fc_norm_hidden"))
        swapped_u = (torch.cat([nh, ne], -1) @ fc.t()).float()
        assert rel_l2(swapped_u, g["draft_u"]) > 0.5
    m.close()
    st.close()


def test_verify_without_draft_is_refused(eng, pkg, golden):
    """A rejecting round drops k rows from the draft cache, so a verify that no draft preceded is
    refused on the host (status 4) instead of driving the cache length negative."""
    ids = prompts(golden, 2)
    st = eng.allocate_state(2, 64)
    m = eng.mtp_allocate(st, 64)
    t, h = eng.prefill(st, ids, want_normed=True)
    with pytest.raises(pkg.Q35Error) as ei:
        eng.mtp_verify(st, m, t, t)
    assert ei.value.code == 4
    d = eng.mtp_draft(m, h, t, (st.positions + 1).int())
    eng.mtp_verify(st, m, t, d)                       # one draft: one verify is fine
    with pytest.raises(pkg.Q35Error):
        eng.mtp_verify(st, m, t, d)                   # ... a second one is not
    m.reset()
    with pytest.raises(pkg.Q35Error):
        eng.mtp_verify(st, m, t, d)
    assert eng.status() == 0
    m.close()
    st.close()


def test_rounds_equal_plain_greedy_and_sequential_state(eng, golden):
    lanes, rounds = 3, 8
    ids = prompts(golden, lanes)
    # plain greedy
    sp = eng.allocate_state(lanes, 64)
    mp = eng.mtp_allocate(sp, 64)          # a speculative session: decode and verify share kernels
    y0, _ = eng.prefill(sp, ids)
    plain = [y0.clone()]
    cur = y0
    for _ in range(rounds):
        cur = eng.decode_step(sp, cur)
        plain.append(cur.clone())
    plain = torch.stack(plain).cpu()                       # [rounds+1, lanes]

    # speculative loop, everything chained on the device
    ss = eng.allocate_state(lanes, 64)
    m = eng.mtp_allocate(ss, 64)
    t, h = eng.prefill(ss, ids, want_normed=True)
    emitted = [[int(x)] for x in t.tolist()]
    accepted = 0
    for _ in range(rounds):
        pos = (ss.positions + 1).int()
        d = eng.mtp_draft(m, h, t, pos)
        emit, n_emit, h = eng.mtp_verify(ss, m, t, d)
        em, ne = emit.cpu(), n_emit.cpu()
        for i in range(lanes):
            emitted[i].extend(em[i, :int(ne[i])].tolist())
            accepted += int(ne[i]) - 1
        t = torch.where(n_emit == 2, emit[:, 1], emit[:, 0]).int().contiguous()
    for i in range(lanes):
        n = min(len(emitted[i]), rounds + 1)
        assert emitted[i][:n] == plain[:n, i].tolist(), f"lane {i}"
    # lanes that never accepted consumed exactly `rounds` tokens: state equals the plain run bit for bit
    for i in range(lanes):
        if len(emitted[i]) == rounds + 1:
            a, b = ss.export_lane(i, 64), sp.export_lane(i, 64)
            assert a["prefix_len"] == b["prefix_len"] == 16 + rounds
            assert torch.equal(a["gdn_state"], b["gdn_state"])
            assert torch.equal(a["conv_window"], b["conv_window"])
            assert torch.equal(a["kv_keys"][:, :, :16 + rounds], b["kv_keys"][:, :, :16 + rounds])
    # reference tokens (speculative 'steps' loop of the reference == its plain greedy)
    ref = golden["mtp"]["tokens_steps"].tolist()
    common = 0
    for x, y in zip(emitted[0], ref):
        if x != y:
            break
        common += 1
    assert common >= 1
    m.close(); mp.close(); ss.close(); sp.close()


def test_accept_and_reject_branches(eng, golden):
    lanes = 2
    ids = prompts(golden, lanes)
    sp = eng.allocate_state(lanes, 64)
    mp = eng.mtp_allocate(sp, 64)          # keeps the plain run on the kernels the verify body uses
    y0, _ = eng.prefill(sp, ids)
    seq = [y0.clone()]
    for _ in range(4):
        seq.append(eng.decode_step(sp, seq[-1]).clone())
    # sp has consumed y0..seq[3]; position 16 + 4
    ss = eng.allocate_state(lanes, 64)
    m = eng.mtp_allocate(ss, 64)
    t, h = eng.prefill(ss, ids, want_normed=True)
    assert torch.equal(t, y0)
    # round 1: candidate = the true next token -> accept in every lane
    d = eng.mtp_draft(m, h, t, (ss.positions + 1).int())
    emit, n_emit, h = eng.mtp_verify(ss, m, t, seq[1])
    assert n_emit.tolist() == [2, 2]
    assert torch.equal(emit[:, 0], seq[1]) and torch.equal(emit[:, 1], seq[2])
    assert ss.positions.tolist() == [18, 18]
    # round 2: lane 0 gets a wrong candidate (reject), lane 1 the true one (accept)
    t = emit[:, 1].contiguous()
    wrong = ((seq[3] + 1) % 248320).int()
    cand = torch.stack([wrong[0], seq[3][1]]).int().contiguous()
    d = eng.mtp_draft(m, h, t, (ss.positions + 1).int())
    emit, n_emit, h = eng.mtp_verify(ss, m, t, cand)
    assert n_emit.tolist() == [1, 2]
    assert int(emit[0, 0]) == int(seq[3][0]) and int(emit[0, 1]) == -1
    assert int(emit[1, 0]) == int(seq[3][1]) and int(emit[1, 1]) == int(seq[4][1])
    assert ss.positions.tolist() == [19, 20]
    # lane 1 consumed y0..seq[3] like the plain run: identical state; lane 0 is one token behind
    a, b = ss.export_lane(1, 64), sp.export_lane(1, 64)
    assert torch.equal(a["gdn_state"], b["gdn_state"]) and torch.equal(a["conv_window"], b["conv_window"])
    # lane 0: feed seq[3] through a plain step and it must land on the plain run's state too
    nxt = eng.decode_step(ss, torch.stack([seq[3][0], seq[4][1]]).int().contiguous())
    a0, b0 = ss.export_lane(0, 64), sp.export_lane(0, 64)
    assert a0["prefix_len"] == b0["prefix_len"] == 20
    assert torch.equal(a0["gdn_state"], b0["gdn_state"]) and torch.equal(a0["conv_window"], b0["conv_window"])
    assert int(nxt[0]) == int(seq[4][0])
    m.close(); mp.close(); ss.close(); sp.close()


def test_verify_needs_mtp_state(eng, pkg, golden):
    st = eng.allocate_state(1, 32)
    other = eng.allocate_state(1, 32)
    m = eng.mtp_allocate(other, 32)
    z = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(pkg.Q35Error) as ei:
        eng.mtp_verify(st, m, z, z)
    assert ei.value.code == 4
    m.close(); st.close(); other.close()


# ------------------------------------------------------------------------------------ depth 2
def test_chained_drafts_match_the_oracle(eng, weights, golden):
    """Two chained drafts on the reference's own (h, y_next, pos): the first proposal is the
    fixture's, the second the oracle's wherever its f32 top-2 margin exceeds 1e-2."""
    g = golden["mtp"]
    st = eng.allocate_state(1, 64)
    m = eng.mtp_allocate(st, 64, depth=2)
    h = bf(g["draft_h"])
    y, pos = int(g["draft_y"][0]), int(g["draft_pos"][0])
    props = eng.mtp_draft_k(m, h.cuda(), torch.tensor([y], dtype=torch.int32).cuda(),
                            torch.tensor([pos], dtype=torch.int32).cuda(), 2).cpu()
    om = O.MtpLane(weights, kv_bf16=True)
    d1, x1 = om.draft(y, h, pos)
    dbg = {}
    d2, _ = om.draft(d1, x1, pos + 1, dbg)
    assert int(props[0, 0]) == d1 == int(g["draft_id"][0])
    best, margin = O.top2_margin(dbg["logits"][-1].float())
    if margin > 1e-2:
        assert int(props[0, 1]) == d2 == best
    # a single draft on a fresh cache proposes the same first token
    m1 = eng.mtp_allocate(st, 64)
    p1 = eng.mtp_draft(m1, h.cuda(), torch.tensor([y], dtype=torch.int32).cuda(), torch.tensor([pos], dtype=torch.int32).cuda())
    assert int(p1[0]) == int(props[0, 0])
    m.close(); m1.close(); st.close()


def test_depth2_rounds_equal_plain_greedy(eng, golden):
    lanes, rounds = 3, 6
    ids = prompts(golden, lanes)
    sp = eng.allocate_state(lanes, 64)
    mp = eng.mtp_allocate(sp, 64, depth=2)
    y0, _ = eng.prefill(sp, ids)
    plain = [y0.clone()]
    for _ in range(3 * rounds):
        plain.append(eng.decode_step(sp, plain[-1]).clone())
    plain = torch.stack(plain).cpu()

    ss = eng.allocate_state(lanes, 64)
    m = eng.mtp_allocate(ss, 64, depth=2)
    t, h = eng.prefill(ss, ids, want_normed=True)
    emitted = [[int(x)] for x in t.tolist()]
    for _ in range(rounds):
        d = eng.mtp_draft_k(m, h, t, (ss.positions + 1).int(), 2)
        emit, n_emit, h = eng.mtp_verify_k(ss, m, t, d)
        em, ne = emit.cpu(), n_emit.cpu()
        for i in range(lanes):
            emitted[i].extend(em[i, :int(ne[i])].tolist())
        t = emit.gather(1, (n_emit - 1).long()[:, None])[:, 0].int().contiguous()
    for i in range(lanes):
        assert emitted[i] == plain[:len(emitted[i]), i].tolist(), f"lane {i}"
    assert ss.positions.tolist() == [16 + len(e) - 1 for e in emitted]
    m.close(); mp.close(); ss.close(); sp.close()


def test_depth2_longest_prefix_and_rollback(eng, golden):
    """Forced candidates: lane 0 rejects both (n = 0), lane 1 accepts one (n = 1), lane 2 accepts
    both (n = 2); then a second round with the pattern rotated, so every lane's live buffer index
    moves twice.  After each round a lane's state is bit-identical to the plain run that consumed
    the same tokens."""
    lanes = 3
    ids = prompts(golden, lanes)
    sp = eng.allocate_state(lanes, 64)
    mp = eng.mtp_allocate(sp, 64, depth=2)
    y0, _ = eng.prefill(sp, ids)
    seq, snaps = [y0.clone()], []
    for _ in range(8):
        seq.append(eng.decode_step(sp, seq[-1]).clone())
        snaps.append([sp.export_lane(i, 64) for i in range(lanes)])      # snaps[j]: after consuming seq[0..j]
    S = torch.stack(seq).cpu()                                            # S[j, lane]

    ss = eng.allocate_state(lanes, 64)
    m = eng.mtp_allocate(ss, 64, depth=2)
    t, h = eng.prefill(ss, ids, want_normed=True)
    assert torch.equal(t, y0)
    consumed = [0, 0, 0]                      # tokens of seq consumed per lane
    for accept in ([0, 1, 2], [2, 0, 1]):
        cands = torch.empty((lanes, 2), dtype=torch.int32)
        for i in range(lanes):
            c = consumed[i]
            true1, true2 = int(S[c + 1, i]), int(S[c + 2, i])
            wrong = lambda x: (x + 1) % 248320
            cands[i, 0] = true1 if accept[i] >= 1 else wrong(true1)
            cands[i, 1] = true2 if accept[i] >= 2 else wrong(true2)
        eng.mtp_draft_k(m, h, t, (ss.positions + 1).int(), 2)             # fills the draft cache like a real round
        emit, n_emit, h = eng.mtp_verify_k(ss, m, t, cands.cuda())
        assert n_emit.tolist() == [a + 1 for a in accept]
        for i in range(lanes):
            c, a = consumed[i], accept[i]
            want = [int(S[c + 1 + j, i]) for j in range(a + 1)] + [-1] * (2 - a)
            assert emit[i].tolist() == want, (i, emit[i].tolist(), want)
            consumed[i] = c + a + 1
            got, ref = ss.export_lane(i, 64), snaps[consumed[i] - 1][i]
            assert got["prefix_len"] == ref["prefix_len"] == 16 + consumed[i]
            assert torch.equal(got["gdn_state"], ref["gdn_state"]), f"lane {i} accept {a}"
            assert torch.equal(got["conv_window"], ref["conv_window"])
            n = got["prefix_len"]
            assert torch.equal(got["kv_keys"][:, :, :n], ref["kv_keys"][:, :, :n])
            assert torch.equal(got["kv_values"][:, :, :n], ref["kv_values"][:, :, :n])
        t = emit.gather(1, (n_emit - 1).long()[:, None])[:, 0].int().contiguous()
    # a depth-1 round still works on the three-buffer state, whatever buffer is live
    d1 = eng.mtp_draft(m, h, t, (ss.positions + 1).int())
    emit, n_emit, h = eng.mtp_verify(ss, m, t, torch.stack([S[consumed[i] + 1, i] for i in range(lanes)]).int().cuda())
    assert n_emit.tolist() == [2, 2, 2]
    for i in range(lanes):
        got, ref = ss.export_lane(i, 64), snaps[consumed[i] + 1][i]
        assert torch.equal(got["gdn_state"], ref["gdn_state"])
    m.close(); mp.close(); ss.close(); sp.close()


def test_depth_must_be_reserved(eng, pkg, golden):
    st = eng.allocate_state(1, 32)
    m = eng.mtp_allocate(st, 32)                  # depth 1 only
    z = torch.zeros(1, dtype=torch.int32, device="cuda")
    z2 = torch.zeros((1, 2), dtype=torch.int32, device="cuda")
    with pytest.raises(pkg.Q35Error) as ei:
        eng.mtp_verify_k(st, m, z, z2)
    assert ei.value.code == 4
    with pytest.raises(pkg.Q35Error):
        eng.mtp_draft_k(m, torch.zeros((1, 1024), dtype=torch.bfloat16, device="cuda"), z, z, 2)
    with pytest.raises(pkg.Q35Error):
        eng.mtp_allocate(st, 32, depth=3)
    m.close(); st.close()


@pytest.mark.parametrize("depth", [1, 2])
def test_round_graph_equals_eager_rounds(eng, pkg, golden, depth):
    """A replayed CUDA graph of one round against the same rounds launched one call at a time:
    identical emitted tokens and counts every round, identical positions and layer-0 state after,
    and the host bounds refuse a replay that could overrun the draft cache."""
    lanes, rounds = 3, 6
    ids = prompts(golden, lanes)

    def start(cache_rows):
        st = eng.allocate_state(lanes, 96)
        m = eng.mtp_allocate(st, cache_rows, depth=depth)
        t, h = eng.prefill(st, ids, want_normed=True)
        return st, m, t, h

    # eager
    st, m, t, h = start(64)
    eager = []
    for _ in range(rounds):
        pos = (st.positions + 1).int()
        if depth == 1:
            d = eng.mtp_draft(m, h, t, pos)
            emit, n_emit, h = eng.mtp_verify(st, m, t, d)
        else:
            d = eng.mtp_draft_k(m, h, t, pos, depth)
            emit, n_emit, h = eng.mtp_verify_k(st, m, t, d)
        t = emit.gather(1, (n_emit - 1).long()[:, None])[:, 0].int().contiguous()
        eager.append((emit.cpu(), n_emit.cpu()))
    pos_e = st.positions.cpu()
    S_e = st.export_lane(0, 96)["gdn_state"][0].cpu()
    m.close()
    st.close()

    # graph
    st, m, t, h = start(64)
    g = pkg.MtpRoundGraph(eng, st, m, depth=depth)
    g.tok.copy_(t)
    g.h.copy_(h)
    for r in range(rounds):
        g.replay()
        emit, n_emit = g.emit.cpu(), g.n_emit.cpu()
        assert torch.equal(n_emit, eager[r][1]), r
        for i in range(lanes):
            n = int(n_emit[i])
            assert torch.equal(emit[i, :n], eager[r][0][i, :n]), (r, i)
    assert torch.equal(st.positions.cpu(), pos_e)
    assert torch.equal(st.export_lane(0, 96)["gdn_state"][0].cpu(), S_e)
    assert int(g.emitted_total) == sum(int(n.sum()) for _, n in eager)
    assert eng.status() == 0
    m.close()
    st.close()

    # a cache of 2 * depth rows holds two rounds by the host's worst-case bound: the third replay is refused
    st, m, t, h = start(2 * depth)
    g = pkg.MtpRoundGraph(eng, st, m, depth=depth)
    g.tok.copy_(t)
    g.h.copy_(h)
    g.replay()
    g.replay()
    with pytest.raises(pkg.Q35Error):
        g.replay()
    torch.cuda.synchronize()
    m.close()
    st.close()

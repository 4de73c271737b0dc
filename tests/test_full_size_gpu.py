"""The benchmark's full size (4,032 lanes on one GPU) through size-independent properties: the
oracle takes ~0.1 s per lane-step, so 4,032 lanes cannot be replayed on the CPU; instead

* replication: the lanes are copies of a few distinct prompts, so every copy must produce the same
  tokens and the same state bit for bit (a lane's arithmetic must not depend on which row tile, CTA
  or cluster it lands in), and
* anchoring: the distinct prompts, run alone at 5 lanes through the few-row kernels, are compared
  with the oracle by the other test files; here the wide-margin tokens of the 4,032-lane run must
  equal those of the 5-lane run (different kernels: tcgen05 GEMMs vs weight-streaming GEMVs).
"""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu

LANES, DISTINCT, PROMPT, STEPS = 4032, 5, 40, 6


def greedy(eng, ids, steps, want_logits_at=None):
    lanes = ids.shape[0]
    st = eng.allocate_state(lanes, PROMPT + steps + 8)
    cur, _ = eng.prefill(st, ids)
    toks, margins = [cur.clone()], []
    for s in range(steps):
        lg = torch.empty((lanes, eng.vocab), dtype=torch.float32, device="cuda") if want_logits_at else None
        cur = eng.decode_step(st, cur, logits=lg)
        toks.append(cur.clone())
        if lg is not None:
            top = lg.topk(2, dim=1).values
            margins.append((top[:, 0] - top[:, 1]).cpu())
    return st, torch.stack(toks), (torch.stack(margins) if margins else None)


def test_replicated_lanes_agree_at_full_size(pkg, weights):
    pkg.build_lib.build()
    gen = torch.Generator().manual_seed(77)
    base = torch.randint(0, 248320, (DISTINCT, PROMPT), generator=gen, dtype=torch.int32)
    which = torch.arange(LANES) % DISTINCT
    # scatter the copies so that equal prompts sit in different row tiles and different CTAs
    perm = torch.randperm(LANES, generator=gen)
    which = which[perm]
    ids = base[which].cuda()

    big = pkg.Engine(weights, max_rows=LANES * PROMPT)
    st, toks, _ = greedy(big, ids, STEPS)
    assert big.status() == 0
    toks = toks.cpu()
    for d in range(DISTINCT):
        cols = (which == d).nonzero()[:, 0]
        ref = toks[:, cols[0]]
        assert torch.equal(toks[:, cols], ref[:, None].expand(-1, len(cols))), f"prompt {d}: copies disagree"
        # state of the first, a middle and the last copy: bit-identical
        a = st.export_lane(int(cols[0]), PROMPT + STEPS + 8)
        for c in (cols[len(cols) // 2], cols[-1]):
            b = st.export_lane(int(c), PROMPT + STEPS + 8)
            assert a["prefix_len"] == b["prefix_len"] == PROMPT + STEPS
            assert torch.equal(a["gdn_state"], b["gdn_state"])
            assert torch.equal(a["conv_window"], b["conv_window"])
            assert torch.equal(a["kv_keys"], b["kv_keys"]) and torch.equal(a["kv_values"], b["kv_values"])
    st.close()
    big.close()

    # the same prompts alone, through the few-row kernels
    small = pkg.Engine(weights, max_rows=DISTINCT * PROMPT)
    st5, toks5, margins = greedy(small, base.cuda(), STEPS, want_logits_at=True)
    toks5 = toks5.cpu()
    first = torch.stack([(which == d).nonzero()[0, 0] for d in range(DISTINCT)])
    agree = wide = 0
    for d in range(DISTINCT):
        alive = True                          # compare while the two runs are still on the same token path
        for s in range(STEPS + 1):
            if not alive:
                break
            same = int(toks[s, first[d]]) == int(toks5[s, d])
            if s >= 1 and float(margins[s - 1, d]) > 0.25:
                wide += 1
                assert same, f"prompt {d} step {s}: wide-margin token differs between 4032-lane and 5-lane runs"
            agree += same
            alive = same
    assert wide >= 1 and agree >= DISTINCT    # at least the prefill tokens and one wide-margin step were checked
    st5.close()
    small.close()

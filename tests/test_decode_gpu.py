"""Whole-step parity of the engine (through the C-ABI) against the CPU oracle and the
reference-generated config-0 fixture: decode steps from an imported state, the engine's own
prefill, determinism, lane independence, CUDA-graph replay, and the host-side error paths.

End-to-end numbers are cascade numbers: the reference's own legal variants (chunked vs
recurrent prefill, one-pass vs online softmax) differ by 3-7e-2 rel-L2 in the final logits on
these random-init weights, because 1-ULP bf16 differences are amplified through 24 residual
layers.  The 1e-2 / 1e-4 contract is asserted per stage with shared inputs in test_ops_gpu.py;
here the cascade is held under 8e-2 and its measured value is written to parity_decode.json in
the run's output folder.
"""
from __future__ import annotations

import json

import numpy as np
import pytest
import torch

from oracle import q35_oracle as O

from conftest import REPO, rel_l2

pytestmark = pytest.mark.gpu

CASCADE = 8e-2
REPORT = {}


def note(key, val):
    REPORT[key] = val
    out = REPO / "gpurun_out"
    out.mkdir(exist_ok=True)
    (out / "parity_decode.json").write_text(json.dumps(REPORT, indent=1, sort_keys=True))


@pytest.fixture(scope="module")
def eng(pkg, weights):
    pkg.build_lib.build()
    e = pkg.Engine(weights, max_rows=1024)
    yield e
    e.close()


def lane_tuple(lane: O.Lane, cap: int):
    """The oracle lane's state in the reference layouts (engine/state.h:86-92), on the device."""
    S = torch.stack([lane.S[l] for l in O.GDN_LAYERS]).float()
    win = torch.stack([lane.window[l].float() for l in O.GDN_LAYERS])
    k = torch.zeros((6, 2, cap, 256), dtype=torch.bfloat16)
    v = torch.zeros((6, 2, cap, 256), dtype=torch.bfloat16)
    for a, l in enumerate(O.ATTN_LAYERS):
        K = torch.cat(lane.kv[l]["k"], 0)
        V = torch.cat(lane.kv[l]["v"], 0)
        k[a, :, :K.shape[0]] = K.permute(1, 0, 2).to(torch.bfloat16)
        v[a, :, :V.shape[0]] = V.permute(1, 0, 2)
    return S.cuda(), win.cuda(), k.cuda(), v.cuda()


@pytest.fixture(scope="module")
def prefilled(weights, golden):
    """Oracle lanes after the config-0 prompt (lane 0) and a second prompt (lane 1)."""
    g = golden["config0_greedy"]
    a = O.Lane(weights, gdn_prefill="chunk")
    na = a.forward(g["prompt"])
    gen = torch.Generator().manual_seed(99)
    ids_b = torch.randint(0, 248320, (64,), generator=gen)
    b = O.Lane(weights, gdn_prefill="chunk")
    nb = b.forward(ids_b)
    return dict(a=a, b=b, ids_b=ids_b, y0_a=int(a.logits(na)[-1].argmax()), y0_b=int(b.logits(nb)[-1].argmax()))


def test_decode_teacher_forced_from_imported_state(eng, weights, golden, prefilled):
    """Import the oracle's post-prefill state, feed the reference's own tokens for 32 steps."""
    g = golden["config0_greedy"]
    st = eng.allocate_state(2, 128)
    for i, key in enumerate(("a", "b")):
        st.import_lane(i, *lane_tuple(prefilled[key], 128), prefix_len=64)
    back = st.export_lane(0, 128)
    S_or = torch.stack([prefilled["a"].S[l] for l in O.GDN_LAYERS])
    assert torch.equal(back["gdn_state"].cpu(), S_or)
    assert back["prefix_len"] == 64
    toks = g["tokens"]
    lane_b = O.Lane(weights)
    lane_b.restore(prefilled["b"].snapshot())
    tok_b = prefilled["y0_b"]
    margins = g["top2_vals_f32"][:, 0] - g["top2_vals_f32"][:, 1]
    logits = torch.empty((2, eng.vocab), dtype=torch.float32, device="cuda")
    normed = torch.empty((2, 1024), dtype=torch.bfloat16, device="cuda")
    errs_n, errs_l, agree, strong, strong_ok, b_agree = [], [], 0, 0, 0, 0
    for s in range(32):
        in_tok = torch.tensor([int(toks[s]), tok_b], dtype=torch.int32, device="cuda")
        out = eng.decode_step(st, in_tok, logits=logits, normed=normed)
        errs_n.append(rel_l2(normed[0].float().cpu(), g["normed"][s + 1]))
        errs_l.append(rel_l2(logits[0].cpu()[::97], g["logits_f32_sub"][s + 1]))
        ok = int(out[0]) == int(g["top2_ids_f32"][s + 1, 0])
        agree += ok
        if margins[s + 1] > 0.25:
            strong += 1
            strong_ok += ok
        # lane 1 against the oracle run live (its own greedy continuation, teacher-forced by the oracle)
        nb = lane_b.forward([tok_b])
        ref_b, margin_b = O.top2_margin(lane_b.logits_f32(nb)[-1])
        b_agree += int(out[1]) == ref_b
        if margin_b > 0.25:
            assert int(out[1]) == ref_b, f"lane 1 step {s}: wide-margin token differs"
        tok_b = ref_b
    note("teacher_forced_normed_rel_l2", [max(errs_n), float(np.mean(errs_n))])
    note("teacher_forced_logits_rel_l2", [max(errs_l), float(np.mean(errs_l))])
    note("teacher_forced_token_agreement", [agree, 32, strong_ok, strong, b_agree])
    assert max(errs_n) <= CASCADE and max(errs_l) <= CASCADE
    assert errs_n[0] <= 4e-2                       # first step: one pass through 24 layers
    assert strong_ok == strong                     # wide-margin steps must agree
    assert agree >= 20 and b_agree >= 20           # narrow-margin steps may flip under the cascade
    assert int(st.positions[0]) == 96 and int(st.positions[1]) == 96
    # GDN state after 32 steps, layer 0 (cascade-free: its inputs depend on embeddings only)
    fin = st.export_lane(0, 128)
    ref_lane = O.Lane(weights)
    ref_lane.restore(prefilled["a"].snapshot())
    for t in toks[:32]:
        ref_lane.forward([int(t)])
    e0 = rel_l2(fin["gdn_state"][0].cpu(), ref_lane.S[0])
    e_last = rel_l2(fin["gdn_state"][17].cpu(), ref_lane.S[22])
    note("state_after_32_steps_rel_l2_layer0_layer22", [e0, e_last])
    assert e0 <= 5e-3 and e_last <= 0.15
    st.close()


def test_prefill_then_greedy_config0(eng, weights, golden, prefilled):
    """The engine's own prefill (wave bodies) + free-running greedy decode on config 0."""
    g = golden["config0_greedy"]
    ids = torch.stack([torch.from_numpy(g["prompt"]).int(), prefilled["ids_b"].int()]).cuda()
    st = eng.allocate_state(2, 128)
    y0, nl = eng.prefill(st, ids, want_normed=True)
    assert st.positions.tolist() == [64, 64]
    e_n = rel_l2(nl[0].float().cpu(), g["normed"][0])
    exp = st.export_lane(0, 128)
    a = prefilled["a"]
    e_s0 = rel_l2(exp["gdn_state"][0].cpu(), a.S[0])
    e_s17 = rel_l2(exp["gdn_state"][17].cpu(), a.S[22])
    assert torch.equal(exp["conv_window"][0].cpu(), a.window[0].float()) or \
        rel_l2(exp["conv_window"][0].cpu(), a.window[0].float()) < 5e-3
    Kor = torch.cat(a.kv[3]["k"], 0).permute(1, 0, 2)
    e_k = rel_l2(exp["kv_keys"][0, :, :64].float().cpu(), Kor)
    note("prefill_rel_l2_normed_state0_state17_k3", [e_n, e_s0, e_s17, e_k])
    assert e_n <= CASCADE and e_s0 <= 5e-3 and e_s17 <= 0.15 and e_k <= 2e-2
    margins = g["top2_vals_f32"][:, 0] - g["top2_vals_f32"][:, 1]
    if margins[0] > 0.25:
        assert int(y0[0]) == int(g["tokens"][0])
    # free-running greedy: count the common prefix with the reference's tokens
    toks = [int(y0[0])]
    cur = y0
    for _ in range(32):
        cur = eng.decode_step(st, cur)
        toks.append(int(cur[0]))
    common = 0
    for x, y in zip(toks, g["tokens"].tolist()):
        if x != y:
            break
        common += 1
    note("free_running_common_prefix_of_33", common)
    assert common >= 1
    st.close()


def test_determinism_lane_independence_and_graph(eng, pkg, golden):
    g = golden["config0_greedy"]
    prompt = torch.from_numpy(g["prompt"]).int()
    gen = torch.Generator().manual_seed(5)
    other1 = torch.randint(0, 248320, (2, 64), generator=gen).int()
    other2 = torch.randint(0, 248320, (2, 64), generator=gen).int()

    def run(others, use_graph):
        st = eng.allocate_state(3, 128)
        ids = torch.cat([prompt[None], others], 0).cuda()
        y0, _ = eng.prefill(st, ids)
        out = [y0.clone()]
        if use_graph:
            eng.decode_step(st, y0)            # warm-up outside capture (same step is replayed below)
            st2 = eng.allocate_state(3, 128)
            y0b, _ = eng.prefill(st2, ids)
            gr = pkg.StepGraph(eng, st2, steps=1)
            cur = y0b
            for _ in range(8):
                gr.tok_in.copy_(cur)
                gr.replay()
                cur = gr.tok_out.clone()
                out.append(cur)
            gr2 = pkg.StepGraph(eng, st2, steps=2)      # even-length graph chains through buf[0]
            gr2.tok_in.copy_(cur)
            gr2.replay()
            gr2.replay()
            S = st2.export_lane(0, 128)["gdn_state"]
            pos = st2.positions.tolist()
            st2.close()
        else:
            cur = y0
            for _ in range(8):
                cur = eng.decode_step(st, cur)
                out.append(cur.clone())
            S = st.export_lane(0, 128)["gdn_state"]
            pos = st.positions.tolist()
        st.close()
        return torch.stack(out).cpu(), S.cpu(), pos

    t1, S1, p1 = run(other1, False)
    t2, S2, p2 = run(other1, False)
    assert torch.equal(t1, t2) and torch.equal(S1, S2)              # run twice, byte-compare
    t3, S3, _ = run(other2, False)
    assert torch.equal(t1[:, 0], t3[:, 0]) and torch.equal(S1, S3)  # lane 0 ignores its neighbours
    t4, S4, p4 = run(other1, True)
    assert torch.equal(t1, t4) and p1 == [72, 72, 72] and p4 == [76, 76, 76]


@pytest.mark.parametrize("lanes", [1, 3, 16])
def test_small_step_kernel_matches_multi_kernel_path(pkg, weights, golden, monkeypatch, lanes):
    """At <= 16 lanes one persistent kernel runs the whole step.  Against the multi-kernel path on the
    same prompts: same positions, final-norm rows within the cascade band (the two paths sum their
    dot products in different orders), same GDN state in layer 0 to 5e-3, and equal tokens wherever
    the multi-kernel path's top-2 logit margin exceeds twice the largest logit difference of that row
    (on random-init weights the margins are tiny, so a share of equal tokens means nothing at 1 lane)."""
    g = golden["config0_greedy"]
    gen = torch.Generator().manual_seed(31 + lanes)
    ids = torch.randint(0, 248320, (lanes, 70), generator=gen).int()
    ids[0, :64] = torch.from_numpy(g["prompt"]).int()
    ids = ids.cuda()
    outs = {}
    head = weights[pkg.weights.LM + "embed_tokens.weight"].cuda().float()
    for mode in ("0", "1"):               # the multi-kernel run goes first; its tokens are fed to both
        monkeypatch.setenv("Q35_SMALL_STEP", mode)
        e = pkg.Engine(weights, max_rows=2048)
        st = e.allocate_state(lanes, 128)
        y0, _ = e.prefill(st, ids)
        toks, rows, lgs = [y0.clone()], [], []
        cur = y0
        for _ in range(6):
            nrm = torch.empty((lanes, 1024), dtype=torch.bfloat16, device="cuda")
            feed = cur if mode == "0" else outs["0"]["toks"][len(toks) - 1].cuda()
            cur = e.decode_step(st, feed, normed=nrm)         # no logits asked: that would leave the one-kernel path
            toks.append(cur.clone())
            rows.append(nrm.float().cpu())
            lgs.append((nrm.float() @ head.T).cpu())          # the tied head applied by the checker
        outs[mode] = dict(toks=torch.stack(toks).cpu(), rows=torch.stack(rows), lg=torch.stack(lgs), pos=st.positions.tolist(),
                          S=st.export_lane(0, 128)["gdn_state"][0].cpu(), status=e.status())
        st.close()
        e.close()
    a, b = outs["1"], outs["0"]
    assert a["status"] == 0 and b["status"] == 0
    assert a["pos"] == b["pos"] == [76] * lanes
    assert torch.equal(a["toks"][0], b["toks"][0])
    same = (a["toks"] == b["toks"]).float().mean().item()
    first = rel_l2(a["rows"][0], b["rows"][0])
    note(f"small_step_vs_multi_kernel_lanes{lanes}", [first, rel_l2(a["rows"], b["rows"]), same, rel_l2(a["S"], b["S"])])
    assert first <= 5e-2 and rel_l2(a["rows"], b["rows"]) <= CASCADE
    assert rel_l2(a["S"], b["S"]) <= 5e-3
    top2 = b["lg"].topk(2, dim=-1).values
    margin = top2[..., 0] - top2[..., 1]                       # [steps, lanes], multi-kernel path
    diff = (a["lg"] - b["lg"]).abs().amax(dim=-1)
    flipped = a["toks"][1:] != b["toks"][1:]
    assert bool((margin[flipped] <= 2 * diff[flipped]).all())  # every flip is explained by the logit band


def test_host_error_paths(eng, pkg):
    st = eng.allocate_state(2, 64)
    ids = torch.zeros((2, 65), dtype=torch.int32, device="cuda")
    with pytest.raises(pkg.Q35Error) as ei:
        eng.prefill(st, ids)                                  # prompt longer than max_ctx: refused, no launch
    assert ei.value.code == 3
    y0, _ = eng.prefill(st, ids[:, :64].contiguous())
    with pytest.raises(pkg.Q35Error) as ei:
        eng.decode_step(st, y0)                               # cache full
    assert ei.value.code == 3
    st.reset()
    assert st.positions.tolist() == [0, 0]
    bad = torch.tensor([0, 248320], dtype=torch.int32).pin_memory()
    with pytest.raises(pkg.Q35Error):
        eng.decode_step_host(st, bad, torch.empty(2, dtype=torch.int32).pin_memory())
    with pytest.raises(pkg.Q35Error) as ei:
        eng.allocate_state(2000, 64)                          # more lanes than the engine's scratch rows
    assert ei.value.code == 3
    with pytest.raises(pkg.Q35Error):
        eng.allocate_state(1, 100000)
    st.close()

"""Whole-step parity of the engine (through the C-ABI) against the CPU oracle and the
reference-generated config-0 fixture: decode steps from an imported state, the engine's own
prefill, determinism, lane independence, CUDA-graph replay, and the host-side error paths.

End-to-end numbers are cascade numbers: the reference's own legal variants (chunked vs
recurrent prefill, one-pass vs online softmax) differ by 3-7e-2 rel-L2 in the final logits on
these random-init weights, because 1-ULP bf16 differences are amplified through 24 residual
layers.  The 1e-2 / 1e-4 contract is asserted per stage with shared inputs in test_ops_gpu.py;
here the cascade is held under the oracle's own spread between its legal forms (measured on the CPU
by tests/test_oracle_spread.py and stored in tests/golden/oracle_self_spread.json) times a stated
factor, every token that differs from the reference's must be explained by the measured logit
difference of its row, and the measured figures go to $Q35_REPORT_DIR/parity_decode.json.
"""
from __future__ import annotations

import json
import os
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import q35_oracle as O

from conftest import REPO, rel_l2

pytestmark = pytest.mark.gpu

SPREAD = json.loads((REPO / "tests" / "golden" / "oracle_self_spread.json").read_text())
# the oracle's chunked vs recurrent prefill and f32 vs bf16 key cache differ by this much in the final
# logits (rel-L2, worst step); an independent implementation is held to 1.5 x that
CASCADE = 1.5 * SPREAD["logits_rel_l2_max"]
STATE_LAST = 1.5 * SPREAD["state_last_gdn_rel_l2_max"]
REPORT = {}


def note(key, val):
    """Measured parity figures; written to $Q35_REPORT_DIR/parity_decode.json when that variable is set."""
    REPORT[key] = val
    out = os.environ.get("Q35_REPORT_DIR")
    if out:
        Path(out).mkdir(parents=True, exist_ok=True)
        (Path(out) / "parity_decode.json").write_text(json.dumps(REPORT, indent=1, sort_keys=True))


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
    """Import the oracle's post-prefill state, feed the reference's own tokens for 32 steps.  Both lanes
    are followed by the oracle run live, so every step has the oracle's full f32 logits beside it.
    Token rule: a step whose token differs from the oracle's must be explained by the measured logit
    difference of that row (oracle top-2 margin <= 2 x max |logit difference|); its margin is recorded."""
    g = golden["config0_greedy"]
    st = eng.allocate_state(2, 128)
    for i, key in enumerate(("a", "b")):
        st.import_lane(i, *lane_tuple(prefilled[key], 128), prefix_len=64)
    back = st.export_lane(0, 128)
    S_or = torch.stack([prefilled["a"].S[l] for l in O.GDN_LAYERS])
    assert torch.equal(back["gdn_state"].cpu(), S_or)
    assert back["prefix_len"] == 64
    toks = g["tokens"]
    lanes_or = []
    for key in ("a", "b"):
        ln = O.Lane(weights)
        ln.restore(prefilled[key].snapshot())
        lanes_or.append(ln)
    tok_b = prefilled["y0_b"]
    logits = torch.empty((2, eng.vocab), dtype=torch.float32, device="cuda")
    normed = torch.empty((2, 1024), dtype=torch.bfloat16, device="cuda")
    errs_n, errs_l, agree, flips = [], [], [0, 0], []
    for s in range(32):
        feed = [int(toks[s]), tok_b]
        in_tok = torch.tensor(feed, dtype=torch.int32, device="cuda")
        out = eng.decode_step(st, in_tok, logits=logits, normed=normed)
        errs_n.append(rel_l2(normed[0].float().cpu(), g["normed"][s + 1]))
        errs_l.append(rel_l2(logits[0].cpu()[::97], g["logits_f32_sub"][s + 1]))
        lg = logits.cpu()
        for i in range(2):
            ref_lg = lanes_or[i].logits_f32(lanes_or[i].forward([feed[i]]))[-1]
            best, margin = O.top2_margin(ref_lg)
            diff = float((lg[i] - ref_lg).abs().max())
            if int(out[i]) == best:
                agree[i] += 1
            else:
                flips.append({"lane": i, "step": s, "oracle_margin": float(margin), "max_logit_diff": diff})
                assert margin <= 2 * diff, f"lane {i} step {s}: token differs at margin {margin} with logits only {diff} apart"
            if i == 0:
                assert best == int(g["top2_ids_f32"][s + 1, 0])     # the live oracle follows the fixture
            else:
                tok_b = best
    note("teacher_forced_normed_rel_l2", [max(errs_n), float(np.mean(errs_n))])
    note("teacher_forced_logits_rel_l2", [max(errs_l), float(np.mean(errs_l))])
    note("teacher_forced_token_agreement_of_32", agree)
    note("teacher_forced_flipped_tokens", flips)
    note("cascade_bound_from_oracle_self_spread", [CASCADE, STATE_LAST])
    assert max(errs_n) <= CASCADE and max(errs_l) <= CASCADE
    assert errs_n[0] <= 4e-2                       # first step: one pass through 24 layers, no cascade in time
    assert int(st.positions[0]) == 96 and int(st.positions[1]) == 96
    # GDN state after 32 steps, layer 0 (cascade-free: its inputs depend on embeddings only)
    fin = st.export_lane(0, 128)
    e0 = rel_l2(fin["gdn_state"][0].cpu(), lanes_or[0].S[0])
    e_last = rel_l2(fin["gdn_state"][17].cpu(), lanes_or[0].S[22])
    note("state_after_32_steps_rel_l2_layer0_layer22", [e0, e_last])
    assert e0 <= 1e-4 and e_last <= STATE_LAST
    st.close()


@pytest.mark.parametrize("fused", [0, 1])
def test_layer_teacher_forced(eng, weights, golden, prefilled, fused):
    """The reference's per-layer gate (specification/10-reference-dumps-and-gates.md:37; taps
    speccheck/specimpl.py:431-451): every block alone, fed the reference's own input residual row of
    decode step 0 on the oracle's post-prefill state, must reproduce the reference's output row to
    1e-2 - in both forms of the residual stream."""
    g = golden["config0_greedy"]
    st = eng.allocate_state(1, 128)
    st.import_lane(0, *lane_tuple(prefilled["a"], 128), prefix_len=64)
    errs = []
    for l in range(24):
        x_in = torch.from_numpy(g["dec0_s_in"][l]).to(torch.bfloat16)[None].cuda()
        out = eng.op_layer(st, l, x_in, T=1, fused=fused)
        errs.append(rel_l2(out[0].float().cpu(), g["dec0_s_out"][l]))
    note(f"layer_teacher_forced_rel_l2_fused{fused}", [max(errs), float(np.mean(errs))])
    assert max(errs) <= 1e-2, errs
    assert int(st.positions[0]) == 64                  # a single block does not advance the lane
    # the GDN state the blocks left behind is the reference's state after that token
    ref = O.Lane(weights)
    ref.restore(prefilled["a"].snapshot())
    ref.forward([int(g["tokens"][0])])
    fin = st.export_lane(0, 128)
    e0 = rel_l2(fin["gdn_state"][0].cpu(), ref.S[0])
    e17 = rel_l2(fin["gdn_state"][17].cpu(), ref.S[22])
    assert e0 <= 1e-4 and e17 <= 1e-4, (e0, e17)      # teacher-forced inputs: no cascade, the state contract holds in every layer
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
    assert e_n <= CASCADE and e_s0 <= 1e-4 and e_s17 <= STATE_LAST and e_k <= 2e-2
    margins = g["top2_vals_f32"][:, 0] - g["top2_vals_f32"][:, 1]
    head = weights[O.LM + "embed_tokens.weight"].float()
    d0 = float((nl[0].float().cpu() @ head.t() - torch.from_numpy(g["normed"][0]).float() @ head.t()).abs().max())
    if int(y0[0]) != int(g["tokens"][0]):
        assert margins[0] <= 2 * d0
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
def test_fused_stream_matches_add_norm_path(pkg, weights, golden, monkeypatch, lanes):
    """Bodies of at most 16 rows fold the residual add + norm into the weight-streaming projections.
    Against the path that runs the add + norm kernels on the same
    prompts: same positions, final-norm rows within the cascade band (the sums of squares are added in
    another order, a rare 1-ULP difference per norm), same GDN state in layer 0, and every differing
    token explained by the logit difference of its row."""
    g = golden["config0_greedy"]
    gen = torch.Generator().manual_seed(31 + lanes)
    ids = torch.randint(0, 248320, (lanes, 70), generator=gen).int()
    ids[0, :64] = torch.from_numpy(g["prompt"]).int()
    ids = ids.cuda()
    outs = {}
    head = weights[pkg.weights.LM + "embed_tokens.weight"].cuda().float()
    for mode in ("0", "1"):               # the add + norm run goes first; its tokens are fed to both
        monkeypatch.setenv("Q35_FUSE", mode)
        e = pkg.Engine(weights, max_rows=2048)
        st = e.allocate_state(lanes, 128)
        y0, _ = e.prefill(st, ids)
        before = e.launch_count()
        toks, rows, lgs = [y0.clone()], [], []
        cur = y0
        for _ in range(6):
            nrm = torch.empty((lanes, 1024), dtype=torch.bfloat16, device="cuda")
            feed = cur if mode == "0" else outs["0"]["toks"][len(toks) - 1].cuda()
            cur = e.decode_step(st, feed, normed=nrm)
            toks.append(cur.clone())
            rows.append(nrm.float().cpu())
            lgs.append((nrm.float() @ head.T).cpu())          # the tied head applied by the checker
        outs[mode] = dict(toks=torch.stack(toks).cpu(), rows=torch.stack(rows), lg=torch.stack(lgs), pos=st.positions.tolist(),
                          S=st.export_lane(0, 128)["gdn_state"][0].cpu(), status=e.status(),
                          launches=(e.launch_count() - before) // 6)
        st.close()
        e.close()
    a, b = outs["1"], outs["0"]
    assert a["status"] == 0 and b["status"] == 0
    assert a["pos"] == b["pos"] == [76] * lanes
    assert b["launches"] == 172 and a["launches"] == 125      # 48 add + norm kernels gone, one final norm added
    same = (a["toks"] == b["toks"]).float().mean().item()
    first = rel_l2(a["rows"][0], b["rows"][0])
    note(f"fused_vs_add_norm_path_lanes{lanes}", [first, rel_l2(a["rows"], b["rows"]), same, rel_l2(a["S"], b["S"])])
    assert first <= 4e-2 and rel_l2(a["rows"], b["rows"]) <= CASCADE
    assert rel_l2(a["S"], b["S"]) <= 1e-4
    top2 = b["lg"].topk(2, dim=-1).values
    margin = top2[..., 0] - top2[..., 1]                       # [steps, lanes], add + norm path
    diff = (a["lg"] - b["lg"]).abs().amax(dim=-1)
    flipped = a["toks"][1:] != b["toks"][1:]
    assert bool((margin[flipped] <= 2 * diff[flipped]).all())  # every flip is explained by the logit band


def test_incremental_equals_batch(eng, golden):
    """The reference's G5 gate on the engine (speccheck/gates/run_g5.py:60-105): prefill(64) and
    prefill(40) + 24 decode steps over the same ids must leave the same lane: equal positions, KV rows
    of the first attention layer and the layer-0 GDN state at the state tolerance (layer 0 sees only
    embeddings, so no cascade), later layers and the next token within the cascade band."""
    g = golden["config0_greedy"]
    gen = torch.Generator().manual_seed(77)
    ids = torch.stack([torch.from_numpy(g["prompt"]).int(), torch.randint(0, 248320, (64,), generator=gen).int()]).cuda()
    sa = eng.allocate_state(2, 128)
    ya, na = eng.prefill(sa, ids, want_normed=True)
    sb = eng.allocate_state(2, 128)
    eng.prefill(sb, ids[:, :40].contiguous())
    nb = torch.empty((2, 1024), dtype=torch.bfloat16, device="cuda")
    for t in range(40, 64):
        yb = eng.decode_step(sb, ids[:, t].contiguous(), normed=nb)
    assert sa.positions.tolist() == sb.positions.tolist() == [64, 64]
    res = {}
    for lane in range(2):
        A, B = sa.export_lane(lane, 128), sb.export_lane(lane, 128)
        e_s0 = rel_l2(B["gdn_state"][0].cpu(), A["gdn_state"][0].cpu())
        e_s17 = rel_l2(B["gdn_state"][17].cpu(), A["gdn_state"][17].cpu())
        e_k = rel_l2(B["kv_keys"][0, :, :64].float().cpu(), A["kv_keys"][0, :, :64].float().cpu())
        e_v = rel_l2(B["kv_values"][0, :, :64].float().cpu(), A["kv_values"][0, :, :64].float().cpu())
        # raw projection rows of layer 0: the same bf16 operands through two kernels (tensor-core tiles vs the
        # weight-streaming form), so single values may round the other way
        assert rel_l2(B["conv_window"][0].cpu(), A["conv_window"][0].cpu()) <= 2e-3
        e_n = rel_l2(nb[lane].float().cpu(), na[lane].float().cpu())
        res[lane] = [e_s0, e_s17, e_k, e_v, e_n]
        assert e_s0 <= 1e-4 and e_k <= 1e-2 and e_v <= 1e-2, res[lane]
        assert e_s17 <= STATE_LAST and e_n <= CASCADE, res[lane]
    note("incremental_vs_batch_state0_state17_k_v_normed", res)
    sa.close()
    sb.close()


def test_injected_bugs_leave_the_band(pkg, eng, weights, golden, prefilled):
    """The gate must bite: the reference's three injected bugs (speccheck/specimpl.py:255-258
    `conv_write_first`, :330-331 `deinterleave`, :435-436 `no_state_persist`; driver
    speccheck/gates/run_negative.py) are reproduced on the host - a conv window rolled before its taps
    are read, a q_proj whose [q | gate] halves are swapped, a GDN state that was not kept - and each must
    push the per-layer comparison far outside the 1e-2 band the healthy engine passes."""
    g = golden["config0_greedy"]

    def layer_err(engine, state, l):
        x_in = torch.from_numpy(g["dec0_s_in"][l]).to(torch.bfloat16)[None].cuda()
        return rel_l2(engine.op_layer(state, l, x_in)[0].float().cpu(), g["dec0_s_out"][l])

    S, win, k, v = lane_tuple(prefilled["a"], 128)
    # healthy baseline on the same call path
    st = eng.allocate_state(1, 128)
    st.import_lane(0, S, win, k, v, prefix_len=64)
    healthy = [layer_err(eng, st, 0), layer_err(eng, st, 3)]
    st.close()
    assert max(healthy) <= 1e-2
    # (1) conv window rolled one row too early: row 0 (the oldest) is gone, the newest is duplicated
    st = eng.allocate_state(1, 128)
    st.import_lane(0, S, torch.cat([win[:, 1:], win[:, 2:]], 1).contiguous(), k, v, prefix_len=64)
    e_conv = layer_err(eng, st, 0)
    st.close()
    # (2) GDN state not persisted: the block starts from zeros
    st = eng.allocate_state(1, 128)
    st.import_lane(0, torch.zeros_like(S), win, k, v, prefix_len=64)
    e_state = layer_err(eng, st, 0)
    st.close()
    # (3) q_proj de-interleaved wrongly: per head [gate | q] instead of [q | gate]
    name = O.LM + "layers.3.self_attn.q_proj.weight"
    bad = dict(weights)
    bad[name] = weights[name].view(8, 2, 256, 1024).flip(1).reshape(4096, 1024).contiguous()
    e2 = pkg.Engine(bad, max_rows=64, mtp=False)
    st = e2.allocate_state(1, 128)
    st.import_lane(0, S, win, k, v, prefix_len=64)
    e_gate = layer_err(e2, st, 3)
    st.close()
    e2.close()
    note("injected_bugs_layer_rel_l2_healthy_conv_state_gate", [healthy, e_conv, e_state, e_gate])
    assert e_conv > 5e-2 and e_state > 5e-2 and e_gate > 5e-2, (e_conv, e_state, e_gate)


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

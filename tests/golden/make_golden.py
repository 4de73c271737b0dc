#!/usr/bin/env python3
"""Generate tests/golden/*.npz by running the REFERENCE's torch implementation.

Needs the reference checkout (speccheck/specimpl.py, speccheck/mtp.py) on disk:

    python tests/golden/make_golden.py --reference /path/to/reference

The reference's checkpoint loader wants a safetensors shard; it is bypassed by building
`Weights` with `__new__` and filling `.p` from the seeded random-init tensors of
`weights.make_weights` (the same tensors every test regenerates from the seed).
Inputs of the isolated-stage fixtures are stored next to the outputs, so the tests do not
depend on reproducing a random stream.
"""
from __future__ import annotations

import argparse
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parents[1]


def load_weights_module():
    spec = importlib.util.spec_from_file_location(
        "q35_weights", REPO / "qwen3.5-0.8b_b200" / "weights.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def f32(t):
    return np.asarray(t.detach().float().cpu().numpy())


def fingerprint(t):
    t = t.detach().double().reshape(-1)
    return np.array([t.sum().item(), (t * t).sum().item(), t.abs().max().item()])


def top2(row_f32):
    vals, idx = torch.topk(row_f32, 2)
    return idx.numpy().astype(np.int64), vals.numpy().astype(np.float32)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of erokhins/qwen3.5-0.8b (its speccheck/ package is imported)")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    from speccheck import mtp as ref_mtp          # noqa: E402
    from speccheck import specimpl as ref         # noqa: E402

    torch.set_grad_enabled(False)
    wm = load_weights_module()
    params = wm.make_weights(seed=0)
    w = ref.Weights.__new__(ref.Weights)
    w.dtype = torch.bfloat16
    w.p = params
    E = params["model.language_model.embed_tokens.weight"]

    # weight-stream pins: detect a generator that no longer reproduces these tensors
    pins = {}
    for name in ("model.language_model.embed_tokens.weight",
                 "model.language_model.layers.0.linear_attn.in_proj_qkv.weight",
                 "model.language_model.layers.0.linear_attn.A_log",
                 "model.language_model.layers.0.linear_attn.dt_bias",
                 "model.language_model.layers.0.linear_attn.conv1d.weight",
                 "model.language_model.layers.3.self_attn.q_proj.weight",
                 "mtp.fc.weight"):
        pins[name] = f32(params[name].reshape(-1)[:64])
    np.savez(HERE / "weight_pins.npz", **pins)

    # ---------------------------------------------------------------- config 0
    g = torch.Generator().manual_seed(1234)
    ids = torch.randint(0, wm.VOCAB, (64,), generator=g)
    fwd = ref.Forward(w, gdn_form="chunk")
    dbg_p, dbg_d = {}, {}
    toks = fwd.greedy(ids.tolist(), 32, dbg_p, dbg_d, stop_on_eos=False)
    out = {"prompt": ids.numpy(), "tokens": np.array(toks, dtype=np.int64)}
    # replay teacher-forced to collect the normed row of every step
    fwd2 = ref.Forward(w, gdn_form="chunk")
    normed = [fwd2.prefill(ids)[-1]]
    for t in toks[:-1]:
        normed.append(fwd2.decode(t)[-1])
    normed = torch.stack(normed)                                   # [33,1024] bf16
    lg32 = normed.float() @ E.float().t()
    lgbf = (normed @ E.t()).float()
    out["normed"] = f32(normed)
    t2 = [top2(r) for r in lg32]
    out["top2_ids_f32"] = np.stack([a for a, _ in t2])
    out["top2_vals_f32"] = np.stack([b for _, b in t2])
    out["argmax_bf16"] = lgbf.argmax(-1).numpy()
    out["logits_f32_sub"] = f32(lg32[:, ::97])
    out["prefill_s_out_last"] = np.stack(
        [f32(dbg_p[f"L{l:02d}.s_out"][-1]) for l in range(24)])
    out["prefill_state_fp"] = np.stack(
        [fingerprint(dbg_p[f"L{l:02d}.gdn.state_new"]) for l in ref.GDN_LAYERS])
    d0 = dbg_d["decode0"]
    out["dec0_s_in"] = np.stack([f32(d0[f"L{l:02d}.s_in"][0]) for l in range(24)])
    out["dec0_s_out"] = np.stack([f32(d0[f"L{l:02d}.s_out"][0]) for l in range(24)])
    out["dec0_state_fp"] = np.stack(
        [fingerprint(d0[f"L{l:02d}.gdn.state_new"]) for l in ref.GDN_LAYERS])
    out["dec0_L00_gated_out"] = f32(d0["L00.gdn.gated_out"].reshape(-1))
    out["dec0_L00_o"] = f32(d0["L00.gdn.o_pre_norm"].reshape(-1))
    out["dec0_L00_state_h0"] = f32(d0["L00.gdn.state_new"][0])
    out["dec0_L03_q_rope"] = f32(d0["L03.attn.q_rope"].reshape(-1))
    out["dec0_L03_pre_gate"] = f32(d0["L03.attn.attn_out_pre_gate"].reshape(-1))
    np.savez_compressed(HERE / "config0_greedy.npz", **out)
    print("config0 tokens", toks)

    # ---------------------------------------------------------------- isolated GDN stage
    g = torch.Generator().manual_seed(77)
    l = 0
    o = {}
    x1 = torch.randn((1, 1024), generator=g).to(torch.bfloat16)
    win = torch.randn((3, 6144), generator=g).to(torch.bfloat16)
    S0 = (torch.randn((16, 128, 128), generator=g) * 0.1)
    sub = {}
    mix, nwin, S1 = ref.gdn(w, l, x1, sub, win, S0, "recurrent")
    o.update(x1=f32(x1), win=f32(win), S0_h=f32(S0[[0, 15]]), S0_seed=np.array([77]),
             mix1=f32(mix), nwin1=f32(nwin), S1_h=f32(S1[[0, 15]]), S1_fp=fingerprint(S1),
             o1=f32(sub["o_pre_norm"]), gated1=f32(sub["gated_out"]),
             beta1=f32(sub["beta"]), g1=f32(sub["g_decay_log"]),
             q1=f32(sub["q_post_conv"]), v1=f32(sub["v_post_conv"]))
    # multi-token, both forms, from a zero state
    xT = torch.randn((130, 1024), generator=g).to(torch.bfloat16)
    sr, sc = {}, {}
    mix_r, win_r, S_r = ref.gdn(w, l, xT, sr, None, None, "recurrent")
    mix_c, win_c, S_c = ref.gdn(w, l, xT, sc, None, None, "chunk")
    o.update(xT=f32(xT), mixT_rec=f32(mix_r), mixT_chunk=f32(mix_c),
             ST_rec_h=f32(S_r[[0, 15]]), ST_chunk_h=f32(S_c[[0, 15]]),
             ST_rec_fp=fingerprint(S_r), ST_chunk_fp=fingerprint(S_c),
             oT_rec=f32(sr["o_pre_norm"][[0, 63, 64, 129]]),
             oT_chunk=f32(sc["o_pre_norm"][[0, 63, 64, 129]]), winT=f32(win_r))
    np.savez_compressed(HERE / "stage_gdn.npz", **o)

    # ---------------------------------------------------------------- isolated attention stage
    g = torch.Generator().manual_seed(78)
    l = 3
    o = {}
    xp = torch.randn((37, 1024), generator=g).to(torch.bfloat16)
    xq = torch.randn((1, 1024), generator=g).to(torch.bfloat16)
    kv = {}
    cos, sin = ref.rope_cs(torch.arange(37), xp.device)
    sp = {}
    mix_p = ref.attention(w, l, xp, cos, sin, kv, sp)
    cos, sin = ref.rope_cs(torch.tensor([37]), xq.device)
    sq = {}
    mix_q = ref.attention(w, l, xq, cos, sin, kv, sq)
    o.update(xp=f32(xp), xq=f32(xq), mix_p=f32(mix_p), mix_q=f32(mix_q),
             q_rope=f32(sq["q_rope"]), k_rope=f32(sq["k_rope"]),
             pre_gate_q=f32(sq["attn_out_pre_gate"]), pre_gate_p=f32(sp["attn_out_pre_gate"]),
             K_cache=f32(torch.cat(kv["k"], 0)), V_cache=f32(torch.cat(kv["v"], 0)))
    np.savez_compressed(HERE / "stage_attn.npz", **o)

    # ---------------------------------------------------------------- glue / mlp / head stages
    g = torch.Generator().manual_seed(79)
    o = {}
    xs = torch.randn((3, 1024), generator=g).to(torch.bfloat16)
    dl = torch.randn((3, 1024), generator=g).to(torch.bfloat16)
    wn = params["model.language_model.layers.0.post_attention_layernorm.weight"]
    summed = xs + dl
    o.update(xs=f32(xs), dl=f32(dl), summed=f32(summed), normed=f32(ref.rmsnorm_zc(summed, wn)),
             mlp=f32(ref.mlp(w, 0, xs)), logits_bf16_sub=f32((xs @ E.t())[:, ::97]))
    np.savez_compressed(HERE / "stage_misc.npz", **o)

    # ---------------------------------------------------------------- MTP
    g = torch.Generator().manual_seed(4321)
    ids = torch.randint(0, wm.VOCAB, (16,), generator=g)
    o = {"prompt": ids.numpy()}
    for mode in ("steps", "batch"):
        f = ref.Forward(w, gdn_form="chunk")
        m = ref_mtp.MTPDraft(w)
        toks, st = ref_mtp.greedy_mtp(f, m, ids.tolist(), 8, k=1, stop_on_eos=False, verify=mode)
        o[f"tokens_{mode}"] = np.array(toks, dtype=np.int64)
        o[f"stats_{mode}"] = np.array([st["target_forwards"], st["drafted"], st["accepted"],
                                       st["bonus"], st["verify_tokens"]], dtype=np.int64)
        o[f"final_pos_{mode}"] = np.array([f.P, len(m.kv.get("k", []))])
        o[f"state_fp_{mode}"] = np.stack([fingerprint(f.rec[l]) for l in ref.GDN_LAYERS])
    fplain = ref.Forward(w, gdn_form="chunk")
    o["tokens_plain"] = np.array(fplain.greedy(ids.tolist(), 8, stop_on_eos=False), dtype=np.int64)
    # one isolated draft call
    f = ref.Forward(w, gdn_form="chunk")
    nrm = f.prefill(ids)
    t0 = int(f.logits(nrm)[-1].argmax())
    m = ref_mtp.MTPDraft(w)
    dd = {}
    d, xd = m.draft(t0, nrm[-1:], f.P + 1, dd)
    o.update(draft_h=f32(nrm[-1:]), draft_y=np.array([t0]), draft_pos=np.array([f.P + 1]),
             draft_id=np.array([d]), draft_u=f32(dd["mtp.u"]), draft_xd=f32(dd["mtp.x_d"]),
             draft_logits_sub=f32(dd["mtp.logits_last"][:, ::97]))
    np.savez_compressed(HERE / "mtp.npz", **o)
    print("mtp steps", o["tokens_steps"], "plain", o["tokens_plain"])


if __name__ == "__main__":
    main()

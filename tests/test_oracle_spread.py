"""The oracle's own noise floor on the seeded random-init weights.

Two legal forms of the reference's path are run on the config-0 prompt and compared with each
other: (A) chunked vs token-recurrent GDN prefill (speccheck/specimpl.py:187-235 vs :281-294), and
(B) the f32 key cache of the torch code as executed vs the bf16 key cache of the engine's state
tuple (engine/state.h:90).  One-ULP bf16 differences are amplified through 24 residual layers, so
the two forms of the SAME implementation differ by several 1e-2 in the final logits.  The figures
are stored in tests/golden/oracle_self_spread.json; the GPU cascade test holds the CUDA path to a
stated multiple of them.  This test re-measures them and checks the stored file is still right.

Regenerate the file with:  python tests/test_oracle_spread.py
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np
import torch

REPO = Path(__file__).resolve().parents[1]
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))
STORE = REPO / "tests" / "golden" / "oracle_self_spread.json"
STEPS = 8


def _rel(a, b) -> float:
    a, b = a.double().reshape(-1), b.double().reshape(-1)
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def measure(P: dict, prompt, tokens) -> dict:
    from oracle import q35_oracle as O
    torch.set_grad_enabled(False)
    forms = {"chunk": O.Lane(P, gdn_prefill="chunk"), "recurrent": O.Lane(P, gdn_prefill="recurrent"),
             "chunk_bf16_keys": O.Lane(P, gdn_prefill="chunk", kv_bf16=True)}
    rows = {k: [ln.forward(prompt)[-1:]] for k, ln in forms.items()}
    for t in tokens[:STEPS]:
        for k, ln in forms.items():
            rows[k].append(ln.forward([int(t)]))
    base = forms["chunk"]
    out = {"steps": STEPS + 1, "pairs": {}}
    lg_max, n_max, st_max = 0.0, 0.0, 0.0
    for other in ("recurrent", "chunk_bf16_keys"):
        n_err = [_rel(a.float(), b.float()) for a, b in zip(rows[other], rows["chunk"])]
        l_err = [_rel(forms[other].logits_f32(a), base.logits_f32(b)) for a, b in zip(rows[other], rows["chunk"])]
        last = O.GDN_LAYERS[-1]
        s_err = _rel(forms[other].S[last], base.S[last])
        out["pairs"][f"chunk_vs_{other}"] = {"normed_rel_l2": [max(n_err), float(np.mean(n_err))],
                                              "logits_rel_l2": [max(l_err), float(np.mean(l_err))],
                                              "state_last_gdn_rel_l2": s_err,
                                              "state_layer0_rel_l2": _rel(forms[other].S[0], base.S[0])}
        lg_max, n_max, st_max = max(lg_max, max(l_err)), max(n_max, max(n_err)), max(st_max, s_err)
    out["logits_rel_l2_max"], out["normed_rel_l2_max"], out["state_last_gdn_rel_l2_max"] = lg_max, n_max, st_max
    return out


def test_oracle_self_spread_matches_stored(weights, golden):
    g = golden["config0_greedy"]
    m = measure(weights, torch.from_numpy(g["prompt"]), g["tokens"])
    stored = json.loads(STORE.read_text())
    # the same torch ops on another CPU may round a few bf16 matmul outputs the other way: the cascade
    # figure moves by tens of per cent, its order of magnitude does not
    for key in ("logits_rel_l2_max", "normed_rel_l2_max", "state_last_gdn_rel_l2_max"):
        assert 0.4 * stored[key] <= m[key] <= 2.5 * stored[key], (key, m[key], stored[key])
    # the contract's own tolerances are below the oracle's spread: they can only hold per stage
    assert stored["logits_rel_l2_max"] > 1e-2 and stored["state_last_gdn_rel_l2_max"] > 1e-4
    # cascade-free quantities agree between the forms at the contract's tolerance
    for pair in m["pairs"].values():
        assert pair["state_layer0_rel_l2"] <= 1e-4


if __name__ == "__main__":
    from conftest import load_package
    pkg = load_package()
    P = pkg.weights.make_weights(seed=0)
    g = np.load(REPO / "tests" / "golden" / "config0_greedy.npz")
    res = measure(P, torch.from_numpy(g["prompt"]), g["tokens"])
    STORE.write_text(json.dumps(res, indent=1, sort_keys=True) + "\n")
    print(json.dumps(res, indent=1, sort_keys=True))

"""Weight I/O in the reference's checkpoint format: the loader contract of engine/loader.h
(name normalisation, vision skip, loud failures, tied-head alias, byte verification), exercised
the way engine/loader_test.cpp exercises it, on small synthetic shards."""
from __future__ import annotations

import json
import os
import struct

import pytest
import torch

LAYERS = [0, 3]          # one GatedDeltaNet layer, one attention layer
VOCAB = 512


@pytest.fixture(scope="module")
def ck(pkg):
    return pkg.checkpoint


@pytest.fixture(scope="module")
def params(pkg):
    return pkg.weights.make_weights(seed=5, vocab=VOCAB, layers=LAYERS, mtp=True)


def load(ck, d, **kw):
    kw.setdefault("layers", LAYERS)
    return ck.WeightStore.load(d, **kw)


def test_normalize_name_rules(ck):
    assert ck.normalize_name("model.language_model.layers.3.self_attn.q_proj.weight") == (ck.LOAD, "lm.layers.3.self_attn.q_proj.weight")
    assert ck.normalize_name("model.language_model.embed_tokens.weight") == (ck.LOAD, "lm.embed_tokens.weight")
    assert ck.normalize_name("mtp.layers.0.mlp.up_proj.weight") == (ck.LOAD, "mtp.layer0.mlp.up_proj.weight")
    assert ck.normalize_name("mtp.fc.weight") == (ck.LOAD, "mtp.fc.weight")
    assert ck.normalize_name("model.visual.blocks.0.attn.qkv.weight")[0] == ck.SKIP_VISION
    assert ck.normalize_name("lm_head.weight")[0] == ck.UNKNOWN
    assert ck.normalize_name("mtp.layers.1.mlp.up_proj.weight")[0] == ck.UNKNOWN
    for n in ("lm.layers.0.linear_attn.A_log", "mtp.layer0.input_layernorm.weight", "mtp.norm.weight"):
        assert ck.normalize_name(ck.denormalize_name(n)) == (ck.LOAD, n)


def test_text_path_tables_match_the_reference_counts(ck):
    """The reference's load gate G0 (speccheck/specimpl.py:61-63): 335 of the shard's 488 tensors are
    the text path (153 vision tensors skipped); exactly 36 of them are F32 (A_log and the gated-norm
    weight of the 18 GatedDeltaNet layers, specification/01-weights-and-shapes.md section 01.6)."""
    spec = ck.expected_spec(None, None, True)
    assert len(spec) == 335
    f32 = [n for n, (dt, _) in spec.items() if dt == "F32"]
    assert len(f32) == 36 and all(n.endswith(ck.F32_SUFFIXES) for n in f32)
    assert spec["model.language_model.embed_tokens.weight"] == ("BF16", (248320, 1024))
    assert spec["mtp.fc.weight"] == ("BF16", (1024, 2048))
    assert spec["model.language_model.layers.0.linear_attn.conv1d.weight"] == ("BF16", (6144, 1, 4))
    assert len([n for n in spec if n.startswith("mtp.")]) == 15
    nbytes = sum((4 if dt == "F32" else 2) * __import__("math").prod(shape) for dt, shape in spec.values())
    assert abs(nbytes / 1e9 - 1.5457) < 5e-4          # the text-only total of section 01.7


def test_round_trip_verified(ck, params, tmp_path):
    ck.save_checkpoint(params, tmp_path, n_vision_dummies=7)
    store, stats = load(ck, tmp_path, verify=True)
    assert stats.n_loaded == len(params) and stats.n_skipped_vision == 7 == store.skipped_vision_count
    assert stats.device_verified and stats.n_verified == len(params) and not stats.verify_failures
    assert store.allocation_count() == len(params)
    assert store.lookup_count() == len(params) + 1                     # + the tied-head alias
    assert store.resident_bytes() == sum(t.numel() * 2 for t in params.values())
    got = store.checkpoint_dict()
    assert set(got) == set(params)
    for k, t in params.items():
        assert got[k].dtype == torch.bfloat16 and torch.equal(got[k], t), k
    # forward map is sorted and complete
    assert store.ckpt_to_engine == sorted(store.ckpt_to_engine) and len(store.ckpt_to_engine) == len(params)
    assert ("mtp.layers.0.self_attn.q_proj.weight", "mtp.layer0.self_attn.q_proj.weight") in store.ckpt_to_engine


def test_tied_head_is_an_alias(ck, params, tmp_path):
    ck.save_checkpoint(params, tmp_path)
    store, _ = load(ck, tmp_path)
    head, emb = store.at("lm_head.weight"), store.at("lm.embed_tokens.weight")
    assert head.is_alias() and not emb.is_alias() and head.storage_owner == "lm.embed_tokens.weight"
    assert head.tensor.data_ptr() == emb.tensor.data_ptr() and head.checkpoint_name == ""
    assert emb.shape_string() == f"{VOCAB}x1024"
    assert store.find("lm.nothing") is None
    with pytest.raises(ck.CheckpointError):
        store.at("lm.nothing")


def test_f32_scalars_are_stored_f32_and_resident_bf16(ck, params, tmp_path):
    path = ck.save_checkpoint(params, tmp_path)
    hdr, _ = ck.read_header(path)
    f32 = [n for n, e in hdr.items() if e.dtype == "F32"]
    assert sorted(f32) == ["model.language_model.layers.0.linear_attn.A_log", "model.language_model.layers.0.linear_attn.norm.weight"]
    store, _ = load(ck, tmp_path)
    w = store.at("lm.layers.0.linear_attn.A_log")
    assert w.file_dtype == "F32" and w.tensor.dtype == torch.bfloat16


def test_index_file_and_two_shards(ck, params, tmp_path):
    names = sorted(params)
    a = {n: params[n] for n in names[::2]}
    b = {n: params[n] for n in names[1::2]}
    fix = lambda d: {n: (t.float() if n.endswith(ck.F32_SUFFIXES) else t) for n, t in d.items()}
    ck.write_shard(tmp_path / "a.safetensors", fix(a))
    ck.write_shard(tmp_path / "b.safetensors", fix(b))
    wm = {n: "a.safetensors" for n in a}
    wm.update({n: "b.safetensors" for n in b})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    (tmp_path / "stray.safetensors").write_bytes(b"not a shard")         # ignored: the index decides
    store, stats = load(ck, tmp_path, verify=True)
    assert len(stats.shard_paths) == 2 and stats.device_verified
    assert all(torch.equal(store.checkpoint_dict()[k], params[k]) for k in params)
    os.remove(tmp_path / "b.safetensors")
    with pytest.raises(ck.CheckpointError, match="missing"):
        load(ck, tmp_path)


def test_third_party_reader_and_writer_agree(ck, params, tmp_path):
    st = pytest.importorskip("safetensors.torch")
    path = ck.save_checkpoint(params, tmp_path / "ours")
    theirs = st.load_file(path)
    assert set(theirs) == set(params)
    for k, t in params.items():
        assert torch.equal(theirs[k].to(torch.bfloat16), t), k
    other = tmp_path / "theirs"
    other.mkdir()
    st.save_file({k: (t.float() if k.endswith(ck.F32_SUFFIXES) else t.contiguous()) for k, t in params.items()},
                 str(other / "model.safetensors"))
    store, stats = load(ck, other, verify=True)
    assert stats.device_verified
    assert all(torch.equal(store.checkpoint_dict()[k], params[k]) for k in params)


@pytest.mark.parametrize("case", ["unknown", "missing", "shape", "dtype", "lm_head", "extra_layer"])
def test_loud_failures(ck, params, tmp_path, case):
    p = dict(params)
    match = None
    if case == "unknown":
        p["optimizer.state.step"] = torch.zeros(1, dtype=torch.bfloat16)
        match = "neither loaded nor explicitly skipped"
    elif case == "missing":
        del p["model.language_model.layers.3.self_attn.k_norm.weight"]
        match = "missing"
    elif case == "shape":
        p["model.language_model.layers.0.mlp.down_proj.weight"] = torch.zeros((1024, 3583), dtype=torch.bfloat16)
        match = "shape"
    elif case == "lm_head":
        p["lm_head.weight"] = p["model.language_model.embed_tokens.weight"]
        match = "neither loaded nor explicitly skipped"
    elif case == "extra_layer":
        p["model.language_model.layers.1.input_layernorm.weight"] = torch.ones(1024, dtype=torch.bfloat16)
        match = "outside the text path"
    if case == "dtype":
        fixed = {n: t for n, t in p.items()}                      # A_log left as bf16: not the checkpoint's dtype
        ck.write_shard(tmp_path / "m.safetensors", fixed)
        match = "dtype"
    else:
        ck.save_checkpoint(p, tmp_path)
    with pytest.raises(ck.CheckpointError, match=match):
        load(ck, tmp_path)


def test_truncated_and_garbled_shards(ck, params, tmp_path):
    path = ck.save_checkpoint(params, tmp_path)
    size = os.path.getsize(path)
    with open(path, "r+b") as f:
        f.truncate(size - 4096)
    with pytest.raises(ck.CheckpointError, match="truncated"):
        load(ck, tmp_path)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(ck.CheckpointError, match="header length"):
        load(ck, tmp_path)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", 8) + b"notjson!")
    with pytest.raises(ck.CheckpointError, match="not JSON"):
        load(ck, tmp_path)
    os.remove(path)
    with pytest.raises(ck.CheckpointError, match="no safetensors shard"):
        load(ck, tmp_path)


def test_verification_catches_a_flipped_byte(ck, params, tmp_path):
    """The verification pass hashes resident bytes against file bytes: corrupt the resident copy
    and it must say so (the reference's negative control for its load verification)."""
    import hashlib
    path = ck.save_checkpoint(params, tmp_path)
    store, stats = load(ck, tmp_path, verify=True)
    assert stats.device_verified
    # flip one element of a resident tensor and re-hash by hand through the same rule
    w = store.at("lm.layers.3.self_attn.k_proj.weight")
    hdr, _ = ck.read_header(path)
    e = hdr[w.checkpoint_name]
    with open(path, "rb") as f:
        f.seek(e.begin)
        want = hashlib.sha256(f.read(e.end - e.begin)).hexdigest()
    good = hashlib.sha256(w.tensor.view(torch.uint8).numpy().tobytes()).hexdigest()
    assert good == want
    w.tensor[0, 0] += 1.0
    bad = hashlib.sha256(w.tensor.view(torch.uint8).numpy().tobytes()).hexdigest()
    assert bad != want


def test_text_only_load_ignores_mtp(ck, params, tmp_path):
    ck.save_checkpoint(params, tmp_path)
    store, stats = load(ck, tmp_path, mtp=False)
    assert store.find("mtp.fc.weight") is None
    assert stats.n_loaded == len([n for n in params if not n.startswith("mtp.")])


@pytest.mark.gpu
def test_engine_from_checkpoint_decodes_like_the_in_memory_weights(pkg, tmp_path):
    """Full 24-layer synthetic checkpoint (reduced vocabulary) written in the reference's format,
    loaded to the device with byte verification, and stepped: same tokens and same state as an
    engine built from the in-memory tensors."""
    vocab = 4096
    p = pkg.weights.make_weights(seed=1, vocab=vocab)
    pkg.checkpoint.save_checkpoint(p, tmp_path, n_vision_dummies=3, write_index=True)
    e1, stats = pkg.Engine.from_checkpoint(tmp_path, max_rows=64, verify=True)
    assert stats.device_verified and stats.n_skipped_vision == 3 and stats.n_loaded == len(p)
    e0 = pkg.Engine(p, max_rows=64)
    ids = torch.randint(0, vocab, (2, 24), generator=torch.Generator().manual_seed(2)).int().cuda()
    outs = []
    for e in (e0, e1):
        st = e.allocate_state(2, 64)
        tok, _ = e.prefill(st, ids)
        seq = [tok.clone()]
        for _ in range(6):
            seq.append(e.decode_step(st, seq[-1]).clone())
        outs.append((torch.stack(seq).cpu(), st.export_lane(1, 64)))
        st.close()
    assert torch.equal(outs[0][0], outs[1][0])
    assert torch.equal(outs[0][1]["gdn_state"], outs[1][1]["gdn_state"])
    e0.close(); e1.close()

"""Host-side mirror of the reference engine's step / state / prefill / MTP interface.

Everything here is plumbing over the C-ABI of libq35_b200.so (include/q35_engine.h): torch owns
device memory and streams, ctypes carries raw pointers.  There is no CPU path: if the CUDA
library is missing or no GPU is present, construction fails loudly.

Reference interface mirrored (paths relative to the reference repository):
  Engine            <- WeightStore + allocate_scratch + prepare_weight_adapters (engine/decode_step.h:479,595)
  Engine.allocate_state / LaneState.reset / .sizes   <- engine/state.h:99-120
  Engine.decode_step                                 <- engine/decode_step.h:582
  Engine.prefill                                     <- engine/prefill.h:155
  Engine.mtp_allocate / mtp_draft / mtp_verify       <- engine/mtp_draft.h:137-233, engine/mtp_verify.h:234,
                                                        engine/mtp_accept.h:248
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

from . import weights as W

LIB_PATH = Path(__file__).resolve().parent / "libq35_b200.so"

LAYER_FIELDS = ["input_norm", "post_norm", "mlp_gate", "mlp_up", "mlp_down", "gdn_in_qkv", "gdn_in_z",
                "gdn_in_b", "gdn_in_a", "gdn_conv", "gdn_A_log", "gdn_dt_bias", "gdn_norm", "gdn_out",
                "attn_q", "attn_k", "attn_v", "attn_q_norm", "attn_k_norm", "attn_o"]


class LayerWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in LAYER_FIELDS]


class MtpWeights(C.Structure):
    _fields_ = [("fc", C.c_void_p), ("norm_emb", C.c_void_p), ("norm_hid", C.c_void_p),
                ("norm_out", C.c_void_p), ("layer", LayerWeights)]


class Weights(C.Structure):
    _fields_ = [("embed", C.c_void_p), ("final_norm", C.c_void_p), ("layers", LayerWeights * 24),
                ("has_mtp", C.c_int), ("mtp", MtpWeights)]


class Config(C.Structure):
    _fields_ = [("vocab", C.c_int), ("max_rows", C.c_int), ("rope_inv_freq", C.c_float * 32)]


class StateSizes(C.Structure):
    _fields_ = [(n, C.c_size_t) for n in ("gdn_state_bytes", "conv_window_bytes", "kv_bytes",
                                          "per_token_bytes", "total_bytes")]


class Census(C.Structure):
    _fields_ = [("weight_bytes", C.c_longlong), ("lane_state_bytes", C.c_longlong),
                ("kv_bytes_per_pos", C.c_longlong), ("flops_per_row", C.c_longlong),
                ("launches_decode", C.c_int), ("launches_decode_few_lanes", C.c_int)]


EXPORTS = [
    "q35_last_error", "q35_abi_version", "q35_engine_create", "q35_engine_destroy", "q35_step_census",
    "q35_profile_begin", "q35_profile_end", "q35_engine_status",
    "q35_state_sizes_of", "q35_state_create", "q35_state_destroy", "q35_state_reset",
    "q35_state_positions", "q35_state_note_advance", "q35_state_export_lane", "q35_state_import_lane",
    "q35_decode_step", "q35_prefill", "q35_mtp_state_create", "q35_mtp_state_destroy",
    "q35_mtp_state_reset", "q35_mtp_draft", "q35_mtp_verify", "q35_mtp_state_reserve_depth",
    "q35_mtp_draft_k", "q35_mtp_verify_k", "q35_state_sync_bound", "q35_mtp_state_sync_bound",
    "q35_mtp_state_note_advance",
    "q35_op_add_norm", "q35_op_linear",
    "q35_pack_gate_up", "q35_op_mlp_gateup", "q35_op_lm_head", "q35_op_gdn_step", "q35_op_attn_decode",
    "q35_lm_head_argmax_static", "q35_engine_clear_status", "q35_engine_launch_count",
    "q35_mtp_draft_taps", "q35_ops_status", "q35_op_linear_resid", "q35_op_linear_norm", "q35_op_layer", "q35_op_linear_route",
    "q35_op_proj_residual", "q35_op_proj_residual_route",
]

_lib = None


class Q35Error(RuntimeError):
    """A C-ABI call returned a non-zero status (the reference throws std::runtime_error)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"[q35 status {code}] {message}")
        self.code = code


def load_library() -> C.CDLL:
    """dlopen the in-tree CUDA library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise FileNotFoundError(
            f"{LIB_PATH} is missing: build it with `python __graft_entry__.py build` "
            "(there is no CPU fallback for this path)")
    lib = C.CDLL(str(LIB_PATH))
    lib.q35_last_error.restype = C.c_char_p
    for name in EXPORTS:
        fn = getattr(lib, name)          # AttributeError = symbol not exported
        fn.restype = C.c_char_p if name in ("q35_last_error", "q35_op_linear_route", "q35_op_proj_residual_route") else C.c_int
    _lib = lib
    return lib


def _check(rc: int):
    if rc != 0:
        raise Q35Error(rc, load_library().q35_last_error().decode(errors="replace"))


def _ptr(t):
    if t is None:
        return C.c_void_p(0)
    assert t.is_cuda and t.is_contiguous(), "device-resident contiguous tensor required"
    return C.c_void_p(t.data_ptr())


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def rope_inv_freq() -> torch.Tensor:
    """theta^(-2i/64), i = 0..31, in f32 exactly as the reference builds it (speccheck/specimpl.py:153-154)."""
    i = torch.arange(32, dtype=torch.float32)
    return 1.0 / (1e7 ** (2 * i / 64))


def lm_head_argmax_static(x: torch.Tensor, embed: torch.Tensor, tokens: torch.Tensor | None = None):
    """Greedy token of each row of x [rows<=16, 1024] against the tied table embed [vocab, 1024],
    for callers that may not allocate device memory: needs no Engine, and the library keeps the
    scratch of its two-stage argmax in a fixed device array.  `tokens` (int32 [rows], device) is
    the caller's output buffer; pass it to keep this wrapper allocation-free as well."""
    lib = load_library()
    if tokens is None:
        tokens = torch.empty(x.shape[0], dtype=torch.int32, device=x.device)
    _check(lib.q35_lm_head_argmax_static(_ptr(x), _ptr(embed), embed.shape[0], x.shape[0], _ptr(tokens), _stream()))
    return tokens


class LaneState:
    """`lanes` request state tuples (GDN state, conv window, paged KV, positions)."""

    def __init__(self, engine: "Engine", lanes: int, max_ctx: int):
        self.engine, self.lanes, self.max_ctx = engine, lanes, max_ctx
        self.handle = C.c_void_p()
        _check(engine.lib.q35_state_create(engine.handle, lanes, max_ctx, C.byref(self.handle)))

    @property
    def positions(self) -> torch.Tensor:
        """Copy of the per-lane prefix lengths (position of the next token), int32 on the device."""
        out = torch.empty(self.lanes, dtype=torch.int32, device="cuda")
        _check(self.engine.lib.q35_state_positions(self.handle, _ptr(out), _stream()))
        return out

    def reset(self):
        _check(self.engine.lib.q35_state_reset(self.handle, _stream()))

    def note_advance(self, n: int):
        _check(self.engine.lib.q35_state_note_advance(self.handle, n))

    def sync_bound(self):
        """Tighten the host's position bound to the lanes' true maximum (synchronises the stream)."""
        _check(self.engine.lib.q35_state_sync_bound(self.handle, _stream()))

    @staticmethod
    def sizes(lanes: int, max_ctx: int) -> dict:
        s = StateSizes()
        _check(load_library().q35_state_sizes_of(lanes, max_ctx, C.byref(s)))
        return {n: getattr(s, n) for n, _ in StateSizes._fields_}

    def export_lane(self, lane: int, cap: int | None = None) -> dict:
        """One lane's tuple in the reference layouts (engine/state.h:86-92), as device tensors."""
        cap = cap or self.max_ctx
        S = torch.empty((18, 16, 128, 128), dtype=torch.float32, device="cuda")
        win = torch.empty((18, 3, 6144), dtype=torch.float32, device="cuda")
        k = torch.zeros((6, 2, cap, 256), dtype=torch.bfloat16, device="cuda")
        v = torch.zeros((6, 2, cap, 256), dtype=torch.bfloat16, device="cuda")
        _check(self.engine.lib.q35_state_export_lane(self.handle, lane, _ptr(S), _ptr(win), _ptr(k),
                                                     _ptr(v), cap, _stream()))
        return dict(gdn_state=S, conv_window=win, kv_keys=k, kv_values=v,
                    prefix_len=int(self.positions[lane].item()))

    def import_lane(self, lane: int, gdn_state, conv_window, kv_keys, kv_values, prefix_len: int):
        cap = kv_keys.shape[2] if kv_keys is not None else 0
        _check(self.engine.lib.q35_state_import_lane(
            self.handle, lane, _ptr(gdn_state), _ptr(conv_window), _ptr(kv_keys), _ptr(kv_values),
            cap, prefix_len, _stream()))

    def close(self):
        if self.handle:
            self.engine.lib.q35_state_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class MtpState:
    def __init__(self, engine: "Engine", state: LaneState, max_ctx: int, depth: int = 1):
        self.engine, self.state, self.depth = engine, state, depth
        self.handle = C.c_void_p()
        _check(engine.lib.q35_mtp_state_create(engine.handle, state.handle, max_ctx, C.byref(self.handle)))
        if depth > 1:
            _check(engine.lib.q35_mtp_state_reserve_depth(self.handle, depth))

    def reset(self):
        _check(self.engine.lib.q35_mtp_state_reset(self.handle, _stream()))

    def note_advance(self, n: int):
        _check(self.engine.lib.q35_mtp_state_note_advance(self.handle, n))

    def sync_bound(self):
        """Tighten the host's draft-cache length bound to the true maximum (synchronises the stream)."""
        _check(self.engine.lib.q35_mtp_state_sync_bound(self.handle, _stream()))

    def close(self):
        if self.handle:
            self.engine.lib.q35_mtp_state_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Engine:
    """Device weights (packed by the library) + scratch for bodies of up to `max_rows` rows."""

    def __init__(self, params: dict, max_rows: int, vocab: int | None = None, mtp: bool = True):
        if not torch.cuda.is_available():
            raise RuntimeError("q35 engine needs a CUDA device; there is no CPU path")
        self.lib = load_library()
        dev = {}

        def put(name):
            t = params[name]
            if not t.is_cuda:
                t = t.to("cuda")
            t = t.to(torch.bfloat16).contiguous()
            dev[name] = t
            return C.c_void_p(t.data_ptr())

        w = Weights()
        w.embed = put(W.LM + "embed_tokens.weight")
        w.final_norm = put(W.LM + "norm.weight")
        self.vocab = vocab or dev[W.LM + "embed_tokens.weight"].shape[0]

        def fill(lw, pre, attn):
            lw.input_norm = put(pre + "input_layernorm.weight")
            lw.post_norm = put(pre + "post_attention_layernorm.weight")
            lw.mlp_gate = put(pre + "mlp.gate_proj.weight")
            lw.mlp_up = put(pre + "mlp.up_proj.weight")
            lw.mlp_down = put(pre + "mlp.down_proj.weight")
            if attn:
                a = pre + "self_attn."
                lw.attn_q, lw.attn_k, lw.attn_v = put(a + "q_proj.weight"), put(a + "k_proj.weight"), put(a + "v_proj.weight")
                lw.attn_q_norm, lw.attn_k_norm = put(a + "q_norm.weight"), put(a + "k_norm.weight")
                lw.attn_o = put(a + "o_proj.weight")
            else:
                g = pre + "linear_attn."
                lw.gdn_in_qkv, lw.gdn_in_z = put(g + "in_proj_qkv.weight"), put(g + "in_proj_z.weight")
                lw.gdn_in_b, lw.gdn_in_a = put(g + "in_proj_b.weight"), put(g + "in_proj_a.weight")
                lw.gdn_conv, lw.gdn_A_log = put(g + "conv1d.weight"), put(g + "A_log")
                lw.gdn_dt_bias, lw.gdn_norm = put(g + "dt_bias"), put(g + "norm.weight")
                lw.gdn_out = put(g + "out_proj.weight")

        for l in range(W.N_LAYERS):
            fill(w.layers[l], f"{W.LM}layers.{l}.", W.is_attn_layer(l))
        self.has_mtp = bool(mtp and (W.MTP + "fc.weight") in params)
        w.has_mtp = int(self.has_mtp)
        if self.has_mtp:
            w.mtp.fc = put(W.MTP + "fc.weight")
            w.mtp.norm_emb = put(W.MTP + "pre_fc_norm_embedding.weight")
            w.mtp.norm_hid = put(W.MTP + "pre_fc_norm_hidden.weight")
            w.mtp.norm_out = put(W.MTP + "norm.weight")
            fill(w.mtp.layer, W.MTP + "layers.0.", True)
        cfg = Config()
        cfg.vocab, cfg.max_rows = self.vocab, max_rows
        for i, f in enumerate(rope_inv_freq().tolist()):
            cfg.rope_inv_freq[i] = f
        self.max_rows = max_rows
        self.handle = C.c_void_p()
        _check(self.lib.q35_engine_create(C.byref(cfg), C.byref(w), _stream(), C.byref(self.handle)))
        torch.cuda.synchronize()
        # the library copied everything except the embedding table, which it reads in place
        self.embed = dev[W.LM + "embed_tokens.weight"]
        del dev

    @classmethod
    def from_checkpoint(cls, model_dir, max_rows: int, mtp: bool = True, verify: bool = False, vocab: int | None = None):
        """Engine over a checkpoint directory in the reference's safetensors format
        (engine/loader.h:118-141): shards resolved, names normalised, vision tensors skipped, the
        tied head aliased, weights copied to the device once.  Returns (engine, load stats)."""
        from .checkpoint import WeightStore
        store, stats = WeightStore.load(model_dir, device="cuda", vocab=vocab, mtp=mtp, verify=verify)
        if verify and stats.verify_failures:
            raise Q35Error(1, "checkpoint verification failed: " + "; ".join(stats.verify_failures[:3]))
        return cls(store.checkpoint_dict(), max_rows=max_rows, mtp=mtp), stats

    def status(self) -> int:
        """0 when healthy; non-zero when a kernel's bounded wait expired (synchronises the device)."""
        v = C.c_int(0)
        _check(self.lib.q35_engine_status(self.handle, C.byref(v)))
        return v.value

    def clear_status(self):
        _check(self.lib.q35_engine_clear_status(self.handle, _stream()))

    def launch_count(self) -> int:
        """Kernels enqueued through this engine so far (a captured kernel counts once, at capture)."""
        v = C.c_longlong(0)
        _check(self.lib.q35_engine_launch_count(self.handle, C.byref(v)))
        return v.value

    # ---- census -------------------------------------------------------------------------------
    def census(self) -> dict:
        c = Census()
        _check(self.lib.q35_step_census(self.handle, C.byref(c)))
        return {n: getattr(c, n) for n, _ in Census._fields_}

    def step_bytes(self, lanes: int, ctx: float) -> float:
        """Algorithmic HBM bytes of one decode step: weights once + per lane (state read+write,
        conv window, KV read of `ctx` cached positions + one appended)."""
        c = self.census()
        return c["weight_bytes"] + lanes * (c["lane_state_bytes"] + c["kv_bytes_per_pos"] * (ctx + 1))

    FAMILIES = ["glue", "in_proj", "gdn", "attn", "out_proj", "mlp_gateup", "mlp_down", "head"]

    def profile_begin(self):
        _check(self.lib.q35_profile_begin(self.handle))

    def profile_end(self) -> dict:
        """{family: (milliseconds, launches)} of every kernel launched since profile_begin."""
        ms = (C.c_double * len(self.FAMILIES))()
        n = (C.c_longlong * len(self.FAMILIES))()
        _check(self.lib.q35_profile_end(self.handle, ms, n))
        return {f: (ms[i], n[i]) for i, f in enumerate(self.FAMILIES)}

    # ---- state ---------------------------------------------------------------------------------
    def allocate_state(self, lanes: int, max_ctx: int) -> LaneState:
        return LaneState(self, lanes, max_ctx)

    def mtp_allocate(self, state: LaneState, max_ctx: int, depth: int = 1) -> MtpState:
        """Draft cache + the shadow state buffers of depth-`depth` rounds (1 or 2 candidates per round)."""
        return MtpState(self, state, max_ctx, depth)

    def decode_step(self, state: LaneState, in_tok: torch.Tensor, out_tok: torch.Tensor | None = None,
                    logits: torch.Tensor | None = None, normed: torch.Tensor | None = None):
        """One greedy step for every lane; tokens are int32 device tensors [lanes]."""
        assert in_tok.dtype == torch.int32 and in_tok.numel() == state.lanes
        if out_tok is None:
            out_tok = torch.empty(state.lanes, dtype=torch.int32, device="cuda")
        _check(self.lib.q35_decode_step(self.handle, state.handle, _ptr(in_tok), _ptr(out_tok),
                                        _ptr(logits), _ptr(normed), _stream()))
        return out_tok

    def prefill(self, state: LaneState, ids: torch.Tensor, want_normed: bool = False):
        """ids int32 [lanes, T] on the device -> (y0 [lanes], last final-norm rows or None)."""
        assert ids.dtype == torch.int32 and ids.dim() == 2 and ids.shape[0] == state.lanes
        y0 = torch.empty(state.lanes, dtype=torch.int32, device="cuda")
        nl = torch.empty((state.lanes, 1024), dtype=torch.bfloat16, device="cuda") if want_normed else None
        _check(self.lib.q35_prefill(self.handle, state.handle, _ptr(ids.contiguous()), ids.shape[1],
                                    _ptr(y0), _ptr(nl), _stream()))
        return y0, nl

    def mtp_draft(self, m: MtpState, h_norm, y_next, pos, proposal=None):
        if proposal is None:
            proposal = torch.empty(m.state.lanes, dtype=torch.int32, device="cuda")
        _check(self.lib.q35_mtp_draft(self.handle, m.handle, _ptr(h_norm), _ptr(y_next), _ptr(pos),
                                      _ptr(proposal), _stream()))
        return proposal

    def mtp_verify(self, state: LaneState, m: MtpState, cur, cand, emit=None, n_emit=None, h_next=None):
        L = state.lanes
        emit = emit if emit is not None else torch.empty((L, 2), dtype=torch.int32, device="cuda")
        n_emit = n_emit if n_emit is not None else torch.empty(L, dtype=torch.int32, device="cuda")
        h_next = h_next if h_next is not None else torch.empty((L, 1024), dtype=torch.bfloat16, device="cuda")
        _check(self.lib.q35_mtp_verify(self.handle, state.handle, m.handle, _ptr(cur), _ptr(cand),
                                       _ptr(emit), _ptr(n_emit), _ptr(h_next), _stream()))
        return emit, n_emit, h_next

    # ---- host-buffer step (what a caller of the reference's decode_step does) ------------------
    def mtp_draft_k(self, m: MtpState, h_norm, y_next, pos, k: int, proposals=None):
        """k chained drafts per lane: proposals int32 [lanes, k]."""
        L = m.state.lanes
        if proposals is None:
            proposals = torch.empty((L, k), dtype=torch.int32, device="cuda")
        _check(self.lib.q35_mtp_draft_k(self.handle, m.handle, _ptr(h_norm), _ptr(y_next), _ptr(pos), k,
                                        _ptr(proposals), _stream()))
        return proposals

    def mtp_verify_k(self, state: LaneState, m: MtpState, cur, cands, emit=None, n_emit=None, h_next=None):
        """Depth-k verify: cands int32 [lanes, k] -> (emit [lanes, k+1], n_emit [lanes], h_next [lanes, 1024])."""
        L, k = state.lanes, cands.shape[1]
        emit = torch.empty((L, k + 1), dtype=torch.int32, device="cuda") if emit is None else emit
        n_emit = torch.empty(L, dtype=torch.int32, device="cuda") if n_emit is None else n_emit
        h_next = torch.empty((L, 1024), dtype=torch.bfloat16, device="cuda") if h_next is None else h_next
        _check(self.lib.q35_mtp_verify_k(self.handle, state.handle, m.handle, _ptr(cur), _ptr(cands), k,
                                         _ptr(emit), _ptr(n_emit), _ptr(h_next), _stream()))
        return emit, n_emit, h_next

    def decode_step_host(self, state: LaneState, tok_host: torch.Tensor, out_host: torch.Tensor,
                         graph: "StepGraph | None" = None):
        """tokens in pinned host memory -> H2D, one step, D2H, synchronise.  Validates ids on the
        host like the reference's body guard (engine/decode_step.cpp:450-480)."""
        if int(tok_host.min()) < 0 or int(tok_host.max()) >= self.vocab:
            raise Q35Error(1, "token id outside [0, vocab)")
        if graph is not None:
            graph.tok_in.copy_(tok_host, non_blocking=True)
            graph.replay()
            out_host.copy_(graph.tok_out, non_blocking=True)
        else:
            dev_in = tok_host.to("cuda", non_blocking=True)
            out_host.copy_(self.decode_step(state, dev_in), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return out_host

    # ---- single stages -------------------------------------------------------------------------
    def op_add_norm(self, x, delta, w):
        s, n = torch.empty_like(x), torch.empty_like(x)
        _check(self.lib.q35_op_add_norm(_ptr(x), _ptr(delta), _ptr(w), _ptr(s), _ptr(n), x.shape[0], _stream()))
        return s, n

    def op_linear(self, x, Wt):
        out = torch.empty((x.shape[0], Wt.shape[0]), dtype=torch.bfloat16, device="cuda")
        _check(self.lib.q35_op_linear(_ptr(x), _ptr(Wt), _ptr(out), x.shape[0], Wt.shape[0], Wt.shape[1], _stream()))
        return out

    def pack_gate_up(self, gate, up):
        out = torch.empty((2 * W.D_FF, W.D_MODEL), dtype=torch.bfloat16, device="cuda")
        _check(self.lib.q35_pack_gate_up(_ptr(gate), _ptr(up), _ptr(out), _stream()))
        return out

    def ops_status(self) -> int:
        """Status word of the stage entry points that take no engine (op_linear, op_mlp_gateup); cleared by the read."""
        v = C.c_int(-1)
        _check(self.lib.q35_ops_status(C.byref(v)))
        return v.value

    def op_linear_resid(self, x, Wt, resid):
        """resid [rows, 1024] += x @ Wt.T in place (bf16 roundings of the reference); returns resid."""
        _check(self.lib.q35_op_linear_resid(self.handle, _ptr(x), _ptr(Wt), _ptr(resid), x.shape[0], Wt.shape[1], _stream()))
        return resid

    def op_linear_norm(self, resid, nw, Wt, swiglu: bool = False):
        """N(resid; nw) @ Wt.T for the rows the last op_linear_resid produced."""
        n_out = Wt.shape[0] // 2 if swiglu else Wt.shape[0]
        out = torch.empty((resid.shape[0], n_out), dtype=torch.bfloat16, device="cuda")
        _check(self.lib.q35_op_linear_norm(self.handle, _ptr(resid), _ptr(nw), _ptr(Wt), _ptr(out), resid.shape[0],
                                           Wt.shape[0], int(swiglu), _stream()))
        return out

    def op_layer(self, state: "LaneState", layer: int, x_in, T: int = 1, fused: int = -1):
        """One decoder block on its input residual rows x_in [lanes*T, 1024]; positions are not advanced."""
        out = torch.empty_like(x_in)
        _check(self.lib.q35_op_layer(self.handle, state.handle, layer, _ptr(x_in), _ptr(out), T, fused, _stream()))
        return out

    def mtp_draft_taps(self, m: "MtpState", h_norm, y_next, pos, want_logits: bool = False):
        """One draft with the block's taps: (proposal, u, x_d, logits or None)."""
        L = m.state.lanes
        prop = torch.empty(L, dtype=torch.int32, device="cuda")
        u = torch.empty((L, 1024), dtype=torch.bfloat16, device="cuda")
        xd = torch.empty((L, 1024), dtype=torch.bfloat16, device="cuda")
        lg = torch.empty((L, self.vocab), dtype=torch.float32, device="cuda") if want_logits else None
        _check(self.lib.q35_mtp_draft_taps(self.handle, m.handle, _ptr(h_norm), _ptr(y_next), _ptr(pos), _ptr(prop),
                                           _ptr(u), _ptr(xd), _ptr(lg), _stream()))
        return prop, u, xd, lg

    def op_proj_residual(self, x, Wt, resid, nw, normed=None):
        """Output / down projection stage as a body runs it: resid updated in place, normed written above 16 rows."""
        if normed is None:
            normed = torch.empty_like(resid)
        _check(self.lib.q35_op_proj_residual(self.handle, _ptr(x), _ptr(Wt), _ptr(resid), _ptr(nw), _ptr(normed),
                                             x.shape[0], Wt.shape[1], _stream()))
        return resid, normed

    def op_proj_residual_route(self, rows: int, K: int) -> str:
        return self.lib.q35_op_proj_residual_route(self.handle, rows, K).decode()

    def op_linear_route(self, rows: int, N: int, K: int, epilogue: int = 0) -> str:
        """Kernel a projection of this shape is routed to (0 plain, 1 SwiGLU, 2 head + argmax)."""
        return self.lib.q35_op_linear_route(rows, N, K, epilogue).decode()

    def op_mlp_gateup(self, x, Wgu):
        act = torch.empty((x.shape[0], W.D_FF), dtype=torch.bfloat16, device="cuda")
        _check(self.lib.q35_op_mlp_gateup(_ptr(x), _ptr(Wgu), _ptr(act), x.shape[0], _stream()))
        return act

    def op_lm_head(self, x, want_logits: bool = False):
        rows = x.shape[0]
        tok = torch.empty(rows, dtype=torch.int32, device="cuda")
        lg = torch.empty((rows, self.vocab), dtype=torch.float32, device="cuda") if want_logits else None
        _check(self.lib.q35_op_lm_head(self.handle, _ptr(x), rows, _ptr(tok), _ptr(lg), _stream()))
        return tok, lg

    def op_gdn_step(self, proj, conv_w, A_log, dt_bias, norm_w, S, window, lanes: int, T: int):
        y = torch.empty((lanes * T, 2048), dtype=torch.bfloat16, device="cuda")
        _check(self.lib.q35_op_gdn_step(_ptr(proj), _ptr(conv_w), _ptr(A_log), _ptr(dt_bias), _ptr(norm_w),
                                        _ptr(S), _ptr(window), _ptr(y), lanes, T, _stream()))
        return y

    def op_attn_decode(self, proj, q_norm, k_norm, kpool, vpool, page_table, ctx, lanes: int, T: int = 1):
        out = torch.empty((lanes * T, 2048), dtype=torch.bfloat16, device="cuda")
        _check(self.lib.q35_op_attn_decode(self.handle, _ptr(proj), _ptr(q_norm), _ptr(k_norm), _ptr(kpool),
                                           _ptr(vpool), _ptr(page_table), page_table.shape[1], _ptr(ctx),
                                           _ptr(out), lanes, T, _stream()))
        return out

    def close(self):
        if self.handle:
            self.lib.q35_engine_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class StepGraph:
    """A CUDA graph of `steps` chained decode steps (token i+1 = argmax of step i).

    Tokens ping-pong between two device buffers: step i reads buf[i % 2] and writes buf[(i+1) % 2].
    With an even `steps` the last token lands in buf[0] again, so replays chain with no copy; with
    steps = 1 the caller feeds `tok_in` and reads `tok_out`.  The step's kernels read positions and
    tokens from device memory, so one captured graph serves every step; the host reports replayed
    steps to the state for its capacity check."""

    def __init__(self, engine: Engine, state: LaneState, steps: int = 2):
        assert steps == 1 or steps % 2 == 0
        self.engine, self.state, self.n = engine, state, steps
        self.buf = torch.zeros((2, state.lanes), dtype=torch.int32, device="cuda")
        self.tok_in = self.buf[0]
        self.tok_out = self.buf[steps % 2]
        self.graph = torch.cuda.CUDAGraph()
        self.replays = 0
        before = engine.launch_count()
        with torch.cuda.graph(self.graph):
            for i in range(steps):
                engine.decode_step(state, self.buf[i % 2], self.buf[(i + 1) % 2])
        self.kernels_per_replay = engine.launch_count() - before     # counted while the graph was captured
        # capture ran no kernel but advanced the host-side position bound once per captured step: take
        # that back, every replay reports itself (so a bound tightened between capture and replay stays right)
        state.note_advance(-steps)

    def replay(self):
        self.state.note_advance(self.n)
        self.replays += 1
        self.graph.replay()


class MtpRoundGraph:
    """A CUDA graph of ONE speculative round: `depth` chained MTP drafts, the verify body of
    depth + 1 tokens per lane, the verdict, and the hand-over of the round's last emitted token and
    its final-norm row to the next round.

    The round's kernels read positions, cache lengths, tokens and the live-buffer selector from
    device memory, so one captured graph serves every round; between replays nothing crosses the
    host.  The caller seeds `tok` [lanes] and `h` [lanes, 1024] (what `prefill(..., want_normed=True)`
    returned) once, replays, and reads `emit` [lanes, depth + 1] / `n_emit` [lanes] of the round just
    replayed (copy them out before the next replay); `emitted_total` counts the tokens of all replays
    on the device, so a caller that only wants throughput launches nothing between replays (a kernel
    launched between two graph launches costs the second one ~0.3 ms of start-up on this driver:
    1.64 ms per round back to back against 2.01 ms with a two-kernel tally in between, 16 lanes).
    The host's capacity bounds advance by the
    worst case per replay (depth + 1 positions, depth draft rows); `state.sync_bound()` /
    `mtp.sync_bound()` tighten them when the caller synchronises anyway."""

    def __init__(self, engine: Engine, state: LaneState, mtp: MtpState, depth: int = 1, history: int = 0,
                 forced_tokens: torch.Tensor | None = None):
        """forced_tokens (int32 [lanes, n], optional): the lanes' true greedy continuations (token i of a
        lane = the i-th token after the one seeded into `tok`).  The drafts still run, but the verifier is
        handed forced_tokens[lane, emitted so far ...] as candidates, so every candidate that is the
        target's own next token is accepted: the accept branch of a round can be timed on weights whose
        draft never agrees with the target."""
        L = state.lanes
        self.engine, self.state, self.mtp, self.depth = engine, state, mtp, depth
        self.forced = forced_tokens
        self.emitted_lane = torch.zeros(L, dtype=torch.int64, device="cuda")     # tokens emitted per lane by the replays
        # optional ring of the last `history` rounds' verdicts, written by the graph itself (slot = rounds % history),
        # for a caller that reads verdicts back every few rounds without launching anything between replays
        self.history = history
        self.rounds = torch.zeros((), dtype=torch.int64, device="cuda")
        self.hist_emit = torch.zeros((max(history, 1), L, depth + 1), dtype=torch.int32, device="cuda")
        self.hist_n = torch.zeros((max(history, 1), L), dtype=torch.int32, device="cuda")
        self.tok = torch.zeros(L, dtype=torch.int32, device="cuda")
        self.h = torch.zeros((L, 1024), dtype=torch.bfloat16, device="cuda")
        self.emit = torch.zeros((L, depth + 1), dtype=torch.int32, device="cuda")
        self.n_emit = torch.zeros(L, dtype=torch.int32, device="cuda")
        self.emitted_total = torch.zeros((), dtype=torch.int64, device="cuda")   # tokens emitted by all replays, all lanes
        self.graph = torch.cuda.CUDAGraph()
        self.replays = 0
        with torch.cuda.graph(self.graph):
            pos = (state.positions + 1).int()
            if depth == 1:
                d = engine.mtp_draft(mtp, self.h, self.tok, pos)
            else:
                d = engine.mtp_draft_k(mtp, self.h, self.tok, pos, depth)
            if forced_tokens is not None:
                idx = (self.emitted_lane[:, None] + torch.arange(depth, device="cuda")[None]).clamp_(max=forced_tokens.shape[1] - 1)
                d = forced_tokens.gather(1, idx).to(torch.int32).reshape(L, depth).contiguous()
                if depth == 1:
                    d = d[:, 0].contiguous()
            if depth == 1:
                _, _, h_next = engine.mtp_verify(state, mtp, self.tok, d, emit=self.emit, n_emit=self.n_emit)
            else:
                _, _, h_next = engine.mtp_verify_k(state, mtp, self.tok, d, emit=self.emit, n_emit=self.n_emit)
            self.emitted_lane += self.n_emit
            self.tok.copy_(self.emit.gather(1, (self.n_emit - 1).long()[:, None])[:, 0])
            self.h.copy_(h_next)
            self.emitted_total += self.n_emit.sum()
            if history > 0:
                slot = (self.rounds % history).view(1)
                self.hist_emit.index_copy_(0, slot, self.emit.unsqueeze(0))
                self.hist_n.index_copy_(0, slot, self.n_emit.unsqueeze(0))
            self.rounds += 1
        # capture ran no kernel but advanced the host-side bounds once: take that back, every replay reports itself
        state.note_advance(-(depth + 1))
        mtp.note_advance(-depth)

    def replay(self):
        self.state.note_advance(self.depth + 1)
        self.mtp.note_advance(self.depth)
        self.replays += 1
        self.graph.replay()

    def last_rounds(self, n: int):
        """Verdicts of the last n <= history replays, oldest first: (emit [n, lanes, depth + 1], n_emit [n, lanes]) on
        the host.  Synchronises."""
        assert 0 < n <= self.history
        done = int(self.rounds)
        idx = torch.tensor([(done - n + i) % self.history for i in range(n)], device="cuda")
        return self.hist_emit[idx].cpu(), self.hist_n[idx].cpu()

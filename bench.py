#!/usr/bin/env python3
"""Decode-step benchmark: tok/s of the full Qwen3.5-0.8B text-tower decode step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--lanes L] [--impl reference]

Workload (one "step" = one greedy decode step over every lane of a GPU): random-init weights
(seed 0), `lanes` independent requests per GPU, each prefilled with `--prompt` uniform-random
token ids through the engine's own prefill, then K chained greedy steps with the device argmax
over the 248,320-row tied head.  Lanes are data-parallel: with N GPUs every rank runs the same
`lanes` on its own GPU (weak scaling, no collective on the step).

Reported on ONE JSON line by rank 0:
  value      whole-job tok/s, tokens resident on the device, K steps as CUDA-graph replays,
             timed with CUDA events between barrier + synchronize, max over ranks;
  e2e        the same steps through the host-buffer call (pinned host token ids -> H2D -> step ->
             D2H -> synchronise), every step;
  roofline   the dominant kernel family of the step (by CUDA-event time over K eager steps run
             right after the timed region): algorithmic bytes per launch / mean launch time vs
             the measured HBM copy bandwidth;
  cpu_baseline  the reference's own torch path (or, where it is not staged, the oracle port) on
             the host cores, on a bounded sample (N = 1 only);
  lanes_sweep   the same measurement at the other lane counts the metric is quoted on;
  strong     the benchmark's fixed totals (4,032 and 128 lanes) split evenly over the N GPUs;
  slices     per-shape projection figures and the GatedDeltaNet recurrence in isolation
             (the two kernel-level configurations of the benchmark), N = 1 only;
  mtp        speculative rounds (draft + verify), reject path and forced-accept path.
`--impl reference` times the CPU path alone in the same format.
`--only-slice gdn:LANES | chunk:LANES | head:ROWS | gemv:ROWS` runs a few launches of one kernel and exits (the small
cases the profiler captures of those kernels use).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))
from __graft_entry__ import load_package  # noqa: E402

METRIC = "decode_tok_per_s"
FALLBACK_HBM_GBS = 6650.0
# per (lane, GDN layer) algorithmic bytes of the GDN step kernel: state read + write (2 x 1 MiB),
# conv window 3 rows read + 1 written in the reference's f32 layout, raw qkv row, z row, output row
GDN_BYTES_PER_LANE_LAYER = 2 * 1048576 + 98304 + 12288 + 4096 + 4096
# dram__bytes_read.sum + dram__bytes_write.sum of one gdn_step_kernel launch divided by its lanes, from a
# profiler capture of `--only-slice gdn:1024` (state stores of 1 GiB per launch, 8 x the L2, so that nothing
# of a launch stays behind in the cache); traffic grows in proportion to the lanes.  None = not captured.
GDN_NCU_TRAFFIC_PER_LANE = 2.1366e6      # 1,130.1 MB read + 1,057.0 MB written per launch of 1,024 lanes (mean of 3 launches)
# the 13 projection shapes of the benchmark's projection slice: (name, N, K, epilogue)
PROJ_SHAPES = [("in_proj_qkv", 6144, 1024, 0), ("in_proj_z", 2048, 1024, 0), ("in_proj_a", 16, 1024, 0),
               ("in_proj_b", 16, 1024, 0), ("out_proj", 1024, 2048, 0), ("q_proj", 4096, 1024, 0),
               ("k_proj", 512, 1024, 0), ("v_proj", 512, 1024, 0), ("o_proj", 1024, 2048, 0),
               ("gate_up", 7168, 1024, 1), ("down", 1024, 3584, 0), ("lm_head_argmax", 248320, 1024, 2)]
PROJ_ROWS = [1, 8, 32, 128, 512, 4032]


def peaks():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return FALLBACK_HBM_GBS, "fallback (6650 GB/s, earlier measurement on this pool)"


def tensor_peaks():
    """(burst, sustained) dense bf16 TFLOP/s: measured on this pool, else the earlier measurement."""
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["bf16_tflops"]), float(d["bf16_tflops_sustained"]), "measured"
    return 1590.0, 1400.0, "fallback"


def live_copy_gbs() -> float:
    """STREAM-style copy bandwidth of THIS GPU, measured the way MEASURED_PEAKS.json's figure was
    (b.copy_(a) over 1 Gi bf16 elements, read + write bytes, best of 5, CUDA events).  Reported beside
    the roofline so that GPU-to-GPU spread in the pool can be told from a change in the kernels."""
    n = 1 << 30
    a = torch.empty(n, dtype=torch.bfloat16, device="cuda").fill_(1.0)
    b = torch.empty_like(a)
    best = 0.0
    for _ in range(6):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        b.copy_(a)
        e1.record()
        torch.cuda.synchronize()
        best = max(best, 4.0 * n / (e0.elapsed_time(e1) * 1e-3) / 1e9)
    del a, b
    return round(best, 1)


class ClockSampler:
    """nvidia-smi clocks / throttle reasons of one GPU, sampled every 100 ms while running."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc = index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def measure(pkg, eng, lanes: int, prompt: int, steps: int, warmup: int, dist, sampler=None) -> dict:
    """Prefill `lanes` lanes, then time `steps` decode steps three ways (graph, host-buffer, eager+events)."""
    import torch.distributed as td
    ctx_cap = prompt + 3 * (steps + warmup) + 16
    st = eng.allocate_state(lanes, ctx_cap)
    gen = torch.Generator().manual_seed(1000 + lanes)
    ids = torch.randint(0, eng.vocab, (lanes, prompt), generator=gen, dtype=torch.int32).cuda()
    t0 = time.time()
    y0, _ = eng.prefill(st, ids)
    torch.cuda.synchronize()
    prefill_s = time.time() - t0

    def barrier():
        if dist:
            td.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        ms = torch.tensor([a.elapsed_time(b)], device="cuda")
        if dist:
            td.all_reduce(ms, op=td.ReduceOp.MAX)
        return float(ms.item())

    # ---- device-resident: graph of 2 chained steps, replayed ------------------------------------
    eng.decode_step(st, y0)                         # eager warm-up (also sets kernel attributes)
    g2 = pkg.StepGraph(eng, st, steps=2)
    g2.tok_in.copy_(y0)
    for _ in range((warmup + 1) // 2):
        g2.replay()
    if sampler:
        sampler.start()
    k2 = (steps + 1) // 2
    ms_dev = timed(g2.replay, k2)
    clocks = sampler.stop() if sampler else None
    steps_dev = 2 * k2
    ctx_mid = prompt + 1 + 2 * ((warmup + 1) // 2) + steps_dev / 2.0

    # ---- end to end: host token ids in, host token ids out, every step ---------------------------
    g1 = pkg.StepGraph(eng, st, steps=1)
    h_in = torch.empty(lanes, dtype=torch.int32).pin_memory()
    h_out = torch.empty(lanes, dtype=torch.int32).pin_memory()
    h_in.copy_(g2.tok_out.cpu())

    def host_step():
        eng.decode_step_host(st, h_in, h_out, graph=g1)
        h_in.copy_(h_out)

    for _ in range(max(warmup, 3)):
        host_step()
    ms_e2e = timed(host_step, steps)

    # ---- eager steps with per-family CUDA events (roofline of the dominant kernel) ---------------
    cur = g1.tok_out.clone()
    eng.profile_begin()
    for _ in range(steps):
        cur = eng.decode_step(st, cur)
    fam = eng.profile_end()
    torch.cuda.synchronize()
    # a kernel whose bounded wait ran out makes every later kernel return at once: such a run is
    # fast and wrong, so it is no measurement
    status = eng.status()
    if status != 0:
        raise RuntimeError(f"device status word is {status} after the timed steps at {lanes} lanes: "
                           "a kernel gave up a bounded wait; no number is reported")
    st.close()
    total_ms = sum(v[0] for v in fam.values()) or 1.0
    return dict(lanes=lanes, ms_dev=ms_dev, steps_dev=steps_dev, ms_e2e=ms_e2e, steps_e2e=steps,
                kernels_per_step=g2.kernels_per_replay // 2, kernels_timed=g2.kernels_per_replay * k2,
                families={k: {"ms_per_step": v[0] / steps, "launches_per_step": v[1] / steps,
                              "share": v[0] / total_ms} for k, v in fam.items()},
                ctx_mid=ctx_mid, prefill_s=prefill_s, clocks=clocks, last_tokens=cur.clone())


def measure_mtp(pkg, eng, lanes: int = 16, prompt: int = 1024, rounds: int = 64, warmup: int = 3, depth: int = 1,
                forced: bool = False) -> dict:
    """Chunk-64 prefill of `lanes` x `prompt` ids, then `rounds` speculative rounds (`depth` chained MTP
    drafts, verify of depth + 1 tokens), tokens chained on the device, one replayed CUDA graph per round.
    On random-init weights the draft almost never matches the target, so the plain run times the REJECT
    branch (one token per lane per round).  forced=True times the ACCEPT branch: the lanes' true
    continuations are first collected with rejecting rounds (the same verify kernels produce them), then
    fresh lanes replay rounds whose candidates are those tokens, so every round accepts all of them."""
    gen = torch.Generator().manual_seed(4000)
    ids = torch.randint(0, eng.vocab, (lanes, prompt), generator=gen, dtype=torch.int32).cuda()
    total = rounds + warmup
    forced_tokens = None
    if forced:
        need = (depth + 1) * total + depth + 1            # tokens after the seed that the forced rounds consume
        # rounds of the SAME depth: their bodies have the same row count, so the projections split and sum
        # exactly as in the timed rounds and the tokens are bit-for-bit the ones those rounds will compute
        st0 = eng.allocate_state(lanes, prompt + (depth + 1) * need + 8)
        m0 = eng.mtp_allocate(st0, depth * need + 8, depth=depth)
        t, h = eng.prefill(st0, ids, want_normed=True)
        g0 = pkg.MtpRoundGraph(eng, st0, m0, depth=depth, history=need)
        g0.tok.copy_(t)
        g0.h.copy_(h)
        for _ in range(need):
            g0.replay()
        em, ne = g0.last_rounds(need)                       # [need, lanes, depth + 1], [need, lanes]
        seq = [[] for _ in range(lanes)]
        for r in range(need):
            for i in range(lanes):
                seq[i].extend(em[r, i, :int(ne[r, i])].tolist())
        forced_tokens = torch.tensor([s_[:need] for s_ in seq], dtype=torch.int32, device="cuda")
        m0.close()
        st0.close()
    st = eng.allocate_state(lanes, prompt + (depth + 1) * total + 8)
    m = eng.mtp_allocate(st, depth * total + 8, depth=depth)
    torch.cuda.synchronize()
    t0 = time.time()
    t, h = eng.prefill(st, ids, want_normed=True)
    torch.cuda.synchronize()
    prefill_s = time.time() - t0
    # one captured round (drafts + verify + verdict + hand-over), replayed: nothing crosses the host between rounds
    g = pkg.MtpRoundGraph(eng, st, m, depth=depth, forced_tokens=forced_tokens)
    g.tok.copy_(t)
    g.h.copy_(h)
    for _ in range(warmup):
        g.replay()
    g.emitted_total.zero_()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(rounds):
        g.replay()                      # the graph tallies its emitted tokens on the device
    b.record()
    torch.cuda.synchronize()
    emitted = g.emitted_total
    ms = a.elapsed_time(b)
    n = int(emitted.item())
    if eng.status() != 0:
        raise RuntimeError("device status word raised during the MTP rounds: no number is reported")
    m.close()
    st.close()
    return {"workload": f"configs[4]: {lanes} lanes x {prompt}-token chunk-64 prefill, {rounds} rounds of {depth} chained MTP "
                        f"draft(s) + {depth + 1}-token verify" + (", candidates = the target's own next tokens (accept branch)" if forced else ""),
            "accepted_tok_per_s": round(n / (ms * 1e-3), 1), "accept_rate": round((n - rounds * lanes) / (rounds * lanes * depth), 4),
            "ms_per_round": round(ms / rounds, 4), "prefill_tok_per_s": round(lanes * prompt / prefill_s, 1)}


def timed_launches(fn, n: int) -> float:
    """Mean microseconds per launch of n calls fn(i) captured into ONE CUDA graph and replayed (best of 3
    replays, CUDA events around a replay): the host's launch rate stays out of the figure."""
    fn(0)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(n):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(3):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b) * 1e3 / n)
    del g
    return best


def projection_slices(eng, rows_list=PROJ_ROWS) -> list:
    """The benchmark's projection slice: every shape x row count through the single-stage entry points.
    Each timed launch reads a DIFFERENT copy of the weight matrix from a pool larger than the L2 (so the
    figure is an HBM figure, not a cache figure), back to back between one event pair; the two 16-row
    shapes are too small for that and are marked cache-resident.  bytes = 2NK + 2LK + 2LN, flops = 2LNK."""
    hbm, _ = peaks()
    burst, sustained, _ = tensor_peaks()
    out = []
    gen = torch.Generator(device="cuda").manual_seed(11)
    for name, N, K, epi in PROJ_SHAPES:
        wbytes = 2 * N * K
        if epi == 2:
            pool = [eng.embed]                      # 508 MB: larger than the L2 by itself
        else:
            copies = max(2, min(96, -(-300_000_000 // wbytes)))
            pool = [(torch.randn((N, K), device="cuda", generator=gen) * 0.02).to(torch.bfloat16) for _ in range(copies)]
        for L in rows_list:
            x = torch.randn((L, K), device="cuda", generator=gen).to(torch.bfloat16)
            n = max(len(pool), 4) if epi != 2 else 4
            if epi == 0 and N == 1024:
                # the engine's own stage for these two shapes: projection + residual add + norm of the next block
                resid = torch.randn((L, 1024), device="cuda", generator=gen).to(torch.bfloat16)
                nw = torch.ones(1024, device="cuda", dtype=torch.bfloat16)
                fn = lambda i: eng.op_proj_residual(x, pool[i % len(pool)], resid, nw)
            elif epi == 0:
                fn = lambda i: eng.op_linear(x, pool[i % len(pool)])
            elif epi == 1:
                fn = lambda i: eng.op_mlp_gateup(x, pool[i % len(pool)])
            else:
                fn = lambda i: eng.op_lm_head(x)
            us = timed_launches(fn, n)
            nbytes = wbytes + 2 * L * K + 2 * L * (N // 2 if epi == 1 else N) * (0 if epi == 2 else 1) + (4 * L if epi == 2 else 0)
            flops = 2.0 * L * N * K
            rec = {"shape": name, "N": N, "K": K, "rows": L, "us": round(us, 2),
                   "gbs": round(nbytes / us / 1e3, 1), "frac_hbm": round(nbytes / us / 1e3 / hbm, 4),
                   "tflops": round(flops / us / 1e6, 2), "frac_tensor_sustained": round(flops / us / 1e6 / sustained, 4),
                   "frac_tensor_burst": round(flops / us / 1e6 / burst, 4),
                   "kernel": eng.op_linear_route(L, N, K, epi) if not (epi == 0 and N == 1024) else eng.op_proj_residual_route(L, K)}
            if epi == 0 and N == 1024:
                rec["stage"] = "projection + residual add (+ RMSNorm kernel above 16 rows)"
            if len(pool) * wbytes < 200_000_000 and epi != 2:
                rec["note"] = "weights stay in L2 between launches: not an HBM figure"
            out.append(rec)
            del x
        del pool
        torch.cuda.empty_cache()
    return out


def gdn_inputs(eng, L: int, nbuf: int, gen):
    """Inputs of the recurrence slice in the benchmark's distributions: state N(0, 0.1) f32, raw q|k|v|z|b|a rows
    N(0, 1) bf16, conv window N(0, 1), one layer's own weights."""
    P = {"conv": (torch.randn((6144, 4), device="cuda", generator=gen) * 0.1).to(torch.bfloat16),
         "A_log": torch.log(1 + 15 * torch.rand(16, device="cuda", generator=gen)).to(torch.bfloat16),
         "dt_bias": (-4 + 2 * torch.rand(16, device="cuda", generator=gen)).to(torch.bfloat16),
         "norm": torch.ones(128, device="cuda", dtype=torch.bfloat16)}
    bufs = []
    for _ in range(nbuf):
        S = torch.randn((L, 16, 128, 128), device="cuda", generator=gen) * 0.1
        win = torch.randn((L, 3, 6144), device="cuda", generator=gen).to(torch.bfloat16)
        proj = torch.randn((L, 8224), device="cuda", generator=gen).to(torch.bfloat16)
        bufs.append((S, win, proj))
    return P, bufs


def gdn_slices(eng, lanes_list=(1, 128, 4032)) -> list:
    """The benchmark's recurrence slice: conv roll + gates + delta rule + gated norm of ONE layer per launch,
    over `nbuf` distinct (state, window, projection row) sets so that consecutive launches never reuse cached
    state (18 = the model's GDN layers where that is already larger than the L2; more at 1 lane, fewer at 4,032
    to bound memory)."""
    hbm, _ = peaks()
    gen = torch.Generator(device="cuda").manual_seed(12)
    out = []
    for L in lanes_list:
        per = L * GDN_BYTES_PER_LANE_LAYER
        nbuf = max(4, min(600, -(-600_000_000 // per)))
        if L * 18 * 1.05e6 > 600e6:
            nbuf = 18 if L * 18 * 1.06e6 < 30e9 else 4
        P, bufs = gdn_inputs(eng, L, nbuf, gen)
        fn = lambda i: eng.op_gdn_step(bufs[i % nbuf][2], P["conv"], P["A_log"], P["dt_bias"], P["norm"],
                                       bufs[i % nbuf][0], bufs[i % nbuf][1], L, 1)
        us = timed_launches(fn, max(nbuf, 8))
        out.append({"lanes": L, "layers_per_launch": 1, "state_sets": nbuf, "us_per_launch": round(us, 2),
                    "bytes_per_launch": per, "gbs": round(per / us / 1e3, 1), "frac_hbm": round(per / us / 1e3 / hbm, 4),
                    "us_per_18_layers": round(18 * us, 1), "kernel": "gdn_step_kernel"})
        del bufs
        torch.cuda.empty_cache()
    return out


def roofline_of(eng, m: dict) -> dict:
    peak, how = peaks()
    fam = m["families"]
    top = max(fam, key=lambda k: fam[k]["ms_per_step"])
    lanes = m["lanes"]
    c = eng.census()
    per_launch_ms = fam[top]["ms_per_step"] / max(fam[top]["launches_per_step"], 1)
    if top == "gdn":
        nbytes = lanes * GDN_BYTES_PER_LANE_LAYER
        kernel = "gdn_step_kernel"
        traffic = GDN_NCU_TRAFFIC_PER_LANE * lanes if GDN_NCU_TRAFFIC_PER_LANE else None
    elif top == "head":
        nbytes = 2 * eng.vocab * 1024 + lanes * 2048
        kernel = "lm_head projection + argmax"
        per_launch_ms = fam[top]["ms_per_step"]          # two launches form one pass over the table
        traffic = None
    else:
        nbytes = {"in_proj": (18 * 8224 + 6 * 5120) * 1024 * 2 / 24, "out_proj": 1024 * 2048 * 2,
                  "mlp_gateup": 7168 * 1024 * 2, "mlp_down": 1024 * 3584 * 2,
                  "attn": lanes * 2048 * (m["ctx_mid"] + 1), "glue": lanes * 1024 * 2 * 4}[top]
        kernel = top
        traffic = None
    achieved = nbytes / (per_launch_ms * 1e-3) / 1e9
    step_bytes = eng.step_bytes(lanes, m["ctx_mid"])
    ms_step = m["ms_dev"] / m["steps_dev"]
    return {"bound": "hbm", "kernel": kernel, "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
            "frac": round(achieved / peak, 4), "traffic": traffic, "peak_source": how,
            "bytes_per_launch": int(nbytes), "ms_per_launch": round(per_launch_ms, 5),
            "traffic_how": ("dram__bytes_read.sum + dram__bytes_write.sum of a profiler capture of this kernel at 1,024 lanes, "
                            "per lane x the lanes of a launch") if traffic else "not captured",
            "how": "CUDA events around every launch of the family over K eager steps run right after the timed region",
            "step": {"algorithmic_bytes": int(step_bytes), "ms": round(ms_step, 5),
                     "achieved_gbs": round(step_bytes / (ms_step * 1e-3) / 1e9, 1),
                     "frac_of_hbm_roofline": round(step_bytes / (ms_step * 1e-3) / 1e9 / peak, 4)},
            "family_ms_per_step": {k: round(v["ms_per_step"], 5) for k, v in fam.items()}}


def cpu_reference(steps: int, warmup: int, lanes_sample: int, prompt: int, P=None) -> dict:
    """The reference's CPU path on all host threads: `lanes_sample` lanes prefilled with `prompt` ids
    (chunk-64 form), then `steps` greedy steps per lane.  Runs the reference's own modules where
    oracle/make_ref.py staged them (kind "reference"), else the oracle port of the same torch code."""
    from oracle import make_ref
    from oracle import q35_oracle as O
    pkg = load_package()
    torch.set_grad_enabled(False)
    # a launcher may pin the process to one thread (torch.distributed.run exports OMP_NUM_THREADS=1)
    torch.set_num_threads(max(os.cpu_count() or 1, 1))
    if P is None:
        P = pkg.weights.make_weights(seed=0)
    cores = torch.get_num_threads()
    gen = torch.Generator().manual_seed(2000)
    mods = make_ref.load()
    lanes = []
    for _ in range(lanes_sample):
        ids = torch.randint(0, 248320, (prompt,), generator=gen)
        if mods is not None:
            f = make_ref.make_forward(mods[0], P, gdn_form="chunk")
            n = f.prefill(ids)
            lanes.append([f, int(f.logits(n)[-1].argmax())])
        else:
            ln = O.Lane(P, gdn_prefill="chunk")
            n = ln.forward(ids)
            lanes.append([ln, int(ln.logits(n)[-1].argmax())])

    def step():
        for rec in lanes:
            if mods is not None:
                rec[1] = int(rec[0].logits(rec[0].decode(rec[1]))[-1].argmax())
            else:
                rec[1] = int(rec[0].logits(rec[0].forward([rec[1]]))[-1].argmax())

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    return {"value": lanes_sample * steps / dt, "unit": "tok/s", "cores": cores,
            "kind": "reference" if mods is not None else "port",
            "ms_per_step": dt / steps * 1e3,
            "sample": f"{lanes_sample} lane(s), {prompt}-token chunked prefill, {steps} greedy steps each, torch CPU bf16, "
                      + ("the reference's speccheck.specimpl.Forward" if mods is not None else "oracle port of the reference's torch path")}


def strong_split(pkg, eng, totals, prompt: int, steps: int, warmup: int, world: int, rank: int) -> list:
    """The benchmark's fixed totals split evenly over the ranks (strong scaling): every rank runs its block of
    lanes (parallel.shard_lanes), barrier + max-over-ranks timing of graph-replayed steps, no collective on the
    step.  Reports, per total, whole-job tok/s and the step's HBM-roofline fraction at the per-GPU lane count."""
    import torch.distributed as td
    peak, _ = peaks()
    out = []
    for total in totals:
        first, mine = pkg.parallel.shard_lanes(total, world, rank)
        st = eng.allocate_state(mine, prompt + 3 * (steps + warmup) + 16)
        ids = torch.randint(0, eng.vocab, (mine, prompt), generator=torch.Generator().manual_seed(3000 + first), dtype=torch.int32).cuda()
        y0, _ = eng.prefill(st, ids)
        eng.decode_step(st, y0)
        g = pkg.StepGraph(eng, st, steps=2)
        g.tok_in.copy_(y0)
        for _ in range((warmup + 1) // 2):
            g.replay()
        k2 = (steps + 1) // 2
        td.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(k2):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        ms = torch.tensor([a.elapsed_time(b)], device="cuda")
        td.all_reduce(ms, op=td.ReduceOp.MAX)
        ms_step = float(ms.item()) / (2 * k2)
        ctx = prompt + 1 + 2 * ((warmup + 1) // 2) + k2
        nbytes = eng.step_bytes(mine, ctx)
        if eng.status() != 0:
            raise RuntimeError("device status word raised during the strong-split steps")
        gathered = pkg.parallel.gather_tokens(g.tok_out.clone(), total)
        out.append({"total_lanes": total, "lanes_per_gpu": mine, "n_gpus": world, "ms_per_step": round(ms_step, 5),
                    "tok_per_s": round(total / (ms_step * 1e-3), 1),
                    "frac_of_hbm_roofline_per_gpu": round(nbytes / (ms_step * 1e-3) / 1e9 / peak, 4),
                    "gathered_token_ids": int(gathered.numel()) if gathered is not None else None})
        st.close()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--lanes", type=int, default=4032, help="lanes per GPU of the headline measurement")
    ap.add_argument("--sweep", default="1,16,128", help="extra lane counts measured on rank 0's GPU")
    ap.add_argument("--strong", default="4032,128", help="total lane counts split evenly over the GPUs (N > 1)")
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-mtp", action="store_true", help="skip the MTP (configs[4]) section")
    ap.add_argument("--no-slices", action="store_true", help="skip the projection / recurrence slices (configs[1], configs[2])")
    ap.add_argument("--only-slice", default="", help="gdn:LANES | chunk:LANES | head:ROWS | gemv:ROWS - a few launches of one kernel, then exit (profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    workload = (f"configs[3]: full decode step, {args.lanes} lanes per GPU, each prefilled with "
                f"{args.prompt} uniform-random ids, greedy argmax over 248320")
    config = {"workload": workload, "lanes_per_gpu": args.lanes, "prompt_tokens": args.prompt,
              "l2": "inputs larger than L2 (weights 1.5 GB + per-lane state 18.9 MB stream every step)",
              "parallelism": f"dp{world} (lanes data-parallel, weights replicated, no collective)"}

    if args.impl == "reference":
        if rank != 0:
            return
        r = cpu_reference(min(args.steps, 16), min(args.warmup, 3), 2, args.prompt)
        print(json.dumps({"metric": METRIC, "value": r["value"], "unit": "tok/s", "n_gpus": args.gpus,
                          "steps": min(args.steps, 16), "warmup": min(args.warmup, 3),
                          "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                          "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
                          "impl": "reference", "cpu_baseline": r,
                          "e2e": {"value": r["value"], "unit": "tok/s", "h2d_bytes_per_step": 0,
                                  "d2h_bytes_per_step": 0}}))
        return

    torch.set_grad_enabled(False)
    torch.cuda.set_device(local)
    pkg = load_package()
    pkg.build_lib.build()

    if args.only_slice:
        # small cases for a profiler capture of ONE kernel: a few launches, each on its own operands, then exit
        kind, n_s = args.only_slice.split(":")
        n = int(n_s)
        gen = torch.Generator(device="cuda").manual_seed(12)
        if kind == "head":
            eng = pkg.Engine(pkg.weights.make_weights(seed=0), max_rows=max(n, 64), mtp=False)
            x = torch.randn((n, 1024), device="cuda", generator=gen).to(torch.bfloat16)
            for _ in range(3):
                eng.op_lm_head(x)
            nbytes = 2 * eng.vocab * 1024
        else:
            eng = pkg.Engine(pkg.weights.make_weights(seed=0, vocab=16384), max_rows=max(n, 64), vocab=16384, mtp=False)
            if kind == "gdn":
                P, bufs = gdn_inputs(eng, n, 3, gen)
                for S, win, proj in bufs:
                    eng.op_gdn_step(proj, P["conv"], P["A_log"], P["dt_bias"], P["norm"], S, win, n, 1)
                nbytes = n * GDN_BYTES_PER_LANE_LAYER
            elif kind == "chunk":
                # the chunk-64 prefill scan: n lanes x 64 tokens of one GDN layer (conv pass + scan kernel per launch)
                P, bufs = gdn_inputs(eng, n, 1, gen)
                S, win, _ = bufs[0]
                for _ in range(3):
                    proj = torch.randn((n * 64, 8224), device="cuda", generator=gen).to(torch.bfloat16)
                    eng.op_gdn_step(proj, P["conv"], P["A_log"], P["dt_bias"], P["norm"], S, win, n, 64)
                nbytes = n * (2 * 1048576 + 64 * 4 * 256 + 64 * 256)
            elif kind == "gemv":
                # the GDN in-projection shape (8,224 x 1,024) at n <= 16 rows: the weight-streaming kernel
                assert n <= 16
                x = torch.randn((n, 1024), device="cuda", generator=gen).to(torch.bfloat16)
                pool = [(torch.randn((8224, 1024), device="cuda", generator=gen) * 0.02).to(torch.bfloat16) for _ in range(24)]
                for W in pool:
                    eng.op_linear(x, W)
                nbytes = 2 * 8224 * 1024
            else:
                raise SystemExit(f"unknown slice {kind}")
        torch.cuda.synchronize()
        assert eng.status() == 0
        print(json.dumps({"only_slice": kind, "rows_or_lanes": n, "bytes_per_launch": nbytes}))
        return

    dist = world > 1
    if dist:
        import torch.distributed as td
        # stdout carries exactly one JSON line: NCCL's own banner ("NCCL version ...") goes to stderr.  NCCL
        # honours NCCL_DEBUG_FILE only above the VERSION level, so that level is raised to WARN.
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        td.init_process_group("nccl", device_id=torch.device("cuda", local))
    # this GPU's own copy bandwidth, taken first, on an idle GPU, the way MEASURED_PEAKS.json's figure was
    copy_gbs = live_copy_gbs() if rank == 0 else 0.0
    params = pkg.weights.make_weights(seed=0)
    # scratch rows: 64 prompt tokens per lane per prefill body (the chunk-64 GDN scan), capped at 256 Ki rows
    rows = max(min(64 * args.lanes, 262144), 2 * args.lanes, 1024)
    eng = pkg.Engine(params, max_rows=rows)
    sampler = ClockSampler(local) if rank == 0 else None
    m = measure(pkg, eng, args.lanes, args.prompt, args.steps, args.warmup, dist, sampler)
    # the one exchange of the data-parallel layout: sampled ids of every lane, in lane order, on rank 0
    gathered = pkg.parallel.gather_tokens(m["last_tokens"], world * args.lanes) if dist else m["last_tokens"]
    ms_step = m["ms_dev"] / m["steps_dev"]
    value = world * args.lanes * m["steps_dev"] / (m["ms_dev"] * 1e-3)
    e2e = world * args.lanes * m["steps_e2e"] / (m["ms_e2e"] * 1e-3)
    out = {"metric": METRIC, "value": round(value, 1), "unit": "tok/s", "n_gpus": world, "steps": m["steps_dev"],
           "warmup": args.warmup, "ms_per_step": round(ms_step, 5), "higher_is_better": True,
           "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
           "e2e": {"value": round(e2e, 1), "unit": "tok/s", "h2d_bytes_per_step": 4 * args.lanes,
                   "d2h_bytes_per_step": 4 * args.lanes, "ms_per_step": round(m["ms_e2e"] / m["steps_e2e"], 5)},
           # kernels of this library inside the timed region of `value`, per GPU: counted by the engine while the
           # replayed graph was captured (q35_engine_launch_count) x the replays
           "gpu_launches": int(m["kernels_timed"]), "gpu_launches_per_step": int(m["kernels_per_step"]),
           "clocks": m["clocks"], "roofline": roofline_of(eng, m), "prefill_s": round(m["prefill_s"], 2),
           "prefill_tok_per_s": round(args.lanes * args.prompt / m["prefill_s"], 1)}
    if rank == 0:
        out["roofline"]["copy_gbs_this_gpu"] = copy_gbs
        out["roofline"]["frac_of_this_gpu"] = round(out["roofline"]["achieved"] / copy_gbs, 4)
    strong = None
    if dist and args.strong:
        strong = strong_split(pkg, eng, [int(x) for x in args.strong.split(",") if x], args.prompt, args.steps,
                              args.warmup, world, rank)
    sweep = []
    if rank == 0 and args.sweep:
        for L in [int(x) for x in args.sweep.split(",") if x]:
            if L == args.lanes:
                continue
            ms = measure(pkg, eng, L, args.prompt, args.steps, args.warmup, False)
            rf = roofline_of(eng, ms)
            step_ms = ms["ms_dev"] / ms["steps_dev"]
            rec = {"lanes": L, "tok_per_s": round(L * ms["steps_dev"] / (ms["ms_dev"] * 1e-3), 1),
                   "ms_per_step": round(step_ms, 5),
                   "e2e_tok_per_s": round(L * ms["steps_e2e"] / (ms["ms_e2e"] * 1e-3), 1),
                   "frac_of_hbm_roofline": rf["step"]["frac_of_hbm_roofline"],
                   "kernels_per_step": int(ms["kernels_per_step"]),
                   "us_per_kernel_in_graph": round(step_ms * 1e3 / max(ms["kernels_per_step"], 1), 2),
                   "family_ms_per_step_eager": rf["family_ms_per_step"]}
            if L > 16:          # below that the step is a chain of dependent short kernels: no family has a bandwidth figure
                rec["top_kernel"], rec["top_kernel_frac"] = rf["kernel"], rf["frac"]
            sweep.append(rec)
    if strong is None and rank == 0:
        # one GPU: the strong split of the totals IS the headline / sweep measurement of the same lane count
        strong = []
        for total in [int(x) for x in args.strong.split(",") if x]:
            if total == args.lanes:
                strong.append({"total_lanes": total, "lanes_per_gpu": total, "n_gpus": 1, "ms_per_step": round(ms_step, 5),
                               "tok_per_s": round(value, 1),
                               "frac_of_hbm_roofline_per_gpu": out["roofline"]["step"]["frac_of_hbm_roofline"]})
            for rec in sweep:
                if rec["lanes"] == total:
                    strong.append({"total_lanes": total, "lanes_per_gpu": total, "n_gpus": 1, "ms_per_step": rec["ms_per_step"],
                                   "tok_per_s": rec["tok_per_s"], "frac_of_hbm_roofline_per_gpu": rec["frac_of_hbm_roofline"]})
    mtp = None
    if rank == 0 and not args.no_mtp and eng.has_mtp:
        mtp = measure_mtp(pkg, eng)
        mtp["depth2"] = measure_mtp(pkg, eng, depth=2)      # the reference's default round width
        mtp["forced_accept"] = measure_mtp(pkg, eng, forced=True)
        mtp["forced_accept_depth2"] = measure_mtp(pkg, eng, depth=2, forced=True)
        plain16 = [r for r in sweep if r["lanes"] == 16]
        if plain16:
            mtp["plain_decode_tok_per_s_same_lanes"] = plain16[0]["tok_per_s"]
    slices = None
    if rank == 0 and world == 1 and not args.no_slices:
        slices = {"projection": projection_slices(eng), "gdn_recurrence": gdn_slices(eng),
                  "how": "every launch on its own copy of the weights / state from a pool larger than the L2, all launches of a "
                         "case in one replayed CUDA graph, CUDA events around the replay; peaks: measured HBM copy and bf16 GEMM"}
        if eng.status() != 0:
            raise RuntimeError("device status word raised during the slices")
    if dist:
        import torch.distributed as td
        td.barrier()
    if rank == 0:
        out["lanes_sweep"] = sweep
        out["strong"] = strong
        out["mtp"] = mtp
        out["slices"] = slices
        out["gathered_token_ids"] = int(gathered.numel())
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"] = cpu_reference(12, 1, 1, args.prompt, params)
        print(json.dumps(out))
    eng.close()
    if dist:
        import torch.distributed as td
        td.destroy_process_group()


if __name__ == "__main__":
    main()

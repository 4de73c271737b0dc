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
  cpu_baseline  the CPU oracle (a port of the reference's torch path) on the host cores, on a
             bounded sample (N = 1 only);
  lanes_sweep   the same measurement at the other lane counts the metric is quoted on.
`--impl reference` times the CPU path alone in the same format.
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
# dram__bytes_read.sum + dram__bytes_write.sum per launch of gdn_step_kernel, from the ncu capture
# summarised in profiles/ (per lane; scaled by the lanes of a launch).  None until captured.
GDN_NCU_TRAFFIC_PER_LANE = 1.968e6      # dram read + write per lane per launch, ncu capture at 256 lanes (profiles/gdn_step_kernel_256_lanes.md); grows in proportion to lanes


def peaks():
    p = REPO / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return FALLBACK_HBM_GBS, "fallback (6650 GB/s, earlier measurement on this pool)"


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
                families={k: {"ms_per_step": v[0] / steps, "launches_per_step": v[1] / steps,
                              "share": v[0] / total_ms} for k, v in fam.items()},
                ctx_mid=ctx_mid, prefill_s=prefill_s, clocks=clocks, last_tokens=cur.clone())


def measure_mtp(pkg, eng, lanes: int = 16, prompt: int = 1024, rounds: int = 64, warmup: int = 3, depth: int = 1) -> dict:
    """Chunk-64 prefill of `lanes` x `prompt` ids, then `rounds` speculative rounds (`depth` chained MTP
    drafts, verify of depth + 1 tokens), tokens chained on the device.  On random-init weights the
    draft almost never matches the target, so accepted tok/s is about one token per lane per round."""
    st = eng.allocate_state(lanes, prompt + (depth + 1) * (rounds + warmup) + 8)
    m = eng.mtp_allocate(st, depth * (rounds + warmup) + 8, depth=depth)
    gen = torch.Generator().manual_seed(4000)
    ids = torch.randint(0, eng.vocab, (lanes, prompt), generator=gen, dtype=torch.int32).cuda()
    torch.cuda.synchronize()
    t0 = time.time()
    t, h = eng.prefill(st, ids, want_normed=True)
    torch.cuda.synchronize()
    prefill_s = time.time() - t0
    # one captured round (drafts + verify + verdict + hand-over), replayed: nothing crosses the host between rounds
    g = pkg.MtpRoundGraph(eng, st, m, depth=depth)
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
                        f"draft(s) + {depth + 1}-token verify",
            "accepted_tok_per_s": round(n / (ms * 1e-3), 1), "accept_rate": round((n - rounds * lanes) / (rounds * lanes * depth), 4),
            "ms_per_round": round(ms / rounds, 4), "prefill_tok_per_s": round(lanes * prompt / prefill_s, 1)}


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
    elif top == "step_kernel":
        nbytes = eng.step_bytes(lanes, m["ctx_mid"])
        kernel = "small_step_kernel (whole step, persistent)"
        traffic = None
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
            "how": "CUDA events around every launch of the family over K eager steps run right after the timed region",
            "step": {"algorithmic_bytes": int(step_bytes), "ms": round(ms_step, 5),
                     "achieved_gbs": round(step_bytes / (ms_step * 1e-3) / 1e9, 1),
                     "frac_of_hbm_roofline": round(step_bytes / (ms_step * 1e-3) / 1e9 / peak, 4)},
            "family_ms_per_step": {k: round(v["ms_per_step"], 5) for k, v in fam.items()}}


def cpu_reference(steps: int, warmup: int, lanes_sample: int, prompt: int, P=None) -> dict:
    """The CPU path (oracle port of the reference's torch implementation) on all host threads:
    `lanes_sample` lanes prefilled with `prompt` ids, then `steps` greedy steps per lane."""
    from oracle import q35_oracle as O
    pkg = load_package()
    torch.set_grad_enabled(False)
    if P is None:
        P = pkg.weights.make_weights(seed=0)
    cores = torch.get_num_threads()
    gen = torch.Generator().manual_seed(2000)
    lanes = []
    for _ in range(lanes_sample):
        ln = O.Lane(P, gdn_prefill="chunk")
        n = ln.forward(torch.randint(0, 248320, (prompt,), generator=gen))
        lanes.append([ln, int(ln.logits(n)[-1].argmax())])

    def step():
        for rec in lanes:
            rec[1] = int(rec[0].logits(rec[0].forward([rec[1]]))[-1].argmax())

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    return {"value": lanes_sample * steps / dt, "unit": "tok/s", "cores": cores, "kind": "port",
            "ms_per_step": dt / steps * 1e3,
            "sample": f"{lanes_sample} lane(s), {prompt}-token chunked prefill, {steps} greedy steps each, torch CPU bf16"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--lanes", type=int, default=4032, help="lanes per GPU of the headline measurement")
    ap.add_argument("--sweep", default="1,128", help="extra lane counts measured on rank 0's GPU size")
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-mtp", action="store_true", help="skip the MTP (configs[4]) section")
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
    dist = world > 1
    if dist:
        import torch.distributed as td
        # stdout carries exactly one JSON line: NCCL's own banner ("NCCL version ...") goes to stderr.  NCCL
        # honours NCCL_DEBUG_FILE only above the VERSION level, so that level is raised to WARN.
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        td.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = load_package()
    pkg.build_lib.build()
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
           "gpu_launches": eng.census()["launches_decode" if args.lanes > 16 else "launches_decode_few_lanes"] * m["steps_dev"],
           "clocks": m["clocks"], "roofline": roofline_of(eng, m), "prefill_s": round(m["prefill_s"], 2),
           "prefill_tok_per_s": round(args.lanes * args.prompt / m["prefill_s"], 1)}
    if rank == 0:
        out["roofline"]["copy_gbs_this_gpu"] = copy_gbs
        out["roofline"]["frac_of_this_gpu"] = round(out["roofline"]["achieved"] / copy_gbs, 4)
    sweep = []
    if rank == 0 and args.sweep:
        for L in [int(x) for x in args.sweep.split(",") if x]:
            if L == args.lanes:
                continue
            ms = measure(pkg, eng, L, args.prompt, args.steps, args.warmup, False)
            rf = roofline_of(eng, ms)
            sweep.append({"lanes": L, "tok_per_s": round(L * ms["steps_dev"] / (ms["ms_dev"] * 1e-3), 1),
                          "ms_per_step": round(ms["ms_dev"] / ms["steps_dev"], 5),
                          "e2e_tok_per_s": round(L * ms["steps_e2e"] / (ms["ms_e2e"] * 1e-3), 1),
                          "frac_of_hbm_roofline": rf["step"]["frac_of_hbm_roofline"],
                          "top_kernel": rf["kernel"], "top_kernel_frac": rf["frac"],
                          "family_ms_per_step": rf["family_ms_per_step"]})
    mtp = None
    if rank == 0 and not args.no_mtp and eng.has_mtp:
        mtp = measure_mtp(pkg, eng)
        mtp["depth2"] = measure_mtp(pkg, eng, depth=2)      # the reference's default round width
    if dist:
        import torch.distributed as td
        td.barrier()
    if rank == 0:
        out["lanes_sweep"] = sweep
        out["mtp"] = mtp
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

#!/usr/bin/env python
"""Benchmark of the quantized routed-expert layer (router top-6 -> Q8_K -> IQ2_XXS gate/up + SwiGLU -> Q8_K -> Q2_K
down -> slot sum) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

Prints ONE JSON line. A step is one pass of the layer over one batch of synthetic tokens. Inputs are synthetic with
the distributions of the benchmark configurations (f16 scales |N(0,1)|*1e-3, uniform codebook/sign/scale/quant fields,
hidden states N(0,1) rounded to bf16, router logits N(0,1)); weights are random, no dataset or checkpoint is involved.

Timing: CUDA events on the launching stream, W >= 3 warm-up steps, max over ranks. Every step uses another layer's
weights and another routing, so the packed bytes of a step are never in L2 from the step before (the rotation covers
several times the 126 MB L2). `value` is device-timed with inputs resident in HBM; `e2e` goes through the host-buffer
C-ABI call with pinned host memory, copies inside the timed region. `roofline` is the dominant kernel (gate/up)
timed alone: K back-to-back launches between two CUDA events. `--impl reference` times the CPU oracle (a C port of the reference's CPU
semantics; the reference's Rust cannot be built here) on the host cores.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_EMBD, N_FF, N_EXPERT, TOP_K = 4096, 2048, 256, 6
GATE_EXPERT_BYTES = N_FF * (N_EMBD // 256) * 66       # 2 162 688
DOWN_EXPERT_BYTES = N_EMBD * (N_FF // 256) * 84       # 2 752 512
EXPERT_BYTES = 2 * GATE_EXPERT_BYTES + DOWN_EXPERT_BYTES  # 7 077 888

WORKLOADS = {
    # name: (tokens per step, layers rotated, routing variants)
    "moe_decode_b1": dict(tokens=1, layers=8, zipf=False),
    "moe_decode_b8": dict(tokens=8, layers=4, zipf=False),
    "moe_decode_b64": dict(tokens=64, layers=2, zipf=False),
    "moe_decode_b16": dict(tokens=16, layers=4, zipf=False),
    # prefill chunk: router logits N(0,1) - 1.1 ln(rank) (Zipf s = 1.1 expert popularity), tcgen05 grouped GEMM
    "moe_prefill_4096": dict(tokens=4096, layers=2, zipf=True),
    # FP8 E4M3 block-scaled dense projection (no counterpart in the reference), all six (M, N) shapes in one line
    "fp8_linear": dict(tokens=4096, layers=0, zipf=False),
    # router logits (f16) + shared expert (Q8_0), the steps beside the routed experts; batch 1, 8 and 64 in one line
    "shared_expert": dict(tokens=1, layers=0, zipf=False),
}
DEFAULT_WORKLOAD = "moe_prefill_4096"
METRIC, UNIT = "moe_expert_layer_tokens_per_s", "tokens/s"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def ncu_traffic(workload: str):
    """(bytes, source) of dram__bytes_read.sum + dram__bytes_write.sum per launch of the workload's dominant kernel, from
    the committed ncu capture record. The record names the kernel's source file and its SHA-256 at capture time: when
    the file has changed since, the figure no longer describes the code that runs and is withheld."""
    import hashlib

    try:
        rec = json.load(open(os.path.join(ROOT, "profiles", "traffic.json")))[workload]
        src = os.path.join(ROOT, rec["source_file"])
        digest = hashlib.sha256(open(src, "rb").read()).hexdigest()
        if digest != rec["source_sha256"]:
            return None, f"withheld: {rec['source_file']} has changed since the capture at commit {rec['commit']}"
        return rec["dram_bytes_per_launch"], f"ncu capture at commit {rec['commit']} ({rec['summary']})"
    except Exception as e:  # no record for this workload
        return None, f"no capture on record ({type(e).__name__})"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed regions run."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,utilization.gpu")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, window=None):
        """window = (t0, t1) in host time: only samples taken while the measured load ran are kept."""
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        return self.peek(window)

    def peek(self, window=None):
        """The summary of the samples so far (the sampler keeps running)."""
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, r in self.rows:
            if window and not (window[0] <= ts <= window[1]):
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
                for n, v in zip(names, r[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def gen_layer_gpu(torch, device, seed: int, n_expert: int = 0):
    """One layer's expert tensors generated on the device (see formats.random_layer_device)."""
    from deepseek_rs_b200.formats import random_layer_device

    return random_layer_device(torch, device, seed, n_expert or N_EXPERT, N_EMBD, N_FF)


def run_reference(args, rank: int, world: int):
    """CPU arm: the oracle's routed-expert layer on all host threads, a bounded sample of the workload per step."""
    if rank != 0:
        return
    import numpy as np

    import oracle
    from deepseek_rs_b200 import formats as F

    oracle.build()
    wl = WORKLOADS[args.workload]
    # the launcher of a multi-rank run sets OMP_NUM_THREADS=1 for its children: this arm uses every host core at any N
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    oracle.set_num_threads(cores)
    cores = oracle.num_threads()
    sample_tokens = min(wl["tokens"], 64)  # the same sample at every N
    n_exp = 32  # full-size experts, fewer of them: the CPU path's cost per token does not depend on the expert count
    lw = F.ExpertLayer(seed=1, n_expert=n_exp)
    rng = np.random.default_rng(0)
    x = F.bf16_round(rng.standard_normal((sample_tokens, N_EMBD)).astype(np.float32))
    logits = rng.standard_normal((sample_tokens, n_exp)).astype(np.float32)
    for _ in range(max(1, min(args.warmup, 2))):
        oracle.moe_layer(x, logits, lw.gate, lw.up, lw.down, k=TOP_K)
    steps = max(1, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.moe_layer(x, logits, lw.gate, lw.up, lw.down, k=TOP_K)
    dt = time.perf_counter() - t0
    tps = sample_tokens * steps / dt
    sample = f"{sample_tokens} tokens/step x {steps} steps, {n_exp} full-size experts, oracle port, OpenMP"
    line = {"impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * dt / steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x 2-bit codes, f32 accumulate", "data": "synthetic",
            "config": {"workload": args.workload, "tokens_per_step": sample_tokens, "top_k": TOP_K,
                       "n_embd": N_EMBD, "n_ff": N_FF},
            "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def cpu_baseline(workload: str):
    import numpy as np

    import oracle
    from deepseek_rs_b200 import formats as F

    oracle.build()
    oracle.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    cores = oracle.num_threads()
    n_tok, n_exp = max(4, 4 * cores), 32
    lw = F.ExpertLayer(seed=1, n_expert=n_exp)
    rng = np.random.default_rng(0)
    x = F.bf16_round(rng.standard_normal((n_tok, N_EMBD)).astype(np.float32))
    logits = rng.standard_normal((n_tok, n_exp)).astype(np.float32)
    oracle.moe_layer(x[:2], logits[:2], lw.gate, lw.up, lw.down, k=TOP_K)
    t0 = time.perf_counter()
    reps = 0
    while time.perf_counter() - t0 < 10.0:
        oracle.moe_layer(x, logits, lw.gate, lw.up, lw.down, k=TOP_K)
        reps += 1
    dt = time.perf_counter() - t0
    return {"value": n_tok * reps / dt, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{n_tok} tokens x {reps} passes of the layer ({n_exp} full-size experts), {dt:.1f} s"}


def measured_tflops():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["bf16_tflops"]), "measured"
        except Exception:
            pass
    return 1590.0, "fallback"


def ref_mapping_gpu(torch, device, K, workload_tokens: int, ours_ms_per_step: float):
    """GPU baseline beside the product: the reference kernels' thread mapping restated in CUDA (baseline/ref_mapping.cu),
    in both forms the reference has. LIVE: one token at a time, four launches per token, as its decode and its prefill
    loop run the path. BATCHED: its sorted-pair kernels, which it contains but never calls - the only formulation of a
    whole chunk it has. Both are timed on the workload's full token count (nothing extrapolated), on one layer in the
    reference's own (NATIVE) byte order; routing comes from the product's router."""
    from baseline import RefMapping

    R = RefMapping()
    T = workload_tokens
    gate, up, down = gen_layer_gpu(torch, device, seed=0)
    gen = torch.Generator(device=device)
    gen.manual_seed(99)
    x = torch.randn((T, N_EMBD), device=device, generator=gen).to(torch.bfloat16).to(torch.float32).contiguous()
    rank_e = (torch.randperm(N_EXPERT, device=device, generator=gen) + 1).float()
    lg = (torch.randn((T, N_EXPERT), device=device, generator=gen) - 1.1 * torch.log(rank_e)[None, :]).contiguous()
    probs = torch.empty((T, N_EXPERT), device=device)
    sel = torch.empty((T, TOP_K), dtype=torch.int32, device=device)
    w = torch.empty((T, TOP_K), device=device)
    K.router_select_parallel(lg, None, None, None, probs, sel, w, 0, 0, T, 0, 0)
    xq = torch.empty((N_EMBD // 256) * 292, dtype=torch.uint8, device=device)
    mid = torch.empty((TOP_K, N_FF), device=device)
    midq = torch.empty(TOP_K * (N_FF // 256) * 292, dtype=torch.uint8, device=device)
    out = torch.empty((T, N_EMBD), device=device)
    R.tokens(gate, up, down, x, sel, w, xq, mid, midq, out, N_EMBD, N_FF, min(T, 8), 10.0)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    R.tokens(gate, up, down, x, sel, w, xq, mid, midq, out, N_EMBD, N_FF, T, 10.0)
    e1.record()
    torch.cuda.synchronize()
    live_ms = e0.elapsed_time(e1)
    out_live = out.clone()
    scratch = R.batched(gate, up, down, x, sel, w, out, N_EMBD, N_FF, T, 10.0)  # warm-up, allocates the scratch
    torch.cuda.synchronize()
    same = bool(torch.equal(out, out_live))
    e0.record()
    R.batched_with(scratch, gate, up, down, x, sel, w, out, N_EMBD, N_FF, T, 10.0)
    e1.record()
    torch.cuda.synchronize()
    batched_ms = e0.elapsed_time(e1)
    del gate, up, down, scratch
    return {"kind": "restatement of the reference kernels' thread mapping and scalar loads, not the cuda-oxide binary",
            "tokens_timed": T, "extrapolated": False,
            "live_per_token": {"launches_per_token": 4, "ms_for_this_workload_step": live_ms, "ms_per_token": live_ms / T,
                               "value": T / (live_ms * 1e-3), "unit": UNIT, "product_speedup": live_ms / ours_ms_per_step},
            "batched_sorted_pairs": {"launches_per_chunk": 9, "ms_for_this_workload_step": batched_ms,
                                     "value": T / (batched_ms * 1e-3), "unit": UNIT,
                                     "product_speedup": batched_ms / ours_ms_per_step,
                                     "equals_live_form_bit_for_bit": same},
            "product_speedup": min(live_ms, batched_ms) / ours_ms_per_step,
            "note": "router excluded on the baseline side (it is the product's kernel); product_speedup is against the "
                    "faster of the two reference forms"}


def run_prefill(args, torch, dist, K, layers, layout, device, rank, world, sampler, T, L):
    """The batched (grouped-GEMM) workload: one step = one 4096-token chunk through one layer's routed experts."""
    V = 4
    gen = torch.Generator(device=device)
    gen.manual_seed(7 + rank)
    xs = torch.randn((V, T, N_EMBD), device=device, generator=gen).to(torch.bfloat16).to(torch.float32).contiguous()
    rank_e = (torch.randperm(N_EXPERT, device=device, generator=gen) + 1).float()
    lgs = (torch.randn((V, T, N_EXPERT), device=device, generator=gen) - 1.1 * torch.log(rank_e)[None, None, :]).contiguous()
    out = torch.empty((T, N_EMBD), device=device)
    sel = torch.empty((T, TOP_K), dtype=torch.int32, device=device)
    distinct, max_share, near_ties = [], 0.0, 0
    probs = torch.empty((T, N_EXPERT), device=device)
    sel2, w2 = torch.empty_like(sel), torch.empty((T, TOP_K), device=device)
    for v in range(V):
        K.moe_forward(v % L, xs[v], lgs[v], T, out, sel, None)
        cnt = torch.bincount(sel.flatten().clamp(min=0), minlength=N_EXPERT)
        distinct.append(int((cnt > 0).sum()))
        max_share = max(max_share, float(cnt.max()) / (T * TOP_K))
        # near ties: tokens whose 6th and 7th selection scores are fewer than 4 f32 steps apart. Only there could an
        # exp / ln implementation that rounds differently from this one pick another expert.
        K.router_select_parallel(lgs[v], None, None, None, probs, sel2, w2, 0, 0, T, 0, 0)
        top = torch.topk(probs, TOP_K + 1, dim=1).values  # scores are positive: their bit patterns order like the values
        gap = top[:, TOP_K - 1].contiguous().view(torch.int32) - top[:, TOP_K].contiguous().view(torch.int32)
        near_ties += int((gap < 4).sum())
    torch.cuda.synchronize()
    assert K.device_status() == 0

    def step(i):
        K.moe_forward(i % L, xs[i % V], lgs[i % V], T, out, None, None)

    t_load0 = time.time()
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    # The K timed steps are repeated (each repeat between its own pair of events) until about a second of device time
    # has been measured; the value is taken over all repeats and their spread is reported.
    launches0 = K.launch_count
    rep_ms = []
    while len(rep_ms) < 5 or (sum(rep_ms) < 1000.0 and len(rep_ms) < 200):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            step(args.warmup + i)
        e1.record()
        torch.cuda.synchronize()
        rep_ms.append(e0.elapsed_time(e1))
        if len(rep_ms) == 1:
            launches = K.launch_count - launches0
    if world > 1:
        dist.barrier()
    repeats = len(rep_ms)
    ms_total = sum(rep_ms) / repeats

    # phase times from events recorded inside the library between its kernels
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
    for e in evs:
        e.record()
    K.set_phase_events(evs)
    phase = [0.0] * 5
    reps = min(args.steps, 10)
    for i in range(reps):
        step(i)
        torch.cuda.synchronize()
        for j in range(5):
            phase[j] += evs[j].elapsed_time(evs[j + 1]) / reps
    K.set_phase_events(None)

    # end to end: every step copies its chunk in from pinned host memory and its result back. Two handles take the
    # steps in turn (each with its own stream and staging buffers), so one step's copies overlap the other's kernels;
    # a handle is waited for before it is given its next step, and both at the end, inside the timed region.
    from deepseek_rs_b200.kernels import MoeKernels

    K2 = MoeKernels(device=device.index, max_tokens=T, max_layers=L)
    for il, (gate, up, down) in enumerate(layers):
        K2.layer_register(il, gate, up, down, layout)
    hk = [K, K2]
    xh, lh = xs.cpu().pin_memory(), lgs.cpu().pin_memory()
    ohs = [torch.empty((T, N_EMBD)).pin_memory() for _ in hk]
    for i in range(4):
        hk[i % 2].moe_forward_host(i % L, xh[i % V], lh[i % V], T, ohs[i % 2])
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e2e_steps, e2e_reps = min(args.steps, 20), []
    for _ in range(6):
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            h = hk[i % 2]
            h.host_synchronize()
            h.moe_forward_host_async(i % L, xh[i % V], lh[i % V], T, ohs[i % 2])
        for h in hk:
            h.host_synchronize()
        e2e_reps.append((time.perf_counter() - t0) * 1e3 / e2e_steps)
    e2e_ms_step = statistics.median(e2e_reps)
    assert K2.device_status() == 0
    K2.close()
    while time.time() - t_load0 < 2.0:
        step(0)
        torch.cuda.synchronize()
    clocks = sampler.peek(window=(t_load0, time.time()))

    times = torch.tensor([ms_total, e2e_ms_step] + phase, dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms_step, *phase = (float(v) for v in times.tolist())
    # the decode workloads (batch 1, 8, 64) on the same layers: the packed-weight bandwidth half of the metric
    decode = []
    if world == 1 and not args.no_decode_block:
        for t in (1, 8, 64):
            Kd = MoeKernels(device=device.index, max_tokens=t, max_layers=L)
            for il, (gate, up, down) in enumerate(layers):
                Kd.layer_register(il, gate, up, down, layout)
            d = run_decode(args, torch, dist, Kd, layers, layout, device, rank, world, sampler, t, L, f"moe_decode_b{t}",
                           emit=False, steps=200)
            Kd.close()
            decode.append({"workload": d["config"]["workload"], "tokens_per_step": t, "ms_per_step": d["ms_per_step"],
                           "tokens_per_s": d["value"], "distinct_experts_per_step": d["config"]["distinct_experts_per_step"],
                           "packed_weight_gbs": d["packed_weight_gbs"],
                           "frac_of_measured_hbm": d["packed_weight_frac_of_measured_hbm"],
                           "frac_of_8000": d["packed_weight_frac_of_8000"],
                           "gate_up": {k: d["roofline"][k] for k in ("kernel", "achieved", "frac", "avg_launch_ms", "traffic")},
                           "down": {k: d["roofline_down"][k] for k in ("kernel", "achieved", "frac", "avg_launch_ms")},
                           "e2e_tokens_per_s": d["e2e"]["value"], "gpu_launches_per_step": d["gpu_launches"] / d["steps"],
                           "clocks": d["clocks"]})
    sampler.stop()
    if rank != 0:
        return
    peak_tf, peak_kind = measured_tflops()
    hbm, _ = measured_peaks()
    pairs = T * TOP_K
    gu_flops, dn_flops = 2.0 * pairs * 2 * N_FF * N_EMBD, 2.0 * pairs * N_EMBD * N_FF
    u_mean = sum(distinct) / len(distinct)
    tokens = T * args.steps * world
    ms_step = ms_total / args.steps
    line = {
        "metric": METRIC, "value": tokens / (ms_total * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 integer codes x int8 (exact), f32 accumulate in TMEM", "data": "synthetic",
        "config": {"workload": args.workload, "tokens_per_step_per_gpu": T, "top_k": TOP_K, "n_expert": N_EXPERT,
                   "n_embd": N_EMBD, "n_ff": N_FF, "layout": args.layout, "router": "Zipf s=1.1 expert popularity",
                   "parallelism": "single GPU" if world == 1 else f"{world} independent replicas",
                   "l2": f"inputs rotate over {L} layers (1.8 GB each) x {V} routings: larger than the 126 MB L2",
                   "distinct_experts_per_step": u_mean, "largest_expert_share_of_pairs": max_share,
                   "near_tie_tokens_lt_4ulp": near_ties, "tokens_checked_for_near_ties": V * T},
        "repeats": repeats, "ms_per_step_min": min(rep_ms) / args.steps, "ms_per_step_max": max(rep_ms) / args.steps,
        "packed_weight_gbs": u_mean * EXPERT_BYTES * world / (ms_step * 1e-3) / 1e9,
        "roofline": {"bound": "tensor", "kernel": "pf_grouped_gemm_kernel<IQ2> (gate+up+SwiGLU, tcgen05 kind::f16)",
                     "achieved": gu_flops / (phase[1] * 1e-3) / 1e12, "peak": peak_tf, "peak_kind": f"of {peak_kind}",
                     "unit": "TFLOP/s", "frac": gu_flops / (phase[1] * 1e-3) / 1e12 / peak_tf,
                     "traffic": ncu_traffic(args.workload)[0], "traffic_source": ncu_traffic(args.workload)[1],
                     "algorithmic_flops_per_launch": gu_flops, "avg_launch_ms": phase[1]},
        "roofline_down": {"bound": "tensor", "kernel": "pf_grouped_gemm_kernel<Q2K> (down, tcgen05 kind::f16)",
                          "achieved": dn_flops / (phase[3] * 1e-3) / 1e12, "peak": peak_tf, "unit": "TFLOP/s",
                          "frac": dn_flops / (phase[3] * 1e-3) / 1e12 / peak_tf, "avg_launch_ms": phase[3]},
        "phases_ms": {"group+gather": phase[0], "gate_up_gemm": phase[1], "q8k_mid+gather": phase[2],
                      "down_gemm": phase[3], "slot_sum": phase[4]},
        "e2e": {"value": T * world / (e2e_ms_step * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": T * (N_EMBD + N_EXPERT) * 4, "d2h_bytes_per_step": T * N_EMBD * 4,
                "repeats": len(e2e_reps), "value_min": T * world / (max(e2e_reps) * 1e-3),
                "value_max": T * world / (min(e2e_reps) * 1e-3)},
        "gpu_launches": launches, "timed_with": f"CUDA events around K back-to-back steps, {repeats} repeats", "clocks": clocks,
    }
    if decode:
        line["decode"] = decode
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args.workload)
    if world == 1 and not args.no_ref_mapping:
        line["ref_mapping_gpu"] = ref_mapping_gpu(torch, device, K, T, ms_step)
    print(json.dumps(line), flush=True)


def run_fp8(args, torch, dist, K, device, rank, world, sampler):
    """Activations f32 -> E4M3 codes + 1x128 scales -> GEMM with 128x128-block-scaled weights -> bf16. A step is one
    projection of M rows; the headline shape is M = 4096, N = K = 4096."""
    Kdim, R = 4096, 16  # R weight matrices rotate so that no step finds its weights in L2 (16 x 16.8 MB)
    gen = torch.Generator(device=device)
    gen.manual_seed(11 + rank)
    results, t_load0 = [], time.time()
    for N in (4096, 1536):
        ws = []
        for r in range(R):
            w = torch.randn((N, Kdim), device=device, generator=gen)
            wc = torch.empty((N, Kdim), dtype=torch.uint8, device=device)
            wsc = torch.empty((N // 128, Kdim // 128), device=device)
            K.fp8_quantize(w, wc, wsc, N, Kdim, 128)
            ws.append((wc, wsc))
        for M in (1, 128, 4096):
            x = torch.randn((M, Kdim), device=device, generator=gen)
            ac = torch.empty((M, Kdim), dtype=torch.uint8, device=device)
            asc = torch.empty((M, Kdim // 128), device=device)
            out = torch.empty((M, N), dtype=torch.bfloat16, device=device)
            K.fp8_quantize(x, ac, asc, M, Kdim, 1)
            steps = args.steps if M >= 128 else max(args.steps, 200)
            for i in range(args.warmup):
                K.fp8_linear(ac, asc, *ws[i % R], out, M, N, Kdim)
            g = torch.cuda.CUDAGraph()
            cs = torch.cuda.Stream()
            cs.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(cs):
                torch.cuda.synchronize()
                with torch.cuda.graph(g, stream=cs):
                    for i in range(R):
                        K.fp8_linear(ac, asc, *ws[i], out, M, N, Kdim)
            torch.cuda.current_stream().wait_stream(cs)
            g.replay()
            torch.cuda.synchronize()
            reps = max(1, steps // R)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                g.replay()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / (reps * R)
            # end to end: pinned f32 rows in, quantise, project, bf16 rows back
            xh, oh = x.cpu().pin_memory(), torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
            n_e2e = 20
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for i in range(n_e2e):
                xd = xh.to(device, non_blocking=True)
                K.fp8_quantize(xd, ac, asc, M, Kdim, 1)
                K.fp8_linear(ac, asc, *ws[i % R], out, M, N, Kdim)
                oh.copy_(out, non_blocking=True)
                torch.cuda.synchronize()
            e2e_ms = (time.perf_counter() - t0) * 1e3 / n_e2e
            results.append(dict(M=M, N=N, K=Kdim, ms=ms, tflops=2.0 * M * N * Kdim / (ms * 1e-3) / 1e12,
                                weight_gbs=N * Kdim / (ms * 1e-3) / 1e9, e2e_ms=e2e_ms, steps=reps * R))
        del ws
    assert K.device_status() == 0
    while time.time() - t_load0 < 2.0:
        g.replay()
        torch.cuda.synchronize()
    clocks = sampler.stop(window=(t_load0, time.time()))
    if rank != 0:
        return
    head = next(r for r in results if r["M"] == 4096 and r["N"] == 4096)
    mv = next(r for r in results if r["M"] == 1 and r["N"] == 4096)
    peak_tf, kind = measured_tflops()
    hbm, _ = measured_peaks()
    line = {
        "metric": METRIC, "value": head["M"] * world / (head["ms"] * 1e-3), "unit": UNIT, "n_gpus": world,
        "steps": head["steps"], "warmup": args.warmup, "ms_per_step": head["ms"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp8 e4m3 x fp8 e4m3, f32 accumulate, bf16 out",
        "data": "synthetic",
        "config": {"workload": "fp8_linear", "M": 4096, "N": 4096, "K": 4096, "block_scales": "1x128 act, 128x128 weight",
                   "parallelism": "single GPU" if world == 1 else f"{world} independent replicas",
                   "l2": f"{R} weight matrices rotate (268 MB > 126 MB L2)"},
        "roofline": {"bound": "tensor", "kernel": "fp8_gemm_ws_kernel<TMA> (tcgen05 kind::f8f6f4, 128x256 tiles, tensor-map loads)", "achieved": head["tflops"],
                     "peak": peak_tf, "peak_kind": f"of {kind} bf16 GEMM (dense fp8 is nominally twice that)",
                     "unit": "TFLOP/s", "frac": head["tflops"] / peak_tf, "traffic": None, "avg_launch_ms": head["ms"],
                     "fp8_peak_nominal": 2.0 * peak_tf, "frac_of_fp8_peak_nominal": head["tflops"] / (2.0 * peak_tf),
                     "fp8_peak_kind": "2 x the measured bf16 burst (no fp8 measurement exists for this pool; nominal ratio)"},
        "roofline_matvec": {"bound": "hbm", "kernel": "fp8_matvec_kernel (M = 1)", "achieved": mv["weight_gbs"],
                            "peak": hbm, "unit": "GB/s", "frac": mv["weight_gbs"] / hbm, "avg_launch_ms": mv["ms"]},
        "shapes": results,
        "e2e": {"value": head["M"] * world / (head["e2e_ms"] * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": head["M"] * Kdim * 4, "d2h_bytes_per_step": head["M"] * head["N"] * 2},
        "gpu_launches": head["steps"], "timed_with": f"CUDA graph of {R} launches replayed", "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


def run_shared(args, torch, dist, K, device, rank, world, sampler):
    """Router logits (matmul_f16, 2 MB of f16 weights) and the shared expert (three Q8_0 matrices, 26.7 MB) for
    batches of 1, 8 and 64 tokens. R layers' weights rotate so that a step never finds its weights in L2."""
    R = 8  # 8 x 28.8 MB = 231 MB > 126 MB L2
    gen = torch.Generator(device=device)
    gen.manual_seed(21 + rank)

    def q8_0(rows, cols):
        t = torch.randint(0, 256, (rows * (cols // 32), 34), dtype=torch.uint8, device=device, generator=gen)
        sc = (torch.randn(rows * (cols // 32), device=device, generator=gen).abs() * 1e-3).to(torch.float16)
        t[:, 0:2] = sc.view(torch.uint8).view(-1, 2)
        return t.view(-1)

    layers = [(q8_0(N_FF, N_EMBD), q8_0(N_FF, N_EMBD), q8_0(N_EMBD, N_FF),
               (torch.randn((N_EXPERT, N_EMBD), device=device, generator=gen) * 0.05).to(torch.float16)) for _ in range(R)]
    sh_bytes = (2 * N_FF * (N_EMBD // 32) + N_EMBD * (N_FF // 32)) * 34
    results, t_load0, g = [], time.time(), None
    for T in (1, 8, 64):
        x = torch.randn((T, N_EMBD), device=device, generator=gen).to(torch.bfloat16).to(torch.float32)
        out = torch.empty((T, N_EMBD), device=device)
        logits = torch.empty((T, N_EXPERT), device=device)

        def step(i):
            gw, uw, dw, rw = layers[i % R]
            K.matmul_f16(rw, x, logits, N_EMBD, N_EXPERT, T)
            K.shared_expert(gw, uw, dw, x, T, out)

        for i in range(args.warmup):
            step(i)
        l0 = K.launch_count
        step(0)
        launches_per_step = K.launch_count - l0  # counted by the library: it depends on the batch (3 up to 4 tokens, 5 above)
        g = torch.cuda.CUDAGraph()
        cs = torch.cuda.Stream()
        cs.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(cs):
            torch.cuda.synchronize()
            with torch.cuda.graph(g, stream=cs):
                for i in range(R):
                    step(i)
        torch.cuda.current_stream().wait_stream(cs)
        g.replay()
        torch.cuda.synchronize()
        reps = max(1, max(args.steps, 200) // R)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / (reps * R)
        xh, oh = x.cpu().pin_memory(), torch.empty((T, N_EMBD)).pin_memory()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(20):
            xd = xh.to(device, non_blocking=True)
            gw, uw, dw, rw = layers[i % R]
            K.matmul_f16(rw, xd, logits, N_EMBD, N_EXPERT, T)
            K.shared_expert(gw, uw, dw, xd, T, out)
            oh.copy_(out, non_blocking=True)
            torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / 20
        results.append(dict(tokens=T, ms=ms, weight_gbs=(sh_bytes + N_EXPERT * N_EMBD * 2) / (ms * 1e-3) / 1e9,
                            e2e_ms=e2e_ms, steps=reps * R, launches_per_step=launches_per_step))
    assert K.device_status() == 0
    while time.time() - t_load0 < 2.0:
        g.replay()
        torch.cuda.synchronize()
    clocks = sampler.stop(window=(t_load0, time.time()))
    if rank != 0:
        return
    hbm, kind = measured_peaks()
    head = results[0]
    line = {
        "metric": "shared_expert_and_router_logits_tokens_per_s", "value": head["tokens"] * world / (head["ms"] * 1e-3),
        "unit": UNIT, "n_gpus": world, "steps": head["steps"], "warmup": args.warmup, "ms_per_step": head["ms"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 x int8 (dp4a) with f32 block scales; f16 x f32 for the router", "data": "synthetic",
        "config": {"workload": "shared_expert", "tokens_per_step_per_gpu": 1, "n_embd": N_EMBD, "n_ff": N_FF,
                   "n_expert": N_EXPERT, "parallelism": "single GPU" if world == 1 else f"{world} independent replicas",
                   "l2": f"{R} layers' weights rotate ({R} x 28.8 MB > 126 MB L2)"},
        "roofline": {"bound": "hbm", "kernel": "matmul_f16_staged_kernel + shared_staged_kernel x2 (whole step)",
                     "achieved": head["weight_gbs"], "peak": hbm, "peak_kind": f"of {kind}", "unit": "GB/s",
                     "frac": head["weight_gbs"] / hbm, "traffic": None,
                     "algorithmic_bytes_per_step": sh_bytes + N_EXPERT * N_EMBD * 2, "avg_launch_ms": head["ms"]},
        "batches": results,
        "e2e": {"value": head["tokens"] * world / (head["e2e_ms"] * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": N_EMBD * 4, "d2h_bytes_per_step": N_EMBD * 4},
        "gpu_launches": head["steps"] * head["launches_per_step"],
        "timed_with": f"CUDA graph of {R} steps ({head['launches_per_step']} kernels each at batch 1) replayed", "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


def run_prefill_ep(args, torch, dist, device, rank, world, local_rank, sampler, T_chunk):
    """Expert-parallel prefill through the C ABI (dsmoe_ep_init / dsmoe_moe_forward_ep): rank r owns experts
    [r*256/G, (r+1)*256/G) and routes its own tokens; counting, placement, row gather, NCCL dispatch (Q8_K rows) and
    combine (f32 rows), the owner's grouped GEMM and the slot sum all run inside the library. `value` is weak scaling
    (every rank brings its own 4096-token chunk); the same line carries the strong-scaling figure (ONE 4096-token chunk
    split evenly over the ranks), the figure without replicated experts, and a comparison of the outputs with a
    single-GPU run of the same layer on rank 0."""
    from deepseek_rs_b200.ep import ExpertParallelHandle
    from deepseek_rs_b200.kernels import LAYOUT_ROWSOA, MoeKernels

    T, per, R = T_chunk, N_EXPERT // world, args.ep_replicate
    L, V = 2, 4
    K = MoeKernels(device=local_rank, max_tokens=T, max_layers=L)
    ep = ExpertParallelHandle(K, rank, world, max_replicas=R, recv_capacity_rows=3 * T * TOP_K)
    ep_fused = bool(ep.combine_is_fused)
    progress(rank, f"library communicator up, peer-mapped exchanges: {ep_fused}")
    g_exp, d_exp = GATE_EXPERT_BYTES, DOWN_EXPERT_BYTES
    shards = []
    for il in range(L):  # shard of layer il in ROWSOA order, with R empty replica slots behind the rank's own experts
        gate, up, down = gen_layer_gpu(torch, device, seed=1000 * rank + il, n_expert=per)
        bufs = []
        for t, nb, relay, rows, blocks in ((gate, g_exp, K.relayout_iq2xxs, per * N_FF, N_EMBD // 256),
                                          (up, g_exp, K.relayout_iq2xxs, per * N_FF, N_EMBD // 256),
                                          (down, d_exp, K.relayout_q2k, per * N_EMBD, N_FF // 256)):
            buf = torch.zeros((per + R) * nb, dtype=torch.uint8, device=device)
            relay(t, buf[: per * nb], rows, blocks)
            bufs.append(buf)
        torch.cuda.synchronize()
        del gate, up, down
        ep.layer_register(il, bufs[0], bufs[1], bufs[2], LAYOUT_ROWSOA)
        shards.append(bufs)

    # expert popularity is the same on every rank (the router subtracts 1.1 ln(popularity rank) from the logits); the
    # library is never told: replicas are chosen below from its own running counts of `selected`
    gen = torch.Generator(device=device)
    gen.manual_seed(7)
    rank_e = (torch.randperm(N_EXPERT, device=device, generator=gen) + 1).float()
    xl, ll = [], []
    for v in range(V):
        gen.manual_seed(100 + v + 1000 * rank)
        x = torch.randn((T, N_EMBD), device=device, generator=gen).to(torch.bfloat16).to(torch.float32)
        lg = torch.randn((T, N_EXPERT), device=device, generator=gen) - 1.1 * torch.log(rank_e)[None, :]
        xl.append(x.contiguous())
        ll.append(lg.contiguous())
    out = torch.empty((T, N_EMBD), device=device)
    sel = torch.empty((T, TOP_K), dtype=torch.int32, device=device)

    def step(i, n_tok=T):
        ep.forward(i % L, xl[i % V][:n_tok], ll[i % V][:n_tok], out=out[:n_tok])

    def timed(n_steps, n_tok=T):
        for i in range(max(3, args.warmup // 2)):
            step(i, n_tok)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n_steps):
            step(args.warmup + i, n_tok)
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1) / n_steps], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    t_load0 = time.time()
    progress(rank, "shards and inputs ready; unreplicated steps")
    # pure sharding first: its time is reported, and its steps fill the running per-expert counts
    ms_unreplicated = timed(min(args.steps, 10))
    progress(rank, f"unreplicated {ms_unreplicated:.3f} ms per step; installing replicas")
    max_recv_unrep = torch.tensor([float(sum(ep.last_recv_rows()))], dtype=torch.float64, device=device)
    dist.all_reduce(max_recv_unrep, op=dist.ReduceOp.MAX)
    hot = []
    if R:
        counts = ep.expert_counts().to(device)
        dist.all_reduce(counts)  # every rank sees the same totals, hence picks the same replicas
        hot = [int(e) for e in torch.argsort(counts, descending=True, stable=True)[:R].tolist()]
        for il in range(L):  # each owner broadcasts the (already re-laid) bytes of its hot experts into everyone's slots
            for slot, e in enumerate(hot):
                for buf, nb in zip(shards[il], (g_exp, g_exp, d_exp)):
                    piece = buf[(per + slot) * nb:(per + slot + 1) * nb]
                    if e // per == rank:
                        piece.copy_(buf[(e % per) * nb:(e % per + 1) * nb])
                    dist.broadcast(piece, src=e // per)
        torch.cuda.synchronize()
        ep.set_replicas(hot)

    # correctness before timing: routing against the single-GPU router, outputs against a single-GPU run of the layer
    progress(rank, "replicas installed; checking routing and outputs against one GPU")
    K_solo = MoeKernels(device=local_rank, max_tokens=T, max_layers=1)
    probs = torch.empty((T, N_EXPERT), device=device)
    sel_solo, w_solo = torch.empty_like(sel), torch.empty((T, TOP_K), device=device)
    same_routing = True
    for v in range(V):
        ep.forward(0, xl[v], ll[v], out=out, selected_out=sel)
        K_solo.router_select_parallel(ll[v], None, None, None, probs, sel_solo, w_solo, 0, 0, T, 0, 0)
        same_routing = same_routing and bool(torch.equal(sel, sel_solo))
    out_match, out_maxdiff = True, 0.0
    if rank == 0:  # all shards of layer 0 regenerated from their seeds: 1.8 GB + its re-laid copy, freed afterwards
        parts = [gen_layer_gpu(torch, device, seed=1000 * r + 0, n_expert=per) for r in range(world)]
        full = [torch.cat([p[i] for p in parts]) for i in range(3)]
        del parts
        g2, u2, d2 = (torch.empty_like(t) for t in full)
        K_solo.relayout_iq2xxs(full[0], g2, N_EXPERT * N_FF, N_EMBD // 256)
        K_solo.relayout_iq2xxs(full[1], u2, N_EXPERT * N_FF, N_EMBD // 256)
        K_solo.relayout_q2k(full[2], d2, N_EXPERT * N_EMBD, N_FF // 256)
        torch.cuda.synchronize()
        del full
        K_solo.layer_register(0, g2, u2, d2, LAYOUT_ROWSOA)
        want = torch.empty((T, N_EMBD), device=device)
        K_solo.moe_forward(0, xl[1], ll[1], T, want, None, None)
        torch.cuda.synchronize()
    ep.forward(0, xl[1], ll[1], out=out)  # collective: every rank takes part
    torch.cuda.synchronize()
    if rank == 0:
        out_match = bool(torch.equal(out, want))
        out_maxdiff = float((out - want).abs().max() / want.abs().max())
        del g2, u2, d2, want
    K_solo.close()
    flags = torch.tensor([1 if same_routing else 0, 1 if out_match else 0], device=device)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if not int(flags[0].item()):
        raise SystemExit("expert-parallel routing differs from the single-GPU router")
    if rank == 0 and out_maxdiff > 1e-5:
        raise SystemExit(f"expert-parallel output differs from the single-GPU layer (max diff {out_maxdiff} of scale)")

    # timed: weak scaling (the line's value), then strong scaling (one chunk split over the ranks)
    progress(rank, "checks done; timed weak-scaling steps")
    l0 = K.launch_count
    ms_step = timed(args.steps)
    progress(rank, f"weak {ms_step:.3f} ms per step; strong-scaling steps")
    launches = K.launch_count - l0  # the route-side handle; the owner-side launches are counted inside the library call
    recv_rows = float(sum(ep.last_recv_rows()))
    ms_strong = timed(args.steps, T // world)
    assert K.device_status() == 0

    # phase times on this rank from events recorded inside the library
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
    for e in evs:
        e.record()
    ep.set_phase_events(evs)
    names = ["plan", "dispatch", "experts", "combine", "sum"]
    phase = {n: 0.0 for n in names}
    reps = min(args.steps, 5)
    for i in range(reps):
        step(i)
        torch.cuda.synchronize()
        for j, n in enumerate(names):
            phase[n] += evs[j].elapsed_time(evs[j + 1]) / reps
    ep.set_phase_events(None)

    # end to end: pinned host slices in, result back on the host, every step
    progress(rank, "phases done; end-to-end steps")
    xh = [t.cpu().pin_memory() for t in xl]
    lh = [t.cpu().pin_memory() for t in ll]
    e2e_steps = min(args.steps, 20)

    def e2e_one_at_a_time():
        """Copy in, compute, copy out, wait: nothing overlaps."""
        oh = torch.empty((T, N_EMBD)).pin_memory()
        xd, ld = torch.empty_like(xl[0]), torch.empty_like(ll[0])
        dist.barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            xd.copy_(xh[i % V], non_blocking=True)
            ld.copy_(lh[i % V], non_blocking=True)
            ep.forward(i % L, xd, ld, out=out)
            oh.copy_(out, non_blocking=True)
            torch.cuda.synchronize()
        return (time.perf_counter() - t0) * 1e3 / e2e_steps

    def e2e_double_buffered():
        """Two sets of device buffers and two copy streams: the next step's chunk comes in and the previous step's result
        goes out while the current step computes (the library call returns once the step's kernels are queued)."""
        main, s_in, s_out = torch.cuda.current_stream(), torch.cuda.Stream(), torch.cuda.Stream()
        xd = [torch.empty_like(xl[0]) for _ in range(2)]
        ld = [torch.empty_like(ll[0]) for _ in range(2)]
        od = [torch.empty((T, N_EMBD), device=device) for _ in range(2)]
        ohs = [torch.empty((T, N_EMBD)).pin_memory() for _ in range(2)]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_done = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]
        torch.cuda.synchronize()
        dist.barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            b = i % 2
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_done[b])  # the step that last read these input buffers
                xd[b].copy_(xh[i % V], non_blocking=True)
                ld[b].copy_(lh[i % V], non_blocking=True)
                ev_in[b].record(s_in)
            main.wait_event(ev_in[b])
            if i >= 2:
                main.wait_event(ev_out[b])       # the copy that last read this output buffer
            ep.forward(i % L, xd[b], ld[b], out=od[b])
            ev_done[b].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[b])
                ohs[b].copy_(od[b], non_blocking=True)
                ev_out[b].record(s_out)
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) * 1e3 / e2e_steps

    e2e_plain_ms = e2e_one_at_a_time()
    try:
        e2e_ms_step, e2e_note = e2e_double_buffered(), "device buffers double-buffered, copies on their own streams"
    except Exception as exc:  # the same on every rank (same code, same sizes): report the plain figure
        e2e_ms_step, e2e_note = e2e_plain_ms, f"one step at a time (double buffering failed: {type(exc).__name__})"
    while time.time() - t_load0 < 2.0:
        step(0)
        torch.cuda.synchronize()
    clocks = sampler.stop(window=(t_load0, time.time()))
    times = torch.tensor([e2e_ms_step, recv_rows, e2e_plain_ms], dtype=torch.float64, device=device)
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
    e2e_ms_step, max_recv, e2e_plain_ms = (float(v) for v in times.tolist())
    if rank != 0:
        return
    T_total = T * world
    line = {
        "metric": METRIC, "value": T_total / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16 integer codes x int8 (exact), f32 accumulate in TMEM", "data": "synthetic",
        "config": {"workload": args.workload, "tokens_per_step_all_gpus": T_total, "tokens_per_step_per_gpu": T,
                   "top_k": TOP_K, "n_expert": N_EXPERT, "experts_per_gpu": per, "replicated_hot_experts": R,
                   "replicas_chosen_from": "running counts of `selected` inside the library over the unreplicated steps",
                   "n_embd": N_EMBD, "n_ff": N_FF, "layout": "rowsoa", "router": "Zipf s=1.1 expert popularity",
                   "parallelism": f"ep{world}: dsmoe_moe_forward_ep, " + (
                       "dispatch (Q8_K rows) and combine (f32 rows) as kernel stores into peer-mapped buffers over NVLink"
                       if ep_fused else "grouped ncclSend / ncclRecv dispatch (Q8_K rows) and combine (f32 rows)"),
                   "l2": f"inputs rotate over {L} layers x {V} routings",
                   "routing_bit_exact_vs_single_gpu": bool(int(flags[0].item())),
                   "outputs_match_single_gpu": bool(int(flags[1].item())), "outputs_max_diff_of_scale": out_maxdiff,
                   "max_pairs_received_by_a_rank": int(max_recv), "mean_pairs_per_rank": T * TOP_K},
        "strong": {"tokens_per_step_all_gpus": T, "ms_per_step": ms_strong, "value": T / (ms_strong * 1e-3), "unit": UNIT,
                   "note": "one 4096-token chunk split evenly over the ranks"},
        "unreplicated": {"ms_per_step": ms_unreplicated, "value": T_total / (ms_unreplicated * 1e-3), "unit": UNIT,
                         "max_pairs_received_by_a_rank": int(max_recv_unrep.item())},
        "roofline": {"bound": "tensor", "kernel": "pf_grouped_gemm_kernel<IQ2> (per-rank shard)", "achieved": None,
                     "peak": measured_tflops()[0], "unit": "TFLOP/s", "frac": None, "traffic": None,
                     "note": "kernel-level figures are reported by the 1-GPU run; this line is the whole EP step"},
        "e2e": {"value": T_total / (e2e_ms_step * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": T * (N_EMBD + N_EXPERT) * 4 * world, "d2h_bytes_per_step": T * N_EMBD * 4 * world,
                "how": e2e_note, "value_one_step_at_a_time": T_total / (e2e_plain_ms * 1e-3)},
        "phases_ms_rank0": phase,
        "gpu_launches": launches, "timed_with": "CUDA events around K back-to-back steps, max over ranks",
        "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


def run_decode(args, torch, dist, K, layers, layout, device, rank, world, sampler, T, L, workload, emit=True, steps=0):
    """A decode workload (batch T): the whole step replayed from a CUDA graph, the two dominant kernels timed alone, the
    host-buffer call end to end. Returns the JSON line (rank 0; printed when `emit`)."""
    if steps:
        args = argparse.Namespace(**{**vars(args), "steps": steps})
    # routing / activation variants: enough of them that (layer, routing) pairs repeat only after far more than the
    # L2 capacity has streamed through
    V = 16
    gen = torch.Generator(device=device)
    gen.manual_seed(7 + rank)
    xs = torch.randn((V, T, N_EMBD), device=device, generator=gen).to(torch.bfloat16).to(torch.float32).contiguous()
    lgs = torch.randn((V, T, N_EXPERT), device=device, generator=gen).contiguous()
    out = torch.empty((T, N_EMBD), device=device)
    sel = torch.empty((T, TOP_K), dtype=torch.int32, device=device)
    wts = torch.empty((T, TOP_K), device=device)

    # distinct experts per variant (for the algorithmic byte count)
    distinct = []
    for v in range(V):
        K.moe_forward(v % L, xs[v], lgs[v], T, out, sel, wts)
        distinct.append(int(torch.unique(sel).numel()))
    torch.cuda.synchronize()

    def step(i):
        K.moe_forward(i % L, xs[i % V], lgs[i % V], T, out, None, None)

    t_load0 = time.time()
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()

    # The timed steps are replayed from a CUDA graph holding G consecutive steps (G divides K), so that the host's
    # launch cost (several microseconds per ctypes call) does not sit between kernels of a 40-microsecond step.
    G = max(g for g in range(1, min(args.steps, 32) + 1) if args.steps % g == 0)
    launches0 = K.launch_count
    graph = torch.cuda.CUDAGraph()
    cap_stream = torch.cuda.Stream()
    cap_stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(cap_stream):
        step(args.warmup)  # the capture stream's first use of every kernel happens outside the capture
        torch.cuda.synchronize()
        launches0 = K.launch_count
        with torch.cuda.graph(graph, stream=cap_stream):
            for i in range(G):
                step(args.warmup + i)
    launches = (K.launch_count - launches0) * (args.steps // G)
    torch.cuda.current_stream().wait_stream(cap_stream)
    graph.replay()  # one untimed replay
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps // G):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms_total = e0.elapsed_time(e1)
    u_mean = sum(distinct[(args.warmup + i) % V] for i in range(G)) / G
    assert K.device_status() == 0

    # The two dominant kernels timed alone: K back-to-back launches each (inputs prepared beforehand, same rotation
    # over layers and routings), CUDA events around the batch.
    xb, mb = N_EMBD // 256, N_FF // 256
    probs = torch.empty((T, N_EXPERT), device=device)
    pre = []
    for v in range(V):
        xq = torch.empty((T, xb, 292), dtype=torch.uint8, device=device)
        mid = torch.empty((T * TOP_K, N_FF), device=device)
        midq = torch.empty((T * TOP_K, mb, 292), dtype=torch.uint8, device=device)
        sv, wv = torch.empty_like(sel), torch.empty_like(wts)
        gate, up, down = layers[v % L]
        K.router_select_parallel(lgs[v], None, None, None, probs, sv, wv, 0, 0, T, 0, 0)
        K.q8k_quantize(xs[v], xq, N_EMBD, T)
        K.moe_gate_up_mid_qwarp32(gate, up, xq, sv, wv, None, None, mid, GATE_EXPERT_BYTES, xb * 66, xb, N_FF, TOP_K,
                                  10.0, n_tokens=T, layout=layout)
        K.q8k_quantize(mid, midq, N_FF, T * TOP_K)
        pre.append((xq, sv, wv, midq))
    mid = torch.empty((T * TOP_K, N_FF), device=device)
    torch.cuda.synchronize()

    def run_gate_up(i):
        gate, up, _ = layers[i % L]
        xq, sv, wv, _ = pre[i % V]
        K.moe_gate_up_mid_qwarp32(gate, up, xq, sv, wv, None, None, mid, GATE_EXPERT_BYTES, xb * 66, xb, N_FF, TOP_K,
                                  10.0, n_tokens=T, layout=layout)

    def run_down(i):
        _, _, down = layers[i % L]
        _, sv, _, midq = pre[i % V]
        K.moe_down_sum6_qwarp32(down, midq, sv, out, DOWN_EXPERT_BYTES, mb * 84, mb, N_EMBD, n_expert=TOP_K,
                                n_tokens=T, layout=layout)

    def time_alone(fn):
        # L must divide V for (layer, routing) pairs to stay matched; replay from a graph for the same reason as above
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.stream(cap_stream):
            fn(0)
            torch.cuda.synchronize()
            with torch.cuda.graph(g2, stream=cap_stream):
                for i in range(G):
                    fn(i)
        torch.cuda.current_stream().wait_stream(cap_stream)
        g2.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps // G):
            g2.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / args.steps

    gu_ms_mean = time_alone(run_gate_up)
    dn_ms_mean = time_alone(run_down)

    # end to end through the host-buffer C-ABI call
    xh = xs.cpu().pin_memory()
    lh = lgs.cpu().pin_memory()
    oh = torch.empty((T, N_EMBD)).pin_memory()
    for i in range(3):
        K.moe_forward_host(i % L, xh[i % V], lh[i % V], T, oh)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        K.moe_forward_host(i % L, xh[i % V], lh[i % V], T, oh)
    e2e_s = time.perf_counter() - t0
    # nvidia-smi samples every 100 ms: keep the same load running (untimed) until the window holds enough samples
    while time.time() - t_load0 < 2.0:
        for _ in range(8):
            graph.replay()
        torch.cuda.synchronize()
    clocks = sampler.stop(window=(t_load0, time.time())) if emit else sampler.peek(window=(t_load0, time.time()))

    # max over ranks
    times = torch.tensor([ms_total, e2e_s * 1e3, gu_ms_mean], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, gu_ms_mean = (float(v) for v in times.tolist())

    line = None
    if rank == 0:
        peak, peak_kind = measured_peaks()
        tokens = T * args.steps * world
        value = tokens / (ms_total * 1e-3)
        gu_bytes = u_mean * 2 * GATE_EXPERT_BYTES
        achieved = gu_bytes / (gu_ms_mean * 1e-3) / 1e9
        layer_gbs = u_mean * EXPERT_BYTES * world / (ms_total / args.steps * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x 2-bit codes, f32 accumulate", "data": "synthetic",
            "config": {"workload": workload, "tokens_per_step_per_gpu": T, "top_k": TOP_K, "n_expert": N_EXPERT,
                       "n_embd": N_EMBD, "n_ff": N_FF, "layout": args.layout,
                       "parallelism": "single GPU" if world == 1 else f"{world} independent replicas",
                       "l2": f"inputs rotate over {L} layers x {V} routings; packed bytes between reuse >> 126 MB L2",
                       "distinct_experts_per_step": u_mean},
            "packed_weight_gbs": layer_gbs,
            "packed_weight_frac_of_measured_hbm": layer_gbs / world / peak,
            "packed_weight_frac_of_8000": layer_gbs / world / 8000.0,
            "roofline": {"bound": "hbm", "kernel": "gate_up_x16_kernel (IQ2_XXS gate+up+SwiGLU)", "achieved": achieved,
                         "peak": peak, "peak_kind": f"of {peak_kind}", "unit": "GB/s", "frac": achieved / peak,
                         "traffic": ncu_traffic(workload)[0], "traffic_source": ncu_traffic(workload)[1], "algorithmic_bytes_per_launch": gu_bytes,
                         "avg_launch_ms": gu_ms_mean},
            "roofline_down": {"bound": "hbm", "kernel": "down_m8_kernel (Q2_K down + slot sum)",
                              "achieved": u_mean * DOWN_EXPERT_BYTES / (dn_ms_mean * 1e-3) / 1e9, "peak": peak,
                              "unit": "GB/s", "frac": u_mean * DOWN_EXPERT_BYTES / (dn_ms_mean * 1e-3) / 1e9 / peak,
                              "avg_launch_ms": dn_ms_mean},
            "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": T * (N_EMBD + N_EXPERT) * 4, "d2h_bytes_per_step": T * N_EMBD * 4},
            "gpu_launches": launches, "timed_with": f"CUDA graph of {G} steps replayed {args.steps // G} times",
            "clocks": clocks,
        }
        if emit and world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(workload)
        if emit and world == 1 and not args.no_ref_mapping:
            line["ref_mapping_gpu"] = ref_mapping_gpu(torch, device, K, T, ms_total / args.steps)
        if emit:
            print(json.dumps(line), flush=True)
    return line




T_START = time.time()


def progress(rank: int, msg: str):
    """Stage marks of a multi-rank run on stderr (the JSON line owns stdout): if a run stops, its log says where."""
    if rank == 0:
        print(f"[bench {time.time() - T_START:6.1f}s] {msg}", file=sys.stderr, flush=True)


def start_watchdog(args, rank: int, world: int):
    """Multi-rank runs only. A collective whose peer never arrives blocks inside a library call; this thread lets the
    job end with a line that says so (value null: nothing was measured) instead of hanging until someone kills it."""

    def give_up():
        time.sleep(args.watchdog_s)
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": None, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                              "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True,
                              "error": f"the {world}-rank run did not finish within {args.watchdog_s} s "
                                       "(a rank or a collective never arrived); nothing was measured"}), flush=True)
        os._exit(4)

    threading.Thread(target=give_up, daemon=True).start()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=0, help="timed steps (default 200, or 20 for the prefill workload)")
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layout", default="rowsoa", choices=["rowsoa", "native"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-ref-mapping", action="store_true", help="skip the GPU baseline (restated reference mapping)")
    ap.add_argument("--no-decode-block", action="store_true", help="prefill workload: skip the batch 1 / 8 / 64 decode block")
    ap.add_argument("--ep-replicate", type=int, default=32, choices=[0, 32, 64],
                    help="N > 1: this many of the most popular experts are held by every rank (0 = pure sharding)")
    ap.add_argument("--watchdog-s", type=int, default=240, help="N > 1: give up (error line, exit 4) when the run has not "
                    "finished after this many seconds, instead of waiting on a collective for ever")
    ap.add_argument("--layers", type=int, default=0, help="layers to rotate over (0 = the workload's default; 1 keeps "
                    "device memory small for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.steps <= 0:
        args.steps = 20 if WORKLOADS[args.workload]["tokens"] >= 1024 else 200
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if args.steps <= 0:
            args.steps = 5
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    from deepseek_rs_b200.kernels import LAYOUT_NATIVE, LAYOUT_ROWSOA, MoeKernels

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        # The exchanges here are kernel stores into peer memory plus tiny all-gathers, so NCCL's in-switch (NVLS) paths
        # buy nothing; leaving them off keeps communicator set-up independent of the switch's multicast state.
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        start_watchdog(args, rank, world)
        progress(rank, f"starting the process group ({world} ranks)")
        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=args.watchdog_s))
        progress(rank, "process group up")

    sampler = ClockSampler(local_rank)
    sampler.start()  # started early (nvidia-smi takes a while to come up); samples are filtered to the load window
    wl = WORKLOADS[args.workload]
    if args.workload == "shared_expert":
        run_shared(args, torch, dist, MoeKernels(device=local_rank, max_tokens=64), device, rank, world, sampler)
        if world > 1:
            dist.destroy_process_group()
        return
    if args.workload == "fp8_linear":
        run_fp8(args, torch, dist, MoeKernels(device=local_rank, max_tokens=1), device, rank, world, sampler)
        if world > 1:
            dist.destroy_process_group()
        return
    if wl["tokens"] >= 1024 and world > 1:
        run_prefill_ep(args, torch, dist, device, rank, world, local_rank, sampler, wl["tokens"])
        dist.destroy_process_group()
        return
    T, L = wl["tokens"], (args.layers if args.layers > 0 else wl["layers"])
    K = MoeKernels(device=local_rank, max_tokens=T, max_layers=L)
    layout = LAYOUT_ROWSOA if args.layout == "rowsoa" else LAYOUT_NATIVE
    layers = []
    for il in range(L):
        gate, up, down = gen_layer_gpu(torch, device, seed=1000 * rank + il)
        if layout == LAYOUT_ROWSOA:
            g2, u2, d2 = torch.empty_like(gate), torch.empty_like(up), torch.empty_like(down)
            K.relayout_iq2xxs(gate, g2, N_EXPERT * N_FF, N_EMBD // 256)
            K.relayout_iq2xxs(up, u2, N_EXPERT * N_FF, N_EMBD // 256)
            K.relayout_q2k(down, d2, N_EXPERT * N_EMBD, N_FF // 256)
            torch.cuda.synchronize()
            gate, up, down = g2, u2, d2
        K.layer_register(il, gate, up, down, layout)
        layers.append((gate, up, down))

    if wl["tokens"] >= 1024:
        run_prefill(args, torch, dist, K, layers, layout, device, rank, world, sampler, T, L)
        if world > 1:
            dist.destroy_process_group()
        return

    run_decode(args, torch, dist, K, layers, layout, device, rank, world, sampler, T, L, args.workload)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

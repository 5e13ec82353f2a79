#!/usr/bin/env python
"""MoE-layer throughput benchmark.

  python bench.py --gpus N --steps K --warmup W [--workload c1] [--tokens T]

A step is one pass of the MoE layer over one batch of synthetic tokens.  Prints ONE JSON line
(rank 0).  `value` is tokens/s with the inputs resident in HBM; `e2e` is the same metric through
the host-buffer entry point (pinned host activations in, fp32 result out, copies inside the
timed region); `roofline` describes the dominant kernel, timed live with CUDA events on the
stream it is launched on; `cpu_baseline` times the reference's own CPU expert kernels
(oracle/_ref) on this box's host cores on a bounded sample.

  python bench.py --impl reference ...   times only that CPU arm.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np
import torch


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]),
                    bf16_tflops_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(np.max(mx)) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def measured_traffic(workload, tokens, kernel):
    """DRAM bytes per launch of `kernel` from the committed ncu summary (profiles/traffic.json), or None."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        table = json.load(f)
    return table.get(f"{workload}/T{tokens}/{kernel}")


def expert_weight_bytes(cfg):
    from strata_b200 import synth
    return sum(sum(synth.expert_bytes(cfg, r)) for r in synth.ROLES)


def gate_up_bytes(cfg):
    from strata_b200 import synth
    return sum(sum(synth.expert_bytes(cfg, r)) for r in ("gate", "up"))


# ------------------------------------------------------------------------------ CPU arm
def cpu_reference_run(cfg, T, sample_pairs_budget_s=15.0, threads=None):
    """Times the reference's CPU expert kernels on a bounded sample of the workload's
    (token, expert) pairs with every host core; returns (tokens_per_s, info)."""
    from oracle import oracle as O
    from strata_b200 import synth
    from tests import helpers as Hh
    ref = O.ref()
    threads = threads or len(os.sched_getaffinity(0))
    x = synth.gen_inputs(cfg, T)
    w, b = synth.gen_router(cfg)
    logits = O.router_logits(Hh.np_u16(x), Hh.np_u16(w))
    spec = O.router_spec(cfg.E, cfg.k, cfg.score_kind, cfg.normalize, cfg.norm_init, cfg.weight_scale)
    rc, ids, wts = O.route(spec, logits, b.numpy() if b is not None else None)
    assert rc == 0
    # bounded sample: the pairs of the first n_tok tokens, n_tok grown until the budget is met
    flops_per_pair = 6.0 * cfg.H * cfg.I
    est_rate = 2.0e9 * threads * (0.15 if cfg.fmt == synth.FMT_NVFP4 else 1.0)  # scalar NVFP4 is slow
    n_tok = int(max(1, min(T, sample_pairs_budget_s * est_rate / (flops_per_pair * cfg.k))))
    sub_ids = ids[:n_tok]
    counts, offsets, perm = O.group(sub_ids, cfg.E)
    pair_token = (perm // cfg.k).astype(np.uint32)
    needed = np.nonzero(counts)[0]
    ptrs = (O.RefExpertPtrs * cfg.E)()
    keep = []
    for e in needed:
        vals = {}
        for role in synth.ROLES:
            p, s = synth.gen_expert_range(cfg, role, int(e), int(e) + 1, "cpu")
            p, s = np.ascontiguousarray(p[0].numpy()), np.ascontiguousarray(s[0].numpy())
            keep += [p, s]
            vals[role] = (p.ctypes.data, s.ctypes.data)
        ptrs[e].gate_packed, ptrs[e].gate_scales = vals["gate"]
        ptrs[e].up_packed, ptrs[e].up_scales = vals["up"]
        ptrs[e].down_packed, ptrs[e].down_scales = vals["down"]
        g = synth.NVFP4_GLOBAL if cfg.fmt == synth.FMT_NVFP4 else {"gate": 1.0, "up": 1.0, "down": 1.0}
        ptrs[e].gate_global, ptrs[e].up_global, ptrs[e].down_global = g["gate"], g["up"], g["down"]
    xf = np.ascontiguousarray(x.float().numpy())
    y = np.empty((len(perm), cfg.H), np.float32)
    passes = 1
    if ref is not None:
        def one_pass():
            ns = ref.ref_cpu_experts(cfg.fmt, cfg.H, cfg.I, cfg.E, ptrs, xf.ctypes.data_as(O.f32p),
                                     offsets.ctypes.data_as(O.u32p), pair_token.ctypes.data_as(O.u32p),
                                     y.ctypes.data_as(O.f32p), threads)
            assert ns > 0
            return ns * 1e-9
        kind = "reference"
        secs = one_pass()
        # a whole workload that takes well under the budget is repeated and the passes averaged
        if n_tok == T and secs < sample_pairs_budget_s / 8:
            passes = int(min(50, max(2, sample_pairs_budget_s / 2 / max(secs, 1e-4))))
            secs = float(np.mean([one_pass() for _ in range(passes)]))
    else:
        # compiled reference missing on this machine: time the plain-C restatement instead
        kind = "port"
        experts, keep2 = Hh.oracle_experts(cfg, needed)
        desc = Hh.oracle_desc(cfg, n_tok)
        t0 = time.perf_counter()
        rc = O.port().orc_experts_all(desc, Hh.np_u16(x).ctypes.data_as(O.u16p), experts,
                                      sub_ids.ctypes.data_as(O.u32p),
                                      np.ascontiguousarray(wts[:n_tok]).ctypes.data_as(O.f32p),
                                      offsets.ctypes.data_as(O.u32p), perm.ctypes.data_as(O.u32p),
                                      y.ctypes.data_as(O.f32p))
        secs = time.perf_counter() - t0
        assert rc == 0
    bytes_read = float(len(needed)) * expert_weight_bytes(cfg)
    info = dict(kind=kind, cores=threads, sample=f"{n_tok} of {T} tokens ({len(perm)} token-expert rows over "
                f"{len(needed)} experts), routed experts only, mean of {passes} pass(es), {secs:.3f} s each",
                eff_gbs=bytes_read / secs / 1e9)
    return n_tok / secs, info


# ------------------------------------------------------------------------------ GPU arm
def l2_flush_buffer(device):
    return torch.empty(512 << 20, dtype=torch.uint8, device=device)


def run_gpu(args, cfg, T, rank, world):
    from strata_b200 import MoeContext, MoeLayer, synth
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(device)
    peaks = load_peaks()
    if world > 1:
        from strata_b200 import ep
        return ep.bench(args, cfg, T, rank, world, device, peaks, ClockSampler)

    ctx = MoeContext(device.index)
    torch.cuda.set_stream(ctx.stream)   # flushes, events and the library share one stream
    layer = synth.build_layer(cfg, device, T=T)
    ml = MoeLayer(ctx, cfg, max_tokens=T)
    ml.load_synth(layer)
    out = torch.empty(T, cfg.H, dtype=torch.float32, device=device)
    flush = l2_flush_buffer(device)
    x_host = layer.x.cpu().pin_memory()
    out_host = torch.empty(T, cfg.H, dtype=torch.float32).pin_memory()

    def step():
        ml.forward(layer.x, out)

    sampler = ClockSampler(device.index)     # samples clocks and throttle reasons from the warm-up on
    sampler.start()
    for _ in range(max(args.warmup, 3)):
        flush.zero_()
        step()
    ctx.synchronize()

    launches0 = ctx.stats().kernel_launches
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(args.steps)]
    torch.cuda.synchronize()
    for a, b in evs:
        flush.zero_()          # evict the weights from L2 between timed iterations
        a.record()
        step()
        b.record()
    torch.cuda.synchronize()
    launches = ctx.stats().kernel_launches - launches0
    ms = [a.elapsed_time(b) for a, b in evs]
    ms_per_step = float(np.mean(ms))

    # phase timing (separate iterations: the phase events serialise the host)
    ctx.set_timing(True)
    phase = []
    for _ in range(min(args.steps, 20)):
        flush.zero_()
        step()
        phase.append(ctx.phase_ms())
    ctx.set_timing(False)
    phase_ms = {k: float(np.median([p[k] for p in phase])) for k in phase[0]}

    # end to end through the host-buffer entry point
    for _ in range(3):
        ml.forward_host(x_host, out_host)
    e2e_t = []
    for _ in range(args.steps):
        flush.zero_()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        ml.forward_host(x_host, out_host)
        e2e_t.append(time.perf_counter() - t0)
    # the timed regions above are short: keep the same load running until the clock log has a few samples
    deadline = time.perf_counter() + 2.0
    while len(sampler.rows) < 6 and time.perf_counter() < deadline:
        flush.zero_()
        step()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    e2e_s = float(np.mean(e2e_t))

    # roofline of the dominant kernel
    _, aux = ml.forward(layer.x, want_aux=True)
    ctx.synchronize()
    counts = aux["counts"].cpu().numpy()
    active = int((counts > 0).sum())
    pairs = T * cfg.k
    dominant = max(("gate_up", "down"), key=lambda k: phase_ms[k])
    if dominant == "gate_up":
        alg_bytes = active * gate_up_bytes(cfg) + pairs * cfg.H * 2 + pairs * cfg.I * 4
    else:
        alg_bytes = active * (expert_weight_bytes(cfg) - gate_up_bytes(cfg)) + pairs * cfg.I * 4 + pairs * cfg.H * 4
    flops = 2.0 * pairs * cfg.H * cfg.I * (2 if dominant == "gate_up" else 1)
    hbm_time = alg_bytes / (peaks["hbm_gbs"] * 1e9)
    tc_time = flops / (peaks["bf16_tflops"] * 1e12)
    dur = phase_ms[dominant] * 1e-3
    if hbm_time >= tc_time:
        roof = dict(bound="hbm", achieved=alg_bytes / dur / 1e9, peak=peaks["hbm_gbs"], unit="GB/s")
    else:
        roof = dict(bound="tensor", achieved=flops / dur / 1e12, peak=peaks["bf16_tflops"], unit="TFLOP/s")
    roof["frac"] = roof["achieved"] / roof["peak"]
    roof.update(traffic=measured_traffic(cfg.name, T, dominant), kernel=dominant, kernel_ms=phase_ms[dominant], peak_source=peaks["source"],
                active_experts=active, algorithmic_bytes=int(alg_bytes))
    layer_bytes = active * expert_weight_bytes(cfg) + cfg.E * cfg.H * 2 + 3 * cfg.I_shared * cfg.H * 2

    # batch sweep of the same layer (config 1 names 1/4/16/64/256 tokens): tokens/s and the
    # fraction of HBM peak the whole layer reaches on its algorithmic bytes
    sweep = []
    if args.sweep:
        for Ts in [t for t in (1, 4, 16, 64, 256) if t <= T]:
            xs = layer.x[:Ts].contiguous()
            outs = torch.empty(Ts, cfg.H, dtype=torch.float32, device=device)
            for _ in range(3):
                flush.zero_()
                ml.forward(xs, outs)
            ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(10)]
            for a, b in ev:
                flush.zero_()
                a.record()
                ml.forward(xs, outs)
                b.record()
            torch.cuda.synchronize()
            t_ms = float(np.mean([a.elapsed_time(b) for a, b in ev]))
            _, ax = ml.forward(xs, want_aux=True)
            ctx.synchronize()
            act_s = int((ax["counts"] > 0).sum().item())
            lb = act_s * expert_weight_bytes(cfg) + cfg.E * cfg.H * 2 + 3 * cfg.I_shared * cfg.H * 2
            sweep.append({"tokens": Ts, "ms": t_ms, "tokens_per_s": Ts / (t_ms * 1e-3), "active_experts": act_s,
                          "layer_hbm_frac": lb / (t_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]})

    cpu_v, cpu_info = cpu_reference_run(cfg, T, args.cpu_seconds)
    line = {
        "metric": "MoE layer tokens/s", "value": T / (ms_per_step * 1e-3), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (seeded hash weights, N(0,1) BF16 activations, random-init router)",
        "config": {"workload": f"{cfg.name}: {cfg.description}", "tokens": T, "hidden": cfg.H,
                   "intermediate": cfg.I, "experts": cfg.E, "top_k": cfg.k,
                   "format": ["mxfp4", "nvfp4", "int4g128"][cfg.fmt], "shared_intermediate": cfg.I_shared,
                   "l2": "512 MiB buffer rewritten between timed iterations"},
        "layer_hbm_gbs": layer_bytes / (ms_per_step * 1e-3) / 1e9,
        "layer_hbm_frac": layer_bytes / (ms_per_step * 1e-3) / 1e9 / peaks["hbm_gbs"],
        "phase_ms": phase_ms,
        "sweep": sweep,
        "roofline": roof,
        "cpu_baseline": {"value": cpu_v, "unit": "tokens/s", **cpu_info},
        "e2e": {"value": T / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": T * cfg.H * 2,
                "d2h_bytes_per_step": T * cfg.H * 4},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None)
    ap.add_argument("--tokens", type=int, default=None)
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-sweep", dest="sweep", action="store_false", help="skip the batch sweep")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="multi-GPU row exchange: the library's peer-memory kernels or NCCL all-to-allv")
    ap.add_argument("--scaling", default=None, choices=["weak", "strong"],
                    help="multi-GPU: weak = --tokens per rank (default), strong = --tokens in total")
    args = ap.parse_args()
    from strata_b200 import synth
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    name = args.workload or "c1"
    cfg = synth.CONFIGS[name]
    T = args.tokens or cfg.T
    if args.scaling is None:
        args.scaling = "strong" if name in ("c2", "c3", "c4") else "weak"

    if args.impl == "reference":
        if rank != 0:
            return 0
        vals, info = [], None
        for _ in range(max(1, min(args.steps, 3))):
            v, info = cpu_reference_run(cfg, T, args.cpu_seconds)
            vals.append(v)
        v = float(np.mean(vals))
        print(json.dumps({
            "impl": "reference", "metric": "MoE layer tokens/s", "value": v, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": len(vals), "warmup": 0, "ms_per_step": 1e3 * T / v,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"workload": f"{cfg.name}: {cfg.description}", "tokens": T},
            "cpu_baseline": {"value": v, "unit": "tokens/s", **info},
            "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return 0

    line = run_gpu(args, cfg, T, rank, world)
    if rank == 0 and line is not None:
        print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())

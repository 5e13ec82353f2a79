#!/usr/bin/env python
"""MoE-layer throughput benchmark.

  python bench.py --gpus N --steps K --warmup W [--workload c3] [--tokens T]

A step is one pass of the MoE layer over one batch of synthetic tokens.  Prints ONE JSON line
(rank 0).  The default workload is the expert-parallel MXFP4 prefill configuration (c3: hidden
7168, 256 experts, top-8, 16384 tokens) at EVERY N including 1, strong scaling (the token count is
the whole job's; rank r owns tokens [r T/N, (r+1) T/N) and experts [r E/N, (r+1) E/N)), so that
the 1-GPU line, the scaling curve and the prefill target are one workload.

  value      tokens/s with the inputs resident in HBM (CUDA events, max over ranks per step)
  e2e        the same metric through the host-buffer call (pinned host activations in, fp32 result
             out, both copies inside the timed region)
  roofline   the dominant kernel of the main workload, timed live with CUDA events on the library's
             stream, against the measured peaks
  parity     the timed layer's output for a few tokens against the CPU oracle (ids bit-exact)
  cpu_baseline  the reference's own CPU expert kernels (oracle/_ref) on this box's host cores,
             bounded sample
  sub        (N = 1) the other benchmark configurations, each with its own roofline / e2e /
             cpu_baseline: c0 at 8 tokens (decode, HBM target), the c1_sigmoid batch sweep
             1/4/16/64/256 (the reference's Laguna routing rule; the softmax variant is a second
             arm), c2 at 4096 tokens (prefill, tensor target); (N = 8) c4 with per-rank max latency
  stage_ms_rank0  (N > 1) rank 0's four stages of an expert-parallel step (CUDA events)
  exchange   (N > 1) token rows per token that cross NVLink each way, read back from the library's counters
  host_placement  (N > 1) per rank: the NUMA node of its GPU and whether the rank confined itself to that node's
             CPUs before allocating its pinned staging buffers (strata_b200/hostmem.py; --no-numa leaves it alone)

  python bench.py --impl reference ...   times only the CPU arm on the main workload.
"""
import argparse
import gc
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

FMT_NAMES = ["mxfp4", "nvfp4", "int4g128", "bf16"]
DATA = "synthetic (seeded hash weights, N(0,1) BF16 activations, random-init router)"
L2_NOTE = ("512 MiB buffer rewritten, then 256 MiB of another buffer read, between timed iterations: the inputs are cold and "
           "L2 holds clean lines (a step is not charged the write-back of the flush's own dirty lines)")


class L2Flush:
    """Evicts everything the layer touched from L2: a write pass over 512 MiB (larger than the 126 MB L2), then a read
    pass over 256 MiB of a second buffer, so that what L2 holds afterwards is clean.  After the write pass alone L2 is
    full of the flush's dirty lines and the first ~126 MB a kernel reads would each pay for a write-back that is not
    the kernel's traffic (measured: a 352 MB read-only pass takes 71 us after the write pass alone, 58 us after both)."""

    def __init__(self, device):
        self.w = torch.empty(512 << 20, dtype=torch.uint8, device=device)
        self.r = torch.zeros((256 << 20) // 4, dtype=torch.int32, device=device)
        self.sink = None

    def zero_(self):
        self.w.zero_()
        self.sink = self.r.sum()


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


def reference_gpu_commands():
    """The reference's own CUDA backend (compiled unmodified for sm_100a by oracle/build.py, a checker like the CPU arm)
    and this library, each timing the same GLM INT4 MoE command -- 8 routed experts applied to R rows at hidden 6144 /
    intermediate 2048, host fp32 rows in and out, wall clock around enqueue + collect -- through the same C++ program
    (tests/cpp/backend_shim_test.cpp --time).  None when the prebuilt reference executable did not travel."""
    import re
    import tempfile
    ref_exe = os.path.join(ROOT, "oracle", "_ref", "backend_shim_test_ref")
    if not os.path.exists(ref_exe):
        return None
    pat = re.compile(r"(\d+) experts x (\d+) rows: ([0-9.]+) ms per command")

    def run(exe):
        r = subprocess.run([exe, "--time"], capture_output=True, text=True, timeout=300)
        if r.returncode != 0:
            return None
        return {int(m.group(2)): float(m.group(3)) for m in pat.finditer(r.stdout)}
    try:
        ref = run(ref_exe)
        with tempfile.TemporaryDirectory() as tmp:
            ours_exe = os.path.join(tmp, "shim_time")
            lib_dir, orc_dir = os.path.join(ROOT, "strata_b200"), os.path.join(ROOT, "oracle")
            c = subprocess.run(["g++", "-std=c++20", "-O1", "-I", os.path.join(ROOT, "include"),
                                os.path.join(ROOT, "tests", "cpp", "backend_shim_test.cpp"), "-o", ours_exe,
                                "-L", lib_dir, "-lstrata_moe", "-L", orc_dir, "-lmoe_oracle",
                                f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{orc_dir}"], capture_output=True, text=True)
            ours = run(ours_exe) if c.returncode == 0 else None
    except (OSError, subprocess.SubprocessError):
        return None
    if not ref or not ours:
        return None
    return {"what": "GLM INT4 MoE command, 8 routed experts x R rows, hidden 6144 / intermediate 2048, host fp32 rows in and out, "
                    "wall clock around enqueue + collect, best of 5; the reference's CUDA backend compiled unmodified for sm_100a "
                    "against this library through the C++ shim, same program",
            "rows": sorted(ref), "reference_ms": [ref[r] for r in sorted(ref)],
            "this_library_ms": [ours.get(r) for r in sorted(ref)],
            "speedup": [round(ref[r] / ours[r], 2) if ours.get(r) else None for r in sorted(ref)]}


def expert_weight_bytes(cfg):
    from strata_b200 import synth
    return sum(sum(synth.expert_bytes(cfg, r)) for r in synth.ROLES)


def gate_up_bytes(cfg):
    from strata_b200 import synth
    return sum(sum(synth.expert_bytes(cfg, r)) for r in ("gate", "up"))


def config_dict(cfg, T, **extra):
    d = {"workload": f"{cfg.name}: {cfg.description}", "tokens": T, "hidden": cfg.H,
         "intermediate": cfg.I, "experts": cfg.E, "top_k": cfg.k, "format": FMT_NAMES[cfg.fmt],
         "shared_intermediate": cfg.I_shared, "l2": L2_NOTE}
    d.update(extra)
    return d


# ------------------------------------------------------------------------------ CPU arm
def cpu_reference_run(cfg, T, sample_pairs_budget_s=15.0, threads=None, repeats=1):
    """Times the reference's CPU expert kernels on a bounded sample of the workload's
    (token, expert) pairs with every host core; returns (tokens_per_s, info)."""
    from oracle import layer_check as Hh
    from oracle import oracle as O
    from strata_b200 import synth
    ref = O.ref()
    threads = threads or len(os.sched_getaffinity(0))
    # bounded sample: the pairs of the first n_tok tokens (routing is only computed for those)
    flops_per_pair = 6.0 * cfg.H * cfg.I
    est_rate = 2.0e9 * threads * (0.15 if cfg.fmt == synth.FMT_NVFP4 else 1.0)  # scalar NVFP4 is slow
    n_tok = int(max(1, min(T, sample_pairs_budget_s * est_rate / (flops_per_pair * cfg.k))))
    x = synth.gen_inputs(cfg, T)[:n_tok].contiguous()
    w, b = synth.gen_router(cfg)
    logits = O.router_logits(Hh.np_u16(x), Hh.np_u16(w))
    spec = O.router_spec(cfg.E, cfg.k, cfg.score_kind, cfg.normalize, cfg.norm_init, cfg.weight_scale)
    rc, ids, wts = O.route(spec, logits, b.numpy() if b is not None else None)
    assert rc == 0
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
        secs = float(np.mean([one_pass() for _ in range(max(1, repeats))]))
        passes = max(1, repeats)
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


# ------------------------------------------------------------------------------ parity inside the bench
def oracle_parity(cfg, x_cpu, ids_gpu, out_rows, subset):
    """The timed layer against the CPU oracle: ids of all `x_cpu` tokens bit for bit, output rows of
    `subset` (out_rows[i] belongs to token subset[i]) within the layer tolerance."""
    from oracle import layer_check as Hh
    ref = Hh.run_oracle(cfg, x_cpu, token_subset=np.asarray(subset, np.uint32))
    rel, mx = Hh.error_metrics(out_rows, ref["out"])
    ids_equal = bool(np.array_equal(np.asarray(ids_gpu).astype(np.uint32), ref["ids"]))
    return {"rel_l2": float(rel), "max_abs_rms": float(mx), "ids_equal": ids_equal,
            "tokens_checked": int(len(subset)), "ids_checked": int(ref["ids"].shape[0]),
            "bars": {"rel_l2": 1e-2, "max_abs_rms": 2.0 ** -6},
            "ok": bool(ids_equal and rel <= 1e-2 and mx <= 2.0 ** -6)}


# ------------------------------------------------------------------------------ single GPU
def roofline_of(cfg, T, active, phase_ms, peaks):
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
        # against the BURST cuBLAS figure (the stricter one); the kernel runs inside a many-step loop under the power cap,
        # where cuBLAS itself settles at the sustained figure, reported beside it
        roof = dict(bound="tensor", achieved=flops / dur / 1e12, peak=peaks["bf16_tflops"], unit="TFLOP/s",
                    peak_sustained=peaks["bf16_tflops_sustained"],
                    frac_of_sustained=flops / dur / 1e12 / peaks["bf16_tflops_sustained"])
    roof["frac"] = roof["achieved"] / roof["peak"]
    roof.update(traffic=measured_traffic(cfg.name, T, dominant), kernel=dominant, kernel_ms=phase_ms[dominant],
                peak_source=peaks["source"], active_experts=active, algorithmic_bytes=int(alg_bytes),
                algorithmic_flops=float(flops))
    return roof


def measure_layer(ctx, cfg, T, steps, warmup, peaks, flush, cpu_seconds, want_parity=False, batch_sweep=(),
                  sampler=None):
    """One configuration on one GPU: device-resident throughput, phases, end to end, roofline, CPU arm."""
    from strata_b200 import MoeLayer, synth
    device = ctx.device
    layer = synth.build_layer(cfg, device, T=T)
    ml = MoeLayer(ctx, cfg, max_tokens=T)
    ml.load_synth(layer)
    out = torch.empty(T, cfg.H, dtype=torch.float32, device=device)
    x_host = layer.x.cpu().pin_memory()
    out_host = torch.empty(T, cfg.H, dtype=torch.float32).pin_memory()

    def step():
        ml.forward(layer.x, out)

    for _ in range(max(warmup, 3)):
        flush.zero_()
        step()
    ctx.synchronize()
    st0 = ctx.stats()
    launches0 = st0.kernel_launches
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    torch.cuda.synchronize()
    for a, b in evs:
        flush.zero_()          # evict the weights from L2 between timed iterations
        a.record()
        step()
        b.record()
    torch.cuda.synchronize()
    st1 = ctx.stats()
    launches = st1.kernel_launches - launches0
    router_stats = {"fast_tokens_per_step": (st1.router_fast_tokens - st0.router_fast_tokens) / steps,
                    "rechecked_tokens_per_step": (st1.router_rechecked_tokens - st0.router_rechecked_tokens) / steps}
    ms_per_step = float(np.mean([a.elapsed_time(b) for a, b in evs]))

    # phase timing (separate iterations: the phase events serialise the host)
    ctx.set_timing(True)
    phase = []
    for _ in range(min(steps, 20)):
        flush.zero_()
        step()
        phase.append(ctx.phase_ms())
    ctx.set_timing(False)
    phase_ms = {k: float(np.median([p[k] for p in phase])) for k in phase[0]}

    # end to end through the host-buffer entry point
    for _ in range(3):
        ml.forward_host(x_host, out_host)
    e2e_t = []
    for _ in range(steps):
        flush.zero_()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        ml.forward_host(x_host, out_host)
        e2e_t.append(time.perf_counter() - t0)
    if sampler is not None:
        # the timed regions above can be short: keep the same load running until the clock log has a few samples
        deadline = time.perf_counter() + 2.0
        while len(sampler.rows) < 6 and time.perf_counter() < deadline:
            flush.zero_()
            step()
            torch.cuda.synchronize()
    e2e_s = float(np.mean(e2e_t))

    _, aux = ml.forward(layer.x, want_aux=True)
    ctx.synchronize()
    counts = aux["counts"].cpu().numpy()
    active = int((counts > 0).sum())
    rec = {
        "value": T / (ms_per_step * 1e-3), "unit": "tokens/s", "ms_per_step": ms_per_step,
        "config": config_dict(cfg, T), "phase_ms": phase_ms,
        "roofline": roofline_of(cfg, T, active, phase_ms, peaks),
        "e2e": {"value": T / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": T * cfg.H * 2,
                "d2h_bytes_per_step": T * cfg.H * 4},
        "gpu_launches": int(launches),
        "router": router_stats,
    }
    layer_bytes = active * expert_weight_bytes(cfg) + cfg.E * cfg.H * 2 + 3 * cfg.I_shared * cfg.H * 2
    rec["layer_hbm_gbs"] = layer_bytes / (ms_per_step * 1e-3) / 1e9
    rec["layer_hbm_frac"] = rec["layer_hbm_gbs"] / peaks["hbm_gbs"]
    rec["layer_tflops"] = 6.0 * cfg.H * cfg.I * T * cfg.k / (ms_per_step * 1e-3) / 1e12
    rec["layer_tensor_frac"] = rec["layer_tflops"] / peaks["bf16_tflops"]
    if want_parity:
        sub = sorted(set([0, T // 2, T - 1]))
        ml.forward(layer.x, out)
        ctx.synchronize()
        rec["parity"] = oracle_parity(cfg, layer.x.cpu(), aux["ids"].cpu().numpy(),
                                      out[torch.tensor(sub, device=device)].cpu().numpy(), sub)

    # batch sweep of the same layer: tokens/s and the fraction of HBM peak the whole layer reaches
    sweep = []
    for Ts in [t for t in batch_sweep if t <= T]:
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
        ctx.set_timing(True)
        ph = []
        for _ in range(5):
            flush.zero_()
            ml.forward(xs, outs)
            ph.append(ctx.phase_ms())
        ctx.set_timing(False)
        ph_ms = {k: float(np.median([p[k] for p in ph])) for k in ph[0]}
        _, ax = ml.forward(xs, want_aux=True)
        ctx.synchronize()
        act_s = int((ax["counts"] > 0).sum().item())
        lb = act_s * expert_weight_bytes(cfg) + cfg.E * cfg.H * 2 + 3 * cfg.I_shared * cfg.H * 2
        sweep.append({"tokens": Ts, "ms": t_ms, "tokens_per_s": Ts / (t_ms * 1e-3), "active_experts": act_s,
                      "layer_hbm_frac": lb / (t_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                      "roofline": roofline_of(cfg, Ts, act_s, ph_ms, peaks)})
    if sweep:
        rec["sweep"] = sweep
    ml.close()
    del layer, ml, out, aux
    gc.collect()
    torch.cuda.empty_cache()
    if cpu_seconds > 0:
        cpu_v, cpu_info = cpu_reference_run(cfg, T, cpu_seconds)
        rec["cpu_baseline"] = {"value": cpu_v, "unit": "tokens/s", **cpu_info}
    return rec


def run_single(args, cfg, T):
    from strata_b200 import MoeContext, synth
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(device)
    peaks = load_peaks()
    ctx = MoeContext(device.index)
    torch.cuda.set_stream(ctx.stream)   # flushes, events and the library share one stream
    flush = L2Flush(device)
    sampler = ClockSampler(device.index)     # samples clocks and throttle reasons from the warm-up on
    sampler.start()
    main = measure_layer(ctx, cfg, T, args.steps, args.warmup, peaks, flush, args.cpu_seconds,
                         want_parity=args.parity, sampler=sampler,
                         batch_sweep=(1, 4, 16, 64, 256) if cfg.name.startswith("c1") and args.sub else ())
    clocks = sampler.stop()
    sub = []
    if args.sub:
        sub_steps = max(5, min(args.steps, 20))
        sub_cpu = min(args.cpu_seconds, 4.0)
        plan = [("c0", 8, ()), ("c1_sigmoid", 256, (1, 4, 16, 64, 256)), ("c1", 256, ()), ("c2", 4096, ()),
                ("c3", 16384, ())]
        for name, Ts, sweep in plan:
            if name == cfg.name and Ts == T:
                continue
            rec = measure_layer(ctx, synth.CONFIGS[name], Ts, sub_steps, 3, peaks, flush, sub_cpu,
                                want_parity=args.parity, batch_sweep=sweep)
            rec["name"], rec["steps"] = name, sub_steps
            sub.append(rec)
    line = {
        "metric": "MoE layer tokens/s", "value": main["value"], "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": main["ms_per_step"],
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "bf16", "data": DATA,
        "config": dict(main["config"], parallelism="ep1"),
    }
    for k in ("layer_hbm_gbs", "layer_hbm_frac", "layer_tflops", "layer_tensor_frac", "phase_ms", "roofline",
              "cpu_baseline", "e2e", "gpu_launches", "router", "parity", "sweep"):
        if k in main:
            line[k] = main[k]
    line["clocks"] = clocks
    if sub:
        line["sub"] = sub
    if args.sub:
        ref_gpu = reference_gpu_commands()
        if ref_gpu:
            line["reference_gpu"] = ref_gpu
    return line


# ------------------------------------------------------------------------------ multi GPU
def measure_ep(args, cfg, T, rank, world, device, ctx, peaks, flush, strong, want_parity, sampler=None):
    """One layer over `world` ranks, E/world experts per rank.  Strong scaling: T tokens in total,
    T/world per rank.  Weak: T tokens per rank.  Returns the record (every rank; rank 0 prints)."""
    import torch.distributed as dist
    from strata_b200 import MoeLayer, synth
    from strata_b200.ep import EpMoe, EpMoePeer, owner_block
    if strong:
        assert T % world == 0
        Tl = T // world
    else:
        Tl, T = T, T * world
    B = owner_block(cfg, world)
    pairs_total = T * cfg.k
    avg = pairs_total // world
    max_pairs = min(pairs_total, max(2 * avg, avg + 4096))
    layer = synth.build_layer(cfg, device, expert_begin=rank * B, expert_end=(rank + 1) * B, T=T)
    x_local = layer.x[rank * Tl:(rank + 1) * Tl].contiguous()
    ml = MoeLayer(ctx, cfg, max_tokens=Tl, expert_begin=rank * B, expert_count=B, max_pairs=max_pairs)
    ml.load_synth(layer)
    parts = max(1, int(getattr(args, "microbatches", 1)))
    if args.exchange == "peer" and parts > 1 and Tl >= 2 * parts:
        from strata_b200.ep import EpMoePeerPipelined

        def make_layer(c, n, cap):
            m = MoeLayer(c, cfg, max_tokens=n, expert_begin=rank * B, expert_count=B, max_pairs=cap)
            m.load_synth(layer)
            return m
        ep = EpMoePeerPipelined(make_layer, cfg, rank, world, Tl, max_pairs, parts=parts)
        exchange_text = (f"library kernels over peer memory (NVLink stores / loads, no collective on the data path), "
                         f"{parts} token micro-batches in flight")
    elif args.exchange == "peer":
        try:
            ep = EpMoePeer(ml, cfg, rank, world, max_pairs)
            exchange_text = "library kernels over peer memory (NVLink stores / loads, no collective on the data path)"
        except RuntimeError as e:    # every rank raises together; the NCCL exchange is the other GPU path
            exchange_text = f"NCCL all-to-allv (counts, rows, outputs); peer windows failed: {e}"
            ep = EpMoe(ml, cfg, rank, world)
    else:
        ep = EpMoe(ml, cfg, rank, world)
        exchange_text = "NCCL all-to-allv (counts, rows, outputs)"

    warm = max(args.warmup, 3)
    for _ in range(warm):
        flush.zero_()
        out = ep.forward(x_local)
    ctx.synchronize()
    launches0 = ctx.stats().kernel_launches
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    dist.barrier()
    torch.cuda.synchronize()
    for a, b in evs:
        flush.zero_()
        dist.barrier()
        a.record()
        out = ep.forward(x_local)
        b.record()
    torch.cuda.synchronize()
    dist.barrier()
    launches = ctx.stats().kernel_launches - launches0
    ms_local = torch.tensor([a.elapsed_time(b) for a, b in evs], device=device, dtype=torch.float64)
    ms = ms_local.clone()
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)           # per step: the slowest rank
    ms_per_step = float(ms.mean())
    per_rank_ms = [torch.zeros(1, device=device, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(per_rank_ms, ms_local.mean().reshape(1))
    ctx.synchronize()    # raises if any step tripped the device status word (overflow, timeout, non-finite)
    if hasattr(ep, "synchronize"):
        ep.synchronize()
    ids_loc, _ = ml.route(x_local)
    per_rank = torch.bincount((ids_loc.reshape(-1) // B).long(), minlength=world).double()
    dist.all_reduce(per_rank)     # rows every rank receives in one step
    recv_max = per_rank.max()

    # end to end: pinned host activations in, fp32 result out, every step
    x_host = x_local.cpu().pin_memory()
    out_host = torch.empty(Tl, cfg.H, dtype=torch.float32).pin_memory()
    x_dev = torch.empty_like(x_local)
    e2e = []
    for i in range(args.steps + 2):
        flush.zero_()
        torch.cuda.synchronize()
        dist.barrier()
        t0 = time.perf_counter()
        x_dev.copy_(x_host, non_blocking=True)
        o = ep.forward(x_dev)
        out_host.copy_(o, non_blocking=True)
        torch.cuda.synchronize()
        e2e.append(time.perf_counter() - t0)
    e2e_t = torch.tensor(e2e[2:], device=device, dtype=torch.float64)
    dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    if sampler is not None:
        t_end = time.perf_counter() + 2.0
        go = torch.ones(1, device=device)
        while True:     # same load until rank 0's clock log has a few samples (all ranks leave together)
            if rank == 0:
                go.fill_(1.0 if (len(sampler.rows) < 6 and time.perf_counter() < t_end) else 0.0)
            dist.broadcast(go, 0)
            if go.item() == 0.0:
                break
            flush.zero_()
            ep.forward(x_local)
            torch.cuda.synchronize()
    ctx.synchronize()
    # where a step's time goes: the four stages of the peer exchange, timed on this rank's stream
    # (each stage's time includes waiting for the slowest peer)
    stage_ms = None
    exchange = None
    if isinstance(ep, EpMoePeer):
        st = ep.state
        acc = torch.zeros(4, dtype=torch.float64)
        reps = 5
        for _ in range(reps):
            flush.zero_()
            dist.barrier()
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
            ev[0].record()
            st.begin(x_local)
            ev[1].record()
            st.dispatch()
            ev[2].record()
            st.experts()
            ev[3].record()
            st.finish(out)
            ev[4].record()
            torch.cuda.synchronize()
            acc += torch.tensor([ev[i].elapsed_time(ev[i + 1]) for i in range(4)], dtype=torch.float64)
        ctx.synchronize()
        stage_ms = dict(zip(("route_group_publish", "plan_dispatch", "wait_experts_signal", "wait_combine"),
                            [round(float(v), 4) for v in acc / reps]))
        # what crossed: token rows per token each way (a token counts once per owning rank), beside k rows per token
        # that an exchange per (token, expert) pair would move
        sent, _, _ = st.last_counts()
        remote = torch.tensor([float(sum(v for r, v in enumerate(sent) if r != rank)), float(sum(sent))],
                              device=device, dtype=torch.float64)
        dist.all_reduce(remote)
        exchange = {"rows_per_token_over_nvlink": round(float(remote[0].item()) / T, 3),
                    "rows_per_token_with_local": round(float(remote[1].item()) / T, 3),
                    "pairs_per_token": cfg.k, "bytes_per_row_each_way": cfg.H * 2}

    parity = None
    if want_parity:
        # rank 0's tokens against the CPU oracle (every rank takes part in the step that produces them)
        out = ep.forward(x_local)
        ctx.synchronize()
        if rank == 0:
            sub = sorted(set([0, Tl // 2, Tl - 1]))
            parity = oracle_parity(cfg, x_local.cpu(), ids_loc.cpu().numpy(),
                                   out[torch.tensor(sub, device=device)].cpu().numpy(), sub)
        dist.barrier()

    flops = 6.0 * cfg.H * cfg.I * pairs_total
    # per rank: the expert GEMMs (tensor bound for the prefill shapes, HBM bound when each resident expert
    # sees only a few rows)
    rank_flops = flops / world
    rank_bytes = B * expert_weight_bytes(cfg) + (pairs_total / world) * (cfg.H * 2 + cfg.H * 4)
    t_tc = rank_flops / (peaks["bf16_tflops"] * 1e12)
    t_hbm = rank_bytes / (peaks["hbm_gbs"] * 1e9)
    if t_tc >= t_hbm:
        roof = {"bound": "tensor", "achieved": rank_flops / (ms_per_step * 1e-3) / 1e12, "peak": peaks["bf16_tflops"],
                "unit": "TFLOP/s"}
    else:
        roof = {"bound": "hbm", "achieved": rank_bytes / (ms_per_step * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                "unit": "GB/s"}
    roof.update(frac=roof["achieved"] / roof["peak"], traffic=None, peak_source=peaks["source"],
                kernel="whole step of one rank (route + exchange + expert GEMMs + combine)",
                algorithmic_flops=rank_flops, algorithmic_bytes=int(rank_bytes))
    rec = {
        "value": T / (ms_per_step * 1e-3), "unit": "tokens/s", "ms_per_step": ms_per_step,
        "config": config_dict(cfg, T, tokens_per_rank=Tl, experts_per_rank=B, parallelism=f"ep{world}",
                              exchange=exchange_text),
        "roofline": roof,
        "per_rank_ms": [round(float(v.item()), 4) for v in per_rank_ms],
        "per_rank_max_ms": round(max(float(v.item()) for v in per_rank_ms), 4),
        "max_rank_pairs": int(recv_max.item()), "mean_rank_pairs": pairs_total / world,
        "e2e": {"value": T / float(e2e_t.mean()), "unit": "tokens/s",
                "h2d_bytes_per_step": Tl * cfg.H * 2, "d2h_bytes_per_step": Tl * cfg.H * 4},
        "gpu_launches": int(launches), "stage_ms_rank0": stage_ms,
    }
    if exchange is not None:
        rec["exchange"] = exchange
    if parity is not None:
        rec["parity"] = parity
    if hasattr(ep, "close"):
        ep.close()
    ml.close()
    del layer, ml, ep
    gc.collect()
    torch.cuda.empty_cache()
    dist.barrier()
    return rec


def run_multi(args, cfg, T, rank, world):
    import torch.distributed as dist
    from strata_b200 import MoeContext, synth
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(device)
    # before any pinned buffer exists: staging memory on the GPU's own NUMA node.  Best effort: a virtual machine that
    # reports one node and no node for its GPUs is left alone, and the record in the JSON line says so.  (Eight ranks
    # copying at once were measured at 14 GB/s each against 40 - 57 GB/s with two or four ranks on such a machine.)
    from strata_b200 import hostmem
    placement = hostmem.bind_near_gpu(device.index) if not args.no_numa else {"bound": False, "why": "--no-numa"}
    peaks = load_peaks()
    dist.init_process_group("nccl", device_id=device)
    ctx = MoeContext(device.index)
    torch.cuda.set_stream(ctx.stream)
    flush = L2Flush(device)
    sampler = ClockSampler(device.index)      # only rank 0 starts it; the others take part in its keep-busy loop
    if rank == 0:
        sampler.start()
    strong = args.scaling == "strong"
    main = measure_ep(args, cfg, T, rank, world, device, ctx, peaks, flush, strong, args.parity, sampler=sampler)
    clocks = sampler.stop() if rank == 0 else None
    sub = []
    if args.sub and world == 8 and cfg.name != "c4":
        c4 = synth.CONFIGS["c4"]
        keep_steps = args.steps
        args.steps = max(5, min(args.steps, 20))
        rec = measure_ep(args, c4, c4.T, rank, world, device, ctx, peaks, flush, True, False)
        rec["name"], rec["steps"] = "c4", args.steps
        args.steps = keep_steps
        sub.append(rec)
    line = None
    if rank == 0:
        line = {
            "metric": "MoE layer tokens/s", "value": main["value"], "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": main["ms_per_step"],
            "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": "bf16", "data": DATA,
        }
        for k in ("config", "roofline", "per_rank_ms", "per_rank_max_ms", "max_rank_pairs", "mean_rank_pairs", "e2e",
                  "gpu_launches", "stage_ms_rank0", "exchange", "parity"):
            if k in main:
                line[k] = main[k]
        line["clocks"] = clocks
        if sub:
            line["sub"] = sub
    placements = [None] * world
    dist.all_gather_object(placements, placement)
    if rank == 0:
        line["host_placement"] = placements
    dist.barrier()
    dist.destroy_process_group()
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None)
    ap.add_argument("--tokens", type=int, default=None)
    ap.add_argument("--experts", type=int, default=None,
                    help="override the expert count of the workload (profiler captures of a full-shape tile on a small device footprint)")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-sub", dest="sub", action="store_false", help="skip the sub-records of the other configurations")
    ap.add_argument("--no-parity", dest="parity", action="store_false", help="skip the oracle check of the timed layer")
    ap.add_argument("--no-numa", action="store_true",
                    help="N > 1: leave the ranks' CPU affinity alone (default: confine each rank to its GPU's NUMA node)")
    ap.add_argument("--microbatches", type=int, default=1,
                    help="multi-GPU, peer exchange: token micro-batches in flight per step (each on its own stream)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="multi-GPU row exchange: the library's peer-memory kernels or NCCL all-to-allv")
    ap.add_argument("--scaling", default=None, choices=["weak", "strong"],
                    help="multi-GPU: strong = --tokens in total (default), weak = --tokens per rank")
    args = ap.parse_args()
    from strata_b200 import synth
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    name = args.workload or "c3"
    cfg = synth.CONFIGS[name]
    if args.experts:
        import dataclasses
        cfg = dataclasses.replace(cfg, E=args.experts, name=f"{cfg.name}_e{args.experts}",
                                  description=f"{cfg.description} ({args.experts} experts)")
    T = args.tokens or cfg.T
    if args.scaling is None:
        args.scaling = "strong"

    if args.impl == "reference":
        if rank != 0:
            return 0
        reps = max(1, min(args.steps, 3))     # the weights are generated once, the timed pass repeats
        v, info = cpu_reference_run(cfg, T, args.cpu_seconds, repeats=reps)
        vals = [v] * reps
        print(json.dumps({
            "impl": "reference", "metric": "MoE layer tokens/s", "value": v, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": len(vals), "warmup": 0, "ms_per_step": 1e3 * T / v,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32",
            "data": DATA, "config": dict(config_dict(cfg, T), parallelism=f"ep{max(args.gpus, 1)}"),
            "cpu_baseline": {"value": v, "unit": "tokens/s", **info},
            "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return 0

    line = run_single(args, cfg, T) if world == 1 else run_multi(args, cfg, T, rank, world)
    if rank == 0 and line is not None:
        print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())

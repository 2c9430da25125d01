#!/usr/bin/env python
"""Benchmark of the mixed NVFP4/MXFP8 linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the configuration the headline metric is quoted on): prefill with
M = 8192 tokens through the four Llama-3-8B linear shapes.  One step =
    RMSNorm + Hadamard + pack of X[8192,4096]  -> fused mixed GEMM 4096 -> 6144   (QKV)
    Hadamard + pack of X[8192,4096]            -> fused mixed GEMM 4096 -> 4096   (O)
    RMSNorm + Hadamard + pack of X[8192,4096]  -> fused mixed GEMM 4096 -> 28672  (gate_up)
    Hadamard + pack of X[8192,14336]           -> fused mixed GEMM 14336 -> 4096  (down)
with K split 31/32 NVFP4 + 1/32 MXFP8, weights pre-packed once.  Inputs are synthetic
(N(0,1) with 1% outlier channels x20, weights N(0,0.02)); the per-step working set (~1.1 GB)
is far larger than the 126 MB L2, so no explicit flush is needed between iterations.

`value` is GEMM+pack throughput with inputs resident in HBM; `e2e` is the same step driven
from pinned host buffers (host->device copy of both activation matrices and device->host copy
of the down-projection output inside the timed region; the other three outputs are inputs of later
kernels in a real layer and would never leave the device, so only the layer's last output is read
back).  With N > 1 every rank runs the same step on its own GPU (the per-op configurations do not
shard: replicas only, weak scaling).  After the headline step every run, at every N, also runs the
configuration that does shard - the tensor-parallel decoder stack (`model_tp` in the JSON line:
strong scaling over the N ranks, column-/row-parallel linears, one all-reduce per row-parallel linear).

`--impl reference` times the reference's own CPU code for the path on a bounded sample of the same
workload, with all host threads: its ActQuantizer (NVFP4 + MXFP8) and Hadamard matrix from the staged
copy under oracle/_ref (see oracle/build_ref.py) followed by torch's bf16 F.linear, as the reference's
fake-quant forward does; when oracle/_ref is absent, the C port oracle/plq_oracle.c instead.
The one JSON line on stdout is kept short; the full per-case tables go to stderr as a second JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = [("qkv", 4096, 6144, True), ("o", 4096, 4096, False), ("gate_up", 4096, 28672, True),
          ("down", 14336, 4096, False)]   # name, K, N, fused RMSNorm on the input
M_TOKENS = 8192
NOMINAL_FP4_TFLOPS = 9000.0     # B200 dense FP4 (NVIDIA's sparse figure halved)
NOMINAL_HBM_GBS = 8000.0
GEMM_QKV_DRAM_BYTES = 90.8e6       # ncu: dram bytes read + written by one QKV-shape GEMM launch (profiles/)


def flops_of(m, shapes=SHAPES):
    return sum(2.0 * m * n * k for _, k, n, _ in shapes)


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p["bf16_tflops_sustained"]), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None
        self.t0 = self.t1 = None

    def mark_begin(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "10",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        rows = self.rows
        if self.t0 is not None and self.t1 is not None:
            # nvidia-smi is started before the warm-up (its start-up takes longer than a short timed region);
            # keep the samples that fall inside the timed region, or, if it was shorter than three sampling
            # periods, all samples taken under load since the start
            inside = [r for r in rows if self.t0 <= r[0] <= self.t1 + 0.02]
            rows = inside if len(inside) >= 3 else rows
        for _, r in rows:
            try:
                sm.append(float(r[0])); mx = float(r[1])
            except Exception:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        busy = [v for v in sm if mx and v > 0.5 * mx] or sm
        return {"sm_mhz": busy[len(busy) // 2] if busy else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# CPU arm: the reference's own code (oracle/_ref) or, without it, the C port; bounded sample
# ------------------------------------------------------------------------------------------------
SAMPLE_M, SAMPLE_N = 256, 2048


def host_threads() -> int:
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


SHAPES_70B = [("qkv", 8192, 10240, True), ("o", 8192, 8192, False), ("gate_up", 8192, 57344, True),
              ("down", 28672, 8192, False)]     # one Llama-3-70B decoder layer's linears (fused q/k/v and gate/up)


def _sample_tensors(torch, shapes=None, m=None, n_rows=None):
    shapes, m, n_rows = shapes or SHAPES, m or SAMPLE_M, n_rows or SAMPLE_N
    g = torch.Generator().manual_seed(1234)
    out = []
    for name, k, n, norm in shapes:
        x = torch.randn(m, k, generator=g)
        x[:, torch.randperm(k, generator=g)[: k // 100]] *= 20.0
        w = torch.randn(n_rows, k, generator=g) * 0.02
        gamma = (torch.rand(k, generator=g) + 0.5).to(torch.bfloat16)
        out.append((name, k, x.to(torch.bfloat16), w.to(torch.bfloat16), gamma if norm else None))
    return out


def _cpu_step_reference(torch, shapes=None, m=None, n_rows=None):
    """One step = for each of the four shapes: [RMSNorm] -> block-Hadamard(128) as a float32 matmul with the
    reference's own matrix -> the reference's ActQuantizer (bits "nvfp4", high_bits "mxfp8", last K/32 channels)
    -> torch's bf16 F.linear against weights the reference's quantiser prepared once (untimed)."""
    import torch.nn.functional as Fn
    from oracle import build_ref
    qu, get_hadamard_matrix = build_ref.load()
    torch.set_num_threads(host_threads())
    h128 = get_hadamard_matrix(128, "cpu").float()

    def rotate(t):
        k = t.shape[-1]
        return (t.float().view(-1, k // 128, 128) @ h128).view(-1, k).to(t.dtype)

    work = []
    with torch.no_grad():
        for name, k, x, w, gamma in _sample_tensors(torch, shapes, m, n_rows):
            k_hi = k // 32
            wr = rotate(w)
            wq = torch.cat([qu.fake_quantize_nvfp4(wr[:, : k - k_hi]), qu.fake_quantize_mxfp8(wr[:, k - k_hi:])], -1)
            q = qu.ActQuantizer()
            q.configure(bits="nvfp4", high_bits="mxfp8", high_bits_length=k_hi)
            work.append((x, gamma, q, wq.to(torch.bfloat16)))

    def step():
        with torch.no_grad():
            for x, gamma, q, wq in work:
                if gamma is not None:           # inference/forward_pass.py:33-39 of the reference
                    xf = x.float()
                    x = (gamma.float() * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6))).to(x.dtype)
                Fn.linear(q(rotate(x)), wq)
    return step, "reference", torch.get_num_threads()


def _cpu_step_port(torch, shapes=None, m=None, n_rows=None):
    """The same step on the C port (oracle/plq_oracle.c, OpenMP) with torch's float32 matmul for the product."""
    import numpy as np
    from oracle import cport
    cport.set_num_threads(host_threads())
    torch.set_num_threads(host_threads())

    def bits(t):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)

    work = []
    for name, k, x, w, gamma in _sample_tensors(torch, shapes, m, n_rows):
        wdq = torch.from_numpy(cport.dequant(cport.prepare(bits(w), k // 32, hadamard=True)))
        work.append((bits(x), None if gamma is None else bits(gamma), k, wdq))

    def step():
        for xb, gb, k, wdq in work:
            a = torch.from_numpy(cport.dequant(cport.prepare(xb, k // 32, gb, 1e-6, True)))
            torch.matmul(a, wdq.T)
    return step, "port", cport.num_threads()


def run_cpu_sample(steps: int, warmup: int, budget_s: float = 60.0):
    """Times the CPU arm on SAMPLE_M token rows x SAMPLE_N weight rows of each of the four shapes (full K); stops
    early once `budget_s` seconds of timed work are done, and says how many steps it timed."""
    import torch
    from oracle import build_ref
    step, kind, cores = (_cpu_step_reference if build_ref.available() else _cpu_step_port)(torch)
    for _ in range(warmup):
        step()
    done, t0 = 0, time.perf_counter()
    while done < steps and (done == 0 or time.perf_counter() - t0 < budget_s):
        step()
        done += 1
    dt = (time.perf_counter() - t0) / done
    fl = sum(2.0 * SAMPLE_M * SAMPLE_N * k for _, k, _, _ in SHAPES)
    what = ("the reference's ActQuantizer + Hadamard matrix (oracle/_ref) and torch bf16 F.linear" if kind == "reference"
            else "C port oracle/plq_oracle.c + torch float32 matmul (oracle/_ref not staged)")
    return {"value": fl / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": kind,
            "sample": f"{SAMPLE_M} token rows x {SAMPLE_N} weight rows of each of the 4 shapes, full K, [RMSNorm] + "
                      f"rotation + activation quantiser + product per step, weight quantisation excluded; {what}",
            "ms_per_step": dt * 1e3, "steps_timed": done}


def config_dict(n_gpus):
    return {"workload": "prefill M=8192 x Llama-3-8B linear shapes (4096->6144, 4096->4096, 4096->28672, "
                        "14336->4096), K split 31/32 NVFP4 + 1/32 MXFP8, RMSNorm/Hadamard/pack on device",
            "m_tokens": M_TOKENS, "l2": "per-step working set ~1.1 GB >> 126 MB L2, no flush needed",
            "parallelism": f"replicas x{n_gpus}" if n_gpus > 1 else "single GPU"}


def cpu_model_estimate(budget_s: float = 8.0):
    """configs[4] on the host, extrapolated: the CPU arm's code on 64 token rows x 1024 weight rows of each of the
    four linears of one Llama-3-70B decoder layer (full K), and from its rate the tokens/s the 80 layers' linears
    alone would allow (a full 70B forward does not fit a host's memory or a benchmark's time)."""
    import torch
    from oracle import build_ref
    m, n_rows = 64, 1024
    step, kind, cores = (_cpu_step_reference if build_ref.available() else _cpu_step_port)(torch, SHAPES_70B, m, n_rows)
    step()
    done, t0 = 0, time.perf_counter()
    while done == 0 or time.perf_counter() - t0 < budget_s:
        step()
        done += 1
    dt = (time.perf_counter() - t0) / done
    rate = sum(2.0 * m * n_rows * k for _, k, _, _ in SHAPES_70B) / dt               # flop/s on the sample
    per_token = 80 * sum(2.0 * n * k for _, k, n, _ in SHAPES_70B)                    # flop per token, linears only
    return {"tokens_per_s": rate / per_token, "tflops": rate / 1e12, "cores": cores, "kind": kind, "extrapolated": True,
            "sample": f"{m} token rows x {n_rows} weight rows of each of one layer's four linears, full K, x 80 layers; "
                      "attention, LM head and weight quantisation not counted"}


def main_reference(args, rank):
    if rank != 0:
        return
    warm = min(args.warmup, 2)
    b = run_cpu_sample(max(args.steps, 1), warm, budget_s=90.0)   # a step is 0.1-1 s of host work
    line = {"impl": "reference", "metric": "mixed NVFP4/MXFP8 GEMM TFLOP/s", "value": b["value"], "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": b["steps_timed"], "warmup": warm, "ms_per_step": b["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4+mxfp8 (f32 accumulate)",
            "data": "synthetic", "config": config_dict(args.gpus),
            "cpu_baseline": {k: b[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": b["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def main_ours(args, rank, local_rank, world):
    import torch
    import plaquant_b200 as plq

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: plaquant_b200 has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    plq.lib()
    peaks = load_peaks()

    # ---- synthetic data: host (pinned) masters and device copies ---------------------------------
    g = torch.Generator().manual_seed(1000 * 3 + rank)
    def activ(k):
        x = torch.randn(M_TOKENS, k, generator=g, dtype=torch.float32)
        x[:, torch.randperm(k, generator=g)[: k // 100]] *= 20.0
        return x.to(torch.bfloat16).pin_memory()
    x_host = {4096: activ(4096), 14336: activ(14336)}
    x_dev = {k: torch.empty_like(v, device=dev) for k, v in x_host.items()}
    for k in x_host:
        x_dev[k].copy_(x_host[k])
    layers = []
    for name, k, n, norm in SHAPES:
        w = (torch.randn(n, k, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16).to(dev)
        pw = plq.pack(w, k // 32, hadamard=True, sf_layout="tiled")
        gamma = (torch.rand(k, generator=g) + 0.5).to(torch.bfloat16).to(dev) if norm else None
        pa = plq.alloc_packed(M_TOKENS, k, k // 32, "tiled", dev)
        y = torch.empty(M_TOKENS, n, dtype=torch.bfloat16, device=dev)
        layers.append({"name": name, "k": k, "n": n, "pw": pw, "gamma": gamma, "pa": pa, "y": y})
        del w
    y_host = torch.empty(M_TOKENS, SHAPES[-1][2], dtype=torch.bfloat16).pin_memory()
    torch.cuda.synchronize()

    gemm_events = []

    def step(record=False, x_src=None):
        x_src = x_dev if x_src is None else x_src
        for L in layers:
            plq.pack(x_src[L["k"]], L["k"] // 32, hadamard=True, gamma=L["gamma"], eps=1e-6, out=L["pa"])
            if record:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            plq.mixed_gemm(L["pa"], L["pw"], out=L["y"])
            if record:
                e1.record()
                gemm_events.append((L["name"], e0, e1))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world > 1:
            import torch.distributed as dist
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    # ---- device-resident timing -------------------------------------------------------------------
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(args.warmup):
        step()
    plq.check_device_status()
    barrier()
    sampler.mark_begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step(record=True)
    e1.record()
    barrier()
    sampler.mark_end()
    clocks = sampler.stop()
    plq.check_device_status()
    ms_step = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    per_gemm = {}
    for name, a, b in gemm_events:
        per_gemm.setdefault(name, []).append(a.elapsed_time(b))
    gemm_ms = sum(sum(v) / len(v) for v in per_gemm.values())
    fl = flops_of(M_TOKENS)
    value = world * fl / (ms_step * 1e-3) / 1e12

    # ---- end to end from pinned host buffers ----------------------------------------------------------
    # Every step copies its inputs host -> device and its result device -> host.  The input copy of step
    # i + 1 runs on a second stream into the other of two device buffers while step i computes.
    copy_stream = torch.cuda.Stream(device=dev)
    main_stream = torch.cuda.current_stream(dev)
    x_in = [x_dev, {k: torch.empty_like(v) for k, v in x_dev.items()}]
    ev_ready = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]
    for e in ev_free:
        e.record(main_stream)
    e2e_count = [0]

    def step_e2e():
        b = e2e_count[0] & 1
        e2e_count[0] += 1
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(ev_free[b])          # the step that last read this buffer has finished
            for k in x_host:
                x_in[b][k].copy_(x_host[k], non_blocking=True)
            ev_ready[b].record(copy_stream)
        main_stream.wait_event(ev_ready[b])
        step(x_src=x_in[b])
        ev_free[b].record(main_stream)
        y_host.copy_(layers[-1]["y"], non_blocking=True)
    for _ in range(min(args.warmup, 3)):
        step_e2e()
    barrier()
    e0.record()
    for _ in range(args.steps):
        step_e2e()
    e1.record()
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    h2d = sum(v.numel() * 2 for v in x_host.values())
    d2h = y_host.numel() * 2

    # ---- the other two kernels of the path, timed alone (rank 0 reports) -------------------------------
    extra = {}
    if rank == 0:
        extra = side_benchmarks(plq, torch, dev, peaks)

    # free the per-op operands, then the configuration that shards: the tensor-parallel decoder stack
    model_tp = None
    if args.tp_layers > 0:
        for L in layers:
            L["pw"] = L["pa"] = L["y"] = None
        x_dev.clear(); x_in.clear()
        torch.cuda.empty_cache()
        try:
            model_tp = run_model_tp(args, torch, plq, rank, world, dev, peaks)
        except Exception as exc:  # noqa: BLE001 - the headline line below is still printed, with the failure in it
            model_tp = {"error": f"{type(exc).__name__}: {exc}"[:400]} if rank == 0 else None
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    gemm_tflops = fl / (gemm_ms * 1e-3) / 1e12
    # Comparator: no FP4 peak is measured on this pool, so the tensor roofline is 4 x the measured cuBLAS bf16 rate
    # (FP4 is nominally 4 x bf16): the burst figure when the timed region is shorter than a second (the SM clock
    # has not settled under the power cap yet), the sustained one otherwise.
    timed_s = ms_step * 1e-3 * args.steps
    which = "bf16_tflops" if timed_s < 1.0 else "bf16_tflops_sustained"
    fp4_peak = 4.0 * peaks[which]
    per_gemm_ms = {k: sum(v) / len(v) for k, v in per_gemm.items()}
    line = {
        "metric": "mixed NVFP4/MXFP8 GEMM TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4+mxfp8 (f32 accumulate)", "data": "synthetic",
        "config": config_dict(world),
        "e2e": {"value": world * fl / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e},
        "gpu_launches": 2 * len(layers) * args.steps,
        "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "mixed_gemm_kernel<256, 2>", "achieved": gemm_tflops,
                     "peak": fp4_peak, "unit": "TFLOP/s", "frac": gemm_tflops / fp4_peak,
                     "peak_source": f"4 x {peaks['source']} cuBLAS {which} ({peaks[which]} TF/s; timed region "
                                    f"{timed_s:.2f} s); no FP4 peak is measured on this pool",
                     "frac_of_nominal_fp4": gemm_tflops / NOMINAL_FP4_TFLOPS, "nominal_fp4_tflops": NOMINAL_FP4_TFLOPS,
                     "flops_per_step": fl, "gemm_ms_per_step": gemm_ms, "pack_ms_per_step": ms_step - gemm_ms,
                     "per_gemm_tflops": {L["name"]: round(2.0 * M_TOKENS * L["n"] * L["k"] / (per_gemm_ms[L["name"]] * 1e-3) / 1e12, 1)
                                         for L in layers},
                     "traffic": GEMM_QKV_DRAM_BYTES,
                     "traffic_note": "dram__bytes_read+write of one QKV-shape launch (412 GFLOP, 134.6 MB of operands "
                                     "and output) from the ncu capture in profiles/; part of the output is still in L2 "
                                     "when the kernel ends"},
    }
    detail = {"per_gemm_ms": per_gemm_ms, **extra}
    # short forms of the side results for the one-line record
    if "pack" in extra:
        line["pack"] = {k: extra["pack"][k] for k in ("us", "gbs", "frac_of_measured_hbm", "frac_of_nominal_hbm")}
    if "gemv" in extra:
        gv = extra["gemv"]
        line["gemv_m8"] = {name: {"us": round(gv[f"{name}_m8"]["us"], 2),
                                  "frac_of_measured_hbm": round(gv[f"{name}_m8"]["frac_of_measured_hbm"], 3)}
                           for name, _, _, _ in SHAPES}
        tot_b = sum(gv[f"{name}_m8"]["bytes"] for name, _, _, _ in SHAPES)
        tot_us = sum(gv[f"{name}_m8"]["us"] for name, _, _, _ in SHAPES)
        line["gemv_m8"]["layer"] = {"us": round(tot_us, 2), "frac_of_measured_hbm": round(tot_b / tot_us / 1e3 / peaks["hbm_gbs"], 3)}
    line["hbm_peak_gbs"] = {"measured": peaks["hbm_gbs"], "nominal": NOMINAL_HBM_GBS, "source": peaks["source"]}
    if model_tp is not None:
        line["model_tp"] = model_tp
    if world == 1:
        try:
            line["cpu_baseline"] = {k: v for k, v in run_cpu_sample(20, 1, budget_s=15.0).items()
                                    if k not in ("ms_per_step", "steps_timed")}
            if model_tp is not None:
                model_tp["cpu_baseline_extrapolated"] = cpu_model_estimate()
        except Exception as exc:  # the checker could not be built or staged on this host
            line["cpu_baseline"] = {"value": None, "unit": "TFLOP/s", "cores": 0, "kind": "port", "sample": f"failed: {exc}"}
    print(json.dumps(line), flush=True)
    print(json.dumps({"detail": detail}), file=sys.stderr, flush=True)


def run_model_tp(args, torch, plq, rank, world, dev, peaks):
    """configs[4] on the ranks of this run: the Llama-3-70B-architecture decoder stack (random init, `--tp-layers`
    of its 80 layers), tensor-parallel over the N ranks (column-parallel QKV / gate_up, row-parallel O / down, one
    reduction per row-parallel linear, done inside the following RMSNorm-quant kernel over peer memory: all-reduce
    form for decode batches, reduce-scatter + all-gather of the packed rows for the prefill),
    batch 16, 2048 prefill tokens + 128 greedy decode steps.  Strong scaling: the job is fixed.  Returns the
    `model_tp` block (rank 0) or None."""
    import torch.distributed as dist
    from plaquant_b200 import tp
    from plaquant_b200.forward_pass import LlamaConfig, ResQForwardB200
    ctx = tp.TPContext(rank, world, None)
    cfg = LlamaConfig.llama3_70b()
    layers = args.tp_layers
    batch, prefill, decode = args.batch, args.prefill, args.decode
    scattered = args.fused_reduce and args.scatter_prefill and world > 1 and (batch * prefill) % world == 0
    model = ResQForwardB200(cfg, dev, ctx, seed=4, num_layers=layers, fused_reduce_rows=16 if args.fused_reduce else 0,
                            scatter_prefill_rows=batch * prefill if scattered else 0)
    ids = torch.randint(0, cfg.vocab_size, (batch, prefill), generator=torch.Generator().manual_seed(40)).to(dev)

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
    out = model.generate(ids, decode)                # warm-up run (also builds the caches' allocator pools)
    plq.check_device_status()
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    out = model.generate(ids, decode)
    e1.record()
    sync()
    plq.check_device_status()
    ms = e0.elapsed_time(e1)
    tev = model.timing_events
    prefill_ms, decode_ms = tev[0].elapsed_time(tev[1]), tev[1].elapsed_time(tev[2])
    same = True
    ar = {}
    if world > 1:
        t = torch.tensor([ms, prefill_ms, decode_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, prefill_ms, decode_ms = (float(v) for v in t.tolist())
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        same = all(torch.equal(g, gathered[0]) for g in gathered)
        # the all-reduces of the path, timed alone: 2 per layer, [batch * prefill, hidden] bf16 in the prefill
        # (NCCL) and [batch, hidden] per decode step (inside the fused kernel unless --nccl-reduce)
        for name, rows, reps in (("prefill", batch * prefill, 4), ("decode", batch, 50)):
            buf = torch.zeros(rows, cfg.hidden_size, dtype=torch.bfloat16, device=dev)
            dist.all_reduce(buf)
            sync()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                dist.all_reduce(buf)
            b.record()
            sync()
            ar[name] = {"bytes_per_allreduce": buf.numel() * 2, "nccl_ms_each": a.elapsed_time(b) / reps,
                        "per_pass": 2 * layers}
            del buf
        if scattered:
            # the kernel that replaces each of those all-reduces AND the add + RMSNorm-quant behind it in the
            # prefill, timed alone on the model's own buffers (an even number of calls keeps the buffer parity)
            from plaquant_b200 import ops
            sr, R = model.scatter, batch * prefill
            h_my = torch.zeros(R // world, cfg.hidden_size, dtype=torch.bfloat16, device=dev)
            gamma = model.layers[0].ln2
            for _ in range(2):
                ops.reduce_scatter_add_rmsnorm_pack(sr, R, h_my, gamma, cfg.rms_eps)
            sync()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(4):
                ops.reduce_scatter_add_rmsnorm_pack(sr, R, h_my, gamma, cfg.rms_eps)
            b.record()
            sync()
            t = torch.tensor([a.elapsed_time(b) / 4], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ar["prefill"]["fused_reduce_scatter_norm_quant_gather_ms_each"] = float(t.item())
            ar["prefill"]["share_of_prefill_ms"] = float(t.item()) * 2 * layers / prefill_ms
            ar["prefill"]["note"] = "nccl_ms_each is the all-reduce this run does NOT make, for comparison"
            del h_my
        else:
            ar["prefill"]["share_of_prefill_ms"] = ar["prefill"]["nccl_ms_each"] * 2 * layers / prefill_ms
    # bytes one decode step must read on a rank: packed weights of the linears (tiled copy), the unquantised LM
    # head, and the key/value caches up to the current position (mean over the decode steps)
    w_bytes = sum(lin._gemm_w.nbytes() for L in model.layers for lin in (L.qkv, L.o, L.gate_up, L.down))
    head_bytes = model.lm_head.numel() * 2
    kv_bytes = layers * 2 * batch * (prefill + decode / 2) * model.kv_heads * cfg.head_dim * 2
    step_ms = decode_ms / decode
    step_bytes = w_bytes + head_bytes + kv_bytes
    del model
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    tokens = batch * (prefill + decode)
    return {"metric": "decoder tokens/s (prefill + greedy decode)", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
            "scaling": "strong", "parallelism": f"tp{world}", "layers": layers, "of_layers": cfg.num_layers,
            "batch": batch, "prefill_tokens": prefill, "decode_steps": decode, "ms": ms, "prefill_ms": prefill_ms,
            "decode_ms": decode_ms, "decode_ms_per_step": step_ms, "ranks_agree_on_tokens": same,
            "reduce": ("fused into the RMSNorm-quant kernel over peer memory: all-reduce form (decode), "
                       + ("reduce-scatter + all-gather of the packed rows (prefill)" if scattered else "NCCL (prefill)"))
                      if (args.fused_reduce and world > 1)
                      else ("NCCL" if world > 1 else "none (one rank)"),
            "allreduce": ar,
            "decode_roofline": {"bound": "hbm", "bytes_per_step_per_rank": step_bytes,
                                "packed_weight_bytes": w_bytes, "lm_head_bytes": head_bytes, "kv_cache_bytes": kv_bytes,
                                "achieved": step_bytes / (step_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                "frac": step_bytes / (step_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}}


def main_model(args, rank, local_rank, world):
    """configs[4]: random-init Llama-3-70B-architecture decoder stack, tensor-parallel over the ranks
    (column-parallel QKV / gate_up, row-parallel O / down, one NCCL all-reduce after each row-parallel
    linear), batch 16, prefill of 2048 random token ids + 128 greedy decode steps.  Strong scaling:
    the job is fixed, the ranks share it."""
    import torch
    import torch.distributed as dist
    import plaquant_b200 as plq
    from plaquant_b200 import tp
    from plaquant_b200.forward_pass import LlamaConfig, ResQForwardB200

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ctx = tp.TPContext(rank, world, None)
    cfg = LlamaConfig.llama3_70b()
    layers = args.layers or cfg.num_layers
    batch, prefill, decode = args.batch, args.prefill, args.decode
    scattered = args.fused_reduce and args.scatter_prefill and world > 1 and (batch * prefill) % world == 0
    model = ResQForwardB200(cfg, dev, ctx, seed=4, num_layers=layers, fused_reduce_rows=16 if args.fused_reduce else 0,
                            scatter_prefill_rows=batch * prefill if scattered else 0)
    ids = torch.randint(0, cfg.vocab_size, (batch, prefill), generator=torch.Generator().manual_seed(40)).to(dev)

    def run():
        return model.generate(ids, decode)

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
    for _ in range(max(1, min(args.warmup, 2))):
        out = run()
    plq.check_device_status()
    sampler = ClockSampler(local_rank)
    sync()
    sampler.start()
    sampler.mark_begin()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    steps = max(1, min(args.steps, 5))
    e0.record()
    for _ in range(steps):
        out = run()
    e1.record()
    sync()
    sampler.mark_end()
    clocks = sampler.stop()
    plq.check_device_status()
    ms = e0.elapsed_time(e1) / steps
    tev = getattr(model, "timing_events", None)
    phases = {"prefill_ms": tev[0].elapsed_time(tev[1]), "decode_ms": tev[1].elapsed_time(tev[2])} if tev else {}
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        same = all(torch.equal(g, gathered[0]) for g in gathered)
    else:
        same = True
    if rank == 0:
        tokens = batch * (prefill + decode)
        print(json.dumps({
            "metric": "decoder tokens/s (prefill + greedy decode)", "value": tokens / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": steps, "warmup": max(1, min(args.warmup, 2)), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4+mxfp8 (f32 accumulate)",
            "data": "synthetic", "clocks": clocks, "ranks_agree_on_tokens": same, "last_run_phases": phases,
            "config": {"workload": f"Llama-3-70B architecture, {layers} of 80 layers, random init, batch {batch}, "
                                   f"prefill {prefill} + {decode} greedy decode steps", "parallelism": f"tp{world}",
                       "prefill_reduce": "fused reduce-scatter / all-gather" if scattered else ("NCCL" if world > 1 else "none")}}),
            flush=True)
    if world > 1:
        dist.destroy_process_group()


def time_cuda(torch, fn, iters, flush=None):
    """Average milliseconds of fn() over `iters` runs, each preceded by an L2 flush when given."""
    tot = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.add_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record()
        torch.cuda.synchronize()
        tot += a.elapsed_time(b)
    return tot / iters


def clone_packed(plq, p, copies):
    """`copies` independent device copies of a packed matrix (to cycle through operands larger than L2)."""
    return [plq.PackedMatrix(p.rows, p.k_lo, p.k_hi, p.lo_codes.clone(), p.lo_sf.clone(), p.hi_codes.clone(),
                             p.hi_sf.clone(), p.sf_layout) for _ in range(copies)]


def time_rotating(torch, fns, rounds):
    """Average milliseconds per call of the callables in `fns`: one pass over them is captured in a CUDA
    graph (so the Python/ctypes launch path, ~15 us per call, is not what gets timed) and the graph
    is replayed `rounds` times between one pair of CUDA events.  Each callable works on its own copy of
    the operands and the copies together exceed L2 several times, so every launch streams from HBM."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        for f in fns:
            f()
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for f in fns:
                f()
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(rounds):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / (rounds * len(fns))


def side_benchmarks(plq, torch, dev, peaks):
    """configs[1] (fused RMSNorm-quant + Hadamard-pack, [4096, 4096]) and configs[2] (decode GEMV
    sweep), each kernel timed alone with an L2 flush before every launch; HBM roofline."""
    flush = torch.zeros(256 * 1024 * 1024 // 4, dtype=torch.int32, device=dev)     # 256 MB > L2
    out = {}
    g = torch.Generator().manual_seed(77)
    x = torch.randn(4096, 4096, generator=g)
    x[:, torch.randperm(4096, generator=g)[:40]] *= 20.0
    x = x.to(torch.bfloat16).to(dev)
    gamma = (torch.rand(4096, generator=g) + 0.5).to(torch.bfloat16).to(dev)
    pa = plq.alloc_packed(4096, 4096, 128, "tiled", dev)
    fn = lambda: plq.pack(x, 128, hadamard=True, gamma=gamma, eps=1e-6, out=pa)
    xs = [x.clone() for _ in range(12)]                       # 12 x 33.5 MB of input > 3 x L2
    pas = [plq.alloc_packed(4096, 4096, 128, "tiled", dev) for _ in range(12)]
    fns = [(lambda xi=xi, pi=pi: plq.pack(xi, 128, hadamard=True, gamma=gamma, eps=1e-6, out=pi)) for xi, pi in zip(xs, pas)]
    ms = time_rotating(torch, fns, 5)
    del xs, pas, fns
    nbytes = 2 * 4096 * 4096 + 2 * 4096 + 4096 * 2364
    out["pack"] = {"workload": "RMSNorm + Hadamard128 + NVFP4/MXFP8 pack, bf16 [4096, 4096]", "us": ms * 1e3,
                   "timing": "back-to-back launches over 12 operand copies (> 3 x L2), one event pair",
                   "bytes": nbytes, "gbs": nbytes / (ms * 1e-3) / 1e9,
                   "frac_of_measured_hbm": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                   "frac_of_nominal_hbm": nbytes / (ms * 1e-3) / 1e9 / NOMINAL_HBM_GBS}
    gv = {}
    for name, k, n, _ in SHAPES:
        w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16).to(dev)
        pw = plq.pack(w, k // 32, hadamard=True, sf_layout="tiled")
        del w
        pws = clone_packed(plq, pw, max(2, int(400e6 // pw.nbytes())))      # >= 400 MB of weights in rotation
        for m in (1, 2, 4, 8):
            xa = plq.pack(x[:m, :k] if k <= 4096 else torch.randn(m, k, generator=g).to(torch.bfloat16).to(dev),
                          k // 32, hadamard=True, sf_layout="tiled")
            y = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
            fns = [(lambda w=w_: plq.gemv_tc(xa, w, out=y, static_weights=True)) for w_ in pws]   # weights packed at load time
            ms = time_rotating(torch, fns, 5)
            nb = pw.nbytes() + xa.nbytes() + m * n * 2
            gv[f"{name}_m{m}"] = {"us": ms * 1e3, "bytes": nb, "gbs": nb / (ms * 1e-3) / 1e9,
                                  "frac_of_measured_hbm": nb / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                  "frac_of_nominal_hbm": nb / (ms * 1e-3) / 1e9 / NOMINAL_HBM_GBS}
        del pw, pws
    out["gemv"] = gv
    out["gemv_timing"] = "back-to-back launches cycling >= 400 MB of weight copies (> 3 x L2), one event pair"
    out["hbm_peak_gbs"] = {"measured": peaks["hbm_gbs"], "nominal": NOMINAL_HBM_GBS, "source": peaks["source"]}
    return out


def main_case(args):
    """One kernel of the path on one fixed case, `warmup` + `steps` launches: the command the
    ncu captures under profiles/ were taken from (small enough for a multi-pass capture)."""
    import torch
    import plaquant_b200 as plq
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(5)
    def activ(m, k):
        x = torch.randn(m, k, generator=g)
        x[:, torch.randperm(k, generator=g)[: k // 100]] *= 20.0
        return x.to(torch.bfloat16).to(dev)
    name, k, n, _ = next(s for s in SHAPES if s[0] == args.shape)
    if args.case == "decode_step":
        # two layers of the Llama-3-70B-architecture stack on one GPU, batch 16, 2048 prefill tokens, a few decode
        # steps (two eager, the rest replayed from the captured graph): the launch list of one step under profiles/
        from plaquant_b200.forward_pass import LlamaConfig, ResQForwardB200
        model = ResQForwardB200(LlamaConfig.llama3_70b(), dev, seed=4, num_layers=2)
        ids = torch.randint(0, 128256, (16, 2048), generator=g).to(dev)
        out = model.generate(ids, max(args.steps, 3))
        torch.cuda.synchronize()
        tev = model.timing_events
        print(json.dumps({"case": "decode_step", "layers": 2, "decode_steps": int(out.shape[1]),
                          "prefill_ms": tev[0].elapsed_time(tev[1]), "decode_ms": tev[1].elapsed_time(tev[2])}), flush=True)
        return
    if args.case == "pack":
        x = activ(4096, 4096)
        gamma = (torch.rand(4096, generator=g) + 0.5).to(torch.bfloat16).to(dev)
        pa = plq.alloc_packed(4096, 4096, 128, "tiled", dev)
        fn = lambda: plq.pack(x, 128, hadamard=True, gamma=gamma, eps=1e-6, out=pa)
        work, unit = 2 * 4096 * 4096 + 2 * 4096 + 4096 * 2364, "GB/s"
    elif args.case == "silu_pack":
        f = 14336                                           # Llama-3-8B FFN width: gate_up output [m, 2 f] -> down_proj input
        gu = activ(args.m, 2 * f)
        pa = plq.alloc_packed(args.m, f, f // 32, "tiled", dev)
        fn = lambda: plq.silu_mul_pack(gu, f // 32, out=pa)
        work, unit = args.m * (2 * f * 2 + pa.nbytes() // args.m), "GB/s"
    elif args.case == "rope":
        # the fused QKV output of one Llama-3-70B layer, `m` token rows of 4 sequences: RoPE on q / k, append of k / v
        from plaquant_b200 import ops
        heads, kvh, b = 64, 8, 4
        t = args.m // b
        qkv = activ(args.m, (heads + 2 * kvh) * 128).view(b, t, -1)
        ang = torch.outer(torch.arange(t, dtype=torch.float32), 1.0 / (500000.0 ** (torch.arange(0, 128, 2, dtype=torch.float32) / 128)))
        cos, sin = torch.cat([ang.cos(), ang.cos()], -1).to(dev), torch.cat([ang.sin(), ang.sin()], -1).to(dev)
        kc = torch.empty(b, t, kvh, 128, dtype=torch.bfloat16, device=dev)
        vc = torch.empty_like(kc)
        fn = lambda: ops.rope_kv_append(qkv, cos, sin, heads, kvh, kc, vc, 0)
        work, unit = 2 * qkv.numel() * 2, "GB/s"
    elif args.case in ("gemv", "gemv_tc"):
        layout, op = (("rowmajor", plq.gemv) if args.case == "gemv" else
                      ("tiled", lambda a_, b_, out: plq.gemv_tc(a_, b_, out=out, static_weights=True)))
        w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16).to(dev)
        pw = plq.pack(w, k // 32, hadamard=True, sf_layout=layout)
        pa = plq.pack(activ(args.m, k), k // 32, hadamard=True, sf_layout=layout)
        y = torch.empty(args.m, n, dtype=torch.bfloat16, device=dev)
        pws = clone_packed(plq, pw, max(2, int(400e6 // pw.nbytes())))
        rot = [(lambda w=w_: op(pa, w, out=y)) for w_ in pws]
        fn = lambda: op(pa, pw, out=y)
        work, unit = pw.nbytes() + pa.nbytes() + y.numel() * 2, "GB/s"
    else:
        w = (torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16).to(dev)
        pw = plq.pack(w, k // 32, hadamard=True, sf_layout="tiled")
        pa = plq.pack(activ(args.m, k), k // 32, hadamard=True, sf_layout="tiled")
        y = torch.empty(args.m, n, dtype=torch.bfloat16, device=dev)
        fn = lambda: plq.mixed_gemm(pa, pw, out=y, variant=args.variant)
        pws = clone_packed(plq, pw, max(2, int(400e6 // pw.nbytes())))
        rot = [(lambda w=w_: plq.mixed_gemm(pa, w, out=y, variant=args.variant)) for w_ in pws]
        work, unit = 2.0 * args.m * n * k, "TFLOP/s"
    flush = torch.zeros(256 * 1024 * 1024 // 4, dtype=torch.int32, device=dev)
    for _ in range(args.warmup):
        fn()
    torch.cuda.synchronize()
    ms = time_cuda(torch, fn, args.steps, flush)
    if args.case in ("gemv", "gemv_tc", "gemm"):
        ms_rot = time_rotating(torch, rot, max(1, args.steps // 4))
    plq.check_device_status()
    rate = work / (ms * 1e-3) / (1e9 if unit == "GB/s" else 1e12)
    line = {"case": args.case, "shape": name, "m": args.m, "us_per_launch": ms * 1e3, "rate": rate, "unit": unit,
            "work": work}
    if args.case in ("gemv", "gemv_tc", "gemm"):
        line["us_back_to_back"] = ms_rot * 1e3
        line["rate_back_to_back"] = work / (ms_rot * 1e-3) / (1e9 if unit == "GB/s" else 1e12)
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default=None, choices=["pack", "silu_pack", "rope", "gemv", "gemv_tc", "gemm", "decode_step"],
                    help="run one kernel on one fixed case instead of the full step")
    ap.add_argument("--shape", default="qkv", choices=[s[0] for s in SHAPES])
    ap.add_argument("--m", type=int, default=None)
    ap.add_argument("--variant", default=None, choices=["128x128", "128x256", "pair256x256"])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--nccl-prefill", dest="scatter_prefill", action="store_false",
                    help="model_tp: all-reduce the prefill's row-parallel outputs with NCCL instead of the fused "
                         "reduce-scatter / all-gather kernel")
    ap.add_argument("--nccl-reduce", dest="fused_reduce", action="store_false",
                    help="model workload: NCCL all-reduces in the decode step instead of the reduction fused into "
                         "the RMSNorm-quant kernel over peer memory")
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="linears", choices=["linears", "model"],
                    help="linears: the per-op step (default); model: the tensor-parallel decoder stack")
    ap.add_argument("--layers", type=int, default=None, help="model workload: number of decoder layers (default 80)")
    ap.add_argument("--tp-layers", type=int, default=16,
                    help="layers of the 80-layer decoder stack in the model_tp block of the default run (0 = skip it)")
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--prefill", type=int, default=2048)
    ap.add_argument("--decode", type=int, default=128)
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.case is not None:
        if args.m is None:
            args.m = 8 if args.case in ("gemv", "gemv_tc") else M_TOKENS
        return main_case(args)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.workload == "model" and args.impl == "ours":
        return main_model(args, rank, local_rank, world)
    if args.impl == "reference":
        main_reference(args, rank)
    else:
        main_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Benchmark of the fused 4-bit AdamW step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one optimizer step over the whole parameter list of the workload: at every N the
Llama-7B-shaped parameter set (bf16 parameters and gradients, per-tensor gradient sigma log-uniform in
[1e-5, 1e-2], 0.1 % of entries x100); at N > 1 the optimizer state is sharded over the ranks and the updated
parameters are delivered to every rank inside the step (the Llama-13B-shaped set runs beside it, under `also`).
All data is synthetic and seeded.  Rank 0 prints one JSON line.

`value`      Gparams/s with everything resident in HBM, device time over exactly K steps.
`e2e`        the same metric through the public optimizer class with the step's input (the gradients)
             copied from pinned host memory inside the timed region and the step's status word read back.
`roofline`   algorithmic HBM bytes of one step / device time of one step, against the measured copy peak.
`cpu_baseline` the CPU oracle (C form, all host threads) on a bounded sample of the same workload.
`--impl reference` times the reference's CPU path (its torch-operator restatement, the oracle) instead.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from quantfour_adamw_cuda_b200 import shapes as S  # noqa: E402

HP = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes per algorithmic byte of a step, from one ncu capture of the two step kernels on the GPT-2-medium-shaped
# set (dram__bytes_read.sum + dram__bytes_write.sum = 3.712 GB over 2.869 GB algorithmic; the first pass re-reads
# gradients and second-moment codes).  Traffic grows in proportion to the elements processed, so the figure for the bench workload
# is this factor times its algorithmic bytes; the result line says that it is scaled, not captured.
TRAFFIC_PER_ALGORITHMIC_BYTE = 3.712 / 2.869


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.t0, self.t1 = index, None, 0.0, 0.0

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # the busiest half of the samples stands for "under load" (the sampler also sees the idle edges)
        load = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(load) if load else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def synth_tensor(shape, sigma, gen, device, dtype=torch.bfloat16, outliers=True):
    x = torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * sigma
    if outliers:
        mask = torch.rand(shape, generator=gen, device=device) < 1e-3
        x = torch.where(mask, x * 100, x)
    return x.to(dtype)


def sigmas(n, seed=1234):
    g = torch.Generator().manual_seed(seed)
    return (10 ** torch.empty(n).uniform_(-5, -2, generator=g)).tolist()


# ------------------------------------------------------------------------------------------------
# CPU legs (oracle)
# ------------------------------------------------------------------------------------------------

def cpu_sample_shapes(workload: str):
    """Bounded sample of the workload: one decoder layer's nine tensors (Llama shapes) or the first
    transformer block plus the position table (GPT-2 shape)."""
    sh = S.WORKLOADS[workload]()
    if workload.startswith("llama"):
        return sh[1:10], "one decoder layer (4 attention + 3 MLP matrices + 2 norm vectors), bf16, warm state"
    return sh[1:14], "position table + first transformer block, bf16, warm state"


def run_cpu(workload: str, form: str, steps: int, warmup: int, budget_s: float = 25.0):
    """Time the CPU oracle on the bounded sample.  form: 'c' (plain C, OpenMP) or 'torch' (the
    reference's torch operators).  Returns (Gparams/s, cores, seconds per step, sample text)."""
    from oracle import c_oracle, torch_oracle
    shapes, text = cpu_sample_shapes(workload)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    c_oracle.set_threads(cores)
    step_fn = c_oracle.step_tensor if form == "c" else torch_oracle.step_tensor
    gen = torch.Generator().manual_seed(0)
    sig = sigmas(len(shapes))
    params = [synth_tensor(s, 0.02, gen, "cpu", outliers=False) for s in shapes]
    grads = [synth_tensor(s, sg, gen, "cpu") for s, sg in zip(shapes, sig)]
    states = [torch_oracle.TensorState.zeros(s) for s in shapes]
    hp = (HP["lr"], HP["betas"][0], HP["betas"][1], HP["eps"], HP["weight_decay"])

    def one():
        for p, g, st in zip(params, grads, states):
            step_fn(p, g, st, *hp)

    t0 = time.perf_counter()
    one()
    first = time.perf_counter() - t0
    warm = max(1, min(warmup, int(budget_s * 0.3 / max(first, 1e-3))))
    for _ in range(warm - 1):
        one()
    k = max(1, min(steps, int(budget_s * 0.7 / max(first, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(k):
        one()
    dt = (time.perf_counter() - t0) / k
    n = S.numel(shapes)
    return n / dt / 1e9, cores, dt, f"{text}; {n} params, {k} timed steps after {warm} warm-up"


def reference_arm(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    workload = args.workload or "llama7b"     # the same workload as the main arm, at every N
    value, cores, dt, text = run_cpu(workload, "torch", args.steps, args.warmup, budget_s=120.0)
    print(json.dumps({
        "impl": "reference", "metric": "4-bit AdamW step throughput", "value": value, "unit": "Gparams/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "sample": text},
        "cpu_baseline": {"value": value, "unit": "Gparams/s", "cores": cores, "kind": "port", "sample": text},
        "e2e": {"value": value, "unit": "Gparams/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "the reference's pure-PyTorch path cannot complete a step (it stops itself); timed here is its "
                "torch-operator restatement (oracle/torch_oracle.py) on all host threads",
    }))


# ------------------------------------------------------------------------------------------------
# GPU arm, one GPU
# ------------------------------------------------------------------------------------------------

def build_problem(shapes, device, seed=0, grad_sets=2):
    gen = torch.Generator(device=device).manual_seed(seed)
    sig = sigmas(len(shapes))
    params = [torch.nn.Parameter(synth_tensor(s, 0.02, gen, device, outliers=False), requires_grad=False) for s in shapes]
    grads = [[synth_tensor(s, sg, gen, device) for s, sg in zip(shapes, sig)] for _ in range(grad_sets)]
    return params, grads


def single_gpu(args):
    import ctypes as C

    import quantfour_adamw_cuda_b200 as qf
    from quantfour_adamw_cuda_b200 import _lib

    workload = args.workload or "llama7b"
    shapes = S.WORKLOADS[workload]()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    n_params = S.numel(shapes)
    alg_bytes = S.algorithmic_bytes(shapes)
    params, grads = build_problem(shapes, dev)
    opt = qf.FourBitAdamW(params, **HP)

    def set_grads(k):
        for p, g in zip(params, grads[k % len(grads)]):
            p.grad = g

    # ---- warm-up through the public API (also builds the state and the descriptor table) ----------
    for i in range(max(3, args.warmup)):
        set_grads(i)
        opt.step()
    torch.cuda.synchronize(dev)
    if args.start_step:
        for st in opt.state.values():
            st["step"].fill_(float(args.start_step))
        set_grads(0)
        opt.step()      # the optimizer notices the rewritten counters and rebuilds its per-step constants
        torch.cuda.synchronize(dev)

    # ---- timed region: exactly K steps, device time -----------------------------------------------
    sampler = ClockSampler(dev.index)
    sampler.start()
    time.sleep(0.3)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    torch.cuda.synchronize(dev)
    ev[0].record()
    for i in range(args.steps):
        set_grads(i)
        opt.step(grad_scale=args.grad_scale)
        ev[i + 1].record()
    torch.cuda.synchronize(dev)
    total_ms = ev[0].elapsed_time(ev[-1])
    per_step = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]
    clocks = sampler.stop()
    ms_per_step = total_ms / args.steps
    value = n_params / (ms_per_step * 1e-3) / 1e9

    # ---- per-kernel split: the two halves of the step through the C ABI, events around each --------
    L = _lib.lib()
    plan = next(iter(opt._plans.values()))
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    pre_ms = main_ms = 0.0
    reps = min(args.steps, 10)
    e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    for i in range(reps):
        for st in opt.state.values():
            st["step"] += 1
        h = (_lib.QfHyper * 1)(qf.make_hyper(HP["lr"], *HP["betas"], HP["eps"], HP["weight_decay"],
                                             float(next(iter(opt.state.values()))["step"]), args.grad_scale or 1.0))
        a = (plan.descs, len(plan.descs), h, 1, plan.workspace.data_ptr(), plan.workspace.numel(), dev.index, stream)
        e[0].record()
        _lib.check(L.qf_step_pre(*a), "qf_step_pre")
        e[1].record()
        _lib.check(L.qf_step_main(*a), "qf_step_main")
        e[2].record()
        torch.cuda.synchronize(dev)
        pre_ms += e[0].elapsed_time(e[1]) / reps
        main_ms += e[1].elapsed_time(e[2]) / reps

    # ---- end to end: gradients arrive from pinned host memory every step ----------------------------
    e2e = None
    if not args.no_e2e:
        host = [g.cpu().pin_memory() for g in grads[0]]
        h2d = sum(t.numel() * t.element_size() for t in host)
        dst = grads[0]
        k = max(1, min(args.steps, 5))
        for p, g in zip(params, dst):
            p.grad = g

        # The way a host that holds the gradients would drive the public API: the parameter list in eight groups of about
        # equal bytes, one optimizer each; the copies of all groups go out on a copy stream, and the step of group k
        # starts when its gradients have arrived, while those of group k + 1 are still crossing PCIe.
        n_groups = 8
        bounds, acc, target = [0], 0, h2d / n_groups
        for i, t in enumerate(host):
            acc += t.numel() * t.element_size()
            if acc >= target * len(bounds) and len(bounds) < n_groups:
                bounds.append(i + 1)
        if bounds[-1] != len(host):
            bounds.append(len(host))
        groups = [(bounds[j], bounds[j + 1]) for j in range(len(bounds) - 1)]
        del opt
        torch.cuda.empty_cache()
        # In its steady state (same tensors, same gradient buffers) a step copies nothing from the host, so its kernels
        # cannot get stuck on the copy engine behind the gradient copies that were submitted before it.
        opts = [qf.FourBitAdamW(params[a:b], **HP) for a, b in groups]
        copy_stream = torch.cuda.Stream(dev)
        arrived = [torch.cuda.Event() for _ in groups]
        cur = torch.cuda.current_stream(dev)

        def e2e_step():
            copy_stream.wait_stream(cur)           # the last step has finished with the gradient buffers
            for (a, b), ev, o in zip(groups, arrived, opts):
                with torch.cuda.stream(copy_stream):
                    for hsrc, d in zip(host[a:b], dst[a:b]):
                        d.copy_(hsrc, non_blocking=True)
                    ev.record(copy_stream)
                cur.wait_event(ev)
                o.step()
            return any([o.nonfinite_seen() for o in opts])   # device -> host reads of the status words; synchronise

        e2e_step()
        e2e_step()
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        for _ in range(k):
            e2e_step()
        dt = (time.perf_counter() - t0) / k
        e2e = {"value": n_params / dt / 1e9, "unit": "Gparams/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * len(opts),
               "ms_per_step": dt * 1e3, "steps": k,
               "how": "%d groups of tensors, one optimizer each; group k steps while group k + 1 is still being copied" % len(opts)}
        del host, opts
        opt = None

    peak, peak_kind = measured_peak()
    achieved = alg_bytes / (ms_per_step * 1e-3) / 1e9
    out = {
        "metric": "4-bit AdamW step throughput", "value": value, "unit": "Gparams/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "tensors": len(shapes), "params": n_params, "param_dtype": "bf16",
                   "start_step": args.start_step, "grad_scale": args.grad_scale,
                   "state": "4-bit m (block-128) + 4-bit v (rank-1 / block-128), fp32 for numel <= 4096",
                   "l2": "inputs (%.1f GB per step) are far larger than L2" % (alg_bytes / 1e9),
                   "ms_per_step_min": min(per_step), "ms_per_step_max": max(per_step),
                   "ms_per_step_median": float(np.median(per_step)), "ms_per_step_p10": float(np.percentile(per_step, 10)),
                   "ms_per_step_p90": float(np.percentile(per_step, 90))},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": alg_bytes * TRAFFIC_PER_ALGORITHMIC_BYTE,
                     "traffic_kind": "scaled from an ncu capture of the same kernels on the 355 M-parameter set",
                     "peak_kind": peak_kind, "frac_of_8TBs": achieved / 8000.0,
                     "algorithmic_bytes_per_step": alg_bytes, "kernels_ms": {"pre": pre_ms, "main": main_ms},
                     "note": "whole step (clear, pre, reciprocals, main panel, main flat, commit: 6 launches) over algorithmic bytes"},
        "e2e": e2e, "gpu_launches": 6 * args.steps, "clocks": clocks,
    }
    if not args.no_also:
        del opt, params, grads
        torch.cuda.empty_cache()
        out["also"] = also_block(dev, peak)
    if not args.no_cpu:
        v, cores, dt, text = run_cpu(workload, "c", 3, 1)
        out["cpu_baseline"] = {"value": v, "unit": "Gparams/s", "cores": cores, "kind": "port", "sample": text,
                               "form": "plain-C oracle with OpenMP"}
    print(json.dumps(out))


def timed_steps(opt, params, grads, steps, dev):
    """Device time per step over `steps` steps of `opt` with the gradient sets rotated."""
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    ev0.record()
    for i in range(steps):
        for p, g in zip(params, grads[i % len(grads)]):
            p.grad = g
        opt.step()
    ev1.record()
    torch.cuda.synchronize(dev)
    return ev0.elapsed_time(ev1) / steps


def graph_replay_ms(params, grads, steps, dev):
    """Device time per step of the capturable step (FourBitAdamW(capturable=True)) recorded once into a CUDA graph and
    replayed: no host work per step.  The optimizer starts from zero state and takes three eager steps first."""
    import quantfour_adamw_cuda_b200 as qf
    opt = qf.FourBitAdamW(params, capturable=True, **HP)
    for p, g in zip(params, grads):
        p.grad = g
    for _ in range(3):
        opt.step()
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            opt.step()
    torch.cuda.current_stream(dev).wait_stream(side)
    for _ in range(3):
        graph.replay()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    ev0.record()
    for _ in range(steps):
        graph.replay()
    ev1.record()
    torch.cuda.synchronize(dev)
    return ev0.elapsed_time(ev1) / steps, opt.schedule_exhausted()


def also_block(dev, peak):
    """The other configurations of the benchmark list on this GPU, outside the timed region of the headline: the
    single fp32 4096 x 4096 parameter, the stand-alone quantize / dequantize kernels, the GPT-2-medium-shaped list
    (first step from zero state, and warm), and the Llama-13B-shaped set unsharded."""
    import quantfour_adamw_cuda_b200 as qf
    out = {}
    # one fp32 4096 x 4096 parameter, 10 steps with fresh gradients (the reference's CPU-runnable case, here on the GPU)
    gen = torch.Generator(device=dev).manual_seed(0)
    p = torch.nn.Parameter(torch.randn(4096, 4096, generator=gen, device=dev) * 0.02, requires_grad=False)
    gs = [[torch.randn(4096, 4096, generator=gen, device=dev) * 1e-3] for _ in range(10)]
    opt = qf.FourBitAdamW([p], **HP)
    timed_steps(opt, [p], gs, 10, dev)                      # the ten steps of the configuration (from zero state)
    ms = timed_steps(opt, [p], gs, 20, dev)                 # the same gradients again, warm
    nbytes = S.algorithmic_bytes([(4096, 4096)], elem_bytes=4)
    out["fp32_4096x4096"] = {"ms_per_step": ms, "GBps": nbytes / ms / 1e6, "frac": nbytes / ms / 1e6 / peak,
                             "algorithmic_bytes": nbytes, "note": "fp32 parameter and gradient: 14 bytes per element"}
    del opt
    p.grad = None
    gms, _ = graph_replay_ms([p], gs[0], 50, dev)
    out["fp32_4096x4096"]["cuda_graph_replay"] = {"ms_per_step": gms, "GBps": nbytes / gms / 1e6, "frac": nbytes / gms / 1e6 / peak}
    del p, gs
    # stand-alone quantize / dequantize
    out["quantize"] = quantize_kernels(dev, peak, steps=20, warmup=3)
    torch.cuda.empty_cache()
    # GPT-2-medium-shaped ragged list
    shapes = S.WORKLOADS["gpt2m"]()
    params, grads = build_problem(shapes, dev, grad_sets=1)
    opt = qf.FourBitAdamW(params, **HP)
    first = timed_steps(opt, params, grads, 1, dev)         # includes state allocation and the exact arithmetic of a zero state
    timed_steps(opt, params, grads, 3, dev)
    ms = timed_steps(opt, params, grads, 50, dev)
    nbytes = S.algorithmic_bytes(shapes)
    out["gpt2m"] = {"ms_per_step": ms, "first_step_ms": first, "params": S.numel(shapes), "tensors": len(shapes),
                    "GBps": nbytes / ms / 1e6, "frac": nbytes / ms / 1e6 / peak}
    del opt
    gms, exhausted = graph_replay_ms(params, grads[0], 50, dev)
    out["gpt2m"]["cuda_graph_replay"] = {"ms_per_step": gms, "GBps": nbytes / gms / 1e6, "frac": nbytes / gms / 1e6 / peak,
                                         "schedule_exhausted": exhausted}
    del params, grads
    torch.cuda.empty_cache()
    # Llama-13B-shaped set on one GPU (the sharded runs use it at 2, 4 and 8 GPUs)
    shapes = S.WORKLOADS["llama13b"]()
    params, grads = build_problem(shapes, dev, grad_sets=1)
    opt = qf.FourBitAdamW(params, **HP)
    timed_steps(opt, params, grads, 4, dev)
    ms = timed_steps(opt, params, grads, 8, dev)
    nbytes = S.algorithmic_bytes(shapes)
    out["llama13b"] = {"ms_per_step": ms, "params": S.numel(shapes), "Gparams_per_s": S.numel(shapes) / ms / 1e6,
                       "GBps": nbytes / ms / 1e6, "frac": nbytes / ms / 1e6 / peak}
    del opt
    # the same set with relaxed_update=True (an option, off by default: uncorrected bf16 parameter update, new parameters
    # within a few bf16 units of the exact ones, codes and scales bit-identical)
    for p in params:
        p.grad = None
    opt = qf.FourBitAdamW(params, relaxed_update=True, **HP)
    timed_steps(opt, params, grads, 4, dev)
    rms = timed_steps(opt, params, grads, 8, dev)
    out["llama13b"]["relaxed_update"] = {"ms_per_step": rms, "GBps": nbytes / rms / 1e6, "frac": nbytes / rms / 1e6 / peak}
    del opt, params, grads
    torch.cuda.empty_cache()
    return out


def quantize_kernels(dev, peak, steps, warmup):
    """Times of the four stand-alone kernels at the sizes of the quantize / dequantize configuration."""
    import quantfour_adamw_cuda_b200 as qf
    n = 1 << 28
    x = torch.randn(n, generator=torch.Generator(device=dev).manual_seed(0), device=dev) * 1e-3
    x = torch.where(torch.rand(n, generator=torch.Generator(device=dev).manual_seed(1), device=dev) < 1e-3, x * 100, x)
    R = C = 16384
    v = (torch.randn(R, C, generator=torch.Generator(device=dev).manual_seed(2), device=dev) * 1e-3) ** 2
    codes_m, sc_m = qf.quantize_m(x)
    codes_v, row, col = qf.quantize_v(v)
    cases = {
        "quantize_m": (lambda: qf.quantize_m(x), n * 4.5 + n // 32),
        "dequantize_m": (lambda: qf.dequantize_m(codes_m, sc_m, n), n * 4.5 + n // 32),
        "quantize_v_rank1": (lambda: qf.quantize_v(v), R * C * 4.5 + 8 * R),
        "dequantize_v_rank1": (lambda: qf.dequantize_v(codes_v, row, col), R * C * 4.5 + 8 * R),
    }
    out = {}
    for name, (fn, nbytes) in cases.items():
        for _ in range(max(3, warmup)):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(dev)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1) / steps
        out[name] = {"ms": ms, "GBps": nbytes / ms / 1e6, "frac_of_peak": nbytes / ms / 1e6 / peak}
    out["quantize_v_rank1"]["two_read_bound_frac"] = (R * C * 4.5 + 8 * R) / (R * C * 8.5 + 8 * R)
    out["note"] = ("2^28 fp32 values (block-128, dynamic-exponent map) and a 16384 x 16384 fp32 matrix (rank-1); GB/s over the "
                   "compulsory bytes of each call; the rank-1 quantize has to read its input twice (maxima, then codes), which "
                   "caps it at two_read_bound_frac of the peak on this scale; timings include the allocation of the outputs by "
                   "torch's caching allocator")
    return out


def quantize_micro(args):
    """Stand-alone quantize / dequantize micro-benchmark: first-moment path on 2^28 fp32 values ~N(0, 1e-3) with 0.1 %
    of the entries x100 (block-128, dynamic-exponent map), second-moment path on a 16384 x 16384 fp32 matrix of squared
    N(0, 1e-3) values (rank-1 row / column maxima).  One JSON line; GB/s over the compulsory bytes of each call."""
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peak, peak_kind = measured_peak()
    out = quantize_kernels(dev, peak, args.steps, args.warmup)
    note = out.pop("note")
    print(json.dumps({"metric": "stand-alone quantize / dequantize", "unit": "GB/s over compulsory bytes", "n_gpus": 1,
                      "steps": args.steps, "data": "synthetic", "peak": peak, "peak_kind": peak_kind,
                      "config": {"workload": "quantize", "m": "2^28 fp32", "v": "16384x16384 fp32", "note": note},
                      "kernels": out}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=[None, *S.WORKLOADS, "quantize"])
    ap.add_argument("--comm", default="auto", choices=["auto", "nccl", "p2p", "ce"],
                    help="N>1: how the updated parameters reach the other ranks (copy engines piece by piece, peer stores from "
                         "the update kernel, or an all-gather afterwards)")
    ap.add_argument("--start-step", type=int, default=0,
                    help="N=1: set every step counter to this value after the warm-up (>= 20000 shows the late-training "
                         "regime where sqrt(1 - beta2^t) has rounded to 1)")
    ap.add_argument("--reduce-grads", action="store_true",
                    help="N>1: the step starts with the mean of the per-rank gradients kept in a flat buffer, each rank over its own range "
                         "(peer loads inside a node, NCCL's reduce-scatter timed beside it)")
    ap.add_argument("--grad-scale", type=float, default=None,
                    help="N=1: pass this factor to every timed step (the first pass then rewrites the gradients scaled); "
                         "use a value next to 1, e.g. 1.0000001, so that repeated steps do not drive the data to zero")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-also", action="store_true", help="skip the other configurations reported beside the headline")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU arm")
    if args.workload == "quantize":
        return quantize_micro(args)
    if args.gpus == 1 and int(os.environ.get("WORLD_SIZE", "1")) == 1:
        return single_gpu(args)
    import bench_zero1
    return bench_zero1.run(args, HP)


if __name__ == "__main__":
    main()

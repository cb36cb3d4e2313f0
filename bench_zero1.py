"""Multi-GPU leg of bench.py: the Llama-13B-shaped parameter set with the 4-bit optimizer state sharded over
the ranks (ShardedFourBitAdamW), one process per GPU under torchrun.  NCCL carries the max exchange; the updated
bf16 parameters reach the other ranks through peer stores issued by the update kernel itself (comm "p2p", the
default where it can be set up) or through an NCCL all-gather after it (comm "nccl").  Both are timed; the
headline is the mode the optimizer picked."""
from __future__ import annotations

import json
import os
import time

import torch
import torch.distributed as dist

from quantfour_adamw_cuda_b200 import shapes as S
from quantfour_adamw_cuda_b200.zero1 import ShardedFourBitAdamW


def _max_over_ranks(x: float, dev) -> float:
    t = torch.tensor([x], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _step_ms(bench, shapes, hp, comm, steps, warm, dev) -> dict:
    """Device time of the sharded step over `shapes` (max over ranks), set up and torn down in place."""
    params, grads = bench.build_problem(shapes, dev, seed=0, grad_sets=1)
    opt = ShardedFourBitAdamW(params, comm=comm, **hp)
    for p, g in zip(params, grads[0]):
        p.grad = g
    for _ in range(warm):
        opt.step()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize(dev)
    ev0.record()
    for _ in range(steps):
        opt.step()
    ev1.record()
    dist.barrier()
    torch.cuda.synchronize(dev)
    ms = _max_over_ranks(ev0.elapsed_time(ev1) / steps, dev)
    out = {"params": S.numel(shapes), "ms_per_step": ms, "Gparams_per_s": S.numel(shapes) / (ms * 1e-3) / 1e9, "comm": opt.comm}
    opt.close()
    dist.barrier()
    return out


def run(args, hp) -> None:
    import bench  # the repo-root script: synthetic data, clock sampler, peaks, CPU leg

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    workload = args.workload or "llama13b"
    shapes = S.WORKLOADS[workload]()
    n_params, alg_bytes = S.numel(shapes), S.algorithmic_bytes(shapes)
    params, grads = bench.build_problem(shapes, dev, seed=0, grad_sets=1)   # same seed: replicated parameters
    reduce_grads = bool(getattr(args, "reduce_grads", False))
    opt = ShardedFourBitAdamW(params, comm=getattr(args, "comm", None) or "auto", reduce_grads=reduce_grads, **hp)
    if reduce_grads:     # the gradients live in the optimizer's flat buffer; every rank holds the same values here,
        for p, g in zip(params, grads[0]):   # so their mean leaves them unchanged from step to step
            p.grad.copy_(g)
        grads = None
        torch.cuda.empty_cache()
    else:
        for p, g in zip(params, grads[0]):
            p.grad = g
    warm = max(3, args.warmup)
    for _ in range(warm):
        opt.step()
    torch.cuda.synchronize(dev)

    sampler = bench.ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    torch.cuda.synchronize(dev)
    ev0.record()
    for _ in range(args.steps):
        opt.step()
    ev1.record()
    dist.barrier()
    torch.cuda.synchronize(dev)
    ms_per_step = _max_over_ranks(ev0.elapsed_time(ev1) / args.steps, dev)
    clocks = sampler.stop() if rank == 0 else None

    # the parts of a step, each timed on the device and maxed over ranks
    reps = min(args.steps, 5)
    e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    parts = [0.0, 0.0, 0.0]
    for _ in range(reps):
        dist.barrier()
        e[0].record()
        opt.step_pre()
        if opt.shared_new.numel():
            dist.all_reduce(opt.shared_new, op=dist.ReduceOp.MAX)
        e[1].record()
        opt.step_main()
        e[2].record()
        opt._all_gather()
        e[3].record()
        torch.cuda.synchronize(dev)
        for k in range(3):
            parts[k] += e[k].elapsed_time(e[k + 1]) / reps
    parts = [_max_over_ranks(x, dev) for x in parts]
    reduce_ms = None
    if reduce_grads:
        reduce_ms = 0.0
        for _ in range(reps):
            dist.barrier()
            e[0].record()
            opt._reduce_gradients()
            e[1].record()
            torch.cuda.synchronize(dev)
            reduce_ms += e[0].elapsed_time(e[1]) / reps
        reduce_ms = _max_over_ranks(reduce_ms, dev)
    push_ms = None
    if opt.comm == "p2p":   # the fused main pass: update + peer stores, closed by the small collective
        push_ms = 0.0
        for _ in range(reps):
            opt.step_pre()
            if opt.shared_new.numel():
                dist.all_reduce(opt.shared_new, op=dist.ReduceOp.MAX)
            dist.barrier()
            e[0].record()
            opt.backend.main_push(opt.states, opt._hyper, opt.peer_deltas)
            dist.all_reduce(opt._token, op=dist.ReduceOp.MAX)
            e[1].record()
            torch.cuda.synchronize(dev)
            push_ms += e[0].elapsed_time(e[1]) / reps
        push_ms = _max_over_ranks(push_ms, dev)

    shard_elements, flat_total = opt.layout.shard, opt.layout.total
    # kernels of this library per step on this rank: clear / reciprocals / commit, plus one pre and one main kernel
    # per mapping that has work (whole-row pieces with a column count that is a multiple of 256 take the panel mapping)
    from quantfour_adamw_cuda_b200.zero1 import RANK1
    recs = [st.rec for st in opt.states]
    panel = any(r.kind == RANK1 and not r.partial and r.cols % 256 == 0 for r in recs)
    flat_r1 = any(r.kind == RANK1 and (r.partial or r.cols % 256) for r in recs)
    flat_other = any(r.kind != RANK1 for r in recs)
    launches_per_step = 3 + 2 * int(panel) + int(flat_r1) + int(flat_r1 or flat_other)
    # end to end: this rank's slices of the gradients arrive from pinned host memory every step
    e2e = None
    if reduce_grads:
        args.no_e2e = True    # the end-to-end leg feeds only this rank's slices, which is not what a reduce-scatter consumes
    if not args.no_e2e:
        host = [st.g.cpu().pin_memory() for st in opt.states]
        h2d = sum(t.numel() * t.element_size() for t in host)
        k = max(1, min(args.steps, 5))

        def e2e_step():
            for src, st in zip(host, opt.states):
                st.g.copy_(src, non_blocking=True)
            opt.step()
            torch.cuda.current_stream(dev).synchronize()
            return float(opt.flat[0])            # device -> host read of one updated parameter

        e2e_step()
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(k):
            e2e_step()
        dist.barrier()
        dt = _max_over_ranks((time.perf_counter() - t0) / k, dev)
        h2d_all = torch.tensor([h2d], dtype=torch.float64, device=dev)
        dist.all_reduce(h2d_all)
        e2e = {"value": n_params / dt / 1e9, "unit": "Gparams/s", "h2d_bytes_per_step": int(h2d_all.item()),
               "d2h_bytes_per_step": 2 * world, "ms_per_step": dt * 1e3, "steps": k}

    # the 7B shape sharded the same way (the metric also asks for its step time at 2/4/8 GPUs)
    also = None
    if workload == "llama13b":
        opt.close()
        dist.barrier()
        torch.cuda.synchronize(dev)
        comm_used = opt.comm_selected
        del opt, params, grads
        if not args.no_e2e:
            del host, e2e_step     # the closure holds the optimizer
        torch.cuda.empty_cache()
        also = {"llama7b": _step_ms(bench, S.WORKLOADS["llama7b"](), hp, comm_used, max(3, min(args.steps, 10)), 3, dev)}
    else:
        comm_used = opt.comm_selected

    if rank == 0:
        peak, peak_kind = bench.measured_peak()
        shard_bytes = alg_bytes / world
        compute_ms = parts[0] + parts[1]
        gather_bytes = (world - 1) / world * 2 * flat_total
        out = {
            "metric": "4-bit AdamW step throughput", "value": n_params / (ms_per_step * 1e-3) / 1e9, "unit": "Gparams/s",
            "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload, "tensors": len(shapes), "params": n_params, "param_dtype": "bf16",
                       "parallelism": f"zero1-dp{world}", "shard_elements": shard_elements, "comm": comm_used, "reduce_grads": reduce_grads,
                       "l2": "inputs (%.1f GB per rank and step) are far larger than L2" % (shard_bytes / 1e9)},
            "roofline": {"bound": "hbm", "achieved": shard_bytes / (compute_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": shard_bytes / (compute_ms * 1e-3) / 1e9 / peak, "traffic": None, "peak_kind": peak_kind,
                         "note": "per rank: algorithmic bytes of the rank's shard over the device time of its fused step "
                                 "(both halves incl. the max exchange), all-gather excluded",
                         "parts_ms": {"pre+max_exchange": parts[0], "main": parts[1], "all_gather": parts[2],
                                      "grad_reduce_scatter": reduce_ms},
                         "all_gather": {"bytes_received_per_gpu": gather_bytes,
                                        "GBps_per_gpu": gather_bytes / (parts[2] * 1e-3) / 1e9 if parts[2] else None,
                                        "link_peak_GBps": 770.0},
                         "main_with_peer_stores": None if push_ms is None else {
                             "ms": push_ms, "bytes_sent_per_gpu": gather_bytes,
                             "GBps_per_gpu": gather_bytes / (push_ms * 1e-3) / 1e9, "link_peak_GBps": 770.0,
                             "target_ms": max(parts[1], gather_bytes / 770e9 * 1e3),
                             "note": "target = the slower of the plain main pass and the bytes that must leave the GPU over the measured peer-copy bandwidth"}},
            "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "clocks": clocks, "also": also,
        }
        print(json.dumps(out))
    dist.destroy_process_group()

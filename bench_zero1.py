"""Multi-GPU leg of bench.py: the optimizer state sharded over the ranks (ShardedFourBitAdamW), one process per GPU
under torchrun.  The headline workload is the same at every N -- the Llama-7B-shaped set, so the lines at N = 1, 2, 4, 8
form one strong-scaling curve -- and the Llama-13B-shaped set is reported beside it.  NCCL carries the max exchange; the
updated bf16 parameters reach the other ranks while the update computes -- through peer stores issued by the update kernel
itself (comm "p2p", the default where it can be set up) or in pieces through the copy engines (comm "ce") -- or through an
NCCL all-gather after it (comm "nccl").

Every measured workload ends with two checks: the flat parameter buffers of all ranks must be identical (a 64-bit
checksum, minimum and maximum over the ranks), and one whole tensor -- one that is cut between ranks where there is
one -- is recomputed by the CPU oracle on rank 0 for the same number of steps and compared bit for bit."""
from __future__ import annotations

import json
import os
import time

import torch
import torch.distributed as dist

from quantfour_adamw_cuda_b200 import shapes as S
from quantfour_adamw_cuda_b200.zero1 import RANK1, ShardedFourBitAdamW


def _max_over_ranks(x: float, dev) -> float:
    t = torch.tensor([x], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _checksum(flat: torch.Tensor) -> int:
    """Order-dependent 64-bit checksum of a buffer's bytes (wrapping integer arithmetic on the device, in chunks)."""
    words = flat.view(torch.int16)
    total, chunk = 0, 1 << 26
    for lo in range(0, words.numel(), chunk):
        w = words[lo:lo + chunk].to(torch.int64)
        idx = torch.arange(lo, lo + w.numel(), device=flat.device, dtype=torch.int64)
        total = (total + int(((w + 40503) * ((idx % 65521) * 2 + 1)).sum().item())) & 0x7fffffffffffffff
    return total


def peer_copy_rates(dev, rank: int, world: int) -> dict:
    """Device-to-device copy rate out of this GPU with every GPU copying at once, measured with plain copies: to the
    next rank only (a ring, 1 GiB), and to all other ranks at the same time (1 GiB each, 512 MiB at eight ranks).  GB/s
    per GPU and direction, best of three rounds, minimum over the ranks."""
    n_ring, n_all = 1 << 30, (1 << 30 if world <= 4 else 1 << 29)
    src = torch.empty(n_ring, dtype=torch.uint8, device=dev)
    peers = [(rank + k) % world for k in range(1, world)]
    dst = {r: torch.empty(n_ring if r == peers[0] else n_all, dtype=torch.uint8, device=torch.device("cuda", r)) for r in peers}
    streams = {r: torch.cuda.Stream(dev) for r in peers}
    out = {}
    for name, targets, nbytes in (("ring", peers[:1], n_ring), ("all_to_all", peers, n_all)):
        best = 0.0
        for rep in range(4):
            dist.barrier()
            torch.cuda.synchronize(dev)
            t0 = time.perf_counter()
            for r in targets:
                with torch.cuda.stream(streams[r]):
                    dst[r][:nbytes].copy_(src[:nbytes], non_blocking=True)
            for r in targets:
                streams[r].synchronize()
            dt = time.perf_counter() - t0
            best = max(best, len(targets) * nbytes / dt / 1e9) if rep else best   # the first round opens the peer mappings
        t = torch.tensor([best], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        out[name] = float(t.item())
    del src, dst
    torch.cuda.empty_cache()
    return out


def measure(bench, workload: str, hp, args, dev, rank: int, world: int, detail: bool) -> dict:
    """Build the workload, run warm-up + timed steps of the sharded optimizer, time the parts of a step, and check
    the result (replicas identical; one tensor against the CPU oracle)."""
    from oracle import c_oracle as CO
    from oracle import torch_oracle as TO

    shapes = S.WORKLOADS[workload]()
    n_params, alg_bytes = S.numel(shapes), S.algorithmic_bytes(shapes)
    params, grads = bench.build_problem(shapes, dev, seed=0, grad_sets=1)   # same seed: replicated parameters
    reduce_grads = bool(getattr(args, "reduce_grads", False)) and detail
    opt = ShardedFourBitAdamW(params, comm=getattr(args, "comm", None) or "auto", reduce_grads=reduce_grads, **hp)
    # the tensor the oracle recomputes: the first one that is cut between ranks (its maxima go through the exchange)
    lay = opt.layout
    cut = [t for t in range(len(shapes)) if len(lay.owners(t)) > 1 and len(shapes[t]) == 2]
    probe = cut[0] if cut else min(range(len(shapes)), key=lambda t: abs(S.numel([shapes[t]]) - (1 << 24)))
    probe_p0 = params[probe].detach().cpu().clone() if rank == 0 else None
    probe_g = grads[0][probe].detach().cpu().clone() if rank == 0 else None
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

    sampler = bench.ClockSampler(dev.index)
    if rank == 0 and detail:
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
    clocks = sampler.stop() if rank == 0 and detail else None

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
    reduce_ms = nccl_reduce_ms = None
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
        # the yardstick: NCCL's reduce-scatter of the same bytes (what the optimizer falls back to without peer mappings)
        nccl_reduce_ms = None
        if opt.grad_deltas:
            saved, opt.grad_deltas = opt.grad_deltas, []
            nccl_reduce_ms = 0.0
            for i in range(reps + 1):
                dist.barrier()
                e[0].record()
                opt._reduce_gradients()
                e[1].record()
                torch.cuda.synchronize(dev)
                if i:
                    nccl_reduce_ms += e[0].elapsed_time(e[1]) / reps
            nccl_reduce_ms = _max_over_ranks(nccl_reduce_ms, dev)
            opt.grad_deltas = saved
    push_ms = None
    if opt.comm in ("p2p", "ce"):   # the main pass with the delivery inside it (peer stores, or pieces + copy engines), closed by the small collective
        push_ms = 0.0
        for _ in range(reps):
            opt.step_pre()
            if opt.shared_new.numel():
                dist.all_reduce(opt.shared_new, op=dist.ReduceOp.MAX)
            dist.barrier()
            e[0].record()
            if opt.comm == "p2p":
                opt.backend.main_push(opt.states, opt._hyper, opt.peer_deltas)
            else:
                opt._main_ce()
            dist.all_reduce(opt._token, op=dist.ReduceOp.MAX)
            e[1].record()
            torch.cuda.synchronize(dev)
            push_ms += e[0].elapsed_time(e[1]) / reps
        push_ms = _max_over_ranks(push_ms, dev)

    # ---- checks: all replicas hold the same parameters; one tensor equals the oracle's ----------------------
    dist.barrier()
    torch.cuda.synchronize(dev)
    cs = torch.tensor([_checksum(opt.flat)], dtype=torch.int64, device=dev)
    lo, hi = cs.clone(), cs.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    replicas_identical = bool(lo.item() == hi.item())
    oracle_subset = None
    if rank == 0 and not reduce_grads:
        st = TO.TensorState.zeros(shapes[probe])
        want = probe_p0
        CO.set_threads(os.cpu_count() or 1)
        for _ in range(opt.step_count):
            CO.step_tensor(want, probe_g, st, hp["lr"], hp["betas"][0], hp["betas"][1], hp["eps"], hp["weight_decay"])
        same = torch.equal(params[probe].detach().cpu(), want)
        oracle_subset = {"tensor": probe, "shape": list(shapes[probe]), "steps": opt.step_count,
                         "ranks_sharing_it": len(lay.owners(probe)), "result": "bit-exact" if same else "DIFFERS"}

    recs = [st.rec for st in opt.states]
    panel = any(r.kind == RANK1 and not r.partial and r.cols % 256 == 0 for r in recs)
    flat_r1 = any(r.kind == RANK1 and (r.partial or r.cols % 256) for r in recs)
    flat_other = any(r.kind != RANK1 for r in recs)
    launches_per_step = 3 + 2 * int(panel) + int(flat_r1) + int(flat_r1 or flat_other)

    # end to end: this rank's slices of the gradients arrive from pinned host memory every step
    e2e = None
    if detail and not args.no_e2e and not reduce_grads:
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
        del host, e2e_step

    out = {"workload": workload, "tensors": len(shapes), "params": n_params, "alg_bytes": alg_bytes, "ms_per_step": ms_per_step,
           "warm": warm, "parts": parts, "reduce_ms": reduce_ms, "nccl_reduce_ms": nccl_reduce_ms, "push_ms": push_ms, "comm": opt.comm_selected,
           "shard_elements": lay.shard, "flat_total": lay.total, "replicas_identical": replicas_identical,
           "oracle_subset": oracle_subset, "launches_per_step": launches_per_step, "clocks": clocks, "e2e": e2e,
           "reduce_grads": reduce_grads}
    opt.close()
    dist.barrier()
    torch.cuda.synchronize(dev)
    del opt, params, grads
    torch.cuda.empty_cache()
    return out


def run(args, hp) -> None:
    import bench  # the repo-root script: synthetic data, clock sampler, peaks

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    workload = args.workload or "llama7b"
    link = peer_copy_rates(dev, rank, world)
    m = measure(bench, workload, hp, args, dev, rank, world, detail=True)
    also = None
    if workload == "llama7b" and not getattr(args, "no_also", False):
        a = measure(bench, "llama13b", hp, args, dev, rank, world, detail=False)
        gather = (world - 1) / world * 2 * a["flat_total"]
        also = {"llama13b": {
            "params": a["params"], "ms_per_step": a["ms_per_step"], "Gparams_per_s": a["params"] / (a["ms_per_step"] * 1e-3) / 1e9,
            "comm": a["comm"], "shard_step_ms": a["parts"][0] + a["parts"][1],
            "parts_ms": {"pre+max_exchange": a["parts"][0], "main": a["parts"][1], "all_gather": a["parts"][2],
                         "main_with_delivery": a["push_ms"]},
            "delivery_bytes_per_gpu": gather, "delivery_bound_ms": gather / (link["all_to_all"] * 1e9) * 1e3,
            "replicas_identical": a["replicas_identical"], "oracle_subset": a["oracle_subset"]}}

    if rank == 0:
        peak, peak_kind = bench.measured_peak()
        n_params, alg_bytes, parts, push_ms = m["params"], m["alg_bytes"], m["parts"], m["push_ms"]
        shard_bytes = alg_bytes / world
        compute_ms = parts[0] + parts[1]
        gather_bytes = (world - 1) / world * 2 * m["flat_total"]
        rate = link["all_to_all"]
        out = {
            "metric": "4-bit AdamW step throughput", "value": n_params / (m["ms_per_step"] * 1e-3) / 1e9, "unit": "Gparams/s",
            "n_gpus": world, "steps": args.steps, "warmup": m["warm"], "ms_per_step": m["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload, "tensors": m["tensors"], "params": n_params, "param_dtype": "bf16",
                       "parallelism": f"zero1-dp{world}", "shard_elements": m["shard_elements"], "comm": m["comm"],
                       "reduce_grads": m["reduce_grads"],
                       "l2": "inputs (%.1f GB per rank and step) are far larger than L2" % (shard_bytes / 1e9)},
            "replicas_identical": m["replicas_identical"], "oracle_subset": m["oracle_subset"],
            # the part of the step that shards: first pass + max exchange + update of this rank's range (no delivery)
            "shard_step_ms": compute_ms,
            # the part that cannot: every GPU must send and receive (N-1)/N of the parameters
            "delivery": {"bytes_per_gpu": gather_bytes, "measured_peer_copy_GBps": link,
                         "bound_ms": gather_bytes / (rate * 1e9) * 1e3,
                         "note": "bound = bytes that must leave (and enter) every GPU over the copy rate measured at start-up with "
                                 "all GPUs copying to all others; it grows with N, so the whole step cannot scale linearly"},
            "roofline": {"bound": "hbm", "achieved": shard_bytes / (compute_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": shard_bytes / (compute_ms * 1e-3) / 1e9 / peak, "traffic": None, "peak_kind": peak_kind,
                         "note": "per rank: algorithmic bytes of the rank's shard over the device time of its fused step "
                                 "(both halves incl. the max exchange), delivery of the parameters excluded",
                         "parts_ms": {"pre+max_exchange": parts[0], "main": parts[1], "all_gather": parts[2],
                                      "grad_reduce_scatter": m["reduce_ms"], "grad_reduce_scatter_nccl": m["nccl_reduce_ms"]},
                         "all_gather": {"bytes_received_per_gpu": gather_bytes,
                                        "GBps_per_gpu": gather_bytes / (parts[2] * 1e-3) / 1e9 if parts[2] else None},
                         "main_with_delivery": None if push_ms is None else {
                             "how": "peer stores from the update kernel" if m["comm"] == "p2p" else "update in pieces, copy engines deliver each finished piece",
                             "ms": push_ms, "bytes_sent_per_gpu": gather_bytes,
                             "GBps_per_gpu": gather_bytes / (push_ms * 1e-3) / 1e9,
                             "frac_of_measured_copy_rate": gather_bytes / (push_ms * 1e-3) / 1e9 / rate,
                             "target_ms": max(parts[1], gather_bytes / (rate * 1e9) * 1e3),
                             "note": "target = the slower of the plain main pass and the delivery bound"}},
            "e2e": m["e2e"], "gpu_launches": m["launches_per_step"] * args.steps, "clocks": m["clocks"], "also": also,
        }
        print(json.dumps(out))
    dist.destroy_process_group()

"""One process per GPU on every GPU of the machine (2 to 8): the sharded step with the parameters delivered by peer
stores from the update kernel (comm="p2p") or by the copy engines piece by piece (comm="ce") must leave the same bits as
the all-gather path (comm="nccl") and as the unsharded oracle, for bf16 and fp32 parameters, with a shape list whose largest matrix is cut by three or more ranks
at 8 ranks; then the same with per-rank gradients and the reduce-scatter inside the step.  Skipped on a single-GPU
machine."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["QF_ROOT"])
from oracle import c_oracle as CO, torch_oracle as TO
from quantfour_adamw_cuda_b200.zero1 import ShardedFourBitAdamW
rank, local, world = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"]), int(os.environ["WORLD_SIZE"])
dev = torch.device("cuda", local)
torch.cuda.set_device(dev)
dist.init_process_group("nccl", device_id=dev)
SHAPES = [(300, 256), (1000,), (96, 128), (5000,), (64, 77), (1024, 512), (130, 384), (4096,), (512, 512)]
HP = (1e-3, 0.9, 0.999, 1e-8, 0.01)
for dtype in (torch.bfloat16, torch.float32):
    gen = torch.Generator().manual_seed(5)
    init = [(torch.randn(s, generator=gen) * 0.02).to(dtype) for s in SHAPES]
    want = [p.clone() for p in init]
    states = [TO.TensorState.zeros(s) for s in SHAPES]
    runs = {}
    for comm in ("p2p", "ce", "nccl"):
        params = [torch.nn.Parameter(p.to(dev)) for p in init]
        runs[comm] = (params, ShardedFourBitAdamW(params, lr=1e-3, comm=comm))
        assert runs[comm][1].comm == comm, (comm, runs[comm][1].comm)
    for step in range(5):
        gs = [(torch.randn(s, generator=gen) * 1e-3).to(dtype) for s in SHAPES]
        for p, g, st in zip(want, gs, states):
            CO.step_tensor(p, g, st, *HP)
        for params, opt in runs.values():
            for p, g in zip(params, gs):
                p.grad = g.to(dev)
            opt.step()
    torch.cuda.synchronize(dev)
    for comm, (params, opt) in runs.items():
        for i, (p, w) in enumerate(zip(params, want)):
            assert torch.equal(p.detach().cpu(), w), f"rank {rank} {comm} {dtype} tensor {i} {SHAPES[i]}"
    assert torch.equal(runs["p2p"][1].flat, runs["nccl"][1].flat) and torch.equal(runs["ce"][1].flat, runs["nccl"][1].flat)
    if dtype == torch.bfloat16:
        assert len(runs["ce"][1].chunks) >= 1
    lay = runs["p2p"][1].layout
    cut = max(len(lay.owners(t)) for t in range(len(SHAPES)))
    assert cut >= min(world, 3), f"the shape list should put one tensor on {min(world, 3)} or more ranks, got {cut}"
    runs["p2p"][1].close()
    runs["ce"][1].close()
# the ranks hold different gradients; the step starts with the reduce-scatter (mean) of the flat gradient buffer
for dtype in (torch.bfloat16, torch.float32):
    gen = torch.Generator().manual_seed(9)
    init = [(torch.randn(s, generator=gen) * 0.02).to(dtype) for s in SHAPES]
    want = [p.clone() for p in init]
    states = [TO.TensorState.zeros(s) for s in SHAPES]
    params = [torch.nn.Parameter(p.to(dev)) for p in init]
    opt = ShardedFourBitAdamW(params, lr=1e-3, reduce_grads=True)
    for step in range(4):
        opt.zero_grad()
        for p, w, st in zip(params, want, states):
            # small integers times 2^-13: every partial sum is exact in bf16, so the mean does not depend on the order
            # or the precision in which the collective adds the ranks up
            per_rank = [(torch.randint(-8, 9, w.shape, generator=gen).float() * 2.0 ** -13).to(dtype) for _ in range(world)]
            mean = (sum(x.float() for x in per_rank) / world).to(dtype)
            CO.step_tensor(w, mean, st, *HP)
            p.grad.add_(per_rank[rank].to(dev))
        opt.step()
    torch.cuda.synchronize(dev)
    for i, (p, w) in enumerate(zip(params, want)):
        assert torch.equal(p.detach().cpu(), w), f"rank {rank} reduce_grads {dtype} tensor {i} {SHAPES[i]}"
    opt.close()
dist.barrier()
dist.destroy_process_group()
print(f"rank {rank} ok")
'''


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_stores_match_all_gather_and_oracle_on_every_gpu(tmp_path):
    nproc = min(torch.cuda.device_count(), 8)
    nproc = 1 << (nproc.bit_length() - 1)     # 2, 4 or 8: the mean of the per-rank gradients stays exact
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, QF_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", "29631", str(script)]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    for r in range(nproc):
        assert f"rank {r} ok" in out.stdout
    print(f"{nproc} ranks: p2p == ce == nccl == oracle (bf16, fp32), reduce_grads == oracle")

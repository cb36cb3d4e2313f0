"""CPU tests of the sharded optimizer's host logic: the flat layout, the records of each rank, and -- as two
gloo ranks with the oracle standing in for the kernels -- that the sharded step (max exchange + all-gather)
reproduces the unsharded oracle bit for bit."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import torch_oracle as TO
from quantfour_adamw_cuda_b200.zero1 import BLOCKQ, FP32, RANK1, flat_layout, rank_records

SHAPES = [(300, 256), (1000,), (96, 128), (5000,), (64, 77), (40, 50), (130, 384), (4096,)]


def test_layout_is_block_aligned_and_balanced():
    for world in (1, 2, 3, 4, 8):
        lay = flat_layout(SHAPES, world)
        assert all(o % 128 == 0 for o in lay.offsets) and lay.shard % 128 == 0
        assert lay.total >= lay.offsets[-1] + lay.numels[-1] and lay.total - lay.shard < lay.offsets[-1] + lay.numels[-1] + 128 * world
        for a, b in zip(lay.offsets, lay.offsets[1:]):
            assert b >= a


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_records_tile_every_tensor_exactly_once(world):
    lay = flat_layout(SHAPES, world)
    cover = [torch.zeros(n, dtype=torch.int32) for n in lay.numels]
    for rank in range(world):
        for r in rank_records(lay, rank):
            cover[r.tensor][r.a:r.b] += 1
            assert r.a % 128 == 0                                   # pieces start on block boundaries
            shape = lay.shapes[r.tensor]
            if r.kind == RANK1 and not r.partial:
                assert r.numel == r.rows * r.cols and r.a == r.row_lo * shape[1]
            if r.kind == RANK1 and r.partial:
                assert (r.rows, r.cols) == shape and r.flat_offset == r.a
            if r.kind == FP32:
                assert lay.numels[r.tensor] <= 4096
    assert all(bool((c == 1).all()) for c in cover)


def test_whole_row_records_only_when_blocks_do_not_straddle_rows():
    lay = flat_layout([(64, 77)], 2)         # 77 columns: blocks straddle rows -> partial records only
    recs = rank_records(lay, 0, threshold=0) + rank_records(lay, 1, threshold=0)
    assert all(r.partial for r in recs)
    lay = flat_layout([(300, 256)], 2)
    kinds = [(r.partial, r.rows) for r in rank_records(lay, 0, threshold=0)]
    assert (False, 150) in kinds or any(not p for p, _ in kinds)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, steps, out):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from sharded_cpu_backend import CpuBackend
    from quantfour_adamw_cuda_b200.zero1 import ShardedFourBitAdamW
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(0)
        params = [torch.nn.Parameter(torch.randn(s, generator=gen) * 0.02) for s in SHAPES]
        opt = ShardedFourBitAdamW(params, lr=1e-3, backend=CpuBackend())
        for _ in range(steps):
            for p in params:
                p.grad = torch.randn(p.shape, generator=gen) * 1e-3
            opt.step()
        if rank == 0:
            torch.save([p.detach().clone() for p in params], out)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_step_equals_unsharded_oracle_with_gloo_ranks(world, tmp_path):
    steps = 4
    out = str(tmp_path / "params.pt")
    mp.spawn(_worker, args=(world, _free_port(), steps, out), nprocs=world, join=True)
    got = torch.load(out)
    gen = torch.Generator().manual_seed(0)
    params = [torch.randn(s, generator=gen) * 0.02 for s in SHAPES]
    states = [TO.TensorState.zeros(s) for s in SHAPES]
    for _ in range(steps):
        for p, st in zip(params, states):
            TO.step_tensor(p, torch.randn(p.shape, generator=gen) * 1e-3, st, 1e-3, 0.9, 0.999, 1e-8, 0.01)
    for i, (a, b) in enumerate(zip(got, params)):
        assert torch.equal(a, b), f"tensor {i} {SHAPES[i]} differs in {(a != b).sum()} places"


def test_single_process_without_process_group_matches_oracle():
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from sharded_cpu_backend import CpuBackend
    from quantfour_adamw_cuda_b200.zero1 import ShardedFourBitAdamW
    gen = torch.Generator().manual_seed(1)
    params = [torch.nn.Parameter(torch.randn(s, generator=gen) * 0.02) for s in SHAPES]
    ref = [p.detach().clone() for p in params]
    states = [TO.TensorState.zeros(s) for s in SHAPES]
    opt = ShardedFourBitAdamW(params, lr=1e-3, backend=CpuBackend())
    for _ in range(3):
        grads = [torch.randn(p.shape, generator=gen) * 1e-3 for p in params]
        for p, g, r, st in zip(params, grads, ref, states):
            p.grad = g
            TO.step_tensor(r, g, st, 1e-3, 0.9, 0.999, 1e-8, 0.01)
        opt.step()
    assert all(torch.equal(p.detach(), r) for p, r in zip(params, ref))
    sd = opt.state_dict()
    assert sd["step"] == 3 and len(sd["records"]) == len(opt.states)
    opt.load_state_dict(sd)

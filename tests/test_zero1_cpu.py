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
        full = opt.full_state_dict()        # collective: every rank assembles the state of all ranks
        if rank == 0:
            torch.save([p.detach().clone() for p in params], out)
            torch.save(full, out + ".state")
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
    _assert_full_equals_oracle(torch.load(out + ".state"), states)


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


# ---- sharded <-> full state -----------------------------------------------------------------------------------

def _emulated(world, init, threshold=4096):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from sharded_cpu_backend import CpuBackend
    from quantfour_adamw_cuda_b200.zero1 import ShardedFourBitAdamW
    ranks = []
    for r in range(world):
        params = [torch.nn.Parameter(p.clone()) for p in init]
        ranks.append((params, ShardedFourBitAdamW(params, lr=1e-3, backend=CpuBackend(), rank=r, world=world,
                                                  quant_threshold=threshold)))
    return ranks


def _emulated_step(ranks, grads):
    shard = ranks[0][1].layout.shard
    for params, opt in ranks:
        for p, g in zip(params, grads):
            p.grad = g.clone()
        opt.step_pre()
    if ranks[0][1].shared_new.numel():
        combined = torch.stack([opt.shared_new for _, opt in ranks]).max(dim=0).values
        for _, opt in ranks:
            opt.shared_new.copy_(combined)
    for _, opt in ranks:
        opt.step_main()
    for r, (_, src) in enumerate(ranks):
        for _, dst in ranks:
            dst.flat[r * shard:(r + 1) * shard].copy_(src.flat[r * shard:(r + 1) * shard])


def _assert_full_equals_oracle(full, states):
    for t, st in enumerate(states):
        f = full["state"][t]
        if st.kind == "fp32":
            assert torch.equal(f["exp_avg"].reshape(-1), st.m.reshape(-1)) and torch.equal(f["exp_avg_sq"].reshape(-1), st.v.reshape(-1))
            assert not f["momentum_qstate"]["enable"]
            continue
        assert f["exp_avg"].dtype == torch.int8 and f["momentum_qstate"]["enable"]
        assert torch.equal(f["exp_avg"].view(torch.uint8), st.m_codes), f"tensor {t}: m codes"
        assert torch.equal(f["exp_avg_sq"].view(torch.uint8), st.v_codes), f"tensor {t}: v codes"
        assert torch.equal(f["momentum_qstate"]["overhead"]["max1"], st.m_scale)
        vo = f["variance_qstate"]["overhead"]
        if st.kind == "rank1":
            assert torch.equal(vo["max_dims"][0].reshape(-1), st.v_row) and torch.equal(vo["max_dims"][1].reshape(-1), st.v_col)
        else:
            assert torch.equal(vo["max1"], st.v_scale)


@pytest.mark.parametrize("world,world2", [(3, 2), (2, 5), (4, 1)])
def test_full_state_from_shards_and_resharding(world, world2):
    """Pieces of all ranks assemble into exactly the unsharded oracle's state; that state, loaded by a different
    number of ranks, continues exactly like the oracle."""
    from quantfour_adamw_cuda_b200.zero1 import assemble_full_state
    gen = torch.Generator().manual_seed(7)
    init = [torch.randn(s, generator=gen) * 0.02 for s in SHAPES]
    ref = [p.clone() for p in init]
    states = [TO.TensorState.zeros(s) for s in SHAPES]
    ranks = _emulated(world, init)

    def advance(ranks, n):
        for _ in range(n):
            grads = [torch.randn(s, generator=gen) * 1e-3 for s in SHAPES]
            for p, g, st in zip(ref, grads, states):
                TO.step_tensor(p, g, st, 1e-3, 0.9, 0.999, 1e-8, 0.01)
            _emulated_step(ranks, grads)

    advance(ranks, 3)
    opt0 = ranks[0][1]
    pieces = [e for _, opt in ranks for e in opt.pieces()]
    full = assemble_full_state(pieces, opt0.layout.shapes, opt0.step_count, opt0.param_groups[0])
    assert all(float(f["step"]) == 3.0 for f in full["state"].values())
    _assert_full_equals_oracle(full, states)

    ranks2 = _emulated(world2, [p.clone() for p in ref])
    for _, opt in ranks2:
        opt.load_full_state_dict(full)
    advance(ranks2, 2)
    for params, _ in ranks2:
        assert all(torch.equal(p.detach(), r) for p, r in zip(params, ref))
    pieces = [e for _, opt in ranks2 for e in opt.pieces()]
    _assert_full_equals_oracle(assemble_full_state(pieces, opt0.layout.shapes, 5, opt0.param_groups[0]), states)


def test_assemble_rejects_missing_pieces():
    from quantfour_adamw_cuda_b200.zero1 import assemble_full_state
    init = [torch.zeros(s) for s in SHAPES]
    ranks = _emulated(2, init)
    with pytest.raises(ValueError, match="do not tile"):
        assemble_full_state(ranks[0][1].pieces(), ranks[0][1].layout.shapes, 0, ranks[0][1].param_groups[0])


def test_full_state_dict_loads_into_the_unsharded_optimizer():
    """The assembled state dict has the unsharded optimizer's schema: FourBitAdamW.load_state_dict takes it and
    hands the same tensors back."""
    from quantfour_adamw_cuda_b200 import FourBitAdamW
    gen = torch.Generator().manual_seed(3)
    init = [torch.randn(s, generator=gen) * 0.02 for s in SHAPES]
    ranks = _emulated(1, init)
    for _ in range(2):
        _emulated_step(ranks, [torch.randn(s, generator=gen) * 1e-3 for s in SHAPES])
    full = ranks[0][1].full_state_dict()
    plain = FourBitAdamW([torch.nn.Parameter(p.clone()) for p in init], lr=1e-3)
    plain.load_state_dict(full)
    back = plain.state_dict()
    for t in range(len(SHAPES)):
        a, b = full["state"][t], back["state"][t]
        assert torch.equal(a["exp_avg"], b["exp_avg"]) and a["exp_avg"].dtype == b["exp_avg"].dtype
        assert float(b["step"]) == 2.0
        if a["variance_qstate"]["overhead"].get("max_dims") is not None:
            for x, y in zip(a["variance_qstate"]["overhead"]["max_dims"], b["variance_qstate"]["overhead"]["max_dims"]):
                assert torch.equal(x, y) and y.dtype == torch.float32


# ---- gradients reduced inside the step ---------------------------------------------------------------------------

def _worker_reduce(rank, world, port, steps, out):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from sharded_cpu_backend import CpuBackend
    from quantfour_adamw_cuda_b200.zero1 import ShardedFourBitAdamW
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(0)
        params = [torch.nn.Parameter(torch.randn(s, generator=gen) * 0.02) for s in SHAPES]
        opt = ShardedFourBitAdamW(params, lr=1e-3, backend=CpuBackend(), reduce_grads=True)
        for step in range(steps):
            opt.zero_grad()
            for p in params:
                per_rank = [torch.randn(p.shape, generator=gen) * 1e-3 for _ in range(world)]
                if step % 2:
                    p.grad.add_(per_rank[rank])        # accumulate into the flat buffer, like backward does
                else:
                    p.grad = per_rank[rank].clone()    # a gradient produced elsewhere: copied in by the step
            opt.step()
        if rank == 0:
            torch.save([p.detach().clone() for p in params], out)
    finally:
        dist.destroy_process_group()


def test_gradients_reduced_inside_the_step_with_gloo_ranks(tmp_path):
    world, steps = 2, 4
    out = str(tmp_path / "params.pt")
    mp.spawn(_worker_reduce, args=(world, _free_port(), steps, out), nprocs=world, join=True)
    got = torch.load(out)
    gen = torch.Generator().manual_seed(0)
    params = [torch.randn(s, generator=gen) * 0.02 for s in SHAPES]
    states = [TO.TensorState.zeros(s) for s in SHAPES]
    for _ in range(steps):
        for p, st in zip(params, states):
            per_rank = [torch.randn(p.shape, generator=gen) * 1e-3 for _ in range(world)]
            TO.step_tensor(p, (per_rank[0] + per_rank[1]) * 0.5, st, 1e-3, 0.9, 0.999, 1e-8, 0.01)
    for i, (a, b) in enumerate(zip(got, params)):
        assert torch.equal(a, b), f"tensor {i} {SHAPES[i]} differs in {(a != b).sum()} places"


def test_flat_gradient_buffer_without_a_process_group():
    """reduce_grads=True in a single process: gradients become views of one flat buffer, zero_grad keeps them
    attached, a gradient assigned from outside is copied in, and the step matches the oracle."""
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from sharded_cpu_backend import CpuBackend
    from quantfour_adamw_cuda_b200.zero1 import ShardedFourBitAdamW
    gen = torch.Generator().manual_seed(4)
    params = [torch.nn.Parameter(torch.randn(s, generator=gen) * 0.02) for s in SHAPES]
    ref = [p.detach().clone() for p in params]
    states = [TO.TensorState.zeros(s) for s in SHAPES]
    opt = ShardedFourBitAdamW(params, lr=1e-3, backend=CpuBackend(), reduce_grads=True)
    base = opt.flat_grad.data_ptr()
    assert all(p.grad is not None and base <= p.grad.data_ptr() < base + opt.flat_grad.numel() * 4 for p in params)
    for step in range(3):
        opt.zero_grad()
        assert float(opt.flat_grad.abs().sum()) == 0.0
        grads = [torch.randn(p.shape, generator=gen) * 1e-3 for p in params]
        for i, (p, g) in enumerate(zip(params, grads)):
            if i % 2:
                p.grad = g.clone()         # replaced from outside
            else:
                p.grad.add_(g)             # accumulated in place
        for r, g, st in zip(ref, grads, states):
            TO.step_tensor(r, g, st, 1e-3, 0.9, 0.999, 1e-8, 0.01)
        opt.step()
        assert all(base <= p.grad.data_ptr() < base + opt.flat_grad.numel() * 4 for p in params)
    assert all(torch.equal(p.detach(), r) for p, r in zip(params, ref))


def test_constructor_rejects_unknown_comm():
    from quantfour_adamw_cuda_b200.zero1 import ShardedFourBitAdamW
    with pytest.raises(ValueError, match="comm must be"):
        ShardedFourBitAdamW([torch.nn.Parameter(torch.zeros(8))], comm="smoke-signals", backend=object())

"""GPU tests of the sharded optimizer: one rank through the public class, and several ranks emulated in one
process on one GPU (the exchange of maxima and parameter ranges done by the test), against the CPU oracle.
The emulation exercises the partial-record kernels (pieces that start in the middle of a matrix)."""
import pytest
import torch

from oracle import c_oracle as CO
from oracle import torch_oracle as TO
from quantfour_adamw_cuda_b200.zero1 import ShardedFourBitAdamW

pytestmark = pytest.mark.gpu

SHAPES = [(300, 256), (1000,), (96, 128), (5000,), (64, 77), (40, 50), (130, 384), (4096,), (512, 512)]
HP = (1e-3, 0.9, 0.999, 1e-8, 0.01)


def _oracle_run(dtype, steps, seed):
    gen = torch.Generator().manual_seed(seed)
    params = [(torch.randn(s, generator=gen) * 0.02).to(dtype) for s in SHAPES]
    init = [p.clone() for p in params]
    states = [TO.TensorState.zeros(s) for s in SHAPES]
    grads = []
    for _ in range(steps):
        gs = [(torch.randn(s, generator=gen) * 1e-3).to(dtype) for s in SHAPES]
        grads.append(gs)
        for p, g, st in zip(params, gs, states):
            CO.step_tensor(p, g, st, *HP)
    return init, grads, params


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_single_rank_matches_oracle(dtype):
    init, grads, want = _oracle_run(dtype, 4, 0)
    params = [torch.nn.Parameter(p.cuda()) for p in init]
    opt = ShardedFourBitAdamW(params, lr=1e-3)
    for gs in grads:
        for p, g in zip(params, gs):
            p.grad = g.cuda()
        opt.step()
    for i, (p, w) in enumerate(zip(params, want)):
        assert torch.equal(p.detach().cpu(), w), f"tensor {i} {SHAPES[i]}"


@pytest.mark.parametrize("world", [2, 3, 5])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_emulated_ranks_match_unsharded_oracle(world, dtype):
    init, grads, want = _oracle_run(dtype, 4, 1)
    ranks = []
    for r in range(world):
        params = [torch.nn.Parameter(p.cuda()) for p in init]
        ranks.append((params, ShardedFourBitAdamW(params, lr=1e-3, rank=r, world=world)))
    shard = ranks[0][1].layout.shard
    for gs in grads:
        for params, opt in ranks:
            for p, g in zip(params, gs):
                p.grad = g.cuda()
            opt.step_pre()
        if ranks[0][1].shared_new.numel():      # what the all-reduce(MAX) does
            combined = torch.stack([opt.shared_new for _, opt in ranks]).max(dim=0).values
            for _, opt in ranks:
                opt.shared_new.copy_(combined)
        for _, opt in ranks:
            opt.step_main()
        for r, (_, src) in enumerate(ranks):    # what the all-gather does
            for _, dst in ranks:
                dst.flat[r * shard:(r + 1) * shard].copy_(src.flat[r * shard:(r + 1) * shard])
    for params, _ in ranks:
        for i, (p, w) in enumerate(zip(params, want)):
            assert torch.equal(p.detach().cpu(), w), f"tensor {i} {SHAPES[i]} differs in {(p.detach().cpu() != w).sum()} places"


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_emulated_ranks_with_peer_stores(world, dtype):
    """qf_step_main_push with the other ranks' flat buffers standing in for peer mappings (same device):
    the stores issued by the update kernels replace the all-gather."""
    init, grads, want = _oracle_run(dtype, 4, 2)
    ranks = []
    for r in range(world):
        params = [torch.nn.Parameter(p.cuda()) for p in init]
        ranks.append((params, ShardedFourBitAdamW(params, lr=1e-3, rank=r, world=world)))
    for gs in grads:
        for params, opt in ranks:
            for p, g in zip(params, gs):
                p.grad = g.cuda()
            opt.step_pre()
        if ranks[0][1].shared_new.numel():
            combined = torch.stack([opt.shared_new for _, opt in ranks]).max(dim=0).values
            for _, opt in ranks:
                opt.shared_new.copy_(combined)
        for _, opt in ranks:
            deltas = [other.flat.data_ptr() - opt.flat.data_ptr() for _, other in ranks if other is not opt]
            opt.backend.main_push(opt.states, opt._hyper, deltas)
    torch.cuda.synchronize()
    for params, _ in ranks:
        for i, (p, w) in enumerate(zip(params, want)):
            assert torch.equal(p.detach().cpu(), w), f"tensor {i} {SHAPES[i]} differs in {(p.detach().cpu() != w).sum()} places"


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_emulated_ranks_with_pipelined_copies(world, dtype):
    """The update in pieces (one qf_step_main per piece) with qf_peer_copy carrying each finished piece into the
    other ranks' flat buffers (same device here)."""
    init, grads, want = _oracle_run(dtype, 4, 3)
    ranks = []
    for r in range(world):
        params = [torch.nn.Parameter(p.cuda()) for p in init]
        opt = ShardedFourBitAdamW(params, lr=1e-3, rank=r, world=world)
        ranks.append((params, opt))
    for _, opt in ranks:
        opt.peer_deltas = [other.flat.data_ptr() - opt.flat.data_ptr() for _, other in ranks if other is not opt]
        opt.peer_devices = [-1] * len(opt.peer_deltas)
        opt._setup_chunks(max_chunks=3, min_bytes=1)
    assert max(len(opt.chunks) for _, opt in ranks) > 1
    for gs in grads:
        for params, opt in ranks:
            for p, g in zip(params, gs):
                p.grad = g.cuda()
            opt.step_pre()
        if ranks[0][1].shared_new.numel():
            combined = torch.stack([opt.shared_new for _, opt in ranks]).max(dim=0).values
            for _, opt in ranks:
                opt.shared_new.copy_(combined)
        for _, opt in ranks:
            opt._main_ce()
    torch.cuda.synchronize()
    for params, _ in ranks:
        for i, (p, w) in enumerate(zip(params, want)):
            assert torch.equal(p.detach().cpu(), w), f"tensor {i} {SHAPES[i]} differs in {(p.detach().cpu() != w).sum()} places"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("copies,n", [(2, 1 << 16), (4, 100_003), (7, 12_345)])
def test_gradient_mean_over_copies_is_the_fp32_sum_in_the_given_order_rounded_once(dtype, copies, n):
    """qf_grad_mean_peers with the other ranks' gradient buffers standing in as plain buffers of the same device: the
    owner's range becomes RN((g_0 + g_1 + ...) / copies), summed in fp32 in the order of the list; nothing outside the
    range and nothing of the other copies is written."""
    import ctypes as C
    from quantfour_adamw_cuda_b200 import _lib
    gen = torch.Generator().manual_seed(copies * 131 + n)
    pad = 64
    bufs = [(torch.randn(n + 2 * pad, generator=gen) * 1e-2).to(dtype).cuda() for _ in range(copies)]
    before = [b.clone() for b in bufs]
    own = 1 % copies                                     # the owner is not the first of the list
    order = list(range(copies))
    acc = before[order[0]][pad:pad + n].float()
    for k in order[1:]:
        acc = acc + before[k][pad:pad + n].float()
    want = (acc * torch.tensor(1.0 / copies, dtype=torch.float32)).to(dtype)
    g = bufs[own][pad:pad + n]
    deltas = (C.c_int64 * copies)(*[bufs[k].data_ptr() - bufs[own].data_ptr() for k in order])
    code = {torch.float32: _lib.QF_F32, torch.bfloat16: _lib.QF_BF16, torch.float16: _lib.QF_F16}[dtype]
    _lib.check(_lib.lib().qf_grad_mean_peers(C.c_void_p(g.data_ptr()), n, code, deltas, copies, 1.0 / copies, 0,
                                             C.c_void_p(torch.cuda.current_stream().cuda_stream)), "qf_grad_mean_peers")
    torch.cuda.synchronize()
    assert torch.equal(g, want.cuda())
    for k in range(copies):
        if k != own:
            assert torch.equal(bufs[k], before[k])
    assert torch.equal(bufs[own][:pad], before[own][:pad]) and torch.equal(bufs[own][pad + n:], before[own][pad + n:])


def test_push_rejects_bad_peers():
    params = [torch.nn.Parameter(torch.zeros(64, 256, device="cuda"))]
    opt = ShardedFourBitAdamW(params, lr=1e-3)
    params[0].grad = torch.zeros_like(params[0])
    opt.step_pre()
    with pytest.raises(ValueError, match="n_peers"):
        opt.backend.main_push(opt.states, opt._hyper, [1024] * 16)
    with pytest.raises(ValueError, match="multiple of 16"):
        opt.backend.main_push(opt.states, opt._hyper, [8])
    opt.step_main()


def test_peer_export_reports_offset():
    """The handle of a buffer inside a larger allocation comes with the buffer's offset in it."""
    from quantfour_adamw_cuda_b200.zero1 import CudaBackend
    big = torch.zeros(1 << 22, dtype=torch.uint8, device="cuda")
    handle, off = CudaBackend().export_buffer(big[4096:])
    assert len(handle) == 64 and off >= 4096 and (off - 4096) % 512 == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_state_moves_between_sharded_and_unsharded_optimizers(dtype):
    """Three emulated ranks -> one state dict in the unsharded layout -> FourBitAdamW -> back into a sharded
    optimizer of two ranks; the parameters follow the oracle through all three stages."""
    from quantfour_adamw_cuda_b200 import FourBitAdamW
    from quantfour_adamw_cuda_b200.zero1 import assemble_full_state
    init, grads, want = _oracle_run(dtype, 6, 3)

    def emulated(world, start):
        out = []
        for r in range(world):
            params = [torch.nn.Parameter(p.clone().cuda()) for p in start]
            out.append((params, ShardedFourBitAdamW(params, lr=1e-3, rank=r, world=world)))
        return out

    def emulated_step(ranks, gs):
        shard = ranks[0][1].layout.shard
        for params, opt in ranks:
            for p, g in zip(params, gs):
                p.grad = g.cuda()
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

    ranks = emulated(3, init)
    for gs in grads[:2]:
        emulated_step(ranks, gs)
    opt0 = ranks[0][1]
    full = assemble_full_state([e for _, o in ranks for e in o.pieces()], opt0.layout.shapes, opt0.step_count, opt0.param_groups[0])

    params = [torch.nn.Parameter(p.detach().clone()) for p in ranks[0][0]]
    plain = FourBitAdamW(params, lr=1e-3)
    plain.load_state_dict(full)
    for gs in grads[2:4]:
        for p, g in zip(params, gs):
            p.grad = g.cuda()
        plain.step()

    ranks2 = emulated(2, [p.detach().cpu() for p in params])
    for _, opt in ranks2:
        opt.load_full_state_dict(plain.state_dict())
    for gs in grads[4:]:
        emulated_step(ranks2, gs)
    for i, (p, w) in enumerate(zip(ranks2[1][0], want)):
        assert torch.equal(p.detach().cpu(), w), f"tensor {i} {SHAPES[i]} differs in {(p.detach().cpu() != w).sum()} places"


def test_peer_functions_report_errors_instead_of_faulting():
    import ctypes as C
    from quantfour_adamw_cuda_b200 import _lib
    L = _lib.lib()
    base = C.c_void_p(0)
    # a handle of zeros names no allocation: the call must fail with a message, not crash
    rc = L.qf_peer_open(bytes(64), 0, C.byref(base))
    assert rc != 0 and L.qf_last_error()
    # closing something that was never opened
    x = torch.zeros(16, device="cuda")
    with pytest.raises(ValueError, match="not a mapping"):
        _lib.check(L.qf_peer_close(C.c_void_p(x.data_ptr()), 0), "qf_peer_close")
    # exporting a host pointer
    buf = (C.c_char * 64)()
    off = C.c_int64(0)
    host = torch.zeros(16)
    rc = L.qf_peer_export(C.c_void_p(host.data_ptr()), 0, buf, C.byref(off))
    assert rc != 0 and L.qf_last_error()
    torch.cuda.synchronize()
    assert float(x.sum()) == 0.0          # the context is still usable


def test_sharded_optimizer_reports_nonfinite_gradients():
    params = [torch.nn.Parameter(torch.randn(128, 256, device="cuda") * 0.02), torch.nn.Parameter(torch.randn(5000, device="cuda"))]
    opt = ShardedFourBitAdamW(params, lr=1e-3)
    for p in params:
        p.grad = torch.randn_like(p) * 1e-3
    opt.step()
    assert not opt.nonfinite_seen()
    params[0].grad[3, 5] = float("inf")
    opt.step()
    assert opt.nonfinite_seen()
    assert not opt.nonfinite_seen()      # reading clears the word

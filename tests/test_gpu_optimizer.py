"""GPU tests of the FourBitAdamW class: parity with the oracle through the public optimizer API,
state_dict round trip, and the reference's own acceptance test (closeness to torch.optim.AdamW)."""
import copy
import io

import pytest
import torch
import torch.nn as nn

from oracle import c_oracle as CO
from oracle import torch_oracle as TO

pytestmark = pytest.mark.gpu

import quantfour_adamw_cuda_b200 as qf  # noqa: E402

DEV = "cuda"


def _model(dtype):
    torch.manual_seed(7)
    m = nn.Sequential(nn.Linear(256, 512), nn.LayerNorm(512), nn.Linear(512, 130), nn.Linear(130, 64))
    return m.to(DEV, dtype)


def _oracle_for(params):
    cpu = [p.detach().cpu().clone() for p in params]
    return cpu, [TO.TensorState.zeros(p.shape) for p in cpu]


def _check_against_oracle(opt, params, cpu, states):
    for p, c, st in zip(params, cpu, states):
        assert torch.equal(p.detach().cpu(), c)
        s = opt.state[p]
        assert int(s["step"]) == st.step
        if st.kind == "fp32":
            assert torch.equal(s["exp_avg"].cpu().reshape(-1), st.m) and torch.equal(s["exp_avg_sq"].cpu().reshape(-1), st.v)
            assert not s["momentum_qstate"]["enable"]
            continue
        assert s["exp_avg"].dtype == torch.int8 and s["momentum_qstate"]["enable"]
        assert torch.equal(s["exp_avg"].cpu().view(torch.uint8), st.m_codes)
        assert torch.equal(s["exp_avg_sq"].cpu().view(torch.uint8), st.v_codes)
        assert torch.equal(s["momentum_qstate"]["overhead"]["max1"].cpu(), st.m_scale)
        vo = s["variance_qstate"]["overhead"]
        if st.kind == "rank1nd":
            assert vo["dim"] == len(st.shape) and len(vo["max_dims"]) == len(st.shape) and vo["max1"] is None
            for k, (mx, want) in enumerate(zip(vo["max_dims"], st.v_axes)):
                assert list(mx.shape) == [d if a == k else 1 for a, d in enumerate(st.shape)]
                assert torch.equal(mx.cpu().reshape(-1), want), f"maxima of axis {k}"
        elif st.kind == "rank1":
            assert vo["max_dims"][0].shape == (st.shape[0], 1) and vo["max_dims"][1].shape == (1, st.shape[1])
            assert torch.equal(vo["max_dims"][0].cpu().reshape(-1), st.v_row)
            assert torch.equal(vo["max_dims"][1].cpu().reshape(-1), st.v_col)
        else:
            assert torch.equal(vo["max1"].cpu(), st.v_scale)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_optimizer_matches_oracle_and_state_layout(dtype):
    model = _model(dtype)
    params = list(model.parameters())
    opt = qf.FourBitAdamW(params, lr=2e-3, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.05)
    cpu, states = _oracle_for(params)
    for it in range(8):
        x = torch.randn(32, 256, device=DEV, dtype=dtype)
        opt.zero_grad(set_to_none=(it % 2 == 0))
        model(x).float().pow(2).mean().backward()
        for c, p, st in zip(cpu, params, states):
            CO.step_tensor(c, p.grad.detach().cpu(), st, 2e-3, 0.9, 0.99, 1e-8, 0.05)
        opt.step()
        _check_against_oracle(opt, params, cpu, states)
    assert not opt.nonfinite_seen()


def test_params_without_grad_are_skipped_and_closure_loss_is_returned():
    model = _model(torch.float32)
    params = list(model.parameters())
    opt = qf.AdamWFused_QuantFour(params, lr=1e-3)
    before = [p.detach().clone() for p in params]
    x = torch.randn(8, 256, device=DEV)

    def closure():
        opt.zero_grad()
        loss = model(x).sum()
        loss.backward()
        params[0].grad = None
        return loss

    loss = opt.step(closure)
    assert torch.is_tensor(loss) and loss.requires_grad
    assert torch.equal(params[0], before[0]) and len(opt.state[params[0]]) == 0
    assert not torch.equal(params[2], before[2])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_state_dict_round_trip_resumes_bit_identically(dtype):
    model_a = _model(dtype)
    model_b = copy.deepcopy(model_a)
    opt_a = qf.FourBitAdamW(model_a.parameters(), lr=1e-3)
    xs = [torch.randn(16, 256, device=DEV, dtype=dtype) for _ in range(6)]

    def run(model, opt, x):
        opt.zero_grad()
        model(x).float().pow(2).mean().backward()
        opt.step()

    for x in xs[:3]:
        run(model_a, opt_a, x)
    buf = io.BytesIO()
    torch.save({"model": model_a.state_dict(), "opt": opt_a.state_dict()}, buf)
    buf.seek(0)
    ck = torch.load(buf, map_location="cpu")
    model_b.load_state_dict(ck["model"])
    opt_b = qf.FourBitAdamW(model_b.parameters(), lr=1e-3)
    opt_b.load_state_dict(ck["opt"])
    for pa, pb in zip(model_a.parameters(), model_b.parameters()):
        sa, sb = opt_a.state[pa], opt_b.state[pb]
        assert sb["exp_avg"].dtype == sa["exp_avg"].dtype and sb["exp_avg"].device == pb.device
        assert sb["step"].device.type == "cpu"
        if sa["momentum_qstate"]["enable"]:
            assert sb["momentum_qstate"]["overhead"]["max1"].dtype == torch.float32
    for x in xs[3:]:
        run(model_a, opt_a, x)
        run(model_b, opt_b, x)
    for pa, pb in zip(model_a.parameters(), model_b.parameters()):
        assert torch.equal(pa, pb)
        assert torch.equal(opt_a.state[pa]["exp_avg"], opt_b.state[pb]["exp_avg"])
        assert torch.equal(opt_a.state[pa]["exp_avg_sq"], opt_b.state[pb]["exp_avg_sq"])


def test_adam_equivalence_like_the_reference_test():
    """The reference's live test (tests/driver.py:26-72, :120-133): a 5->10->5 MLP, 10 iterations, every
    parameter within atol 0.025 / rtol 1e-5 of torch.optim.AdamW (lr 0.005, betas (0.8, 0.88), wd 0.03),
    and parameters must have moved after the first step."""
    torch.manual_seed(2020)
    model = nn.Sequential(nn.Linear(5, 10), nn.Linear(10, 5)).to(DEV)
    model_ref = copy.deepcopy(model)
    kw = dict(lr=0.005, betas=(0.8, 0.88), weight_decay=0.03, eps=1e-8)
    opt = qf.AdamW_QuantFour(model.parameters(), **kw)
    opt_ref = torch.optim.AdamW(model_ref.parameters(), **kw)
    start = [p.detach().clone() for p in model.parameters()]
    for i in range(10):
        x = torch.randn(5, 5, device=DEV)
        for m, o in ((model, opt), (model_ref, opt_ref)):
            o.zero_grad()
            m(x).sum().backward()
            o.step()
        if i == 0:
            assert all(not torch.equal(a, b) for a, b in zip(start, model.parameters()))
        for a, b in zip(model.parameters(), model_ref.parameters()):
            torch.testing.assert_close(a, b, atol=0.025, rtol=1e-5)


def test_larger_quantized_model_tracks_fp32_adamw():
    torch.manual_seed(1)
    w = nn.Parameter(torch.randn(256, 384, device=DEV) * 0.1)
    w_ref = nn.Parameter(w.detach().clone())
    kw = dict(lr=0.005, betas=(0.8, 0.88), weight_decay=0.03, eps=1e-8)
    opt, opt_ref = qf.FourBitAdamW([w], **kw), torch.optim.AdamW([w_ref], **kw)
    for _ in range(10):
        g = torch.randn_like(w)
        w.grad, w_ref.grad = g.clone(), g.clone()
        opt.step()
        opt_ref.step()
        torch.testing.assert_close(w, w_ref, atol=0.025, rtol=1e-5)
    m, v = opt.dequantized_state(w)
    assert m.shape == w.shape and v.shape == w.shape and float(v.min()) > 0


def test_cpu_parameters_and_bad_dtypes_fail_loudly():
    p = nn.Parameter(torch.randn(64, 128))
    p.grad = torch.randn_like(p)
    with pytest.raises(RuntimeError, match="no CPU path"):
        qf.FourBitAdamW([p]).step()
    h = nn.Parameter(torch.randn(64, 128, device=DEV).double())
    h.grad = torch.randn_like(h)
    with pytest.raises(TypeError):
        qf.FourBitAdamW([h]).step()


def test_tensor_with_more_than_2_to_31_elements():
    """64-bit element indexing: a 1-D tensor of 2^31 + 640 elements steps exactly like the same data cut into two
    tensors at a block boundary (block-128 state is independent per block)."""
    import quantfour_adamw_cuda_b200 as qf
    free, _ = torch.cuda.mem_get_info()
    if free < 40 * 2**30:
        pytest.skip("needs about 30 GB of device memory")
    n, cut = 2**31 + 640, 2**30
    gen = torch.Generator(device="cuda").manual_seed(11)
    base = torch.empty(n, dtype=torch.bfloat16, device="cuda").normal_(0, 0.02, generator=gen)
    whole = torch.nn.Parameter(base.clone())
    halves = [torch.nn.Parameter(base[:cut].clone()), torch.nn.Parameter(base[cut:].clone())]
    del base
    o1, o2 = qf.FourBitAdamW([whole], lr=1e-3), qf.FourBitAdamW(halves, lr=1e-3)
    for _ in range(2):
        g = torch.empty(n, dtype=torch.bfloat16, device="cuda").normal_(0, 1e-3, generator=gen)
        whole.grad = g
        halves[0].grad, halves[1].grad = g[:cut], g[cut:]
        o1.step()
        o2.step()
    assert torch.equal(whole.detach()[:cut], halves[0].detach()) and torch.equal(whole.detach()[cut:], halves[1].detach())
    s1 = o1.state[whole]
    for key in ("exp_avg", "exp_avg_sq"):
        joined = torch.cat([o2.state[h][key] for h in halves])
        assert torch.equal(s1[key], joined), key
    joined = torch.cat([o2.state[h]["momentum_qstate"]["overhead"]["max1"] for h in halves])
    assert torch.equal(s1["momentum_qstate"]["overhead"]["max1"], joined)
    assert not o1.nonfinite_seen()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("scale", [1.0 / 1024, 0.37])
def test_grad_scale_equals_scaling_the_gradients_first(dtype, scale):
    """step(grad_scale=s) leaves the same parameters and state as multiplying every gradient by s (rounded to its
    dtype) and stepping, and the gradients themselves end up scaled in place -- for every mapping: panel and flat
    rank-1, block-128, fp32 state."""
    import numpy as np
    shapes = [(64, 256), (300, 77), (5000,), (1000,), (3, 5, 7, 99), (129, 255), (4096,), (256, 512)]
    gen = torch.Generator().manual_seed(21)
    init = [(torch.randn(s, generator=gen) * 0.02).to(dtype) for s in shapes]
    pa = [nn.Parameter(p.clone().cuda()) for p in init]
    pb = [nn.Parameter(p.clone().cuda()) for p in init]
    oa, ob = qf.FourBitAdamW(pa, lr=1e-3), qf.FourBitAdamW(pb, lr=1e-3)
    s32 = float(np.float32(scale))
    for step in range(4):
        grads = [(torch.randn(s, generator=gen) * 0.5).to(dtype) for s in shapes]
        scaled = [(g.float() * s32).to(dtype) for g in grads]
        for p, g in zip(pa, grads):
            p.grad = g.clone().cuda()
        for p, g in zip(pb, scaled):
            p.grad = g.clone().cuda()
        oa.step(grad_scale=scale)
        ob.step()
        for i, (a, b, g) in enumerate(zip(pa, pb, scaled)):
            assert torch.equal(a.detach(), b.detach()), f"step {step} tensor {i} {shapes[i]}: parameters"
            assert torch.equal(a.grad.cpu(), g), f"step {step} tensor {i} {shapes[i]}: gradient not scaled in place"
    for a, b in zip(pa, pb):
        sa, sb = oa.state[a], ob.state[b]
        assert torch.equal(sa["exp_avg"], sb["exp_avg"]) and torch.equal(sa["exp_avg_sq"], sb["exp_avg_sq"])
    oa.step()       # and a step without the argument goes back to unscaled gradients
    assert not oa.nonfinite_seen()


# ---- capturable=True: the step as kernel launches only, scalars resident on the device ------------------------

def _static_problem(dtype, seed=11):
    gen = torch.Generator().manual_seed(seed)
    shapes = [(256, 384), (5000,), (130, 64), (64,), (128, 256)]
    params = [nn.Parameter((torch.randn(s, generator=gen) * 0.05).to(DEV, dtype)) for s in shapes]
    for p in params:
        p.grad = torch.zeros_like(p)
    return shapes, params, gen


def _new_grads(shapes, gen, dtype, scale=1e-2):
    return [(torch.randn(s, generator=gen) * scale).to(dtype) for s in shapes]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_capturable_step_replayed_from_a_cuda_graph_matches_the_oracle(dtype):
    """One eager step, then the step recorded into a CUDA graph and replayed with new gradients written into the
    same buffers: parameters, codes, scales and the step count follow the oracle bit for bit.  Two param groups."""
    shapes, params, gen = _static_problem(dtype)
    hp = dict(betas=(0.9, 0.99), eps=1e-8)
    opt = qf.FourBitAdamW([{"params": params[:3], "lr": 2e-3, "weight_decay": 0.05},
                           {"params": params[3:], "lr": 5e-4, "weight_decay": 0.0}], capturable=True, **hp)
    cpu, states = _oracle_for(params)
    lrs = [2e-3] * 3 + [5e-4] * 2
    wds = [0.05] * 3 + [0.0] * 2

    def feed_and_oracle():
        gs = _new_grads(shapes, gen, dtype)
        for p, g, c, st, lr, wd in zip(params, gs, cpu, states, lrs, wds):
            p.grad.copy_(g)
            CO.step_tensor(c, g, st, lr, 0.9, 0.99, 1e-8, wd)

    feed_and_oracle()
    opt.step()                                   # eager: builds the tables
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    feed_and_oracle()                            # the capture itself runs nothing; this step happens at the first replay
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            opt.step()
    torch.cuda.current_stream().wait_stream(side)
    graph.replay()
    for _ in range(5):
        feed_and_oracle()
        graph.replay()
    torch.cuda.synchronize()
    opt.state_dict()                             # reads the step count back
    _check_against_oracle(opt, params, cpu, states)
    assert not opt.nonfinite_seen() and not opt.schedule_exhausted()


def test_capturable_eager_steps_equal_the_plain_optimizer_and_survive_an_lr_change():
    dtype = torch.bfloat16
    shapes, params, gen = _static_problem(dtype, seed=12)
    twins = [nn.Parameter(p.detach().clone()) for p in params]
    a = qf.FourBitAdamW(params, lr=1e-3, capturable=True)
    b = qf.FourBitAdamW(twins, lr=1e-3)
    for it in range(9):
        if it == 4:                              # a scheduler's doing: same tables, new rows from the current step on
            a.param_groups[0]["lr"] = b.param_groups[0]["lr"] = 3e-4
        for p, q, g in zip(params, twins, _new_grads(shapes, gen, dtype)):
            if it in (2, 6):                     # gradients in new buffers: only their addresses are written again
                p.grad = g.to(DEV)
            else:
                p.grad.copy_(g)
            q.grad = g.to(DEV)
        a.step()
        b.step()
    sa, sb = a.state_dict()["state"], b.state_dict()["state"]
    for i, (p, q) in enumerate(zip(params, twins)):
        assert torch.equal(p, q)
        assert float(sa[i]["step"]) == float(sb[i]["step"]) == 9.0
        assert torch.equal(sa[i]["exp_avg"], sb[i]["exp_avg"]) and torch.equal(sa[i]["exp_avg_sq"], sb[i]["exp_avg_sq"])


def test_capturable_schedule_that_runs_out_is_reported_and_refresh_continues_exactly():
    dtype = torch.float32
    shapes, params, gen = _static_problem(dtype, seed=13)
    twins = [nn.Parameter(p.detach().clone()) for p in params]
    a = qf.FourBitAdamW(params, lr=1e-3, capturable=True, schedule_rows=3)
    b = qf.FourBitAdamW(twins, lr=1e-3)

    def both(n):
        for _ in range(n):
            for p, q, g in zip(params, twins, _new_grads(shapes, gen, dtype)):
                p.grad.copy_(g)
                q.grad = g.to(DEV)
            a.step()
            b.step()

    both(3)
    assert not a.schedule_exhausted()
    a.refresh_schedule()                         # rows for steps 4..6
    both(3)
    assert not a.schedule_exhausted()
    for p, q in zip(params, twins):
        assert torch.equal(p, q)
    for p, g in zip(params, _new_grads(shapes, gen, dtype)):
        p.grad.copy_(g)
    a.step()                                     # a seventh step on a three-row table: takes row 3 again, and says so
    assert a.schedule_exhausted()
    assert float(a.state_dict()["state"][0]["step"]) == 7.0


def test_capturable_refuses_what_it_cannot_record():
    p = nn.Parameter(torch.zeros(64, 256, device=DEV))
    opt = qf.FourBitAdamW([p], lr=1e-3, capturable=True)
    p.grad = torch.zeros_like(p)
    with pytest.raises(RuntimeError, match="grad_scale"):
        opt.step(grad_scale=0.5)
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with pytest.raises(RuntimeError, match="before capturing"):
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                opt.step()
    torch.cuda.synchronize()


# ---- relaxed_update=True: uncorrected bf16 parameter update, states untouched --------------------------------

def test_relaxed_update_keeps_every_code_and_scale_and_parameters_within_a_few_bf16_units():
    """40 free-running steps of two optimizers on the same gradients, one exact, one with relaxed_update: first and
    second moment never depend on the parameter, so codes and scales must be bit-identical throughout; a bf16
    parameter may differ where an update fell next to a rounding boundary, and such a difference stays (as an absolute
    amount: it counts for more units when the value shrinks later).  Counts are printed; asserted: every difference is
    at most two bf16 units of the largest magnitude the element can have had (|p| + 40 lr), and fewer than 1 % of the
    elements differ at all."""
    torch.manual_seed(3)
    lr, steps = 1e-3, 40
    shapes = [(1024, 1024), (512, 768), (300, 256), (5000,), (64,)]
    a = [nn.Parameter((torch.randn(s) * 0.02).to(DEV, torch.bfloat16)) for s in shapes]
    b = [nn.Parameter(p.detach().clone()) for p in a]
    oa = qf.FourBitAdamW(a, lr=lr)
    ob = qf.FourBitAdamW(b, lr=lr, relaxed_update=True)
    for _ in range(steps):
        for p, q in zip(a, b):
            g = (torch.randn(p.shape, device=DEV) * 1e-2).to(torch.bfloat16)
            p.grad, q.grad = g, g.clone()
        oa.step()
        ob.step()
    differ = total = 0
    worst_units = 0.0
    for i, (p, q) in enumerate(zip(a, b)):
        sa, sb = oa.state[p], ob.state[q]
        assert torch.equal(sa["exp_avg"], sb["exp_avg"]) and torch.equal(sa["exp_avg_sq"], sb["exp_avg_sq"]), i
        if sa["momentum_qstate"]["enable"]:
            assert torch.equal(sa["momentum_qstate"]["overhead"]["max1"], sb["momentum_qstate"]["overhead"]["max1"])
            va, vb = sa["variance_qstate"]["overhead"], sb["variance_qstate"]["overhead"]
            if va.get("max_dims") is not None:
                assert torch.equal(va["max_dims"][0], vb["max_dims"][0]) and torch.equal(va["max_dims"][1], vb["max_dims"][1])
            else:
                assert torch.equal(va["max1"], vb["max1"])
        pf, qf_ = p.detach().float(), q.detach().float()
        d = (pf - qf_).abs()
        if p.dim() != 2 or p.shape[1] % 256:
            assert float(d.max()) == 0.0, f"tensor {i} does not take the relaxed path"
        unit = torch.exp2(torch.floor(torch.log2(pf.abs() + steps * lr)) - 7)     # a bf16 unit at that magnitude
        worst_units = max(worst_units, float((d / unit).max()))
        total += d.numel()
        differ += int((d > 0).sum())
    print(f"relaxed update, {steps} steps: {differ} of {total} parameters differ from the exact ones; "
          f"largest difference {worst_units:.3f} bf16 units of |p| + {steps} lr")
    assert worst_units <= 2.0 and differ < total * 1e-2


# ---- nd_rank1=True: per-axis maxima for tensors of three and more dimensions --------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_nd_rank1_follows_the_per_axis_oracle_and_round_trips_through_a_state_dict(dtype):
    """3-D and 4-D tensors with the reference's per-axis second-moment scaling (last axis 256: panel mapping; 40 and 7:
    flat mapping), beside a matrix, a vector and a small tensor: parameters, codes, block scales and every axis' maxima
    against the oracle for six steps; then a state dict goes into a fresh optimizer, which continues identically."""
    gen = torch.Generator().manual_seed(21)
    shapes = [(6, 20, 256), (3, 4, 10, 40), (9, 11, 7, 7), (64, 256), (5000,), (4, 4, 4)]
    cpu = [(torch.randn(s, generator=gen) * 0.05).to(dtype) for s in shapes]
    params = [nn.Parameter(c.clone().to(DEV)) for c in cpu]
    states = [TO.TensorState.zeros(s, nd_rank1=True) for s in shapes]
    assert [st.kind for st in states] == ["rank1nd", "rank1nd", "rank1nd", "rank1", "block", "fp32"]
    opt = qf.FourBitAdamW(params, lr=2e-3, weight_decay=0.02, nd_rank1=True)

    def one_step(o, ps):
        gs = [(torch.randn(s, generator=gen) * 1e-2).to(dtype) for s in shapes]
        for p, g, c, st in zip(ps, gs, cpu, states):
            p.grad = g.to(DEV)
            CO.step_tensor(c, g, st, 2e-3, 0.9, 0.999, 1e-8, 0.02)
        o.step()

    for _ in range(6):
        one_step(opt, params)
        _check_against_oracle(opt, params, cpu, states)
    m, v = opt.dequantized_state(params[1])
    wm, wv = states[1].dequantized()
    assert torch.equal(m.cpu().reshape(-1), wm) and torch.equal(v.cpu().reshape(-1), wv)
    buf = io.BytesIO()
    torch.save(opt.state_dict(), buf)
    buf.seek(0)
    params2 = [nn.Parameter(p.detach().clone()) for p in params]
    opt2 = qf.FourBitAdamW(params2, lr=2e-3, weight_decay=0.02, nd_rank1=True)
    opt2.load_state_dict(torch.load(buf))
    for _ in range(3):
        one_step(opt2, params2)
        _check_against_oracle(opt2, params2, cpu, states)
    assert not opt2.nonfinite_seen()

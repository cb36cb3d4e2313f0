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
        if st.kind == "rank1":
            assert vo["max_dims"][0].shape == (st.shape[0], 1) and vo["max_dims"][1].shape == (1, st.shape[1])
            assert torch.equal(vo["max_dims"][0].cpu().reshape(-1), st.v_row)
            assert torch.equal(vo["max_dims"][1].cpu().reshape(-1), st.v_col)
        else:
            assert torch.equal(vo["max1"].cpu(), st.v_scale)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
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
    h = nn.Parameter(torch.randn(64, 128, device=DEV).half())
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

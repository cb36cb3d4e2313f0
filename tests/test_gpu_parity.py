"""GPU parity tests: the CUDA kernels, called through the C ABI, against the CPU oracle on the same
seeded inputs.  Bar: packed codes, scales and parameters bit-exact (all arithmetic is IEEE
round-to-nearest in the same order as the oracle; a midpoint tie goes to the lower code on both
sides).  The tolerance asked of the path -- codes may differ on qmap-midpoint ties for at most 1e-6
of the elements by one level, parameters within rtol 1e-5 (fp32) / 1 bf16 ulp -- is asserted in the
long free-running test, where any differing rounding would compound."""
import math
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from helpers import AbiStepper, GpuState, make_grad
from oracle import c_oracle as CO
from oracle import torch_oracle as TO

pytestmark = pytest.mark.gpu

import quantfour_adamw_cuda_b200 as qf  # noqa: E402

DEV = "cuda"
HP = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)


def _hp_args():
    return HP["lr"], HP["betas"][0], HP["betas"][1], HP["eps"], HP["weight_decay"]


@pytest.mark.parametrize("n", [1, 2, 7, 127, 128, 129, 255, 4097, (1 << 20) + 3])
@pytest.mark.parametrize("which", [0, 1])
def test_quantize_dequantize_block(n, which):
    x = torch.randn(n) * 1e-3
    if n > 1000:
        x[::997] *= 100
    if which:
        x = x * x
    codes, scales = (qf.quantize_v_block if which else qf.quantize_m)(x.to(DEV))
    oc, osc = CO.quantize_block(x, which)
    assert torch.equal(codes.cpu().view(torch.uint8), oc)
    assert torch.equal(scales.cpu(), osc)
    back = (qf.dequantize_v_block if which else qf.dequantize_m)(codes, scales, n)
    assert torch.equal(back.cpu(), CO.dequantize_block(oc, osc, n, which))


def test_quantize_block_zero_and_tie_inputs():
    # all-zero block -> scale 0, code of 0.0; exact midpoints -> lower code
    x = torch.zeros(256)
    x[128:128 + 15] = TO.MM            # second block: scale = max|MM| < 1, values not exact midpoints after division
    x[128 + 20] = 1.0                  # force scale 1 so that the midpoints are hit exactly
    codes, scales = qf.quantize_m(x.to(DEV))
    oc, osc = CO.quantize_block(x, 0)
    assert torch.equal(codes.cpu().view(torch.uint8), oc) and torch.equal(scales.cpu(), osc)
    got = TO.unpack(codes.cpu(), 256)
    assert set(got[:128].tolist()) == {7}
    assert got[128:128 + 15].tolist() == list(range(15))   # tie -> lower code


@pytest.mark.parametrize("shape", [(256, 512), (300, 77), (1, 8192), (8192, 1), (33, 256), (17, 1000)])
def test_quantize_dequantize_rank1(shape):
    v = (torch.randn(shape) * 1e-3) ** 2
    v[shape[0] // 2, shape[1] // 3] *= 1e4
    codes, row, col = qf.quantize_v(v.to(DEV))
    oc, orow, ocol = CO.quantize_rank1(v)
    assert torch.equal(row.cpu(), orow) and torch.equal(col.cpu(), ocol)
    assert torch.equal(codes.cpu().view(torch.uint8), oc)
    back = qf.dequantize_v(codes, row, col)
    assert torch.equal(back.cpu(), CO.dequantize_rank1(oc, orow, ocol, *shape))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("n", [1, 50, 4096, 5000])
def test_fused_single_tensor_matches_oracle(dtype, n):
    p = (torch.randn(n) * 0.02).to(dtype)
    st = TO.TensorState("fp32", (n,), m=torch.zeros(n), v=torch.zeros(n))
    pg, mg, vg = p.to(DEV), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    for step in range(1, 6):
        g = make_grad((n,), dtype)
        CO.step_tensor(p, g, st, *_hp_args())
        qf.fused_single_tensor(pg, g.to(DEV), mg, vg, 0.9, 0.999, 1e-3, 0.01, 1e-8, torch.tensor(float(step)))
        assert torch.equal(pg.cpu(), p) and torch.equal(mg.cpu(), st.m) and torch.equal(vg.cpu(), st.v)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("n", [4097, 128 * 33, 100_003])
def test_fused_4bit_matches_oracle(dtype, n):
    p = (torch.randn(n) * 0.02).to(dtype)
    st = TO.TensorState.zeros((n,))
    assert st.kind == "block"
    pg = p.to(DEV)
    exp = torch.zeros((n + 1) // 2, dtype=torch.int8, device=DEV)
    sq = torch.zeros_like(exp)
    es = torch.zeros((n + 127) // 128, device=DEV)
    ss = torch.zeros_like(es)
    for step in range(1, 6):
        g = make_grad((n,), dtype)
        CO.step_tensor(p, g, st, *_hp_args())
        qf.fused_4bit(pg, g.to(DEV), exp, sq, es, ss, 0.9, 0.999, 1e-3, 0.01, 1e-8, step)
        assert torch.equal(pg.cpu(), p)
        assert torch.equal(exp.cpu().view(torch.uint8), st.m_codes) and torch.equal(sq.cpu().view(torch.uint8), st.v_codes)
        assert torch.equal(es.cpu(), st.m_scale) and torch.equal(ss.cpu(), st.v_scale)


RAGGED = [
    ((64, 128), torch.float32), ((256, 512), torch.bfloat16), ((300, 77), torch.float32), ((129, 255), torch.bfloat16),
    ((5001,), torch.float32), ((4097,), torch.bfloat16), ((40, 50), torch.float32), ((1024,), torch.bfloat16),
    ((3, 5, 7, 99), torch.float32), ((1, 8192), torch.bfloat16), ((8192, 1), torch.float32), ((4096,), torch.float32),
    ((512, 768), torch.bfloat16), ((1,), torch.float32), ((48, 256), torch.float32),
    ((96, 256), torch.float16), ((131, 77), torch.float16), ((6001,), torch.float16), ((100,), torch.float16),
    # panel tensors whose row count is odd or not a multiple of the item length: the last row of an item goes alone
    ((77, 256), torch.bfloat16), ((17, 512), torch.float32), ((131, 768), torch.bfloat16),
]


def _make_problem(specs, seed=0):
    gen = torch.Generator().manual_seed(seed)
    params = [(torch.randn(s, generator=gen) * 0.02).to(dt) for s, dt in specs]
    ostates = [TO.TensorState.zeros(s) for s, _ in specs]
    gparams = [p.to(DEV) for p in params]
    gstates = [GpuState(st) for st in ostates]
    return gen, params, ostates, gparams, gstates


def _assert_same(params, ostates, gparams, gstates, what=""):
    for i, (p, st, gp, gs) in enumerate(zip(params, ostates, gparams, gstates)):
        assert torch.equal(gp.cpu(), p), f"{what} tensor {i} {tuple(p.shape)} {p.dtype}: params differ in {(gp.cpu() != p).sum()} places"
        d = gs.diff(st)
        assert not any(v for k, v in d.items()), f"{what} tensor {i} {tuple(p.shape)} {p.dtype} kind {st.kind}: {d}"


@pytest.mark.parametrize("split", [False, True])
def test_multi_tensor_step_free_running_bit_exact(split):
    gen, params, ostates, gparams, gstates = _make_problem(RAGGED)
    stepper = AbiStepper(gparams, gstates, **HP)
    for step in range(12):
        sig = 10 ** float(torch.empty(1).uniform_(-5, -2, generator=gen))
        grads = [make_grad(p.shape, p.dtype, sigma=sig, gen=gen) for p in params]
        if step in (3, 4):          # a parameter without gradient is skipped and keeps its own step count
            grads[2] = None
            grads[5] = None
        for p, g, st in zip(params, grads, ostates):
            if g is not None:
                CO.step_tensor(p, g, st, *_hp_args())
        stepper.step([None if g is None else g.to(DEV) for g in grads], split=split)
        _assert_same(params, ostates, gparams, gstates, f"step {step + 1}")
    assert stepper.status() == 0


def test_workspace_may_be_recycled_between_calls():
    """Identical descriptors on consecutive calls, and the workspace memory rewritten in between (what an allocator
    does when it hands a freed address out again, zero-filled): the step must not work from a stale table."""
    gen, params, ostates, gparams, gstates = _make_problem(RAGGED[:8])
    stepper = AbiStepper(gparams, gstates, **HP)
    gbuf = [torch.empty_like(p) for p in gparams]
    for step in range(3):
        grads = [make_grad(p.shape, p.dtype, gen=gen) for p in params]
        for p, g, st in zip(params, grads, ostates):
            CO.step_tensor(p, g, st, *_hp_args())
        for b, g in zip(gbuf, grads):
            b.copy_(g)
        stepper.step(gbuf)
        torch.cuda.synchronize()
        stepper.ws.zero_()
        _assert_same(params, ostates, gparams, gstates, f"step {step + 1}")


def test_late_steps_where_the_bias_correction_has_rounded_to_one():
    """From about step 17 000 on (beta2 = 0.999) sqrt(1 - beta2^t) is exactly 1.0f and the library runs the kernel
    variant without that division: same bits as the oracle, which still divides."""
    gen, params, ostates, gparams, gstates = _make_problem(RAGGED)
    for st, gs in zip(ostates, gstates):
        st.step = gs.step = 30000
    assert np.float32(TO.Hyper.make(1e-3, 0.9, 0.999, 1e-8, 0.01, 30001).bc2s) == np.float32(1.0)
    stepper = AbiStepper(gparams, gstates, **HP)
    for step in range(4):
        grads = [make_grad(p.shape, p.dtype, gen=gen) for p in params]
        for p, g, st in zip(params, grads, ostates):
            CO.step_tensor(p, g, st, *_hp_args())
        stepper.step([g.to(DEV) for g in grads])
        _assert_same(params, ostates, gparams, gstates, f"step {30001 + step}")


@pytest.mark.parametrize("hp", [
    dict(lr=1.0, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0),
    dict(lr=3e-4, betas=(0.5, 0.9), eps=1e-6, weight_decay=0.1),
    dict(lr=1e-2, betas=(0.99, 0.9999), eps=1e-10, weight_decay=1e-3),
    dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-15, weight_decay=0.01),     # eps below the range of the packed sequences
    dict(lr=1e-5, betas=(0.0001, 0.5), eps=1.0, weight_decay=10.0),
])
def test_other_hyper_parameters_bit_exact(hp):
    gen, params, ostates, gparams, gstates = _make_problem(RAGGED, seed=3)
    stepper = AbiStepper(gparams, gstates, **hp)
    args = (hp["lr"], hp["betas"][0], hp["betas"][1], hp["eps"], hp["weight_decay"])
    for step in range(5):
        scale = [1e-3, 1.0, 1e-6, 30.0, 0.0][step]     # ordinary, large, tiny, huge and all-zero gradients
        grads = [make_grad(p.shape, p.dtype, sigma=1e-3, gen=gen) * scale for p in params]
        for p, g, st in zip(params, grads, ostates):
            CO.step_tensor(p, g, st, *args)
        stepper.step([g.to(DEV) for g in grads])
        _assert_same(params, ostates, gparams, gstates, f"{hp} step {step + 1}")
    assert stepper.status() == 0


def test_multi_tensor_step_teacher_forced():
    """Each step starts from the oracle's state, so a mismatch cannot hide behind an earlier one."""
    gen, params, ostates, gparams, gstates = _make_problem(RAGGED, seed=1)
    stepper = AbiStepper(gparams, gstates, **HP)
    for step in range(6):
        grads = [make_grad(p.shape, p.dtype, gen=gen) for p in params]
        for gp, p, gs, st in zip(gparams, params, gstates, ostates):
            gp.copy_(p)
            gs.load(st)
        for p, g, st in zip(params, grads, ostates):
            CO.step_tensor(p, g, st, *_hp_args())
        stepper.step([g.to(DEV) for g in grads])
        _assert_same(params, ostates, gparams, gstates, f"step {step + 1}")


def test_first_step_against_reference_fixture():
    """Fixture produced by the reference's own _single_tensor_step (tests/golden/make_golden.py)."""
    z = np.load(os.path.join(GOLDEN, "step1.npz"))
    p = torch.from_numpy(z["p0"]).clone()
    gs = GpuState(TO.TensorState.zeros(p.shape))
    gp = p.to(DEV)
    stepper = AbiStepper([gp], [gs], lr=float(z["lr"]), betas=(float(z["beta1"]), float(z["beta2"])), eps=float(z["eps"]),
                         weight_decay=float(z["wd"]))
    stepper.step([torch.from_numpy(z["g"]).to(DEV)])
    assert np.array_equal(gs.m_scale.cpu().numpy(), z["m_max1"].reshape(-1))
    assert np.array_equal(gs.v_row.cpu().numpy(), z["v_row"].reshape(-1))
    assert np.array_equal(gs.v_col.cpu().numpy(), z["v_col"].reshape(-1))
    assert np.array_equal(TO.unpack(gs.m_codes.cpu(), p.numel())[:128].numpy(), z["m_row0_codes"])
    assert np.array_equal(TO.unpack(gs.v_codes.cpu(), p.numel())[:128].numpy(), z["v_row0_codes"])
    diff = (gp.cpu() - torch.from_numpy(z["p1"])).abs()
    # the reference run took torch's CPU float32 sqrt, which is off by one ulp on a few inputs
    assert float(diff.max()) <= 8e-9 and float((diff != 0).float().mean()) < 5e-3


def test_config1_4096x4096_fp32_ten_steps():
    """Single 4096x4096 fp32 parameter, seed 0, param ~N(0, 0.02), grad ~N(0, 1e-3) fresh per step,
    10 steps, lr 1e-3, betas (0.9, 0.999), eps 1e-8, wd 0.01."""
    torch.manual_seed(0)
    p = torch.randn(4096, 4096) * 0.02
    st = TO.TensorState.zeros(p.shape)
    gs, gp = GpuState(st), p.to(DEV)
    stepper = AbiStepper([gp], [gs], **HP)
    for step in range(10):
        g = torch.randn(4096, 4096) * 1e-3
        CO.step_tensor(p, g, st, *_hp_args())
        stepper.step([g.to(DEV)])
    _assert_same([p], [st], [gp], [gs], "after 10 steps")
    # and the result stays close to fp32 AdamW (the reference's own acceptance test, tests/driver.py:71)
    assert stepper.status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_hundred_steps_free_running_within_tolerance(dtype):
    """100 free-running steps: codes may differ only on midpoint ties (<= 1e-6 of the elements, one level),
    parameters and dequantized states within rtol 1e-5 (fp32) or one bf16 ulp (bf16)."""
    specs = [((512, 1024), dtype), ((70_000,), dtype), ((2048,), dtype)]
    gen, params, ostates, gparams, gstates = _make_problem(specs, seed=3)
    stepper = AbiStepper(gparams, gstates, **HP)
    for step in range(100):
        grads = [make_grad(p.shape, p.dtype, gen=gen) for p in params]
        for p, g, st in zip(params, grads, ostates):
            CO.step_tensor(p, g, st, *_hp_args())
        stepper.step([g.to(DEV) for g in grads])
    total = differing = 0
    for p, st, gp, gs in zip(params, ostates, gparams, gstates):
        d = gs.diff(st)
        if st.kind != "fp32":
            total += 2 * p.numel()
            differing += d["m_codes"] + d["v_codes"]
            assert d["max_code_dist"] <= 1
        if dtype == torch.float32:
            torch.testing.assert_close(gp.cpu(), p, rtol=1e-5, atol=0)
        else:
            ulp = (gp.cpu().view(torch.int16).int() - p.view(torch.int16).int()).abs().max()
            assert int(ulp) <= 1
    assert differing / total <= 1e-6, f"differing code fraction {differing / total:.3e}"
    print(f"differing code fraction after 100 steps: {differing / total:.3e} ({differing} of {total})")


def test_two_runs_are_bit_identical():
    outs = []
    for _ in range(2):
        gen, params, ostates, gparams, gstates = _make_problem(RAGGED, seed=5)
        stepper = AbiStepper(gparams, gstates, **HP)
        for _ in range(4):
            stepper.step([make_grad(p.shape, p.dtype, gen=gen).to(DEV) for p in params])
        outs.append([gp.cpu() for gp in gparams] + [gs.m_codes.cpu() for gs in gstates if gs.kind != "fp32"]
                    + [gs.v_codes.cpu() for gs in gstates if gs.kind != "fp32"])
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_nonfinite_gradient_sets_status_and_does_not_hang():
    gen, params, ostates, gparams, gstates = _make_problem([((256, 256), torch.float32), ((5000,), torch.float32)])
    stepper = AbiStepper(gparams, gstates, **HP)
    grads = [make_grad(p.shape, p.dtype, gen=gen).to(DEV) for p in params]
    grads[0][3, 7] = float("inf")
    stepper.step(grads)
    assert stepper.status() & 1
    assert stepper.status() == 0     # reading clears the word


@pytest.mark.parametrize("spec", [((9000,), torch.float32), ((9000,), torch.bfloat16), ((512, 512), torch.bfloat16),
                                  ((300, 300), torch.float32)],
                         ids=["block-f32", "block-bf16", "panel-bf16", "rank1-flat-f32"])
def test_nan_gradient_reaches_the_scales_and_the_status_word(spec):
    """One NaN gradient after two warm steps: every scale the reference's abs().max() would turn into NaN is NaN here
    (the packed block maximum must not drop it), the status word reports it, and everything the NaN cannot reach is
    what the oracle computes.  Codes under a NaN scale are outside the contract (the reference leaves them undefined)."""
    shape, dt = spec
    gen, params, ostates, gparams, gstates = _make_problem([spec], seed=11)
    p, st, gp, gs = params[0], ostates[0], gparams[0], gstates[0]
    stepper = AbiStepper(gparams, gstates, **HP)
    for _ in range(2):
        g = make_grad(shape, dt, gen=gen)
        TO.step_tensor(p, g, st, *_hp_args())
        stepper.step([g.to(DEV)])
    _assert_same(params, ostates, gparams, gstates, "warm")
    assert stepper.status() == 0
    g = make_grad(shape, dt, gen=gen)
    flat = 4321
    g.view(-1)[flat] = float("nan")
    TO.step_tensor(p, g, st, *_hp_args())
    stepper.step([g.to(DEV)])
    assert stepper.status() & 1
    n = math.prod(shape)
    ms, oms = gs.m_scale.cpu(), st.m_scale
    assert torch.equal(torch.isnan(ms), torch.isnan(oms)) and int(torch.isnan(oms).sum()) == 1
    assert torch.equal(ms[~torch.isnan(oms)], oms[~torch.isnan(oms)])
    clean = torch.ones(n, dtype=torch.bool)          # elements whose scales the NaN does not touch
    clean[flat // 128 * 128:(flat // 128 + 1) * 128] = False
    if st.kind == "rank1":
        R, Cc = shape
        for a, b in ((gs.v_row.cpu(), st.v_row), (gs.v_col.cpu(), st.v_col)):
            assert torch.equal(torch.isnan(a), torch.isnan(b)) and int(torch.isnan(b).sum()) == 1
            assert torch.equal(a[~torch.isnan(b)], b[~torch.isnan(b)])
        grid = clean.view(R, Cc)
        grid[flat // Cc, :] = False
        grid[:, flat % Cc] = False
    else:
        vs, ovs = gs.v_scale.cpu(), st.v_scale
        assert torch.equal(torch.isnan(vs), torch.isnan(ovs)) and int(torch.isnan(ovs).sum()) == 1
        assert torch.equal(vs[~torch.isnan(ovs)], ovs[~torch.isnan(ovs)])
    cm, om = TO.unpack(gs.m_codes.cpu(), n), TO.unpack(st.m_codes, n)
    cv, ov = TO.unpack(gs.v_codes.cpu(), n), TO.unpack(st.v_codes, n)
    assert torch.equal(cm[clean], om[clean]) and torch.equal(cv[clean], ov[clean])
    pg, po = gp.cpu().view(-1), p.view(-1)
    assert torch.isnan(pg[flat]) and torch.isnan(po[flat])
    keep = torch.ones(n, dtype=torch.bool)
    keep[flat] = False
    assert torch.equal(pg[keep], po[keep])


def test_unaligned_views_take_the_scalar_path():
    """Buffers that are only element-aligned (views at odd offsets) still give oracle results."""
    n = 5003
    base_p = torch.zeros(n + 8, device=DEV)
    base_g = torch.zeros(n + 8, device=DEV)
    p = torch.randn(n) * 0.02
    st = TO.TensorState.zeros((n,))
    gp, gg = base_p[1:n + 1], base_g[3:n + 3]
    gp.copy_(p)
    gs = GpuState(st)
    stepper = AbiStepper([gp], [gs], **HP)
    for _ in range(3):
        g = make_grad((n,), torch.float32)
        gg.copy_(g)
        CO.step_tensor(p, g, st, *_hp_args())
        stepper.step([gg])
    _assert_same([p], [st], [gp], [gs])


def _shape_list_problem(shapes, dtype, seed, sigma_seed=1234):
    gen = torch.Generator().manual_seed(seed)
    sig = (10 ** torch.empty(len(shapes)).uniform_(-5, -2, generator=torch.Generator().manual_seed(sigma_seed))).tolist()
    params = [(torch.randn(s, generator=gen) * 0.02).to(dtype) for s in shapes]
    return gen, sig, params


def test_config3_gpt2_medium_shaped_list_single_multi_tensor_step():
    """GPT-2-medium-shaped ragged list (292 tensors, 354.8 M parameters, bf16, per-tensor gradient sigma log-uniform in
    [1e-5, 1e-2]): one multi-tensor step from zero state and one from warm state, every tensor against the oracle."""
    from quantfour_adamw_cuda_b200 import shapes as S
    shapes = S.gpt2_medium()
    gen, sig, params = _shape_list_problem(shapes, torch.bfloat16, 7)
    ostates = [TO.TensorState.zeros(s) for s in shapes]
    gparams = [p.to(DEV) for p in params]
    gstates = [GpuState(st) for st in ostates]
    stepper = AbiStepper(gparams, gstates, **HP)
    for step in range(3):
        grads = [make_grad(p.shape, p.dtype, sigma=sg, gen=gen) for p, sg in zip(params, sig)]
        for p, g, st in zip(params, grads, ostates):
            CO.step_tensor(p, g, st, *_hp_args())
        stepper.step([g.to(DEV) for g in grads])
        if step in (0, 2):
            _assert_same(params, ostates, gparams, gstates, f"step {step + 1}")
    assert sum(st.kind == "fp32" for st in ostates) == 194 and sum(st.kind == "rank1" for st in ostates) == 98


def test_config4_llama7b_subset_twenty_steps():
    """Parity subset of the Llama-7B-shaped set: one decoder layer's nine tensors plus a 2048-row slice of the embedding,
    bf16 with 0.1 % x100 outliers, 20 free-running steps (the full set has no CPU oracle run in reasonable time)."""
    from quantfour_adamw_cuda_b200 import shapes as S
    shapes = S.llama_7b()[1:10] + [(2048, 4096)]
    gen, sig, params = _shape_list_problem(shapes, torch.bfloat16, 9)
    ostates = [TO.TensorState.zeros(s) for s in shapes]
    gparams = [p.to(DEV) for p in params]
    gstates = [GpuState(st) for st in ostates]
    stepper = AbiStepper(gparams, gstates, **HP)
    for step in range(20):
        grads = [make_grad(p.shape, p.dtype, sigma=sg, gen=gen) for p, sg in zip(params, sig)]
        for p, g, st in zip(params, grads, ostates):
            CO.step_tensor(p, g, st, *_hp_args())
        stepper.step([g.to(DEV) for g in grads])
    _assert_same(params, ostates, gparams, gstates, "after 20 steps")
    assert stepper.status() == 0


def test_config2_full_size_properties():
    """Quantize / dequantize at the micro-benchmark's full sizes, checked through size-independent properties:
    the round-trip error is bounded by half the widest gap of the map times the scale, re-quantizing the dequantized
    second moment gives the same codes and maxima (idempotence; the first-moment map is not idempotent because its
    lowest value is -0.8875, not -1), and the codes of a slice match the oracle on that slice."""
    n = 1 << 28
    g = torch.Generator(device=DEV).manual_seed(0)
    x = torch.randn(n, generator=g, device=DEV) * 1e-3
    mask = torch.rand(n, generator=torch.Generator(device=DEV).manual_seed(1), device=DEV) < 1e-3
    x = torch.where(mask, x * 100, x)
    codes, scales = qf.quantize_m(x)
    back = qf.dequantize_m(codes, scales, n)
    err = (back - x).abs().view(-1, 128) / scales.view(-1, 1).clamp_min(1e-30)
    assert float(err.max()) <= 0.1126
    sl = slice(12345 * 128, 12345 * 128 + (1 << 20))
    oc, osc = CO.quantize_block(x[sl].cpu(), 0)
    assert torch.equal(codes[sl.start // 2: sl.stop // 2].cpu().view(torch.uint8), oc)
    assert torch.equal(scales[sl.start // 128: sl.stop // 128].cpu(), osc)
    del x, back, err, mask
    torch.cuda.empty_cache()
    R = C = 16384
    v = (torch.randn(R, C, generator=torch.Generator(device=DEV).manual_seed(2), device=DEV) * 1e-3) ** 2
    codes, row, col = qf.quantize_v(v)
    assert torch.equal(row, v.max(dim=1).values) and torch.equal(col, v.max(dim=0).values)
    back = qf.dequantize_v(codes, row, col)
    st = torch.min(row.view(-1, 1), col.view(1, -1))
    assert float(((back - v).abs() / st).max()) <= 0.0625 + 1e-6
    codes2, row2, col2 = qf.quantize_v(back)
    assert torch.equal(row2, row) and torch.equal(col2, col) and torch.equal(codes2, codes)
    rows = slice(5000, 5064)
    oc = TO.pack(TO.codes_of(TO._safe_div(v[rows].cpu(), st[rows].cpu()), TO.MV))
    assert torch.equal(codes[rows.start * C // 2: rows.stop * C // 2].cpu().view(torch.uint8), oc)

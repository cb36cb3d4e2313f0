"""CPU tests that pin the oracle: against fixtures produced by the reference's own Python functions
(tests/golden/make_golden.py) and the two oracle forms against each other."""
import math
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN
from oracle import c_oracle as CO
from oracle import torch_oracle as TO


def _z(name):
    return np.load(os.path.join(GOLDEN, name))


def test_tables_equal_reference_literals():
    z = _z("tables.npz")
    qm, mm, qv, mv = CO.tables()
    for ours_c, ours_t, key in ((qm, TO.QM, "qm"), (mm, TO.MM, "mm"), (qv, TO.QV, "qv"), (mv, TO.MV, "mv")):
        assert np.array_equal(ours_c.numpy(), z[key]), key
        assert np.array_equal(ours_t.numpy(), z[key]), key


@pytest.mark.parametrize("which,name", [(0, "m"), (1, "v")])
def test_search_equals_reference_bsearch(which, name):
    z = _z("search.npz")
    x = torch.from_numpy(z[f"x_{name}"])
    want = z[f"code_{name}"]
    mid = TO.MV if which else TO.MM
    assert np.array_equal(TO.codes_of(x, mid).numpy(), want)
    assert np.array_equal(CO.search(x, which).numpy(), want)
    assert np.array_equal(CO.search(x, which, literal=True).numpy(), want)


@pytest.mark.parametrize("which", [0, 1])
def test_count_form_equals_literal_search_on_random_points(which):
    g = torch.Generator().manual_seed(11 + which)
    x = torch.cat([torch.rand(100_000, generator=g) * 2.4 - 1.2, torch.randn(100_000, generator=g) * 0.01])
    assert torch.equal(CO.search(x, which), CO.search(x, which, literal=True))


def test_scaling_helpers_match_reference():
    z = _z("scaling.npz")
    xm = torch.from_numpy(z["xm"])
    packed, scales = TO.quantize_block(xm, TO.MM)
    assert np.array_equal(scales.numpy(), z["xm_max1"].reshape(-1))
    assert np.array_equal(TO.unpack(packed, xm.numel())[:128].numpy(), z["xm_row0_codes"])
    pc, sc = CO.quantize_block(xm, 0)
    assert torch.equal(pc, packed) and torch.equal(sc, scales)
    xv = torch.from_numpy(z["xv"])
    packed, row, col = TO.quantize_rank1(xv)
    assert np.array_equal(row.numpy(), z["xv_row"].reshape(-1))
    assert np.array_equal(col.numpy(), z["xv_col"].reshape(-1))
    assert np.array_equal(TO.unpack(packed, xv.numel())[:200].numpy(), z["xv_row0_codes"])
    pc, rc, cc = CO.quantize_rank1(xv)
    assert torch.equal(pc, packed) and torch.equal(rc, row) and torch.equal(cc, col)
    # the scaled tensor itself
    st = torch.min(row.view(-1, 1), col.view(1, -1))
    assert np.array_equal(xv.div(st).numpy(), z["xv_scaled"])


def test_tables_against_the_maps_the_reference_generator_creates():
    """qmaps_created.npz: create_qmap('nonlinear', 4, signed) and create_qmap('power-1', 4, unsigned) of the
    reference (quant_opt_base.py:32-52).  The second-moment map is the hard-coded one bit for bit; the generated
    first-moment map differs from the hard-coded literals at +-0.2125 and +-0.0325, each by one unit in the last place
    (its linspace arithmetic lands on 0.21249999 and 0.032499999).  The kernels and this oracle follow the hard-coded
    tables, as both of the reference's own paths do."""
    z, t = _z("qmaps_created.npz"), _z("tables.npz")
    assert np.array_equal(z["qv"], t["qv"]) and np.array_equal(TO.QV.numpy(), t["qv"])
    differ = np.nonzero(z["qm"] != t["qm"])[0]
    assert list(differ) == [3, 5, 9, 11]
    assert np.array_equal(np.abs(z["qm"][differ] - t["qm"][differ]), np.spacing(np.abs(z["qm"][differ])))
    assert np.array_equal(TO.QM.numpy(), t["qm"])


def test_per_axis_scaling_of_tensors_with_more_than_two_axes_matches_reference():
    """scaling_nd.npz: the reference's variance_quant_scaling on a 3-D and a 4-D tensor (its per-axis maxima, the
    scaled tensor) and the scale tensor its dequantize side rebuilds from the maxima."""
    z = _z("scaling_nd.npz")
    for name in ("a", "b"):
        x = torch.from_numpy(z[f"x_{name}"])
        stats = TO.axis_stats(x)
        for k, s in enumerate(stats):
            assert np.array_equal(s.numpy(), z[f"max{k}_{name}"]), (name, k)
        scale = TO.axis_scale(stats)
        assert np.array_equal(scale.numpy(), z[f"scale_{name}"])
        assert np.array_equal(x.div(scale).numpy(), z[f"scaled_{name}"])
        packed, axes = TO.quantize_rank1_nd(x)
        back = TO.dequantize_rank1_nd(packed, axes, x.shape)
        want = TO.QV[TO.codes_of(torch.from_numpy(z[f"scaled_{name}"]), TO.MV).long()].mul(torch.from_numpy(z[f"scale_{name}"]))
        assert torch.equal(back, want)


def test_folding_the_leading_axes_into_rows_gives_the_same_scale():
    """What the CUDA path relies on for rank >= 3: with the leading axes folded into rows and the per-row scale taken as
    the smallest of the leading axes' maxima, min(row scale, column maximum) is the reference's per-axis scale."""
    g = torch.Generator().manual_seed(0)
    for shape in ((5, 7, 12), (2, 3, 4, 9)):
        x = torch.rand(shape, generator=g)
        stats = TO.axis_stats(x)
        lead = TO.axis_scale(stats[:-1]).expand(*shape[:-1], 1).reshape(-1, 1)
        folded = torch.min(lead, stats[-1].reshape(1, -1)).view(shape)
        assert torch.equal(folded, TO.axis_scale(stats))
        # and the leading axes' maxima follow from the row maxima of the folded matrix
        rowmax = x.reshape(-1, shape[-1]).max(dim=1).values.view(shape[:-1])
        for k in range(len(shape) - 1):
            others = [d for d in range(len(shape) - 1) if d != k]
            mk = rowmax.amax(dim=others) if others else rowmax
            assert torch.equal(mk, stats[k].reshape(-1))


@pytest.mark.parametrize("oracle", ["torch", "c"])
def test_first_step_matches_reference_step(oracle):
    """The reference's own _single_tensor_step from zero state: scales, rank-1 maxima and the stored
    codes must be identical; the parameter may differ by one ulp on a few elements because the
    reference run took torch's CPU float32 sqrt, which is not correctly rounded."""
    z = _z("step1.npz")
    p, g = torch.from_numpy(z["p0"]).clone(), torch.from_numpy(z["g"])
    st = TO.TensorState.zeros(p.shape)
    step = TO.step_tensor if oracle == "torch" else CO.step_tensor
    step(p, g, st, float(z["lr"]), float(z["beta1"]), float(z["beta2"]), float(z["eps"]), float(z["wd"]))
    assert st.step == int(z["step"]) == 1
    assert np.array_equal(st.m_scale.numpy(), z["m_max1"].reshape(-1))
    assert np.array_equal(st.v_row.numpy(), z["v_row"].reshape(-1))
    assert np.array_equal(st.v_col.numpy(), z["v_col"].reshape(-1))
    assert np.array_equal(TO.unpack(st.m_codes, p.numel())[:128].numpy(), z["m_row0_codes"])
    assert np.array_equal(TO.unpack(st.v_codes, p.numel())[:128].numpy(), z["v_row0_codes"])
    want = torch.from_numpy(z["p1"])
    diff = (p - want).abs()
    assert float(diff.max()) <= 8e-9            # one ulp of a parameter of magnitude < 0.125
    assert float((diff != 0).float().mean()) < 5e-3


def test_adamw_arithmetic_fixture():
    z = _z("adamw_arith.npz")
    h = TO.Hyper.make(float(z["lr"]), float(z["beta1"]), float(z["beta2"]), float(z["eps"]), float(z["wd"]),
                      int(z["step"]))
    p, g = torch.from_numpy(z["p0"]).clone(), torch.from_numpy(z["g"])
    m, v = torch.from_numpy(z["m0"]).clone(), torch.from_numpy(z["v0"]).clone()
    TO.adamw_update_(p, g, m, v, h)
    assert np.array_equal(p.numpy(), z["p1"]) and np.array_equal(m.numpy(), z["m1"]) and np.array_equal(v.numpy(), z["v1"])
    # the C form on the same inputs (fp32-state path)
    st = TO.TensorState("fp32", (p.numel(),), step=int(z["step"]) - 1, m=torch.from_numpy(z["m0"]).clone(),
                        v=torch.from_numpy(z["v0"]).clone())
    p2 = torch.from_numpy(z["p0"]).clone()
    CO.step_tensor(p2, g, st, float(z["lr"]), float(z["beta1"]), float(z["beta2"]), float(z["eps"]), float(z["wd"]))
    assert np.array_equal(p2.numpy(), z["p1"]) and np.array_equal(st.m.numpy(), z["m1"]) and np.array_equal(st.v.numpy(), z["v1"])


def _states_equal(a: TO.TensorState, b: TO.TensorState) -> bool:
    if a.kind == "fp32":
        return torch.equal(a.m, b.m) and torch.equal(a.v, b.v)
    ok = torch.equal(a.m_codes, b.m_codes) and torch.equal(a.v_codes, b.v_codes) and torch.equal(a.m_scale, b.m_scale)
    if a.kind == "rank1":
        return ok and torch.equal(a.v_row, b.v_row) and torch.equal(a.v_col, b.v_col)
    return ok and torch.equal(a.v_scale, b.v_scale)


@pytest.mark.parametrize("shape,dtype", [
    ((64, 128), torch.float32), ((300, 77), torch.float32), ((5001,), torch.float32), ((40, 50), torch.float32),
    ((128, 256), torch.bfloat16), ((4097,), torch.bfloat16), ((3, 5, 7, 99), torch.float32), ((1, 8192), torch.bfloat16),
    ((8192, 1), torch.float32),
])
def test_c_and_torch_oracles_agree_bit_for_bit(shape, dtype):
    p1 = (torch.randn(shape) * 0.02).to(dtype)
    p2 = p1.clone()
    s1, s2 = TO.TensorState.zeros(shape), TO.TensorState.zeros(shape)
    for _ in range(6):
        g = (torch.randn(shape) * 1e-3).to(dtype)
        if g.numel() > 200:
            g.view(-1)[123] *= 100
        TO.step_tensor(p1, g, s1, 1e-3, 0.9, 0.999, 1e-8, 0.01)
        CO.step_tensor(p2, g, s2, 1e-3, 0.9, 0.999, 1e-8, 0.01)
        assert torch.equal(p1, p2)
        assert _states_equal(s1, s2)


def test_zero_gradient_block_keeps_zero_scale_and_zero_codes():
    p = torch.randn(64, 128) * 0.02
    g = torch.zeros(64, 128)
    for step in (TO.step_tensor, CO.step_tensor):
        st = TO.TensorState.zeros(p.shape)
        step(p.clone(), g, st, 1e-3, 0.9, 0.999, 1e-8, 0.01)
        assert float(st.m_scale.abs().max()) == 0 and float(st.v_row.max()) == 0
        assert set(TO.unpack(st.m_codes, p.numel()).tolist()) == {7}      # x = 0 -> code of 0.0
        assert set(TO.unpack(st.v_codes, p.numel()).tolist()) == {0}
        m, v = st.dequantized()
        assert float(m.abs().max()) == 0 and float(v.abs().max()) == 0


def test_pack_roundtrip_and_odd_tail():
    codes = torch.randint(0, 16, (4099,), dtype=torch.uint8)
    packed = TO.pack(codes)
    assert packed.numel() == 2050 and int(packed[-1]) >> 4 == 0
    assert torch.equal(TO.unpack(packed, 4099), codes)


def test_quantize_dequantize_roundtrip_error_bounds():
    x = torch.randn(1 << 16) * 1e-3
    packed, s = CO.quantize_block(x, 0)
    back = CO.dequantize_block(packed, s, x.numel(), 0)
    assert torch.equal(back, TO.dequantize_block(packed, s, x.numel(), TO.QM))
    # nearest-code property: the error is at most half the widest gap of the map times the block scale
    assert float(((back - x).abs() / s.repeat_interleave(128)).max()) <= 0.1126
    v = (torch.randn(256, 384) * 1e-3) ** 2
    pk, row, col = CO.quantize_rank1(v)
    back = CO.dequantize_rank1(pk, row, col, 256, 384)
    assert torch.equal(back, TO.dequantize_rank1(pk, row, col, 256, 384))
    assert float(((back - v).abs() / torch.min(row.view(-1, 1), col.view(1, -1))).max()) <= 0.0625 + 1e-6


def test_stays_close_to_fp32_adamw_like_the_reference_test():
    """The reference's only numeric pin (tests/driver.py:26-72): parameters stay within atol 0.025 of
    torch.optim.AdamW over 10 steps (lr 0.005, betas (0.8, 0.88), wd 0.03)."""
    p = torch.randn(96, 128) * 0.1
    q = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([q], lr=0.005, betas=(0.8, 0.88), weight_decay=0.03, eps=1e-8)
    st = TO.TensorState.zeros(p.shape)
    for _ in range(10):
        g = torch.randn_like(p)
        q.grad = g.clone()
        opt.step()
        CO.step_tensor(p, g, st, 0.005, 0.8, 0.88, 1e-8, 0.03)
        torch.testing.assert_close(p, q.detach(), atol=0.025, rtol=1e-5)

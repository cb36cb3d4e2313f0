"""Generate the golden fixtures in this directory by running the reference's own Python code.

    python tests/golden/make_golden.py /path/to/reference          (all fixtures)
    python tests/golden/make_golden.py /path/to/reference nd       (scaling_nd.npz only)
    python tests/golden/make_golden.py /path/to/reference qmaps    (qmaps_created.npz only)

Needs the reference checkout (read-only) and no GPU.  The one reference module that holds the
pure-PyTorch path creates a lookup table with ``device="cuda"`` at import time; it is loaded from
source with that literal redirected to ``"cpu"`` in memory (nothing is written to the checkout).
The fixtures are small ``.npz`` files; the tests compare the oracle (and, on a GPU, the CUDA
kernels) against them without needing the reference again.

What the reference can and cannot produce:
  * its four tables, its scalar search ``bsearch``, its scaling helpers and its per-axis maxima
    run as they are;
  * its optimizer step ``_single_tensor_step`` runs from zero state up to the point where it stops
    itself with ``assert False, 'good'`` after storing the quantized states; by then the parameter
    update is complete, the first-moment scales and the rank-1 maxima are stored, and the codes of
    row 0 of each scaled tensor are stored one per byte (its quantize loop only visits row 0);
  * a second step cannot run (the dequantize side calls undefined names), so warm-state fixtures
    use the reference's dequantize formula ``qmap[code] * scale`` and the same torch operator
    sequence as the step (``mul_, lerp_, mul_.addcmul_, sqrt/div/add_, addcdiv_``).
"""
from __future__ import annotations

import contextlib
import io
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root: str):
    sys.path.insert(0, root)
    src = open(os.path.join(root, "optim", "adamw_fourbit_triton.py")).read().replace('device="cuda"', 'device="cpu"')
    pkg = types.ModuleType("optim")
    pkg.__path__ = [os.path.join(root, "optim")]
    sys.modules["optim"] = pkg
    mod = types.ModuleType("optim.adamw_fourbit_triton")
    mod.__package__ = "optim"
    sys.modules[mod.__name__] = mod
    exec(compile(src, "adamw_fourbit_triton.py", "exec"), mod.__dict__)
    return mod


def quiet(fn, *a, **k):
    with contextlib.redirect_stdout(io.StringIO()):
        return fn(*a, **k)


def edge_points(qmap: torch.Tensor, mid: torch.Tensor, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    up, dn = torch.tensor(2.0), torch.tensor(-2.0)
    return torch.cat([
        torch.rand(4000, generator=g) * 2.4 - 1.2,
        qmap, mid,
        torch.nextafter(mid, up), torch.nextafter(mid, dn),
        torch.nextafter(qmap, up), torch.nextafter(qmap, dn),
        torch.tensor([0.0, -0.0, 1e-30, -1e-30, float("inf"), -float("inf")]),
    ]).float()


def nd_scaling(ref) -> None:
    """The reference's second-moment scaling on tensors of more than two dimensions: one vector of maxima per axis,
    scale = the smallest of them at each element (variance_quant_scaling -> get_variance_tensor_statistics,
    compute_variance_tensor_scale), and the scale tensor its dequantize side rebuilds from them (sqs_scale_tensor)."""
    g = torch.Generator().manual_seed(5)
    out = {}
    for name, shape in (("a", (6, 20, 40)), ("b", (3, 4, 5, 16))):
        x = (torch.randn(shape, generator=g) * 1e-3) ** 2
        x[tuple(1 for _ in shape)] *= 1e4
        scaled, meta = quiet(ref.variance_quant_scaling, x.clone(), x.shape)
        assert meta["dim"] == len(shape) and meta["max1"] is None and len(meta["max_dims"]) == len(shape)
        out[f"x_{name}"] = x.numpy()
        out[f"scaled_{name}"] = scaled.numpy()
        out[f"scale_{name}"] = quiet(ref.sqs_scale_tensor, meta["max_dims"]).numpy()
        for k, mx in enumerate(meta["max_dims"]):
            out[f"max{k}_{name}"] = mx.numpy()
    np.savez(os.path.join(HERE, "scaling_nd.npz"), **out)


def created_maps(root: str) -> None:
    """The two 4-bit maps as the reference's generator makes them (optim/quant_opt_base.py:32-52: 'nonlinear' signed for
    the first moment, 'power-1' unsigned for the second), beside the literals its kernels and its PyTorch path hard-code."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("quant_opt_base", os.path.join(root, "optim", "quant_opt_base.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    np.savez(os.path.join(HERE, "qmaps_created.npz"),
             qm=mod.create_qmap("nonlinear", 4, True).numpy(), qv=mod.create_qmap("power-1", 4, False).numpy())


def main(root: str, only: str = "") -> None:
    if only == "qmaps":
        created_maps(root)
        print("wrote qmaps_created.npz")
        return
    ref = load_reference(root)
    if only == "nd":
        nd_scaling(ref)
        print("wrote scaling_nd.npz")
        return
    nd_scaling(ref)
    created_maps(root)
    np.savez(os.path.join(HERE, "tables.npz"),
             qm=ref._momentum_qmap.numpy(), mm=ref._momentum_midpoint_lut.numpy(),
             qv=ref._variance_qmap.numpy(), mv=ref._variance_midpoint_lut.numpy())

    # --- scalar search on both maps -------------------------------------------------------
    out = {}
    for name, qmap, mid, seed in (("m", ref._momentum_qmap, ref._momentum_midpoint_lut, 0),
                                  ("v", ref._variance_qmap, ref._variance_midpoint_lut, 1)):
        pts = edge_points(qmap, mid, seed)
        codes = [quiet(ref.bsearch, float(x), qmap, mid) for x in pts]
        out[f"x_{name}"] = pts.numpy()
        out[f"code_{name}"] = np.asarray(codes, dtype=np.uint8)
    np.savez(os.path.join(HERE, "search.npz"), **out)

    # --- scaling helpers ------------------------------------------------------------------
    g = torch.Generator().manual_seed(2)
    xm = torch.randn(37, 128, generator=g) * 1e-3
    xm[5, 17] *= 100
    sm, meta_m = quiet(ref.momentum_quant_scaling, xm.clone(), {})
    xv = (torch.randn(48, 200, generator=g) * 1e-3) ** 2
    sv, meta_v = quiet(ref.variance_quant_scaling, xv.clone(), xv.shape)
    row0_m = quiet(ref.kernel_quant_nonlinear, sm, ref._momentum_qmap, ref._momentum_midpoint_lut)
    row0_v = quiet(ref.kernel_quant_nonlinear, sv, ref._variance_qmap, ref._variance_midpoint_lut)
    np.savez(os.path.join(HERE, "scaling.npz"),
             xm=xm.numpy(), xm_scaled=sm.numpy(), xm_max1=meta_m["max1"].numpy(),
             xm_row0_codes=row0_m.numpy()[:128].astype(np.uint8),
             xv=xv.numpy(), xv_scaled=sv.numpy(), xv_row=meta_v["max_dims"][0].numpy(),
             xv_col=meta_v["max_dims"][1].numpy(), xv_row0_codes=row0_v.numpy()[:200].astype(np.uint8))

    # --- the reference's own optimizer step, from zero state -------------------------------
    lr, betas, eps, wd = 1e-3, (0.9, 0.999), 1e-8, 0.01
    g = torch.Generator().manual_seed(3)
    p0 = torch.randn(64, 128, generator=g) * 0.02
    grad = torch.randn(64, 128, generator=g) * 1e-3
    grad[3, 100] *= 100
    p = p0.clone()
    exp_avg, exp_avg_sq = torch.zeros(()), torch.zeros(())
    step_t = torch.tensor(0.0)
    meta_m, meta_v = {}, {}
    try:
        quiet(ref._single_tensor_step, [p], [grad], [exp_avg], [exp_avg_sq], [step_t], [meta_m], [meta_v],
              beta1=betas[0], beta2=betas[1], lr=lr, weight_decay=wd, eps=eps)
        raise SystemExit("the reference step was expected to stop itself")
    except AssertionError as e:
        assert str(e) == "good", e
    np.savez(os.path.join(HERE, "step1.npz"),
             lr=lr, beta1=betas[0], beta2=betas[1], eps=eps, wd=wd,
             p0=p0.numpy(), g=grad.numpy(), p1=p.numpy(), step=step_t.numpy(),
             m_max1=meta_m["max1"].numpy(), m_row0_codes=exp_avg.numpy()[:128].astype(np.uint8),
             v_row=meta_v["max_dims"][0].numpy(), v_col=meta_v["max_dims"][1].numpy(),
             v_row0_codes=exp_avg_sq.numpy()[:128].astype(np.uint8))

    # --- warm-state arithmetic with the step's operator sequence ---------------------------
    import math
    g = torch.Generator().manual_seed(4)
    N = 1 << 12
    p = torch.randn(N, generator=g) * 0.02
    gr = torch.randn(N, generator=g) * 1e-3
    m = torch.randn(N, generator=g) * 1e-3
    v = (torch.randn(N, generator=g) * 1e-3) ** 2
    fix = {"p0": p.numpy().copy(), "g": gr.numpy().copy(), "m0": m.numpy().copy(), "v0": v.numpy().copy(),
           "lr": lr, "beta1": betas[0], "beta2": betas[1], "eps": eps, "wd": wd, "step": 7}
    step = 7
    p.mul_(1 - lr * wd)
    m.lerp_(gr, 1 - betas[0])
    v.mul_(betas[1]).addcmul_(gr, gr, value=1 - betas[1])
    bc1, bc2 = 1 - betas[0] ** step, 1 - betas[1] ** step
    # float32 sqrt taken through float64: exact IEEE result (torch's CPU float sqrt is not correctly rounded)
    denom = (v.double().sqrt().float() / math.sqrt(bc2)).add_(eps)
    p.addcdiv_(m, denom, value=-(lr / bc1))
    fix.update(p1=p.numpy(), m1=m.numpy(), v1=v.numpy())
    np.savez(os.path.join(HERE, "adamw_arith.npz"), **fix)
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


if __name__ == "__main__":
    if len(sys.argv) not in (2, 3):
        raise SystemExit(__doc__)
    main(*sys.argv[1:])     # a second argument ("nd", "qmaps") writes that one fixture only

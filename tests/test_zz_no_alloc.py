"""The allocation-free step of one 2-D tensor (qf_step_rank1_noalloc) against the regular multi-tensor
entry point.

Some hosts of this library cannot allocate while they step -- a runtime that has given all device memory
to its own pool, or a plug-in that only passes tensors through -- so this entry point keeps its scratch in
a fixed device array inside the library.  Both entry points run the same kernels, so parameters, codes and
scales must be identical bit for bit; two calls in a row check that nothing left in the shared scratch by
the first call leaks into the second.  The file name makes pytest collect it last.
"""
import ctypes as C

import pytest
import torch

from helpers import AbiStepper, GpuState, make_grad
from oracle import torch_oracle as TO
from quantfour_adamw_cuda_b200 import _lib
from quantfour_adamw_cuda_b200.optimizer import make_hyper

pytestmark = pytest.mark.gpu

HP = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)


def _noalloc_step(p, g, st, step):
    L = _lib.lib()
    h = make_hyper(HP["lr"], HP["betas"][0], HP["betas"][1], HP["eps"], HP["weight_decay"], float(step))
    dev = p.device
    rc = L.qf_step_rank1_noalloc(p.data_ptr(), g.data_ptr(), st.m_codes.data_ptr(), st.v_codes.data_ptr(),
                                 st.m_scale.data_ptr(), st.v_row.data_ptr(), st.v_col.data_ptr(), st.shape[0], st.shape[1],
                                 {torch.float32: 0, torch.bfloat16: 1}[p.dtype], C.byref(h), dev.index,
                                 C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    _lib.check(rc, "qf_step_rank1_noalloc")


@pytest.mark.parametrize("shape,dtype", [((512, 768), torch.bfloat16), ((300, 77), torch.float32), ((64, 256), torch.float32)])
def test_noalloc_step_equals_step_multi_on_two_calls_in_a_row(shape, dtype):
    gen = torch.Generator().manual_seed(11)
    p0 = (torch.randn(shape, generator=gen) * 0.02).to(dtype)
    grads = [make_grad(shape, dtype, gen=gen).cuda() for _ in range(3)]
    # reference: the regular entry point
    pa, sa = p0.cuda(), GpuState(TO.TensorState.zeros(shape))
    stepper = AbiStepper([pa], [sa], **HP)
    # under test: the allocation-free entry point, with a different tensor shape run in between so that the
    # shared scratch holds foreign leftovers when the second call starts
    pb, sb = p0.cuda(), GpuState(TO.TensorState.zeros(shape))
    other_p = torch.zeros(96, 512, device="cuda")
    other_s = GpuState(TO.TensorState.zeros((96, 512)))
    for step, g in enumerate(grads, start=1):
        stepper.step([g])
        _noalloc_step(pb, g, sb, step)
        if step == 1:
            _noalloc_step(other_p, torch.full((96, 512), 0.5, device="cuda"), other_s, 1)
        assert torch.equal(pa, pb), f"step {step}: parameters differ"
        assert torch.equal(sa.m_codes, sb.m_codes) and torch.equal(sa.v_codes, sb.v_codes), f"step {step}: codes differ"
        assert torch.equal(sa.m_scale, sb.m_scale), f"step {step}: first-moment scales differ"
        assert torch.equal(sa.v_row, sb.v_row) and torch.equal(sa.v_col, sb.v_col), f"step {step}: maxima differ"


def test_noalloc_step_refuses_tensors_beyond_its_scratch():
    L = _lib.lib()
    h = make_hyper(1e-3, 0.9, 0.999, 1e-8, 0.01, 1.0)
    x = torch.zeros(8, device="cuda")
    big = _lib.QF_NOALLOC_MAX_ROWS_PLUS_COLS
    rc = L.qf_step_rank1_noalloc(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(),
                                 x.data_ptr(), big, 1, 0, C.byref(h), 0, None)
    assert rc == 1 and b"exceeds the built-in scratch" in L.qf_last_error()

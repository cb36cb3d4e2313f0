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
from oracle import c_oracle as CO
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


def _noalloc_status():
    word = C.c_uint32(0)
    _lib.check(_lib.lib().qf_read_status_noalloc(0, C.c_void_p(torch.cuda.current_stream().cuda_stream), C.byref(word)),
               "qf_read_status_noalloc")
    return word.value


def test_noalloc_step_matches_the_oracle_and_takes_no_device_memory():
    """Directly against the CPU oracle (not only against the other entry point), and the claim in the name: the free
    device memory the driver reports is the same before and after a call once the first call has been made."""
    shape, dtype = (256, 512), torch.bfloat16
    gen = torch.Generator().manual_seed(3)
    p = (torch.randn(shape, generator=gen) * 0.02).to(dtype)
    st = TO.TensorState.zeros(shape)
    gp, gs = p.cuda(), GpuState(st)
    for step in range(1, 4):
        g = make_grad(shape, dtype, gen=gen)
        gg = g.cuda()
        CO.step_tensor(p, g, st, HP["lr"], *HP["betas"], HP["eps"], HP["weight_decay"])
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        _noalloc_step(gp, gg, gs, step)
        torch.cuda.synchronize()
        if step > 1:   # the first call on a device may load the module that holds the built-in array
            assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.equal(gp.cpu(), p), f"step {step}: parameters differ from the oracle"
        assert not any(gs.diff(st).values()), f"step {step}: {gs.diff(st)}"
    assert _noalloc_status() == 0


def test_noalloc_status_word_is_sticky_until_read():
    shape = (64, 256)
    p, st = torch.zeros(shape, device="cuda"), GpuState(TO.TensorState.zeros(shape))
    _noalloc_status()
    g = torch.full(shape, 1e-3, device="cuda")
    g[5, 9] = float("nan")
    _noalloc_step(p, g, st, 1)
    p2, st2 = torch.zeros(shape, device="cuda"), GpuState(TO.TensorState.zeros(shape))
    _noalloc_step(p2, torch.full(shape, 1e-3, device="cuda"), st2, 1)   # a clean call in between must not clear the report
    assert _noalloc_status() & _lib.QF_STATUS_NONFINITE
    assert _noalloc_status() == 0


def test_noalloc_step_refuses_tensors_beyond_its_scratch():
    L = _lib.lib()
    h = make_hyper(1e-3, 0.9, 0.999, 1e-8, 0.01, 1.0)
    x = torch.zeros(8, device="cuda")
    big = _lib.QF_NOALLOC_MAX_ROWS_PLUS_COLS
    rc = L.qf_step_rank1_noalloc(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(),
                                 x.data_ptr(), big, 1, 0, C.byref(h), 0, None)
    assert rc == 1 and b"exceeds the built-in scratch" in L.qf_last_error()

"""CPU tests of the host side: constructor checks, state layout rules, hyper-parameter derivation,
and that the C-ABI library loads and exports every symbol the header declares."""
import ctypes as C
import os
import re

import pytest
import torch

import quantfour_adamw_cuda_b200 as qf
from oracle import torch_oracle as TO
from quantfour_adamw_cuda_b200 import _lib, build
from quantfour_adamw_cuda_b200.optimizer import state_kind

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.lib()


def test_header_symbols_are_all_exported(lib):
    header = open(os.path.join(ROOT, "include", "quantfour_b200.h")).read()
    declared = set(re.findall(r"\b(qf_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.qf_abi_version() == _lib.QF_ABI_VERSION


def test_struct_sizes_match_header(lib):
    assert C.sizeof(_lib.QfTensorDesc) == 11 * 8 + 4 * 8 + 4 * 4
    assert lib.qf_workspace_bytes(0) % 256 == 0 and lib.qf_workspace_bytes(10) > lib.qf_workspace_bytes(1)


def test_argument_errors_are_reported_without_a_gpu(lib):
    assert lib.qf_step_multi(None, 1, None, 1, None, 0, 0, None) == 1
    assert b"hypers" in lib.qf_last_error()
    assert lib.qf_fused_4bit(None, None, None, None, None, None, 10, 7, 0.9, 0.999, 1e-3, 0.0, 1e-8, 1.0, 0, None) == 1
    assert b"dtype" in lib.qf_last_error()
    assert lib.qf_quantize_block(None, -1, 0, None, None, 0, None) == 1
    with pytest.raises(ValueError):
        _lib.check(1, "x")


def test_misaligned_buffers_are_refused_before_anything_is_launched(lib):
    """The single-tensor and stand-alone entry points promise QF_ERR_BAD_ARG for buffers that are not aligned to
    their element; the addresses below are never dereferenced (the checks come before any CUDA call)."""
    A, odd = 0x10000, 0x10002   # 4-byte aligned / not
    sc = (0.9, 0.999, 1e-3, 0.0, 1e-8, 1.0)
    assert lib.qf_fused_4bit(odd, A, A, A, A, A, 256, _lib.QF_F32, *sc, 0, None) == 1 and b"aligned" in lib.qf_last_error()
    assert lib.qf_fused_4bit(A, A, A, A, odd, A, 256, _lib.QF_BF16, *sc, 0, None) == 1 and b"aligned" in lib.qf_last_error()
    assert lib.qf_fused_4bit(A + 1, A, A, A, A, A, 256, _lib.QF_BF16, *sc, 0, None) == 1
    assert lib.qf_fused_single_tensor(A, A, odd, A, 256, _lib.QF_F32, *sc, 0, None) == 1 and b"aligned" in lib.qf_last_error()
    assert lib.qf_quantize_block(odd, 256, 0, A, A, 0, None) == 1 and b"aligned" in lib.qf_last_error()
    assert lib.qf_dequantize_block(A, odd, 256, 0, A, 0, None) == 1 and b"aligned" in lib.qf_last_error()
    assert lib.qf_quantize_rank1(A, 16, 16, A, odd, A, 0, None) == 1 and b"aligned" in lib.qf_last_error()
    assert lib.qf_dequantize_rank1(A, A, odd, 16, 16, A, 0, None) == 1 and b"aligned" in lib.qf_last_error()


def test_release_of_nothing_is_not_an_error(lib):
    assert lib.qf_release_workspace(None, 0) == 0
    assert lib.qf_read_status_noalloc(0, None, None) == 1 and b"status" in lib.qf_last_error()


def test_make_hyper_matches_oracle_and_c_library(lib):
    for step in (1, 2, 3, 10, 1000, 123456):
        h = qf.make_hyper(1e-3, 0.9, 0.999, 1e-8, 0.01, float(step))
        o = TO.Hyper.make(1e-3, 0.9, 0.999, 1e-8, 0.01, step)
        c = _lib.QfHyper()
        lib.qf_make_hyper(1e-3, 0.9, 0.999, 1e-8, 0.01, float(step), C.byref(c))
        for f in ("decay", "w1", "beta2", "w2", "eps", "neg_step", "bc2s"):
            want = torch.tensor(getattr(o, f), dtype=torch.float64).float().item()
            assert getattr(h, f) == want, (step, f)
            assert getattr(c, f) == want, (step, f)


def test_constructor_validation_messages():
    p = [torch.nn.Parameter(torch.zeros(4))]
    for kw, msg in (({"lr": 0.0}, "Invalid learning rate"), ({"eps": 0.0}, "Invalid eps value"),
                    ({"betas": (1.0, 0.9)}, r"Invalid Beta\[0\]"), ({"betas": (0.9, 0.0)}, r"Invalid Beta\[1\]"),
                    ({"weight_decay": -1.0}, "Invalid weight_decay")):
        with pytest.raises(ValueError, match=msg):
            qf.FourBitAdamW(p, **kw)
    opt = qf.FourBitAdamW(p, fused=True)
    assert opt.defaults == dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, fused=True)
    assert qf.AdamWFused_QuantFour is qf.FourBitAdamW and qf.AdamW_QuantFour is qf.FourBitAdamW


def test_threshold_rule_and_kinds():
    assert not qf.enable_param_quantization(torch.zeros(4096), 4096)
    assert qf.enable_param_quantization(torch.zeros(4097), 4096)
    assert state_kind(torch.zeros(64, 64), 4096) == _lib.QF_KIND_FP32
    assert state_kind(torch.zeros(64, 65), 4096) == _lib.QF_KIND_RANK1
    assert state_kind(torch.zeros(4097), 4096) == _lib.QF_KIND_BLOCK
    assert state_kind(torch.zeros(2, 3, 1000), 4096) == _lib.QF_KIND_BLOCK


def test_state_layout_on_cpu_tensors():
    p2, p1, ps = (torch.nn.Parameter(torch.zeros(s, dtype=torch.bfloat16)) for s in ((100, 130), (5001,), (10, 10)))
    opt = qf.FourBitAdamW([p2, p1, ps])
    for p in (p2, p1, ps):
        opt._init_state(p)
    s = opt.state[p2]
    assert s["step"].device.type == "cpu" and s["step"].dtype == torch.float32 and s["step"].dim() == 0
    assert s["exp_avg"].dtype == torch.int8 and s["exp_avg"].shape == (6500,) and s["exp_avg_sq"].shape == (6500,)
    assert s["momentum_qstate"]["overhead"]["max1"].shape == (102,)
    assert [tuple(t.shape) for t in s["variance_qstate"]["overhead"]["max_dims"]] == [(100, 1), (1, 130)]
    assert set(s) == {"step", "exp_avg", "exp_avg_sq", "momentum_qstate", "variance_qstate"}
    assert set(s["momentum_qstate"]) == {"enable", "overhead", "qmap"}
    s = opt.state[p1]
    assert s["exp_avg"].shape == (2501,) and s["variance_qstate"]["overhead"]["max1"].shape == (40,)
    s = opt.state[ps]
    assert s["exp_avg"].dtype == torch.float32 and s["exp_avg"].shape == (10, 10) and not s["variance_qstate"]["enable"]


def test_load_state_dict_keeps_code_and_scale_dtypes_for_bf16_params():
    p = torch.nn.Parameter(torch.zeros(100, 130, dtype=torch.bfloat16))
    a = qf.FourBitAdamW([p])
    a._init_state(p)
    a.state[p]["exp_avg"].fill_(-3)
    a.state[p]["momentum_qstate"]["overhead"]["max1"].fill_(1.0000001)
    q = torch.nn.Parameter(torch.zeros(100, 130, dtype=torch.bfloat16))
    b = qf.FourBitAdamW([q])
    b.load_state_dict(a.state_dict())
    s = b.state[q]
    assert s["exp_avg"].dtype == torch.int8 and int(s["exp_avg"][0]) == -3
    assert s["momentum_qstate"]["overhead"]["max1"].dtype == torch.float32
    assert float(s["momentum_qstate"]["overhead"]["max1"][0]) == torch.tensor(1.0000001).item()
    assert s["variance_qstate"]["overhead"]["max_dims"][0].dtype == torch.float32
    assert s["exp_avg"].data_ptr() != a.state[p]["exp_avg"].data_ptr()


def test_step_raises_without_cuda_parameters():
    p = torch.nn.Parameter(torch.zeros(8))
    p.grad = torch.zeros(8)
    with pytest.raises(RuntimeError, match="no CPU path"):
        qf.FourBitAdamW([p]).step()
    sp = torch.nn.Parameter(torch.zeros(8, 8))
    sp.grad = torch.zeros(8, 8).to_sparse()
    with pytest.raises(RuntimeError, match="sparse"):
        qf.FourBitAdamW([sp]).step()


def test_scheduled_step_validates_its_arguments_before_touching_a_device(lib):
    descs = (_lib.QfTensorDesc * 1)()
    assert lib.qf_step_scheduled(descs, 1, 1, None, 0, 0, None, None, 4, None, 0) == 1 and b"null schedule" in lib.qf_last_error()
    A = 0x10000     # never dereferenced: the checks come before any CUDA call
    assert lib.qf_step_scheduled(descs, 1, 1, None, 0, 0, None, A, 0, A, 0) == 1 and b"at least one row" in lib.qf_last_error()
    assert lib.qf_step_scheduled(descs, 1, 1, None, 0, 0, None, A, 4, A, 8) == 1 and b"unknown flag" in lib.qf_last_error()
    assert lib.qf_step_scheduled(descs, 1, 1, None, 0, 0, None, A + 2, 4, A, 0) == 1 and b"misaligned" in lib.qf_last_error()


def test_general_step_call_validates_what_it_is_asked_to_do(lib):
    descs = (_lib.QfTensorDesc * 1)()
    hyp = (_lib.QfHyper * 1)()
    deltas = (C.c_int64 * 1)(1024)
    args = (descs, 1, hyp, 1, None, 0, 0, None)
    assert lib.qf_step_run(*args, 0, None, 0) == 1 and b"neither half" in lib.qf_last_error()
    assert lib.qf_step_run(*args, 64, None, 0) == 1 and b"unknown bits" in lib.qf_last_error()
    assert lib.qf_step_run(*args, _lib.QF_RUN_PRE, deltas, 1) == 1 and b"second half" in lib.qf_last_error()
    assert lib.qf_step_run(*args, _lib.QF_RUN_MAIN | _lib.QF_RUN_RELAXED_UPDATE, deltas, 1) == 1 and b"relaxed" in lib.qf_last_error()
    assert lib.qf_step_run(*args, _lib.QF_RUN_MAIN, None, 1) == 1 and b"peer_delta_bytes" in lib.qf_last_error()


def test_gradient_mean_validates_its_arguments_before_touching_a_device(lib):
    A = 0x10000     # never dereferenced
    d = (C.c_int64 * 2)(0, 4096)
    assert lib.qf_grad_mean_peers(A, -1, _lib.QF_BF16, d, 2, 0.5, 0, None) == 1 and b"negative" in lib.qf_last_error()
    assert lib.qf_grad_mean_peers(A, 0, _lib.QF_BF16, d, 2, 0.5, 0, None) == 0
    assert lib.qf_grad_mean_peers(None, 8, _lib.QF_BF16, d, 2, 0.5, 0, None) == 1 and b"null" in lib.qf_last_error()
    assert lib.qf_grad_mean_peers(A, 8, 7, d, 2, 0.5, 0, None) == 1 and b"dtype" in lib.qf_last_error()
    assert lib.qf_grad_mean_peers(A, 8, _lib.QF_BF16, d, 0, 0.5, 0, None) == 1 and b"n_copies" in lib.qf_last_error()
    assert lib.qf_grad_mean_peers(A, 8, _lib.QF_BF16, d, 99, 0.5, 0, None) == 1 and b"n_copies" in lib.qf_last_error()
    assert lib.qf_grad_mean_peers(A + 2, 8, _lib.QF_BF16, d, 2, 0.5, 0, None) == 1 and b"16-byte" in lib.qf_last_error()
    bad = (C.c_int64 * 2)(0, 4100)
    assert lib.qf_grad_mean_peers(A, 8, _lib.QF_BF16, bad, 2, 0.5, 0, None) == 1 and b"multiple of 16" in lib.qf_last_error()

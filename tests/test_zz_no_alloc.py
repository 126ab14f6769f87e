"""GPU: the allocation-free gated-RMSNorm backward entry point against the regular one.

Collected last on purpose (file name): a run that stops at the first failure has then already executed every other
test.  The library-owned scratch is shared by all calls and keeps its contents, so the check is made on two calls in a
row with different sizes (the second, smaller call must not see the first call's leftovers)."""
import ctypes

import pytest
import torch

from mogankda_b200 import _lib, ops
from mogankda_b200._lib import STRUCTS

pytestmark = pytest.mark.gpu


def _call_noalloc(dy, o_raw, w, gate, act, eps):
    rows = o_raw.numel() // 128
    d_o = torch.empty(rows, 128, dtype=torch.float32, device="cuda")
    dgate = torch.empty_like(gate)
    dw = torch.full((128,), float("nan"), dtype=torch.float32, device="cuda")
    p = STRUCTS["MkdaEpilogueBwdNoAlloc"]()
    p.rows = rows
    p.dy, p.dy_dtype, p.o_raw = dy.data_ptr(), ops._dt(dy), o_raw.data_ptr()
    p.norm_w, p.norm_w_dtype = w.data_ptr(), ops._dt(w)
    p.gate, p.gate_dtype, p.act, p.eps = gate.data_ptr(), ops._dt(gate), ops.ACTS[act], eps
    p.d_o, p.dgate, p.dgate_dtype, p.dweight = d_o.data_ptr(), dgate.data_ptr(), ops._dt(dgate), dw.data_ptr()
    _lib.call("mkda_epilogue_bwd_noalloc", p, torch.cuda.current_stream().cuda_stream)
    return d_o, dgate, dw


def _inputs(rows, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)                      # noqa: E731
    return (r(rows, 128).cuda(), r(rows, 128).cuda(), (1 + 0.1 * r(128)).cuda(), r(rows, 128).to(dtype).cuda())


def test_noalloc_entry_point_matches_regular_one_on_two_calls_in_a_row():
    # the third size is past 64 * MKDA_EPILOGUE_MAX_PART_ROWS rows, where a block walks more than one group of rows
    assert 64 * 1300 + 5 > 64 * _lib.MKDA_EPILOGUE_MAX_PART_ROWS and 64 * 1300 + 5 <= _lib.MKDA_NOALLOC_MAX_ROWS
    for rows, dtype, act, seed in ((64 * 300 + 17, torch.bfloat16, "silu", 1), (200, torch.float32, "sigmoid", 2),
                                   (64 * 1300 + 5, torch.bfloat16, "silu", 3)):
        dy, o_raw, w, gate = _inputs(rows, dtype, seed)
        ref_do, ref_dgate, ref_dw = ops.epilogue_bwd(dy, o_raw, w, gate, act, 1e-6)
        # the property in the name: between building the argument struct and the end of the call no device memory is
        # taken, neither from the driver nor from torch's caching allocator
        d_o = torch.empty(rows, 128, dtype=torch.float32, device="cuda")
        dgate = torch.empty_like(gate)
        dw = torch.full((128,), float("nan"), dtype=torch.float32, device="cuda")
        p = STRUCTS["MkdaEpilogueBwdNoAlloc"]()
        p.rows = rows
        p.dy, p.dy_dtype, p.o_raw = dy.data_ptr(), ops._dt(dy), o_raw.data_ptr()
        p.norm_w, p.norm_w_dtype = w.data_ptr(), ops._dt(w)
        p.gate, p.gate_dtype, p.act, p.eps = gate.data_ptr(), ops._dt(gate), ops.ACTS[act], 1e-6
        p.d_o, p.dgate, p.dgate_dtype, p.dweight = d_o.data_ptr(), dgate.data_ptr(), ops._dt(dgate), dw.data_ptr()
        stream = torch.cuda.current_stream().cuda_stream
        _lib.call("mkda_epilogue_bwd_noalloc", p, stream)          # the first call on the device may look up the scratch address
        torch.cuda.synchronize()
        free0, alloc0, reserved0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
        _lib.call("mkda_epilogue_bwd_noalloc", p, stream)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free0
        assert torch.cuda.memory_allocated() == alloc0 and torch.cuda.memory_reserved() == reserved0
        # same kernels, same summation tree: the results are expected to be identical, not merely close
        assert torch.equal(d_o, ref_do.view_as(d_o))
        assert torch.equal(dgate, ref_dgate)
        assert torch.equal(dw, ref_dw)


def test_noalloc_entry_point_rejects_sizes_beyond_its_scratch():
    lib = _lib.load()
    p = STRUCTS["MkdaEpilogueBwdNoAlloc"]()
    one = torch.zeros(128, device="cuda")
    p.rows = _lib.MKDA_NOALLOC_MAX_ROWS + 1
    for f in ("dy", "o_raw", "gate", "d_o", "dgate", "dweight"):
        setattr(p, f, one.data_ptr())
    rc = lib.mkda_epilogue_bwd_noalloc(ctypes.byref(p), None)
    assert rc == _lib.MKDA_ERR_ARG and b"exceeds the built-in scratch" in lib.mkda_last_error()
    assert str(_lib.MKDA_NOALLOC_MAX_ROWS).encode() in lib.mkda_last_error()

"""CPU: the C-ABI library builds, loads, exports every symbol include/mkda.h declares and agrees with the header on
struct layout; host-side argument checks fail loudly (no compute is launched here)."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from mogankda_b200 import build, _lib
    build.build()
    return _lib.load()


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "mkda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"^\s*(?:int|const char\*)\s+(mkda_\w+)\s*\(", text, flags=re.M)


def test_every_declared_symbol_is_exported(lib):
    names = _declared_functions()
    assert len(names) >= 17
    for n in names:
        assert hasattr(lib, n), n


def test_struct_sizes_match_header(lib):
    from mogankda_b200 import _lib
    n = len(_lib.STRUCT_ORDER)
    sizes = (ctypes.c_int * n)()
    assert lib.mkda_struct_sizes(sizes, n) == n
    for i, name in enumerate(_lib.STRUCT_ORDER):
        assert sizes[i] == ctypes.sizeof(_lib.STRUCTS[name]), name
    assert lib.mkda_abi_version() == 4


def test_null_arguments_are_rejected_without_launch(lib):
    from mogankda_b200 import _lib
    p = _lib.STRUCTS["MkdaIntraFwd"]()
    rc = lib.mkda_intra_fwd(ctypes.byref(p), None)
    assert rc == _lib.MKDA_ERR_ARG
    assert b"intra_fwd" in lib.mkda_last_error()


def test_cpu_tensors_fail_loudly():
    import mogankda_b200 as mk
    q = torch.randn(1, 64, 2, 128)
    with pytest.raises(RuntimeError, match="CUDA"):
        mk.chunk_kda(q, q, q, -torch.rand(1, 64, 2, 128), torch.rand(1, 64, 2))


def test_api_argument_errors():
    import mogankda_b200 as mk
    q = torch.randn(1, 64, 2, 128)
    with pytest.raises(AssertionError):
        mk.chunk_kda(q, q, q, -torch.rand(1, 64, 2), torch.rand(1, 64, 2))          # scalar gate into chunk_kda
    with pytest.raises(AssertionError):
        mk.chunk_gated_delta_rule(q, q, q, -torch.rand(1, 64, 2), torch.rand(1, 64, 2), head_first=True)


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "mogankda_b200")
    for fn in os.listdir(pkg):
        if fn.endswith(".py"):
            assert "oracle" not in open(os.path.join(pkg, fn)).read(), fn


def test_entry_points_reject_misaligned_tensors_without_launching():
    """The kernels use 16-byte vector accesses and bulk copies: a misaligned device address must come back as an error
    code, not as a device fault.  Checked with fake addresses on a machine without a GPU: the check precedes any launch."""
    import ctypes
    from mogankda_b200 import _lib
    lib = _lib.load()
    p = _lib.STRUCTS["MkdaL2Norm"]()
    p.x, p.dtype, p.rows, p.eps, p.rstd = 0x10004, 1, 4, 1e-6, 0x20000
    assert lib.mkda_l2norm_rstd(ctypes.byref(p), None) == -1
    assert b"16-byte aligned" in lib.mkda_last_error()
    q = _lib.STRUCTS["MkdaQkGrad"]()
    q.L.HK, q.L.HV, q.L.NC = 1, 1, 1
    for f in ("dq_v", "dk_v", "q", "k", "dq"):
        setattr(q, f, 0x30000)
    q.dk = 0x30008
    assert lib.mkda_qk_grad_finish(ctypes.byref(q), None) == -1
    assert b"16-byte aligned" in lib.mkda_last_error()

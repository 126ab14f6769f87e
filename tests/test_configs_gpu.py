"""GPU: the benchmark configurations at (or near) full size against the chunked fp64 oracle, which runs on the device
for these sizes; every gradient is compared, the parameter gradients with their "huge cancellation" included.  The
reference checks its README shape end to end in the same way (tests/test_fused_fwd_kda.py:119-138,
tests/test_kda_bwd_kernels.py:26-29)."""
import os
import sys

import pytest
import torch

import mogankda_b200 as mk
from mogankda_b200 import _lib, ops
from mogankda_b200.index import get_layout
from oracle import kda_oracle as orc
from tests.common import check

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench  # noqa: E402

pytestmark = pytest.mark.gpu


def _both(dev, opts, gdn=False, want_ht=True, extra=None):
    """Runs the CUDA path and the oracle on the same device tensors; returns two dicts name -> tensor."""
    out = []
    for f64 in (False, True):
        lv = {n: ((x.double() if f64 else x).detach().clone().requires_grad_(True)
                  if n in bench.GRAD_LEAVES and x.is_floating_point() else x) for n, x in dev.items()}
        if gdn:
            fn = orc.chunked_delta_rule if f64 else mk.chunk_gated_delta_rule
            o, ht = fn(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], initial_state=lv["h0"], output_final_state=True,
                       state_v_first=True)
        else:
            fn = orc.chunked_delta_rule if f64 else mk.chunk_kda
            norm = dict(weight=lv["ep_w"], gate=lv["ep_gate"], act=opts["epi"], eps=1e-6) if opts["epi"] else None
            o, ht = fn(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], cu_seqlens=lv.get("cu"), gate_mode=opts["gate_mode"],
                       A_log=lv.get("A_log"), dt_bias=lv.get("dt_bias"), lower_bound=opts["lower_bound"],
                       beta_mode=opts["beta_mode"], beta_scale=opts["beta_scale"], use_qk_l2norm_in_kernel=opts["l2"],
                       output_norm=norm, output_final_state=want_ht, **(extra or {}))
        loss = o.double().sum() + (ht.double().sum() if ht is not None else 0.0)
        loss.backward()
        res = dict(o=o.detach(), ht=None if ht is None else ht.detach())
        res.update({"d" + n: t.grad for n, t in lv.items() if torch.is_tensor(t) and t.requires_grad})
        out.append(res)
    return out


def _compare(got, ref):
    for n, r in ref.items():
        if r is not None:
            check(n, got[n], r)


def test_config2_1b_shape_every_gradient():
    """T = 8192, HK8 / HV16, documents 3000 / 2000 / 3192, eda gate, sigmoid beta x 2, in-kernel L2, silu epilogue."""
    host, opts, _, _ = bench.make_workload("1b", 0, "cuda")
    dev = {n: x.cuda() for n, x in host.items()}
    got, ref = _both(dev, opts)
    assert {"dA_log", "ddt_bias", "dep_w", "dep_gate", "dq", "dk", "dv", "dg", "dbeta"} <= set(ref)
    _compare(got, ref)


def test_config4_long_document_against_the_oracle():
    """One kimi-gate document of 16 384 tokens at HK16 / HV32: the chooser cuts it into concurrent segments (state +
    transition pre-pass, prefix combine); the result is compared with the oracle, not with the uncut CUDA run."""
    host, opts, _, _ = bench.make_workload("longdoc", 0, "cuda", tokens=16384)
    dev = {n: x.cuda() for n, x in host.items()}
    assert get_layout(1, 16384, None, dev["q"].device, 32, bench.HV).segmented
    got, ref = _both(dev, opts)
    _compare(got, ref)


def test_config5_scalar_gate_with_vk_initial_state():
    """chunk_gated_delta_rule, one batch row of config 5 (T = 16 384, H = 16), fp32 initial state in [V, K] layout,
    final state on."""
    host, opts, _, _ = bench.make_workload("gdn", 0, "cuda")
    dev = {n: (x[:1].contiguous() if x.dim() >= 3 else x).cuda() for n, x in host.items()}
    got, ref = _both(dev, opts, gdn=True)
    _compare(got, ref)


def test_packed_sub_batch_parameter_gradients():
    """Eight documents (up to ~1500 tokens) cut out of the 64k packed batch, as a packed batch of their own at HK16 / HV32:
    every result against the oracle, the parameter gradients (sums over all tokens) included."""
    host, opts, _, _ = bench.make_workload("packed", 0, "cuda")
    cu = host["cu"].tolist()
    lens = [cu[i + 1] - cu[i] for i in range(len(cu) - 1)]
    order = sorted(range(len(lens)), key=lambda i: abs(lens[i] - 1500))
    picks = sorted(order[:2] + list(range(3, 9)))
    pieces = [(cu[i], cu[i + 1]) for i in picks]
    T = sum(e - s for s, e in pieces)
    dev = {}
    for n, x in host.items():
        if n == "cu":
            acc = [0]
            for s, e in pieces:
                acc.append(acc[-1] + e - s)
            dev[n] = torch.tensor(acc, dtype=torch.int32, device="cuda")
        elif x.dim() >= 3:
            dev[n] = torch.cat([x[:, s:e] for s, e in pieces], 1).contiguous().cuda()
        else:
            dev[n] = x.cuda()
    assert dev["q"].shape[1] == T and max(e - s for s, e in pieces) > 1000
    got, ref = _both(dev, opts)
    _compare(got, ref)


def test_precomputed_gate_is_a_plain_cumsum_bit_for_bit():
    """gate_mode="precomputed" must not touch the values: the kernel's output equals the chunk-local running sum times
    1/ln 2 evaluated in fp32 in the kernel's order (16-row groups: running sum inside a group plus the totals of the
    earlier groups, in order), bit for bit (the reference pins the same property, tests/test_kda_gate.py:101-111)."""
    g = torch.Generator().manual_seed(9)
    B, T, HV = 2, 320, 4
    x = (-5.0 * torch.rand(B, T, HV, 128, generator=g)).cuda()
    lay = get_layout(B, T, None, x.device)
    g_c, _ = ops.gate_cumsum_fwd(lay, x, "precomputed", None, None, None, HV)
    xs = x.view(B, T // 64, 4, 16, HV, 128)
    run = torch.empty_like(xs)
    acc = torch.zeros_like(xs[:, :, :, 0])
    for r in range(16):
        acc = acc + xs[:, :, :, r]
        run[:, :, :, r] = acc
    pre = torch.zeros_like(acc[:, :, 0])
    out = torch.empty_like(xs)
    for w in range(4):
        out[:, :, w] = (pre[:, :, None] + run[:, :, w]) * torch.tensor(1.4426950408889634, dtype=torch.float32, device="cuda")
        pre = pre + run[:, :, w, 15]
    assert torch.equal(g_c.view_as(out), out)


def test_a_wait_that_cannot_complete_expires_and_leaves_the_device_usable():
    """Failure detection on the device without a fault: a kernel whose only wait is on a barrier nothing arrives on gives
    up after the short limit passed in, reports it in its own status word, frees its tensor memory and returns; the next
    kernel runs normally and the process-wide status stays clean."""
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    p = _lib.STRUCTS["MkdaSelfTestWait"]()
    p.limit_cycles, p.status = 1 << 20, status.data_ptr()          # about half a millisecond
    _lib.call("mkda_selftest_wait", p, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert status.tolist() == [1, 0]
    A, Bm = torch.randn(128, 64, device="cuda"), torch.randn(64, 64, device="cuda")
    D = torch.zeros(128, 64, device="cuda")
    q = _lib.STRUCTS["MkdaSelfTest"]()
    q.A, q.B, q.D, q.N, q.K, q.mode = A.data_ptr(), Bm.data_ptr(), D.data_ptr(), 64, 64, 0
    _lib.call("mkda_selftest_umma", q, torch.cuda.current_stream().cuda_stream)
    ref = A.double() @ Bm.double().T
    assert ((D.double() - ref).abs().max() / ref.abs().max()).item() < 5e-5
    assert mk.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_scalar_gate_accepts_any_decay(dtype):
    """chunk_gated_delta_rule has no lower bound on the per-token decay (the reference's scalar kernels form
    exp(g_i - g_j) for i >= j only, mogan_kda/ops/gated_delta_rule/chunk/blackwell/fused_fwd.py:425-445).  Decays of -20 and
    -40 per token, next to mild ones, must neither overflow nor lose the entries that matter: every result against the oracle."""
    from tests.common import make_inputs, run
    lv, do, dht, opts, _ = make_inputs(B=2, T=300, HK=2, HV=4, dtype=dtype, gate="precomputed", scalar=True, beta="precomputed",
                                       l2=False, epi=None, h0=True, seed=77)
    g = torch.Generator().manual_seed(78)
    mild = -0.3 * torch.rand(2, 300, 4, generator=g)
    strong = torch.where(torch.rand(2, 300, 4, generator=g) < 0.15, -20.0 - 20.0 * torch.rand(2, 300, 4, generator=g), mild)
    lv["g"] = strong.cuda()
    opts = dict(opts, lower_bound=None)
    got = run(mk.chunk_delta_rule, lv, do, dht, opts, None)
    ref = run(orc.chunked_delta_rule, lv, do, dht, opts, None, f64=True)
    for n, r in ref.items():
        check(n, got[n], r)

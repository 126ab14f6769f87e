"""GPU: the benchmark-size workloads through size-independent properties (the fp64 oracle cannot run at 65 536 tokens
x 32 heads): exact repeatability, documents of a packed batch equal to the same documents run alone (bitwise),
linearity of the forward in v, and oracle parity on a sample of whole documents cut out of the batch."""
import sys
import os

import pytest
import torch

import mogankda_b200 as mk
from oracle import kda_oracle as orc
from tests.common import check

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench  # noqa: E402

pytestmark = pytest.mark.gpu


def _step(dev, opts, v=None):
    lv = {n: (x.detach().clone().requires_grad_(True) if n in bench.GRAD_LEAVES and x.is_floating_point() else x)
          for n, x in dev.items()}
    if v is not None:
        lv["v"] = v.requires_grad_(True)
    norm = dict(weight=lv["ep_w"], gate=lv["ep_gate"], act=opts["epi"], eps=1e-6) if opts["epi"] else None
    o, ht = mk.chunk_kda(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], cu_seqlens=lv.get("cu"), gate_mode=opts["gate_mode"],
                         A_log=lv.get("A_log"), dt_bias=lv.get("dt_bias"), lower_bound=opts["lower_bound"],
                         beta_mode=opts["beta_mode"], beta_scale=opts["beta_scale"], use_qk_l2norm_in_kernel=opts["l2"],
                         output_norm=norm, output_final_state=True)
    return lv, o, ht


@pytest.fixture(scope="module")
def packed():
    host, opts, desc, dims = bench.make_workload("packed", 0, "cuda")
    return {n: x.cuda() for n, x in host.items()}, opts


def test_packed_64k_step_is_repeatable_and_finite(packed):
    dev, opts = packed
    outs = []
    for _ in range(6):       # several runs: a copy that is read before it has landed shows up only now and then
        lv, o, ht = _step(dev, opts)
        o.sum().backward()
        outs.append((o.detach(), ht.detach()) + tuple(lv[n].grad for n in ("q", "k", "v", "g", "beta", "A_log", "dt_bias", "ep_w", "ep_gate")))
    for a in outs[0]:
        assert torch.isfinite(a.float()).all()
    for other in outs[1:]:
        for a, b in zip(outs[0], other):
            assert torch.equal(a, b)


def test_packed_documents_match_standalone_runs_and_the_oracle(packed):
    dev, opts = packed
    lv, o, ht = _step(dev, opts)
    o.sum().backward()
    cu = dev["cu"].tolist()
    lens = [cu[i + 1] - cu[i] for i in range(len(cu) - 1)]
    picks = sorted(range(len(lens)), key=lambda i: lens[i])
    picks = [picks[0], picks[len(picks) // 3], picks[-1] if lens[picks[-1]] <= 1500 else picks[len(picks) // 2]]
    for n in picks:
        s, e = cu[n], cu[n + 1]
        sub = {k: (t[:, s:e].contiguous() if t.dim() >= 3 and t.shape[0] == 1 and t.shape[1] == cu[-1] else t) for k, t in dev.items()}
        sub.pop("cu")
        lv1, o1, ht1 = _step(sub, opts)
        o1.sum().backward()
        assert torch.equal(o1, o[:, s:e]) and torch.equal(ht1, ht[n:n + 1])
        for name in ("q", "k", "v", "g", "beta", "ep_gate"):
            assert torch.equal(lv1[name].grad, lv[name].grad[:, s:e]), name
        if e - s <= 1500:       # oracle parity on the whole document (HK16 / HV32 / D128)
            x = {k: t.double().clone().requires_grad_(True) if t.is_floating_point() else t for k, t in sub.items()}
            oo, _ = orc.chunked_delta_rule(x["q"], x["k"], x["v"], x["g"], x["beta"], gate_mode=opts["gate_mode"], A_log=x["A_log"],
                                           dt_bias=x["dt_bias"], beta_mode=opts["beta_mode"], beta_scale=opts["beta_scale"],
                                           use_qk_l2norm_in_kernel=True, output_final_state=True,
                                           output_norm=dict(weight=x["ep_w"], gate=x["ep_gate"], act=opts["epi"]))
            oo.sum().backward()
            check("o", o1, oo)
            check("dq", lv1["q"].grad, x["q"].grad)
            check("dg", lv1["g"].grad, x["g"].grad)
            check("dv", lv1["v"].grad, x["v"].grad)


def test_forward_without_epilogue_is_linear_in_v(packed):
    """o(v1 + v2) = o(v1) + o(v2) when the initial state is zero (the delta rule is linear in v); checked at full size."""
    dev, opts = packed
    noep = dict(opts, epi=None)
    dev = dict(dev, q=dev["q"].float(), k=dev["k"].float())               # all-fp32 path: no output quantisation
    g = torch.Generator(device="cuda").manual_seed(5)
    v1 = dev["v"].float()
    v2 = torch.randn(v1.shape, device="cuda", generator=g)
    f = lambda v: _step(dev, noep, v.clone())[1].float()                  # noqa: E731
    lhs, rhs = f(v1 + v2), f(v1) + f(v2)
    mx, mn = orc.rel_err(lhs, rhs)
    assert mx < 2e-3 and mn < 2e-3, (mx, mn)


def test_long_document_64k_segmented_equals_unsegmented():
    host, opts, desc, dims = bench.make_workload("longdoc", 0, "cuda")
    dev = {n: x.cuda()[:, :16384].contiguous() if x.dim() >= 3 else x.cuda() for n, x in host.items()}
    res = []
    for auto in (True, False):
        lv = {n: x.detach().clone().requires_grad_(True) for n, x in dev.items()}
        o, ht = mk.chunk_kda(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], gate_mode="kimi", A_log=lv["A_log"], dt_bias=lv["dt_bias"],
                             beta_mode="sigmoid", use_qk_l2norm_in_kernel=True, output_final_state=True, auto_cp=auto)
        (o.float().sum() + ht.sum()).backward()
        res.append((o.float(), ht, lv["v"].grad.float(), lv["g"].grad))
    for name, a, b in zip(("o", "ht", "dv", "dg"), *res):
        mx, mn = orc.rel_err(a, b)
        assert mx < 2e-3 + 2.0 ** -8 and mn < 2e-3 + 1.6e-3, (name, mx, mn)

"""Warm-up truncation of the segment pre-passes (``MkdaWarmup`` in include/mkda.h; the reference's get_warmup_chunks,
mogan_kda/ops/gated_delta_rule/chunk/blackwell/cp_fwd.py:81-115): the table against a restatement in torch, the truncated
result against the exact fp64 oracle, and no effect at all where the decay never reaches the threshold."""
import math

import pytest
import torch

import mogankda_b200 as mk
from mogankda_b200 import ops
from mogankda_b200.index import get_layout
from oracle import kda_oracle as orc
from tests.common import compare, make_inputs, run

pytestmark = pytest.mark.gpu


def _table(seg_off, gl, thr_log2):
    """warm_start / warm_end per (segment, head) from gl [NC,HV,128], chunk by chunk as the header defines them."""
    NS, HV = len(seg_off) - 1, gl.shape[1]
    lg = torch.log2(gl.double())
    ws = torch.empty(NS, HV, dtype=torch.int32)
    we = torch.empty(NS, HV, dtype=torch.int32)
    for s in range(NS):
        a, b = seg_off[s], seg_off[s + 1]
        for h in range(HV):
            ws[s, h], acc = a, torch.zeros(128, dtype=torch.float64)
            for c in range(b - 1, a, -1):
                acc = acc + lg[c, h].cpu()
                if acc.max() < thr_log2:
                    ws[s, h] = c
                    break
            we[s, h], acc = b, torch.zeros(128, dtype=torch.float64)
            for c in range(a, b - 1):
                acc = acc + lg[c, h].cpu()
                if acc.max() < thr_log2:
                    we[s, h] = c + 1
                    break
    return ws, we


def test_warmup_table_matches_the_restatement():
    torch.manual_seed(3)
    HV, T = 3, 64 * 37 + 20
    lay = get_layout(1, T, None, torch.device("cuda"), 8, 0)          # segments of 8 chunks, the last one shorter
    assert lay.NS == 5 and lay.NC == 38
    # per-chunk decays of very different strength: head 0 never reaches the threshold inside a segment, head 1 after a
    # few chunks, head 2 within one chunk; one channel of head 1 decays slowly in some chunks; some factors underflowed
    expo = torch.rand(lay.NC, HV, 128) * torch.tensor([0.05, 6.0, 40.0]).view(1, 3, 1)
    expo[::3, 1, 17] = 0.01
    gl = torch.exp2(-expo)
    gl[5, 2, :] = 0.0
    gl[20, 1, 3] = 0.0
    gl = gl.cuda()
    thr = -10.0
    ws, we = ops.warmup_chunks(lay, gl, 1, HV, thr)
    rws, rwe = _table(lay.host["seg_chunk_off"], gl.cpu(), thr * math.log2(math.e))
    assert torch.equal(ws.cpu(), rws) and torch.equal(we.cpu(), rwe)
    off = torch.tensor(lay.host["seg_chunk_off"])
    assert (ws[:, 0].cpu() == off[:-1]).all() and (we[:, 0].cpu() == off[1:]).all()      # head 0: nothing skipped
    assert (ws[:4, 2].cpu() > off[:4]).all() and (we[:4, 2].cpu() < off[1:5]).all()      # head 2: truncated in every full segment


def test_truncated_prepass_stays_within_tolerance_of_the_exact_oracle():
    """38 chunks = two segments; the eda gate of the generator decays by far more than e^-10 per segment, so the state +
    transition pre-pass visits a few chunks only.  Everything, gradients included, against the exact oracle."""
    lv, do, dht, opts, epi = make_inputs(B=1, T=2048 + 64 * 5 + 7, dtype=torch.float32, gate="eda", seed=13, HV=2)
    cut = run(mk.chunk_delta_rule, lv, do, dht, opts, epi, vfirst=True, warmup_threshold=-10.0)
    ref = run(orc.chunked_delta_rule, lv, do, dht, opts, epi, f64=True, vfirst=True)
    compare(cut, ref)
    exact = run(mk.chunk_delta_rule, lv, do, dht, opts, epi, vfirst=True)
    assert torch.equal(cut["o"][:, :2048], exact["o"][:, :2048])       # the first segment starts from the given state either way
    d = (cut["ht"] - exact["ht"]).abs().max() / exact["ht"].abs().max()
    assert d < 1e-4, f"truncation moved the final state by {d:.2e}"
    with pytest.raises(ValueError):
        mk.chunk_delta_rule(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], warmup_threshold=1.0)


def test_truncation_changes_nothing_where_the_decay_is_weak():
    """Per-token decay of 1e-4: 2048 tokens accumulate -0.2, far above the threshold; every result is bitwise the exact one."""
    lv, do, dht, opts, epi = make_inputs(B=1, T=2048 + 64 * 5 + 7, dtype=torch.float32, gate="precomputed", seed=14, HV=2)
    lv["g"] = torch.full_like(lv["g"], -1e-4)
    exact = run(mk.chunk_delta_rule, lv, do, dht, opts, epi, vfirst=True)
    cut = run(mk.chunk_delta_rule, lv, do, dht, opts, epi, vfirst=True, warmup_threshold=-10.0)
    for n, t in exact.items():
        assert torch.equal(t, cut[n]), n

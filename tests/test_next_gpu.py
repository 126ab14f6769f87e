"""GPU: the rows next to the hot path -- FLA-style call surface, forward-only prefill with state hand-off, and the
segment chooser on a skewed packed batch."""
import pytest
import torch

import mogankda_b200 as mk
from mogankda_b200 import fla_compat
from mogankda_b200.index import get_layout
from oracle import kda_oracle as orc
from tests.common import check, make_inputs, run

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", ["precomputed", "kimi", "gdn"])
def test_fla_style_surface_matches_the_oracle(case):
    """Keyword mapping of the reference's compatibility wrapper (tests/ref_kda.py:189-218)."""
    gate = case
    lv, do, dht, opts, _ = make_inputs(T=200, gate=gate, beta="sigmoid", l2=True, epi=None, dtype=torch.bfloat16)
    fla_kw = dict(use_qk_l2norm_in_kernel=True, use_beta_sigmoid_in_kernel=True, allow_neg_eigval=True,
                  initial_state=lv["h0"], output_final_state=True, safe_gate=True, chunk_size=64)
    if gate != "precomputed":
        fla_kw.update(use_gate_in_kernel=True, A_log=lv["A_log"], dt_bias=lv["dt_bias"])
    if gate == "kimi":
        fla_kw["lower_bound"] = -5.0
    o, ht = fla_compat.chunk_kda(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], **fla_kw)
    ref = run(orc.recurrent_delta_rule, lv, do, dht, opts, None, f64=True, grads=False)
    check("o", o, ref["o"])
    check("ht", ht, ref["ht"])
    with pytest.raises(NotImplementedError):
        fla_compat.chunk_kda(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], use_graph=True)


def test_prefill_in_two_calls_hands_the_state_over():
    """Forward-only prefill: final_state of one call is the initial_state of the next.  Split at a chunk boundary the
    two calls walk exactly the chunks of the single call, so the results are bitwise equal."""
    lv, do, dht, opts, _ = make_inputs(T=384, gate="kimi", epi=None, dtype=torch.bfloat16, h0=True)
    kw = dict(opts, A_log=lv["A_log"], dt_bias=lv["dt_bias"])
    with torch.no_grad():
        o_all, ht_all = mk.chunk_kda(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], initial_state=lv["h0"], **kw)
        cut = 192
        part = lambda t, a, b: t[:, a:b].contiguous()                 # noqa: E731
        o1, h1 = mk.chunk_kda(*(part(lv[n], 0, cut) for n in ("q", "k", "v", "g", "beta")), initial_state=lv["h0"], **kw)
        o2, h2 = mk.chunk_kda(*(part(lv[n], cut, 384) for n in ("q", "k", "v", "g", "beta")), initial_state=h1, **kw)
    assert torch.equal(torch.cat([o1, o2], 1), o_all)
    assert torch.equal(h2, ht_all)
    # an unaligned cut changes the chunking of the second part: equal to tolerance, not bitwise
    with torch.no_grad():
        cut = 100
        o1, h1 = mk.chunk_kda(*(part(lv[n], 0, cut) for n in ("q", "k", "v", "g", "beta")), initial_state=lv["h0"], **kw)
        o2, h2 = mk.chunk_kda(*(part(lv[n], cut, 384) for n in ("q", "k", "v", "g", "beta")), initial_state=h1, **kw)
    check("o (unaligned cut)", torch.cat([o1, o2], 1), o_all.float())       # both sides carry a bf16 rounding
    check("ht (unaligned cut)", h2, ht_all)


def test_chooser_cuts_a_skewed_packed_batch_and_results_agree():
    """One long document among short ones: the chooser segments the batch (index.wants_segments); the result agrees
    with the uncut run (auto_cp=False) to the usual tolerance and, per document, with the oracle on a short one."""
    HV, T = 4, 64 * 80
    cu = [0, 64 * 70] + [64 * 70 + 16 * i for i in range(1, 41)]            # 70-chunk document + 40 x 16 tokens
    lv, do, dht, opts, _ = make_inputs(T=T, HV=HV, cu=cu, gate="eda", epi=None, dtype=torch.bfloat16, h0=True)
    cu_t = opts["cu_seqlens"]
    lay = get_layout(1, T, cu_t, "cuda", 32, HV)
    assert lay.segmented, "the 70-chunk document should be cut"
    a = run(mk.chunk_kda, lv, do, dht, opts, None)
    b = run(mk.chunk_kda, lv, do, dht, opts, None, auto_cp=False)
    for n in a:
        check(n, a[n], b[n].float())                                         # 16-bit results: both sides are rounded
    # ... and, per document, with the oracle: the long (segmented) document and one short one, each run on its own
    for d in (0, 7):
        s, e = cu[d], cu[d + 1]
        sub = {n: (t[:, s:e].contiguous() if t.dim() >= 3 and t.shape[1] == T else t) for n, t in lv.items()}
        sub["h0"] = lv["h0"][d:d + 1]
        o1 = dict(opts, cu_seqlens=None)
        ref = run(orc.chunked_delta_rule, sub, do[:, s:e], dht[d:d + 1], o1, None, f64=True)
        check(f"o[doc {d}]", a["o"][:, s:e], ref["o"])
        check(f"ht[doc {d}]", a["ht"][d:d + 1], ref["ht"])
        for n in ("dq", "dk", "dv", "dg", "dbeta"):
            check(f"{n}[doc {d}]", a[n][:, s:e], ref[n])
        check(f"dh0[doc {d}]", a["dh0"][d:d + 1], ref["dh0"])


def test_api_errors_follow_the_reference_conventions():
    """ValueError for API misuse, assert for dtype / shape (mogan_kda/ops/kimi_delta_rule/chunk/__init__.py:44-56,
    mogan_kda/ops/gated_delta_rule/chunk/__init__.py:425-439)."""
    lv, do, dht, opts, _ = make_inputs(B=2, T=64, gate="precomputed", beta="precomputed", epi=None, l2=False, h0=True)
    args = (lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"])
    cu = torch.tensor([0, 64], dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="batch size"):
        mk.chunk_kda(*args, cu_seqlens=cu)                                   # varlen needs B == 1
    with pytest.raises(ValueError, match="initial states"):
        mk.chunk_kda(*args, initial_state=lv["h0"][:1])                      # one state per sequence
    with pytest.raises(ValueError, match="gate_mode"):
        mk.chunk_kda(*args, gate_mode="nope")
    with pytest.raises(AssertionError):
        mk.chunk_kda(*args, initial_state=lv["h0"].half())                   # states are float32
    with pytest.raises(AssertionError):
        mk.chunk_kda(lv["q"], lv["k"], lv["v"], lv["g"][..., 0], lv["beta"])  # chunk_kda wants a per-channel gate
    with pytest.raises(AssertionError):
        mk.chunk_gated_delta_rule(*args)                                     # ... and the scalar entry point a scalar one
    with pytest.raises(AssertionError):
        mk.chunk_delta_rule(*args, gate_mode="eda")                          # eda needs A_log

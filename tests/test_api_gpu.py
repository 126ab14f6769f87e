"""GPU: the public API (which calls the C-ABI kernels) against the fp64 oracle and the reference-generated fixtures.
Mirrors the reference's option-matrix / invariance tests (tests/test_kda_unit.py:79-289)."""
import os

import pytest
import torch

import mogankda_b200 as mk
from oracle import kda_oracle as orc
from tests.common import VARLEN_CU, check, compare, make_inputs, run

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_config1_against_reference_fixture():
    """Benchmark config 1 (T=256, HK2/HV4, fp32, precomputed gate): outputs and gradients produced by the reference's
    own tests/ref_kda.py are stored in the fixture."""
    fx = torch.load(os.path.join(GOLD, "ref_config1.pt"))
    lv = {n: t.cuda().requires_grad_(True) for n, t in fx["inputs"].items()}
    o, ht = mk.chunk_kda(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], output_final_state=True)
    grads = torch.autograd.grad(o.sum(), list(lv.values()))
    check("o", o, fx["o"])
    check("ht", ht, fx["ht"])
    for n, gr in zip(lv, grads):
        check("d" + n, gr, fx["grads"][n])


MATRIX = [
    dict(gate="eda", cu=VARLEN_CU, T=704, dtype=torch.float32, HV=4, vfirst=True, epi="silu", h0=True),
    dict(gate="eda", B=2, T=300, dtype=torch.bfloat16, HV=4, vfirst=False, epi="silu", h0=False),
    dict(gate="kimi", cu=VARLEN_CU, T=704, dtype=torch.bfloat16, HV=2, vfirst=False, epi="sigmoid", h0=True),
    dict(gate="kimi", B=2, T=300, dtype=torch.float32, HV=4, vfirst=True, epi=None, h0=True, l2=False),
    dict(gate="gdn", cu=VARLEN_CU, T=704, dtype=torch.float32, HV=2, vfirst=False, epi=None, h0=False, beta="precomputed"),
    dict(gate="gdn", B=2, T=300, dtype=torch.bfloat16, HV=4, vfirst=True, epi="silu", h0=True, x_dtype=torch.bfloat16),
    dict(gate="precomputed", cu=VARLEN_CU, T=704, dtype=torch.bfloat16, HV=4, vfirst=True, epi=None, h0=True, l2=False,
         beta="precomputed"),
    dict(gate="precomputed", B=2, T=300, dtype=torch.float32, HV=2, vfirst=False, epi="sigmoid", h0=False),
    dict(gate="gdn", scalar=True, cu=VARLEN_CU, T=704, dtype=torch.bfloat16, HV=4, vfirst=True, epi=None, h0=True),
    dict(gate="precomputed", scalar=True, B=2, T=300, dtype=torch.float16, HV=2, vfirst=False, epi=None, h0=True,
         beta="precomputed"),
    dict(gate="eda", scalar=True, B=1, T=200, dtype=torch.float32, HV=4, vfirst=False, epi="silu", h0=False),
]


@pytest.mark.parametrize("case", MATRIX, ids=lambda c: f"{c['gate']}{'-scalar' if c.get('scalar') else ''}-{str(c['dtype'])[6:]}-{'varlen' if c.get('cu') else 'dense'}")
def test_option_matrix(case):
    case = dict(case)
    vfirst = case.pop("vfirst")
    lv, do, dht, opts, epi = make_inputs(seed=len(str(case)), **case)
    got = run(mk.chunk_delta_rule, lv, do, dht, opts, epi, vfirst=vfirst)
    ref = run(orc.chunked_delta_rule, lv, do, dht, opts, epi, f64=True, vfirst=vfirst)
    compare(got, ref)


def _all_pairs_cover():
    """A small set of option combinations in which every pair of values of two different options occurs at least once:
    greedy cover over seeded random candidates (the reference builds its matrix the same way, tests/kda_common.py:73-94)."""
    import itertools
    import random
    factors = dict(gate=["eda", "kimi", "gdn", "precomputed"], scalar=[False, True], beta=["sigmoid", "precomputed"],
                   HV=[2, 4], vfirst=[False, True], l2=[True, False], epi=[None, "silu", "sigmoid"], h0=[True, False],
                   dtype=[torch.bfloat16, torch.float32, torch.float16], varlen=[False, True])
    names = list(factors)
    todo = {((a, va), (b, vb)) for a, b in itertools.combinations(names, 2) for va in factors[a] for vb in factors[b]}
    rng, cases = random.Random(1234), []
    while todo:
        best, gain = None, -1
        for _ in range(200):
            cand = {n: rng.choice(v) for n, v in factors.items()}
            g = sum(1 for (a, va), (b, vb) in todo if cand[a] == va and cand[b] == vb)
            if g > gain:
                best, gain = cand, g
        todo = {p for p in todo if not (best[p[0][0]] == p[0][1] and best[p[1][0]] == p[1][1])}
        cases.append(best)
    return cases


def _cover_id(c):
    return "-".join(str(v).replace("torch.", "") for v in c.values())


@pytest.mark.parametrize("case", _all_pairs_cover(), ids=_cover_id)
def test_option_pairs_cover(case):
    case = dict(case)
    vfirst, varlen = case.pop("vfirst"), case.pop("varlen")
    kw = dict(cu=VARLEN_CU, T=704) if varlen else dict(B=2, T=200)
    lv, do, dht, opts, epi = make_inputs(seed=sum(map(ord, _cover_id(case))), **kw, **case)
    got = run(mk.chunk_delta_rule, lv, do, dht, opts, epi, vfirst=vfirst)
    ref = run(orc.chunked_delta_rule, lv, do, dht, opts, epi, f64=True, vfirst=vfirst)
    compare(got, ref)


@pytest.mark.parametrize("P", [1, 15, 17, 63, 77, 193])
def test_prefix_invariance_is_bitwise(P):
    """Outputs of the first P tokens, and (with dO = 0 from row P on) the token gradients of those rows, do not change
    by a single bit when the later tokens are removed (tests/test_kda_unit.py:102-137)."""
    lv, do, dht, opts, epi = make_inputs(B=2, T=300, dtype=torch.bfloat16, gate="eda", seed=3)
    opts = dict(opts, output_final_state=False)
    do = do.clone()
    do[:, P:] = 0

    def go(n):
        cut = {k: (t[:, :n].contiguous() if t.dim() >= 3 and t.shape[1] == 300 else t) for k, t in lv.items()}
        leaves = {k: t.clone().requires_grad_(True) for k, t in cut.items()}
        o, _ = mk.chunk_delta_rule(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"],
                                   A_log=leaves["A_log"], dt_bias=leaves["dt_bias"], initial_state=leaves["h0"],
                                   output_norm=dict(weight=leaves["ep_w"], gate=leaves["ep_gate"], act=epi), **opts)
        names = ("q", "k", "v", "g", "beta", "ep_gate")
        grads = torch.autograd.grad((o.double() * do[:, :n].double()).sum(), [leaves[x] for x in names])
        return o, dict(zip(names, grads))

    o_full, g_full = go(300)
    o_cut, g_cut = go(P)
    assert torch.equal(o_full[:, :P], o_cut)
    for n in g_cut:
        assert torch.equal(g_full[n][:, :P], g_cut[n]), n


def test_varlen_equals_per_document_bitwise():
    lv, do, dht, opts, epi = make_inputs(cu=VARLEN_CU, T=704, dtype=torch.bfloat16, gate="kimi", seed=5)
    full = run(mk.chunk_delta_rule, lv, do, dht, opts, epi)
    for n in range(len(VARLEN_CU) - 1):
        s, e = VARLEN_CU[n], VARLEN_CU[n + 1]
        part = {k: (t[:, s:e].contiguous() if t.dim() >= 3 and t.shape[1] == 704 else (t[n:n + 1] if k == "h0" else t))
                for k, t in lv.items()}
        one = run(mk.chunk_delta_rule, part, do[:, s:e], dht[n:n + 1], dict(opts, cu_seqlens=None), epi)
        assert torch.equal(one["o"], full["o"][:, s:e])
        assert torch.equal(one["ht"], full["ht"][n:n + 1])
        for name in ("dq", "dk", "dv", "dg", "dbeta", "dep_gate"):
            assert torch.equal(one[name], full[name][:, s:e]), name
        assert torch.equal(one["dh0"], full["dh0"][n:n + 1])


def test_gva_equals_expanded_heads():
    lv, do, dht, opts, epi = make_inputs(B=2, T=200, HK=2, HV=4, dtype=torch.float32, gate="eda", seed=6)
    got = run(mk.chunk_delta_rule, lv, do, dht, opts, epi)
    ex = dict(lv, q=lv["q"].repeat_interleave(2, 2), k=lv["k"].repeat_interleave(2, 2))
    ref = run(mk.chunk_delta_rule, ex, do, dht, opts, epi)
    assert torch.equal(got["o"], ref["o"]) and torch.equal(got["ht"], ref["ht"])
    for n in ("dv", "dg", "dbeta", "dh0"):
        assert torch.equal(got[n], ref[n]), n
    B, T = 2, 200
    for n in ("dq", "dk"):
        torch.testing.assert_close(got[n], ref[n].view(B, T, 2, 2, 128).sum(3), rtol=1e-5, atol=1e-6)


def test_state_v_first_is_a_pure_transpose():
    lv, do, dht, opts, epi = make_inputs(cu=VARLEN_CU, T=704, dtype=torch.float32, gate="kimi", seed=7)
    a = run(mk.chunk_delta_rule, lv, do, dht, opts, epi, vfirst=False)
    b = run(mk.chunk_delta_rule, lv, do, dht, opts, epi, vfirst=True)
    assert torch.equal(a["o"], b["o"])
    assert torch.equal(a["ht"], b["ht"].transpose(-1, -2))
    assert torch.equal(a["dh0"], b["dh0"])          # run() transposes h0 itself, so the leaf is the same
    for n in ("dq", "dk", "dv", "dg", "dbeta"):
        assert torch.equal(a[n], b[n]), n


def test_repeated_runs_are_bitwise_identical():
    lv, do, dht, opts, epi = make_inputs(cu=VARLEN_CU, T=704, dtype=torch.bfloat16, gate="eda", seed=8)
    first = run(mk.chunk_delta_rule, lv, do, dht, opts, epi)
    for _ in range(5):
        again = run(mk.chunk_delta_rule, lv, do, dht, opts, epi)
        for n in first:
            assert torch.equal(first[n], again[n]), n


@pytest.mark.parametrize("T", [1, 2, 63, 64, 65, 129])
def test_tiny_and_boundary_lengths(T):
    lv, do, dht, opts, epi = make_inputs(B=1, T=T, dtype=torch.float32, gate="kimi", seed=T)
    compare(run(mk.chunk_delta_rule, lv, do, dht, opts, epi),
            run(orc.recurrent_delta_rule if T <= 65 else orc.chunked_delta_rule, lv, do, dht, opts, epi, f64=True))


def test_documents_of_length_one_and_empty_documents():
    cu = (0, 1, 2, 2, 67, 68)
    lv, do, dht, opts, epi = make_inputs(cu=cu, T=68, dtype=torch.float32, gate="eda", seed=11)
    compare(run(mk.chunk_delta_rule, lv, do, dht, opts, epi), run(orc.recurrent_delta_rule, lv, do, dht, opts, epi, f64=True))


def test_padding_tokens_past_the_last_sequence_are_zero():
    cu = (0, 100, 230)
    lv, do, dht, opts, epi = make_inputs(cu=cu, T=300, dtype=torch.bfloat16, gate="eda", seed=12)
    got = run(mk.chunk_delta_rule, lv, do, dht, opts, epi)
    assert (got["o"][:, 230:] == 0).all()
    for n in ("dq", "dk", "dv", "dg", "dbeta"):
        assert (got[n][:, 230:] == 0).all(), n
    cut = {k: (t[:, :230].contiguous() if t.dim() >= 3 and t.shape[1] == 300 else t) for k, t in lv.items()}
    ref = run(orc.chunked_delta_rule, cut, do[:, :230], dht, opts, epi, f64=True)
    check("o", got["o"][:, :230], ref["o"])
    check("dg", got["dg"][:, :230], ref["dg"])


def test_long_sequences_are_segmented_and_match():
    """T > 32 chunks: the state + transition pre-pass, the prefix combine and the main pass replace the single serial
    recurrence; same numbers within tolerance, and the uncut path still agrees with the oracle."""
    lv, do, dht, opts, epi = make_inputs(B=1, T=2048 + 64 * 5 + 7, dtype=torch.float32, gate="eda", seed=13, HV=2)
    seg = run(mk.chunk_delta_rule, lv, do, dht, opts, epi, vfirst=True)
    ref = run(orc.chunked_delta_rule, lv, do, dht, opts, epi, f64=True, vfirst=True)
    compare(seg, ref)
    flat = run(mk.chunk_delta_rule, lv, do, dht, opts, epi, vfirst=True, auto_cp=False)
    compare(flat, ref)


def test_gdn_clamp_has_zero_gradient_and_kimi_works_without_parameters():
    lv, do, dht, opts, epi = make_inputs(B=1, T=130, dtype=torch.float32, gate="gdn", seed=14, epi=None)
    lv["A_log"] = torch.full_like(lv["A_log"], 3.0)         # -exp(3) softplus(x) < -5 almost everywhere -> clamped
    got = run(mk.chunk_delta_rule, lv, do, dht, opts, epi)
    ref = run(orc.chunked_delta_rule, lv, do, dht, opts, epi, f64=True)
    pre = -lv["A_log"].double().exp()[:, None] * torch.nn.functional.softplus(lv["g"].double() + lv["dt_bias"].double())
    clamped = pre < -5.0 - 1e-4
    assert clamped.float().mean() > 0.5 and (got["dg"][clamped] == 0).all() and (ref["dg"][clamped] == 0).all()
    check("dg", got["dg"], ref["dg"])
    lv, do, dht, opts, epi = make_inputs(B=1, T=130, dtype=torch.float32, gate="kimi", seed=15, epi=None)
    lv.pop("A_log"), lv.pop("dt_bias")
    compare(run(mk.chunk_delta_rule, lv, do, dht, opts, epi), run(orc.chunked_delta_rule, lv, do, dht, opts, epi, f64=True))


def test_gated_delta_rule_entry_point():
    """Scalar-gate entry point on a reduced version of benchmark config 5 ([V,K] initial state, final state)."""
    lv, do, dht, opts, epi = make_inputs(B=2, T=500, HK=2, HV=2, dtype=torch.bfloat16, gate="precomputed", scalar=True,
                                         beta="precomputed", epi=None, seed=16)
    lv["g"] = orc.gate_log_decay(torch.randn_like(lv["g"]), "gdn", torch.randn(2, device="cuda") * 0.1, None, -5.0).float()

    def via_gdr(q, k, v, g, beta, **kw):
        kw = {n: x for n, x in kw.items() if n in ("initial_state", "output_final_state", "cu_seqlens", "state_v_first",
                                                   "use_qk_l2norm_in_kernel")}
        return mk.chunk_gated_delta_rule(q, k, v, g, beta, **kw)

    compare(run(via_gdr, lv, do, dht, opts, epi, vfirst=True),
            run(orc.chunked_delta_rule, lv, do, dht, opts, epi, f64=True, vfirst=True))


def test_inputs_at_odd_storage_offsets_are_accepted():
    """Contiguous views that start 4 bytes into their storage (slices of a flat buffer) are not 16-byte aligned; the
    kernels' vector loads need that, so such inputs are copied on the way in.  Same results, bit for bit, gradients too."""
    lv, do, dht, opts, epi = make_inputs(B=1, T=200, dtype=torch.bfloat16, gate="eda", seed=21)

    def call(x):
        kw = dict(opts, A_log=x["A_log"], dt_bias=x["dt_bias"], initial_state=x["h0"],
                  output_norm=dict(weight=x["ep_w"], gate=x["ep_gate"], act=epi, eps=1e-6))
        o, ht = mk.chunk_delta_rule(x["q"], x["k"], x["v"], x["g"], x["beta"], **kw)
        return o, ht, (o.double() * do.double()).sum() + (ht.double() * dht.double()).sum()

    plain = {n: t.clone().requires_grad_(True) for n, t in lv.items()}
    o0, ht0, loss0 = call(plain)
    g0 = torch.autograd.grad(loss0, list(plain.values()))

    flats, odd = {}, {}
    for n, t in lv.items():
        shift = 4 // t.element_size()
        flat = torch.zeros(t.numel() + shift, dtype=t.dtype, device=t.device)
        flat[shift:] = t.reshape(-1)
        flats[n] = flat.requires_grad_(True)
        odd[n] = flats[n][shift:].view(t.shape)
        assert odd[n].is_contiguous() and odd[n].data_ptr() % 16 == 4
    o1, ht1, loss1 = call(odd)
    g1 = torch.autograd.grad(loss1, list(flats.values()))
    assert torch.equal(o0, o1) and torch.equal(ht0, ht1)
    for (n, t), a, b in zip(lv.items(), g0, g1):
        assert torch.equal(a.reshape(-1), b[4 // t.element_size():]), n

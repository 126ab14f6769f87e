"""CPU: pins oracle/kda_oracle.py to the fixtures produced by the reference's own oracles
(tests/golden/make_golden.py), and the chunk algebra to the token-by-token recurrence."""
import glob
import os

import pytest
import torch

from oracle import kda_oracle as orc
from tests.golden.make_golden import kwargs_of

GOLD = os.path.join(os.path.dirname(__file__), "golden")
SMALL = sorted(glob.glob(os.path.join(GOLD, "ref_small_*.pt")))


def _close(a, b, tol=1e-9):
    mx, _ = orc.rel_err(a, b)
    assert mx < tol, mx


@pytest.mark.parametrize("path", SMALL, ids=[os.path.basename(p)[10:-3] for p in SMALL])
@pytest.mark.parametrize("impl", ["recurrent", "chunked"])
def test_option_surface_matches_reference(path, impl):
    fx = torch.load(path)
    c = fx["case"]
    leaves = {n: t.clone().requires_grad_(True) for n, t in fx["inputs"].items()}
    fn = orc.recurrent_delta_rule if impl == "recurrent" else orc.chunked_delta_rule
    o, ht = fn(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"], **kwargs_of(c, leaves))
    _close(o, fx["o"])
    _close(ht, fx["ht"])
    loss = (o * fx["do"]).sum() + (ht * fx["dht"]).sum()
    grads = torch.autograd.grad(loss, list(leaves.values()), allow_unused=True)
    for n, gr in zip(leaves, grads):
        ref = fx["grads"][n]
        assert (gr is None) == (ref is None), n
        if ref is not None:
            _close(gr, ref, 1e-8)


def test_config1_matches_reference():
    fx = torch.load(os.path.join(GOLD, "ref_config1.pt"))
    i = fx["inputs"]
    o, ht = orc.chunked_delta_rule(i["q"], i["k"], i["v"], i["g"], i["beta"], output_final_state=True)
    _close(o, fx["o"], 1e-6)      # fixture stored as float32
    _close(ht, fx["ht"], 1e-6)


def test_chunk_algebra_matches_reference_intermediates():
    fx = torch.load(os.path.join(GOLD, "chunk_small.pt"))
    i = fx["inputs"]
    cu = torch.tensor(fx["cu"], dtype=torch.int32)
    bw = orc.chunked_backward(i["q"], i["k"], i["v"], i["g"], i["beta"], fx["do"], dht=fx["dht"],
                              initial_state=i["h0"], cu_seqlens=cu)
    fw = bw["fwd"]
    f, b, it = fx["fwd"], fx["bwd"], fx["inter"]
    flat = lambda x: x.reshape(-1, *x.shape[2:])      # noqa: E731  [1,T,..] -> [TT,..]
    for name in ("g_c", "A", "Aqk", "Vd", "o"):
        _close(fw[name], flat(f[name]))
    _close(fw["h"], f["h"][0])
    _close(fw["gl"], f["gl"][0])
    _close(fw["ht"], f["ht"])
    _close(fw["nw"], -flat(it["w"]))
    _close(bw["dh"], it["dh"][0])
    _close(bw["dgl"], it["dgl"][0])
    for name in ("dVd", "dAqk", "dL", "dq_p", "dk_p", "dg_p", "dbeta_w", "dq_v", "dk_v", "dgp"):
        _close(bw[name], flat(it[name]), 1e-8)
    for name in ("dq", "dk", "dv", "dg", "dbeta"):
        _close(bw[name], b[name], 1e-8)
    _close(bw["dh0"], b["dh0"], 1e-8)


@pytest.mark.parametrize("vfirst", [False, True])
def test_chunked_backward_equals_autograd_of_recurrence(vfirst):
    g = torch.Generator().manual_seed(5)
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)      # noqa: E731
    B, T, HK, HV, D = 2, 130, 1, 2, 8
    lv = dict(q=r(B, T, HK, D), k=torch.nn.functional.normalize(r(B, T, HK, D), dim=-1), v=r(B, T, HV, D),
              g=-3 * torch.sigmoid(r(B, T, HV, D)), beta=torch.sigmoid(r(B, T, HV)), h0=r(B, HV, D, D))
    do, dht = r(B, T, HV, D), r(B, HV, D, D)
    leaves = {n: t.clone().requires_grad_(True) for n, t in lv.items()}
    o, ht = orc.recurrent_delta_rule(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"],
                                     initial_state=leaves["h0"], output_final_state=True, state_v_first=vfirst)
    grads = dict(zip(leaves, torch.autograd.grad((o * do).sum() + (ht * dht).sum(), list(leaves.values()))))
    bw = orc.chunked_backward(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], do, dht=dht, initial_state=lv["h0"],
                              state_v_first=vfirst)
    _close(bw["fwd"]["o"].reshape(B, T, HV, D), o)
    for n in ("dq", "dk", "dv", "dg", "dbeta"):
        _close(bw[n], grads[n[1:]], 1e-8)
    dh0 = bw["dh0"].transpose(-1, -2) if vfirst else bw["dh0"]
    _close(dh0, grads["h0"], 1e-8)

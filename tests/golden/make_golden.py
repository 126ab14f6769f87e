"""Generates the golden fixtures in this folder by RUNNING THE REFERENCE'S OWN ORACLES.

Run once, in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference

It imports ``tests/ref_kda.py`` (token-by-token fp64 reference) and, by file path,
``mogan_kda/ops/kimi_delta_rule/chunk/torch_ref.py`` (chunked fp64 forward/backward; loaded by path so the
package's GPU-only imports are not triggered), feeds them seeded inputs and stores inputs + outputs as
``*.pt`` files.  The tests never need the reference checkout: they read these files.

Fixtures
  ref_small_<name>.pt   option-surface cases at K=V=16 (inputs, o, final state, autograd gradients), float64
  ref_config1.pt        the T=256 / HK2 / HV4 / D128 float32 case of the benchmark configs (outputs stored as float32)
  chunk_small.pt        torch_ref chunk_fwd_torch / chunk_bwd_torch intermediates on a ragged varlen layout
"""
import importlib.util
import os
import sys

import torch


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def small_cases():
    """name -> kwargs builder.  Shapes are tiny; every option of the API appears at least once."""
    cu = [0, 1, 98, 165, 230]
    cases = {}

    def mk(name, *, B, T, HK, HV, D, gate, scalar=False, beta_mode="sigmoid", beta_scale=2.0, l2=True, epi=None,
           cu=None, h0=False, vfirst=False, seed=0):
        cases[name] = dict(B=B, T=T, HK=HK, HV=HV, D=D, gate=gate, scalar=scalar, beta_mode=beta_mode,
                           beta_scale=beta_scale, l2=l2, epi=epi, cu=cu, h0=h0, vfirst=vfirst, seed=seed)

    mk("eda_full", B=1, T=230, HK=2, HV=4, D=16, gate="eda", epi="silu", cu=cu, h0=True, vfirst=True)
    mk("kimi_dense", B=2, T=150, HK=2, HV=2, D=16, gate="kimi", epi="sigmoid", h0=True, seed=1)
    mk("gdn_channel", B=1, T=230, HK=1, HV=2, D=16, gate="gdn", beta_mode="precomputed", beta_scale=1.0, l2=False,
       cu=cu, seed=2)
    mk("precomputed", B=2, T=130, HK=2, HV=4, D=16, gate="precomputed", beta_mode="precomputed", beta_scale=1.0,
       l2=False, seed=3)
    mk("gdn_scalar", B=1, T=230, HK=2, HV=4, D=16, gate="gdn", scalar=True, cu=cu, h0=True, vfirst=True, seed=4)
    mk("scalar_precomputed", B=2, T=100, HK=2, HV=2, D=16, gate="precomputed", scalar=True, beta_mode="precomputed",
       beta_scale=1.0, l2=True, h0=True, seed=5)
    return cases


def build_inputs(c):
    """Seeded float64 leaves + the keyword dict for ref_chunk_delta_rule."""
    g = torch.Generator().manual_seed(1000 + c["seed"])
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)      # noqa: E731
    B, T, HK, HV, D = c["B"], c["T"], c["HK"], c["HV"], c["D"]
    N = B if c["cu"] is None else len(c["cu"]) - 1
    lv = dict(q=r(B, T, HK, D), k=r(B, T, HK, D), v=r(B, T, HV, D))
    if not c["l2"]:
        lv["q"] = torch.nn.functional.normalize(lv["q"], dim=-1)
        lv["k"] = torch.nn.functional.normalize(lv["k"], dim=-1)
    gshape = (B, T, HV) if c["scalar"] else (B, T, HV, D)
    if c["gate"] == "precomputed":
        lv["g"] = -5.0 * torch.sigmoid(r(*gshape))
    else:
        lv["g"] = r(*gshape)
        hi = 0.8 if c["gate"] == "gdn" else 4.0
        lv["A_log"] = (torch.rand(HV, generator=g, dtype=torch.float64) * (hi - 0.2) + 0.2).log()
        lv["dt_bias"] = r(*gshape[2:]) * 0.5 - 1.0
    lv["beta"] = r(B, T, HV) if c["beta_mode"] == "sigmoid" else c["beta_scale"] * torch.sigmoid(r(B, T, HV))
    if c["h0"]:
        lv["h0"] = r(N, HV, D, D) * 0.1
    if c["epi"]:
        lv["ep_w"] = 1.0 + 0.1 * r(D)
        lv["ep_gate"] = r(B, T, HV, D)
    do = r(B, T, HV, D)
    dht = r(N, HV, D, D) * 0.1
    return lv, do, dht


def kwargs_of(c, lv):
    kw = dict(gate_mode=c["gate"], A_log=lv.get("A_log"), dt_bias=lv.get("dt_bias"), lower_bound=-5.0,
              beta_mode=c["beta_mode"], beta_scale=c["beta_scale"] if c["beta_mode"] == "sigmoid" else 1.0,
              use_qk_l2norm_in_kernel=c["l2"], initial_state=lv.get("h0"), output_final_state=True,
              state_v_first=c["vfirst"],
              cu_seqlens=None if c["cu"] is None else torch.tensor(c["cu"], dtype=torch.int32))
    if c["epi"]:
        kw["output_norm"] = dict(weight=lv["ep_w"], gate=lv["ep_gate"], act=c["epi"], eps=1e-6)
    return kw


def main(ref_root):
    here = os.path.dirname(os.path.abspath(__file__))
    ref_kda = _load(os.path.join(ref_root, "tests", "ref_kda.py"), "ref_kda")
    torch_ref = _load(os.path.join(ref_root, "mogan_kda", "ops", "kimi_delta_rule", "chunk", "torch_ref.py"),
                      "torch_ref")
    # --- option surface, small dims -----------------------------------------------------------
    for name, c in small_cases().items():
        lv, do, dht = build_inputs(c)
        leaves = {n: t.clone().requires_grad_(True) for n, t in lv.items()}
        o, ht = ref_kda.ref_chunk_delta_rule(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"],
                                             **kwargs_of(c, leaves))
        loss = (o * do).sum() + (ht * dht).sum()
        grads = torch.autograd.grad(loss, list(leaves.values()), allow_unused=True)
        torch.save(dict(case=c, inputs=lv, do=do, dht=dht, o=o.detach(), ht=ht.detach(),
                        grads={n: gr for n, gr in zip(leaves, grads)}),
                   os.path.join(here, f"ref_small_{name}.pt"))
        print("wrote", name, tuple(o.shape))
    # --- benchmark config 1 (float32 inputs, D = 128) -----------------------------------------
    torch.manual_seed(0)
    B, T, HK, HV, D = 1, 256, 2, 4, 128
    q, k, v = torch.randn(B, T, HK, D), torch.randn(B, T, HK, D), torch.randn(B, T, HV, D)
    q, k = torch.nn.functional.normalize(q, dim=-1), torch.nn.functional.normalize(k, dim=-1)
    g = -0.5 * torch.rand(B, T, HV, D)
    beta = torch.sigmoid(torch.randn(B, T, HV))
    leaves = {n: t.clone().requires_grad_(True) for n, t in dict(q=q, k=k, v=v, g=g, beta=beta).items()}
    o, ht = ref_kda.ref_chunk_delta_rule(*leaves.values(), output_final_state=True)
    grads = torch.autograd.grad(o.sum(), list(leaves.values()))
    torch.save(dict(inputs=dict(q=q, k=k, v=v, g=g, beta=beta), o=o.detach().float(), ht=ht.detach().float(),
                    grads={n: gr.float() for n, gr in zip(leaves, grads)}), os.path.join(here, "ref_config1.pt"))
    print("wrote config1")
    # --- chunk algebra intermediates (torch_ref) ------------------------------------------------
    gen = torch.Generator().manual_seed(77)
    r = lambda *s: torch.randn(*s, generator=gen, dtype=torch.float64)    # noqa: E731
    cu = [0, 1, 98, 162, 230]
    B, T, HK, HV, D = 1, 230, 2, 4, 8
    q = torch.nn.functional.normalize(r(B, T, HK, D), dim=-1)
    k = torch.nn.functional.normalize(r(B, T, HK, D), dim=-1)
    v, g, beta = r(B, T, HV, D), -5.0 * torch.sigmoid(r(B, T, HV, D)), torch.sigmoid(r(B, T, HV))
    h0, do, dht = r(4, HV, D, D) * 0.1, r(B, T, HV, D), r(4, HV, D, D) * 0.1
    cu_t = torch.tensor(cu, dtype=torch.int32)
    fw = torch_ref.chunk_fwd_torch(q, k, v, g, beta, initial_state=h0, cu_seqlens=cu_t)
    bw = torch_ref.chunk_bwd_torch(q, k, v, beta, fw["g_c"], fw["A"], fw["Aqk"], fw["h"], do, dht=dht,
                                   cu_seqlens=cu_t)
    it = bw["inter"]
    keep_f = {n: fw[n] for n in ("o", "ht", "g_c", "A", "Aqk", "gl", "h", "Vd")}
    keep_b = {n: bw[n] for n in ("dq", "dk", "dv", "dg", "dbeta", "dh0")}
    keep_i = {n: it[n] for n in ("w", "dh", "dVd", "dgl", "dAqk", "dL", "dq_p", "dk_p", "dg_p", "dbeta_w")}
    keep_i.update(dq_v=it["intra"]["dq"], dk_v=it["intra"]["dk"], dgp=it["intra"]["dg"])
    torch.save(dict(cu=cu, inputs=dict(q=q, k=k, v=v, g=g, beta=beta, h0=h0), do=do, dht=dht, fwd=keep_f, bwd=keep_b,
                    inter=keep_i), os.path.join(here, "chunk_small.pt"))
    print("wrote chunk_small")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])

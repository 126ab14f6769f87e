"""Shared helpers of the GPU parity tests: seeded inputs in the style of the reference's generator
(tests/kda_common.py:133-162), runners for the CUDA path and the fp64 oracle, and the error metric."""
import torch

from oracle import kda_oracle as orc

TOL = 2e-3                     # rel-err bar for fp32-typed results (max|a-b|/max|b| and mean|a-b|/mean|b|)
BF16_MAX = 2.0 ** -8           # worst-case relative rounding of one bf16 store
BF16_MEAN = 1.6e-3             # mean relative rounding of a bf16 store (log-uniform mantissas: 2^-9 / 1.44 ~ 1.36e-3)
VARLEN_CU = (0, 1, 98, 354, 504, 704)


def tolerances(t):
    """(max_rel, mean_rel) allowed for a result stored in t.dtype: the 2e-3 bar plus, for 16-bit outputs, the
    quantum of the store itself (the oracle is never rounded)."""
    if t.dtype == torch.float32:
        return TOL, TOL
    return TOL + BF16_MAX, TOL + BF16_MEAN


def check(name, got, ref):
    assert got is not None, f"{name}: missing"
    assert got.shape == ref.shape, f"{name}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got.float()).all(), f"{name}: non-finite values"
    mx, mn = orc.rel_err(got, ref.to(got.device))
    tmx, tmn = tolerances(got)
    assert mx <= tmx and mn <= tmn, f"{name}: max_rel {mx:.3e} (tol {tmx:.1e}) mean_rel {mn:.3e} (tol {tmn:.1e})"
    return mx, mn


def make_inputs(*, B=1, T=256, HK=2, HV=4, cu=None, dtype=torch.float32, gate="eda", scalar=False, beta="sigmoid",
                l2=True, epi="silu", h0=True, seed=0, device="cuda", x_dtype=torch.float32):
    g = torch.Generator(device="cpu").manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g)                       # noqa: E731
    N = B if cu is None else len(cu) - 1
    q, k = r(B, T, HK, 128), r(B, T, HK, 128)
    if not l2:
        q, k = torch.nn.functional.normalize(q, dim=-1), torch.nn.functional.normalize(k, dim=-1)
    lv = dict(q=q.to(dtype), k=k.to(dtype), v=r(B, T, HV, 128).to(dtype))
    gshape = (B, T, HV) if scalar else (B, T, HV, 128)
    if gate == "precomputed":
        lv["g"] = -5.0 * torch.sigmoid(r(*gshape))
    else:
        lv["g"] = r(*gshape).to(x_dtype)
        hi = 0.8 if gate == "gdn" else 4.0
        lv["A_log"] = (torch.rand(HV, generator=g) * (hi - 0.2) + 0.2).log()
        lv["dt_bias"] = r(*gshape[2:]) * 0.5 - 1.0
    lv["beta"] = r(B, T, HV) if beta == "sigmoid" else torch.sigmoid(r(B, T, HV))
    if h0:
        lv["h0"] = r(N, HV, 128, 128) * 0.1
    if epi:
        lv["ep_w"] = 1.0 + 0.1 * r(128)
        lv["ep_gate"] = r(B, T, HV, 128).to(dtype)
    lv = {n: t.to(device) for n, t in lv.items()}
    do = r(B, T, HV, 128).to(device)
    if not epi:
        do = do.to(dtype).float()      # autograd hands the kernel dO in the dtype of o: give the oracle the same values
    dht = (r(N, HV, 128, 128) * 0.1).to(device)
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32, device=device)
    opts = dict(gate_mode=gate, lower_bound=-5.0, beta_mode=beta, beta_scale=2.0 if beta == "sigmoid" else 1.0,
                use_qk_l2norm_in_kernel=l2, cu_seqlens=cu_t, output_final_state=True)
    return lv, do, dht, opts, (epi or None)


def run(fn, lv, do, dht, opts, epi, *, f64=False, vfirst=False, grads=True, **extra):
    """Calls ``fn`` (the CUDA API or an oracle with the same keywords); returns dict(o, ht, d<leaf>...)."""
    lv = {n: (t.double() if f64 else t).clone().requires_grad_(grads) for n, t in lv.items()}
    kw = dict(opts, A_log=lv.get("A_log"), dt_bias=lv.get("dt_bias"), state_v_first=vfirst, **extra)
    h0 = lv.get("h0")
    if h0 is not None and vfirst:
        h0 = h0.transpose(-1, -2).contiguous()
    kw["initial_state"] = h0
    if epi:
        kw["output_norm"] = dict(weight=lv["ep_w"], gate=lv["ep_gate"], act=epi, eps=1e-6)
    o, ht = fn(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], **kw)
    res = dict(o=o, ht=ht)
    if grads:
        d = dht.transpose(-1, -2) if vfirst else dht
        loss = (o.double() * do.double()).sum() + (ht.double() * d.double()).sum()
        for n, gr in zip(lv, torch.autograd.grad(loss, list(lv.values()))):
            res["d" + n] = gr
    return res


def compare(got, ref):
    for n, r in ref.items():
        check(n, got[n], r)


# ---- state tiles (include/mkda.h, MKDA_STATE_TILE_BYTES): an independent torch restatement of the layout ------------------
def _state_tile_index():
    """int64 [128 (K index), 128 (v)] -> position, in bf16 elements, inside one 32 KB half of a state tile."""
    kk = torch.arange(128).view(128, 1)
    v = torch.arange(128).view(1, 128)
    blk, chunk, e = kk >> 6, (kk & 63) >> 3, kk & 7
    byte = blk * 128 * 128 + (v >> 3) * 1024 + (v & 7) * 128 + ((chunk ^ (v & 7)) << 4) + e * 2
    return (byte // 2).reshape(-1)


def pack_state_tiles(S):
    """fp [..., 128 (K index), 128 (v)] -> float32 tensor of the same shape holding the hi / lo operand tiles."""
    S = S.float()
    lead = S.shape[:-2]
    hi = S.to(torch.bfloat16)
    lo = (S - hi.float()).to(torch.bfloat16)
    idx = _state_tile_index().to(S.device)
    out = torch.empty(*lead, 2, 128 * 128, dtype=torch.bfloat16, device=S.device)
    out[..., 0, idx] = hi.reshape(*lead, -1)
    out[..., 1, idx] = lo.reshape(*lead, -1)
    return out.view(torch.float32).reshape(*lead, 128, 128)


def unpack_state_tiles(T):
    """Inverse of pack_state_tiles: float32-typed tile buffer [..., 128, 128] -> fp32 [..., 128 (K index), 128 (v)]."""
    lead = T.shape[:-2]
    halves = T.contiguous().view(torch.bfloat16).reshape(*lead, 2, 128 * 128)
    idx = _state_tile_index().to(T.device)
    return (halves[..., 0, idx].float() + halves[..., 1, idx].float()).reshape(*lead, 128, 128)


# ---- chunk tiles (include/mkda.h, MKDA_CHUNK_TILE_BYTES): X^T [128][64 tokens] per (chunk, head) ----------------------------
def _chunk_tile_index():
    """int64 [128 (row), 64 (token)] -> position, in bf16 elements, inside one 16 KB half of a chunk tile."""
    r = torch.arange(128).view(128, 1)
    t = torch.arange(64).view(1, 64)
    byte = (r >> 3) * 1024 + (r & 7) * 128 + (((t >> 3) ^ (r & 7)) << 4) + (t & 7) * 2
    return (byte // 2).reshape(-1)


def _chunk_rows(lay):
    starts, lens = lay.chunk_start.tolist(), lay.chunk_len.tolist()
    return [(c, s0, n) for c, (s0, n) in enumerate(zip(starts, lens))]


def pack_chunk_tiles(X, lay):
    """token-major fp [TT, H, 128] -> float32-typed chunk tiles [NC, H, 64, 128] (X^T per chunk, zero past the end)."""
    X = X.float()
    H = X.shape[1]
    dense = torch.zeros(lay.NC, H, 128, 64, device=X.device)
    for c, s0, n in _chunk_rows(lay):
        dense[c, :, :, :n] = X[s0:s0 + n].permute(1, 2, 0)
    hi = dense.to(torch.bfloat16)
    lo = (dense - hi.float()).to(torch.bfloat16)
    idx = _chunk_tile_index().to(X.device)
    out = torch.empty(lay.NC, H, 2, 128 * 64, dtype=torch.bfloat16, device=X.device)
    out[..., 0, idx] = hi.reshape(lay.NC, H, -1)
    out[..., 1, idx] = lo.reshape(lay.NC, H, -1)
    return out.view(torch.float32).reshape(lay.NC, H, 64, 128)


def unpack_chunk_tiles(T, lay, TT):
    """Inverse of pack_chunk_tiles -> fp32 [TT, H, 128] (tokens outside every chunk are zero)."""
    H = T.shape[1]
    halves = T.contiguous().view(torch.bfloat16).reshape(lay.NC, H, 2, 128 * 64)
    idx = _chunk_tile_index().to(T.device)
    dense = (halves[..., 0, idx].float() + halves[..., 1, idx].float()).reshape(lay.NC, H, 128, 64)
    X = torch.zeros(TT, H, 128, device=T.device)
    for c, s0, n in _chunk_rows(lay):
        X[s0:s0 + n] = dense[c, :, :, :n].permute(2, 0, 1)
    return X


# ---- quarter tiles (include/mkda.h, MKDA_QUARTER_TILE_BYTES): a [64][64] matrix per (chunk, head) ------------------------
def _quarter_tile_index():
    i = torch.arange(64).view(64, 1)
    j = torch.arange(64).view(1, 64)
    byte = (i >> 3) * 1024 + (i & 7) * 128 + (((j >> 3) ^ (i & 7)) << 4) + (j & 7) * 2
    return (byte // 2).reshape(-1)


def pack_quarter_tiles(X, lay):
    """token-major rows fp [TT, H, 64] -> float32-typed quarter tiles [NC, H, 32, 128] (row i of chunk c = token start+i)."""
    X = X.float()
    H = X.shape[1]
    dense = torch.zeros(lay.NC, H, 64, 64, device=X.device)
    for c, s0, n in _chunk_rows(lay):
        dense[c, :, :n] = X[s0:s0 + n].permute(1, 0, 2)
    hi = dense.to(torch.bfloat16)
    lo = (dense - hi.float()).to(torch.bfloat16)
    idx = _quarter_tile_index().to(X.device)
    out = torch.empty(lay.NC, H, 2, 64 * 64, dtype=torch.bfloat16, device=X.device)
    out[..., 0, idx] = hi.reshape(lay.NC, H, -1)
    out[..., 1, idx] = lo.reshape(lay.NC, H, -1)
    return out.view(torch.float32).reshape(lay.NC, H, 32, 128)


def unpack_quarter_tiles(T, lay, TT):
    """Inverse of pack_quarter_tiles -> fp32 [TT, H, 64] (rows past the end of a chunk are dropped)."""
    H = T.shape[1]
    halves = T.contiguous().view(torch.bfloat16).reshape(lay.NC, H, 2, 64 * 64)
    idx = _quarter_tile_index().to(T.device)
    dense = (halves[..., 0, idx].float() + halves[..., 1, idx].float()).reshape(lay.NC, H, 64, 64)
    X = torch.zeros(TT, H, 64, device=T.device)
    for c, s0, n in _chunk_rows(lay):
        X[s0:s0 + n] = dense[c, :, :n].permute(1, 0, 2)
    return X


# ---- row tiles (include/mkda.h): a [64 tokens][128] operand per (chunk, head), e.g. kbar and scale q 2^g ---------------------
def _row_tile_index():
    t = torch.arange(64).view(64, 1)
    k = torch.arange(128).view(1, 128)
    byte = (k >> 6) * 64 * 128 + (t >> 3) * 1024 + (t & 7) * 128 + ((((k & 63) >> 3) ^ (t & 7)) << 4) + (k & 7) * 2
    return (byte // 2).reshape(-1)


def pack_row_tiles(X, lay):
    """token-major fp [TT, H, 128] -> float32-typed row tiles [NC, H, 64, 128] (zero rows past the end of a chunk)."""
    X = X.float()
    H = X.shape[1]
    dense = torch.zeros(lay.NC, H, 64, 128, device=X.device)
    for c, s0, n in _chunk_rows(lay):
        dense[c, :, :n] = X[s0:s0 + n].permute(1, 0, 2)
    hi = dense.to(torch.bfloat16)
    lo = (dense - hi.float()).to(torch.bfloat16)
    idx = _row_tile_index().to(X.device)
    out = torch.empty(lay.NC, H, 2, 64 * 128, dtype=torch.bfloat16, device=X.device)
    out[..., 0, idx] = hi.reshape(lay.NC, H, -1)
    out[..., 1, idx] = lo.reshape(lay.NC, H, -1)
    return out.view(torch.float32).reshape(lay.NC, H, 64, 128)


def row_tiles_dense(T, lay):
    """float32-typed row tiles -> fp32 [NC, H, 64, 128] (hi + lo), the rows past the end of each chunk included."""
    H = T.shape[1]
    halves = T.contiguous().view(torch.bfloat16).reshape(lay.NC, H, 2, 64 * 128)
    idx = _row_tile_index().to(T.device)
    return (halves[..., 0, idx].float() + halves[..., 1, idx].float()).reshape(lay.NC, H, 64, 128)


def unpack_row_tiles(T, lay, TT):
    H = T.shape[1]
    dense = row_tiles_dense(T, lay)
    X = torch.zeros(TT, H, 128, device=T.device)
    for c, s0, n in _chunk_rows(lay):
        X[s0:s0 + n] = dense[c, :, :n].permute(1, 0, 2)
    return X


def pack_plain_tiles(X, lay):
    """token-major fp [TT, H, 128] -> fp32 [NC, H, 64, 128]: the rows of each chunk, unsplit (zero rows past the end)."""
    H = X.shape[1]
    out = torch.zeros(lay.NC, H, 64, 128, device=X.device)
    for c, s0, n in _chunk_rows(lay):
        out[c, :, :n] = X[s0:s0 + n].float().permute(1, 0, 2)
    return out


def unpack_plain_tiles(T, lay, TT):
    X = torch.zeros(TT, T.shape[1], 128, device=T.device)
    for c, s0, n in _chunk_rows(lay):
        X[s0:s0 + n] = T[c, :, :n].permute(1, 0, 2)
        assert float(T[c, :, n:].abs().sum()) == 0.0, "rows past the end of a chunk must be zero"
    return X


def scaled_operands(qn, kn, g_c, lay, scale):
    """fp64 reference of the state kernels' scaled operands from normalised q / k [TT,HK,128] and the log2 cumsum g_c
    [TT,HV,128]: kbar = k 2^(gL - g), qs = scale q 2^g (token-major [TT,HV,128]) and gl = 2^gL [NC,HV,128]."""
    G = g_c.shape[1] // qn.shape[1]
    qe, ke, g = qn.double().repeat_interleave(G, 1), kn.double().repeat_interleave(G, 1), g_c.double()
    kbar, gl = torch.zeros_like(g), torch.zeros(lay.NC, g.shape[1], 128, dtype=torch.float64, device=g.device)
    for c, s0, n in _chunk_rows(lay):
        gL = g[s0 + n - 1]
        kbar[s0:s0 + n] = ke[s0:s0 + n] * torch.exp2(gL - g[s0:s0 + n])
        gl[c] = torch.exp2(gL)
    return kbar, scale * qe * torch.exp2(g), gl

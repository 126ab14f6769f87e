"""TEST INFRASTRUCTURE ONLY: float64 CPU/GPU-agnostic restatement of the reference's delta-rule math.

Nothing in the shipped package imports this file.  It is the checker used by ``tests/``, by
``__graft_entry__.smoke()`` and by the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.

Parity status: PINNED.  ``tests/golden/make_golden.py`` ran the reference's own oracles
(``tests/ref_kda.py`` and ``mogan_kda/ops/kimi_delta_rule/chunk/torch_ref.py``) on seeded inputs and
stored their outputs; ``tests/test_oracle.py`` checks every function below against those fixtures.

Two tiers, like the reference's own test chain (``tests/test_kda_bwd_oracle.py`` -> kernel tests):

* ``recurrent_delta_rule``  token-by-token ground truth (follows ``tests/ref_kda.py:102-182``), differentiable.
* ``chunked_forward`` / ``chunked_backward``  the chunk algebra the kernels implement (follows
  ``mogan_kda/ops/kimi_delta_rule/chunk/torch_ref.py:94-359``), vectorised over chunks, returning
  every intermediate in the layout the CUDA kernels use so each kernel can be checked on its own.

All math is float64 whatever the input dtype.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

C = 64                      # chunk length (mogan_kda/ops/kimi_delta_rule/chunk/__init__.py:18)
L2_EPS = 1e-6               # tests/ref_kda.py:38
RCP_LN2 = 1.0 / math.log(2.0)
F64 = torch.float64


# ---------------------------------------------------------------------------------------------
# option math  (tests/ref_kda.py:46-95)
# ---------------------------------------------------------------------------------------------

def gate_log_decay(x, mode="precomputed", A_log=None, dt_bias=None, lower_bound=-5.0):
    """Natural-log per-token decay from the raw gate input (tests/ref_kda.py:46-64).

    x [B,T,HV] (scalar gate) or [B,T,HV,K]; A_log [HV]; dt_bias [HV] / [HV,K] / flat [HV*K].
    """
    s = x.to(F64)
    if mode == "precomputed":
        return s
    if dt_bias is not None:
        s = s + dt_bias.to(F64).reshape(s.shape[2:])
    E = None
    if A_log is not None:
        E = A_log.to(F64).exp().reshape(s.shape[2], *([1] * (s.dim() - 3)))
    if mode == "gdn":
        if E is None:
            raise ValueError("gate_mode='gdn' needs A_log")
        out = -E * F.softplus(s)
        return out if lower_bound is None else out.clamp(min=lower_bound)
    if mode == "kimi":
        if lower_bound is None:
            raise ValueError("gate_mode='kimi' needs lower_bound")
        return lower_bound * torch.sigmoid(s if E is None else E * s)
    if mode == "eda":
        if E is None or lower_bound is None:
            raise ValueError("gate_mode='eda' needs A_log and lower_bound")
        return lower_bound + (-lower_bound) * torch.exp(-(E / abs(lower_bound)) * F.softplus(s))
    raise ValueError(f"unknown gate_mode {mode!r}")


def beta_value(beta, mode="precomputed", scale=1.0):
    """tests/ref_kda.py:67-74."""
    b = beta.to(F64)
    if mode == "precomputed":
        return b
    if mode == "sigmoid":
        return scale * torch.sigmoid(b)
    raise ValueError(f"unknown beta_mode {mode!r}")


def gated_rmsnorm(o, weight, gate, act="silu", eps=1e-6):
    """Per-head gated RMSNorm epilogue (tests/ref_kda.py:77-91)."""
    o = o.to(F64)
    y = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.to(F64)
    z = gate.to(F64)
    if act in ("silu", "swish"):
        return y * z * torch.sigmoid(z)
    if act == "sigmoid":
        return y * torch.sigmoid(z)
    raise ValueError(f"unknown act {act!r}")


def l2norm(x):
    """tests/ref_kda.py:94-95."""
    x = x.to(F64)
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + L2_EPS)


# ---------------------------------------------------------------------------------------------
# tier 1: token-by-token recurrence  (tests/ref_kda.py:102-182)
# ---------------------------------------------------------------------------------------------

def _scan_tokens(q, k, v, g, beta, S):
    """q (scaled), k, g [B,T,HV,K]; v [B,T,HV,V]; beta [B,T,HV]; S [B,HV,K,V]."""
    out = []
    if q.shape[1] == 0:
        return v.new_zeros(v.shape), S
    for t in range(q.shape[1]):
        S = S * g[:, t].exp().unsqueeze(-1)
        kt = k[:, t]
        resid = v[:, t] - torch.einsum("bhk,bhkv->bhv", kt, S)
        S = S + torch.einsum("bhk,bhv->bhkv", beta[:, t].unsqueeze(-1) * kt, resid)
        out.append(torch.einsum("bhk,bhkv->bhv", q[:, t], S))
    return torch.stack(out, 1), S


def sequences(B, T, cu_seqlens):
    """[(batch row, first token, end token)] of every independent sequence."""
    if cu_seqlens is None:
        return [(b, 0, T) for b in range(B)]
    if B != 1:
        raise ValueError("cu_seqlens requires B == 1")
    cu = [int(c) for c in cu_seqlens.tolist()]
    return [(0, cu[i], cu[i + 1]) for i in range(len(cu) - 1)]


def recurrent_delta_rule(q, k, v, g, beta, *, scale=None, initial_state=None, output_final_state=False,
                         cu_seqlens=None, state_v_first=False, gate_mode="precomputed", A_log=None,
                         dt_bias=None, lower_bound=-5.0, beta_mode="precomputed", beta_scale=1.0,
                         use_qk_l2norm_in_kernel=False, output_norm=None):
    """Ground truth with the full option surface (same keywords as tests/ref_kda.py:115-122).

    Returns (o float64 [B,T,HV,V], final_state float64 or None).
    """
    B, T, HK, K = q.shape
    HV = v.shape[2]
    G = HV // HK
    scale = K ** -0.5 if scale is None else scale
    q, k, v = q.to(F64), k.to(F64), v.to(F64)
    if use_qk_l2norm_in_kernel:
        q, k = l2norm(q), l2norm(k)
    q = q.repeat_interleave(G, 2) * scale
    k = k.repeat_interleave(G, 2)
    gd = gate_log_decay(g, gate_mode, A_log, dt_bias, lower_bound)
    if gd.dim() == 3:
        gd = gd.unsqueeze(-1).expand(B, T, HV, K)
    bt = beta_value(beta, beta_mode, beta_scale)
    h0 = None
    if initial_state is not None:
        h0 = initial_state.to(F64)
        if state_v_first:
            h0 = h0.transpose(-1, -2)
    outs, finals = [], []
    if cu_seqlens is None:
        S = q.new_zeros(B, HV, K, v.shape[-1]) if h0 is None else h0
        o, S = _scan_tokens(q, k, v, gd, bt, S)
        outs.append(o)
        finals.append(S)
    else:
        for n, (_, s, e) in enumerate(sequences(B, T, cu_seqlens)):
            S = q.new_zeros(1, HV, K, v.shape[-1]) if h0 is None else h0[n:n + 1]
            o, S = _scan_tokens(q[:, s:e], k[:, s:e], v[:, s:e], gd[:, s:e], bt[:, s:e], S)
            outs.append(o)
            finals.append(S)
    o = torch.cat(outs, 1)
    if output_norm is not None:
        o = gated_rmsnorm(o, output_norm.get("weight"), output_norm["gate"], output_norm.get("act", "silu"),
                          output_norm.get("eps", 1e-6))
    ht = None
    if output_final_state:
        ht = torch.cat(finals, 0)
        if state_v_first:
            ht = ht.transpose(-1, -2).contiguous()
    return o, ht


# ---------------------------------------------------------------------------------------------
# chunk bookkeeping (chunks never straddle a sequence; mogan_kda/utils/index.py:93-116,
# torch_ref.py:43-63).  Tokens are addressed in the flattened [B*T] space.
# ---------------------------------------------------------------------------------------------

def chunk_table(B, T, cu_seqlens=None):
    """Returns dict(start [NC], length [NC], seq [NC], seq_off [N+1]) as python lists.

    Chunk ids are sequence-major.  ``start`` is a flattened token index (b*T + t)."""
    start, length, seq, seq_off = [], [], [], [0]
    for n, (b, s, e) in enumerate(sequences(B, T, cu_seqlens)):
        for c0 in range(s, e, C):
            start.append(b * T + c0)
            length.append(min(C, e - c0))
            seq.append(n)
        seq_off.append(len(start))
    return dict(start=start, length=length, seq=seq, seq_off=seq_off)


def _gather(x_flat, tab):
    """[TT, ...] -> zero padded [NC, C, ...]."""
    NC = len(tab["start"])
    out = x_flat.new_zeros(NC, C, *x_flat.shape[1:])
    for c in range(NC):
        s, n = tab["start"][c], tab["length"][c]
        out[c, :n] = x_flat[s:s + n]
    return out


def _scatter(xc, tab, TT):
    out = xc.new_zeros(TT, *xc.shape[2:])
    for c in range(xc.shape[0]):
        s, n = tab["start"][c], tab["length"][c]
        out[s:s + n] = xc[c, :n]
    return out


def _row_mask(tab, device):
    ln = torch.tensor(tab["length"], device=device)
    return torch.arange(C, device=device)[None, :] < ln[:, None]          # [NC, C]


# ---------------------------------------------------------------------------------------------
# tier 2: chunk algebra
# ---------------------------------------------------------------------------------------------

def chunked_forward(q, k, v, g, beta, *, scale=None, initial_state=None, cu_seqlens=None, state_v_first=False):
    """Chunk-form forward on already-activated operands (torch_ref.py:118-167).

    q, k [B,T,HK,K] (already L2-normalised if wanted); v [B,T,HV,V]; g [B,T,HV,K] natural-log per-token decay;
    beta [B,T,HV] effective beta.  Returns a dict, flattened-token layout ([TT, ...]) for per-token tensors
    and chunk-major ([NC, ...]) for per-chunk ones:

      g_c  [TT,HV,K]  chunk-local inclusive cumsum of g in the log2 domain
      A    [TT,HV,C]  rows of (I + strictlower(diag(beta) Gamma))^-1
      Aqk  [TT,HV,C]  rows of scale * lower(q k^T with decay), diagonal included
      nw   [TT,HV,K]  -A diag(beta) k~                 (k~ = k 2^g_c)
      u    [TT,HV,V]  A (beta * v)
      h    [NC,HV,K,V] state entering each chunk;  gl [NC,HV,K] = 2^(g_c at the last valid row)
      Vd   [TT,HV,V]  u + nw h            o [TT,HV,V];   ht [N,HV,K,V] final state per sequence
    States are returned in [K,V] orientation whatever ``state_v_first`` says (it only describes
    ``initial_state``).
    """
    B, T, HK, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    G = HV // HK
    TT = B * T
    scale = K ** -0.5 if scale is None else scale
    dev = q.device
    tab = chunk_table(B, T, cu_seqlens)
    NC = len(tab["start"])
    N = len(tab["seq_off"]) - 1
    qf = q.to(F64).reshape(TT, HK, K).repeat_interleave(G, 1)
    kf = k.to(F64).reshape(TT, HK, K).repeat_interleave(G, 1)
    vf = v.to(F64).reshape(TT, HV, V)
    gf = g.to(F64).reshape(TT, HV, K)
    bf = beta.to(F64).reshape(TT, HV)
    qc, kc, vc, gc, bc = (_gather(x, tab) for x in (qf, kf, vf, gf, bf))       # [NC,C,HV,*]
    valid = _row_mask(tab, dev)                                                 # [NC,C]
    gcum = gc.cumsum(1) * RCP_LN2                                               # padded rows keep the last value
    ln = torch.tensor(tab["length"], device=dev)
    g_last = gcum[torch.arange(NC, device=dev), ln - 1]                         # [NC,HV,K]
    up, dn = torch.exp2(gcum), torch.exp2(-gcum)                                # fine in fp64: |g_c| <= 64*5/ln2
    vm = valid[:, :, None, None].to(F64)
    qt, kt = qc * up * vm, kc * up * vm                                         # q~, k~
    kdn = kc * dn * vm                                                          # k 2^-g
    kbar = kc * torch.exp2(g_last[:, None] - gcum) * vm
    gl = torch.exp2(g_last)
    idx = torch.arange(C, device=dev)
    strict = (idx[:, None] > idx[None, :]).to(F64)
    lower = (idx[:, None] >= idx[None, :]).to(F64)
    gamma = torch.einsum("cihk,cjhk->chij", kt, kdn) * strict                   # Gamma_ij, i > j
    Lmat = gamma * bc.permute(0, 2, 1)[:, :, :, None]                           # diag(beta) on rows
    eye = torch.eye(C, dtype=F64, device=dev)
    Ainv = torch.linalg.solve_triangular(eye + Lmat, eye.expand(NC, HV, C, C), upper=False)
    Ainv = Ainv * lower
    Aqk = scale * torch.einsum("cihk,cjhk->chij", qt, kdn) * lower
    Ab = Ainv * bc.permute(0, 2, 1)[:, :, None, :]                              # A diag(beta)
    nw = -torch.einsum("chij,cjhk->cihk", Ab, kt)
    u = torch.einsum("chij,cjhv->cihv", Ab, vc)
    h0 = None
    if initial_state is not None:
        h0 = initial_state.to(F64)
        if state_v_first:
            h0 = h0.transpose(-1, -2)
    h = q.new_zeros(NC, HV, K, V, dtype=F64)
    Vd = torch.zeros_like(vc)
    o = torch.zeros_like(vc)
    ht = q.new_zeros(N, HV, K, V, dtype=F64)
    for n in range(N):
        S = q.new_zeros(HV, K, V, dtype=F64) if h0 is None else h0[n]
        for c in range(tab["seq_off"][n], tab["seq_off"][n + 1]):
            h[c] = S
            vd = u[c] + torch.einsum("ihk,hkv->ihv", nw[c], S)
            Vd[c] = vd
            o[c] = scale * torch.einsum("ihk,hkv->ihv", qt[c], S) + torch.einsum("hij,jhv->ihv", Aqk[c], vd)
            S = gl[c][:, :, None] * S + torch.einsum("ihk,ihv->hkv", kbar[c], vd)
        ht[n] = S
    sc = lambda x: _scatter(x, tab, TT)                                          # noqa: E731
    return dict(g_c=sc(gcum), A=sc(Ainv.permute(0, 2, 1, 3)), Aqk=sc(Aqk.permute(0, 2, 1, 3)), nw=sc(nw), u=sc(u),
                h=h, gl=gl, Vd=sc(Vd), o=sc(o * vm), ht=ht, table=tab)


def chunked_backward(q, k, v, g, beta, do, *, dht=None, scale=None, initial_state=None, cu_seqlens=None,
                     state_v_first=False):
    """Chunk-form backward (torch_ref.py:174-359), same operand conventions as ``chunked_forward``.

    do [B,T,HV,V]; dht [N,HV,K,V] (or [N,HV,V,K] with state_v_first) or None.  Returns a dict with the
    kernel-level intermediates (flattened-token layout) and the gradients w.r.t. (q, k, v, g, beta, h0):

      dh  [NC,HV,K,V]  gradient of the state LEAVING each chunk;  dVd [TT,HV,V];  dh0 [N,HV,K,V]
      Vd, dX (= dv) [TT,HV,V];  dbeta_w [TT,HV];  dAqk, dL [TT,HV,C]
      dq_p, dk_p, dg_p [TT,HV,K]  row-local partials;   dq_v, dk_v [TT,HV,K] per v-head;   dgp = dg' [TT,HV,K]
      dq, dk [B,T,HK,K]; dv [B,T,HV,V]; dg [B,T,HV,K] (w.r.t. the natural-log per-token g); dbeta [B,T,HV]
    """
    B, T, HK, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    G = HV // HK
    TT = B * T
    scale = K ** -0.5 if scale is None else scale
    dev = q.device
    fw = chunked_forward(q, k, v, g, beta, scale=scale, initial_state=initial_state, cu_seqlens=cu_seqlens,
                         state_v_first=state_v_first)
    tab = fw["table"]
    NC = len(tab["start"])
    N = len(tab["seq_off"]) - 1
    ga = lambda x: _gather(x, tab)                                               # noqa: E731
    qf = q.to(F64).reshape(TT, HK, K).repeat_interleave(G, 1)
    kf = k.to(F64).reshape(TT, HK, K).repeat_interleave(G, 1)
    qc, kc, vc = ga(qf), ga(kf), ga(v.to(F64).reshape(TT, HV, V))
    bc = ga(beta.to(F64).reshape(TT, HV))
    doc = ga(do.to(F64).reshape(TT, HV, V))
    gcum = ga(fw["g_c"])
    valid = _row_mask(tab, dev)
    vm = valid[:, :, None, None].to(F64)
    ln = torch.tensor(tab["length"], device=dev)
    ar = torch.arange(NC, device=dev)
    g_last = gcum[ar, ln - 1]
    up = torch.exp2(gcum) * vm
    rest = torch.exp2(g_last[:, None] - gcum) * vm                              # 2^(g_L - g)
    qt, kt, kbar, gl = qc * up, kc * up, kc * rest, fw["gl"]
    A = ga(fw["A"]).permute(0, 2, 1, 3)                                          # [NC,HV,i,j]
    Aqk = ga(fw["Aqk"]).permute(0, 2, 1, 3)
    nw = ga(fw["nw"])
    h = fw["h"]
    dht_s = None
    if dht is not None:
        dht_s = dht.to(F64)
        if state_v_first:
            dht_s = dht_s.transpose(-1, -2)
    # reverse state chain (torch_ref.py:187-224)
    dh = torch.zeros_like(h)
    dVd = torch.zeros_like(vc)
    dh0 = q.new_zeros(N, HV, K, V, dtype=F64)
    for n in range(N):
        dS = q.new_zeros(HV, K, V, dtype=F64) if dht_s is None else dht_s[n]
        for c in reversed(range(tab["seq_off"][n], tab["seq_off"][n + 1])):
            dh[c] = dS
            dvd = torch.einsum("hij,ihv->jhv", Aqk[c], doc[c]) + torch.einsum("jhk,hkv->jhv", kbar[c], dS)
            dVd[c] = dvd
            dS = (gl[c][:, :, None] * dS + scale * torch.einsum("ihk,ihv->hkv", qt[c], doc[c])
                  + torch.einsum("ihk,ihv->hkv", nw[c], dvd))
        dh0[n] = dS
    # chunk-parallel part through Vd / A (torch_ref.py:227-283)
    X = vc - torch.einsum("cihk,chkv->cihv", kt, h)
    W = bc[..., None] * X
    Vd = torch.einsum("chij,cjhv->cihv", A, W)
    idx = torch.arange(C, device=dev)
    strict = (idx[:, None] > idx[None, :]).to(F64)
    lower = (idx[:, None] >= idx[None, :]).to(F64)
    dAqk = torch.einsum("cihv,cjhv->chij", doc, Vd) * lower
    dW = torch.einsum("chij,cihv->cjhv", A, dVd)
    dX = bc[..., None] * dW
    dbeta_w = (dW * X).sum(-1)
    dA = torch.einsum("cihv,cjhv->chij", dVd, W)
    At = A.transpose(-1, -2)
    dL = -(At @ dA @ At) * strict
    dqt = scale * torch.einsum("cihv,chkv->cihk", doc, h)
    dkt = -torch.einsum("cihv,chkv->cihk", dX, h)
    dkb = torch.einsum("cjhv,chkv->cjhk", Vd, dh)
    dgl = (h * dh).sum(-1)                                                      # [NC,HV,K]
    dq_p = dqt * up
    dk_p = dkt * up + dkb * rest
    kbd = kbar * dkb
    dg_p = qt * dqt + kt * dkt - kbd
    dg_p[ar, ln - 1] += kbd.sum(1) + gl * dgl
    # gradients through Gamma / Aqk (torch_ref.py:286-324); E_ij = 2^(g_i - g_j)
    dn = torch.exp2(-gcum) * vm
    Wq = scale * dAqk * strict
    dLs = dL * strict
    bdL = dLs * bc.permute(0, 2, 1)[:, :, :, None]
    kdn, qup, kup = kc * dn, qc * up, kc * up
    dq_row = up * torch.einsum("chij,cjhk->cihk", Wq, kdn)
    Trow = up * torch.einsum("chij,cjhk->cihk", dLs, kdn)
    dk_row = bc[..., None] * Trow
    dk_col = dn * (torch.einsum("chij,cihk->cjhk", Wq, qup) + torch.einsum("chij,cihk->cjhk", bdL, kup))
    diag = torch.diagonal(dAqk, dim1=-2, dim2=-1).permute(0, 2, 1)[..., None]   # [NC,C,HV,1]
    dq_v = dq_p + dq_row + scale * diag * kc
    dk_v = dk_p + dk_row + dk_col + scale * diag * qc
    dgp = dg_p + qc * dq_row + kc * dk_row - kc * dk_col
    dbeta_g = (kc * Trow).sum(-1)
    dbeta = dbeta_w + dbeta_g
    dg = dgp.flip(1).cumsum(1).flip(1)                                          # padded rows hold zeros
    sc = lambda x: _scatter(x * (vm if x.dim() == 4 else valid[:, :, None].to(F64)), tab, TT)   # noqa: E731
    out = dict(dh=dh, dVd=sc(dVd), dh0=dh0, Vd=sc(Vd), dX=sc(dX), dbeta_w=sc(dbeta_w),
               dAqk=_scatter(dAqk.permute(0, 2, 1, 3), tab, TT), dL=_scatter(dL.permute(0, 2, 1, 3), tab, TT),
               dq_p=sc(dq_p), dk_p=sc(dk_p), dg_p=sc(dg_p), dq_v=sc(dq_v), dk_v=sc(dk_v), dgp=sc(dgp),
               dgl=dgl, fwd=fw)
    out["dq"] = out["dq_v"].reshape(B, T, HK, G, K).sum(3)
    out["dk"] = out["dk_v"].reshape(B, T, HK, G, K).sum(3)
    out["dv"] = out["dX"].reshape(B, T, HV, V)
    out["dg"] = sc(dg).reshape(B, T, HV, K)
    out["dbeta"] = sc(dbeta).reshape(B, T, HV)
    return out


# ---------------------------------------------------------------------------------------------
# full option surface on top of the chunk algebra, differentiable by autograd (for sizes where the
# token loop is too slow).  Pinned to ``recurrent_delta_rule`` in tests/test_oracle.py.
# ---------------------------------------------------------------------------------------------

def chunked_delta_rule(q, k, v, g, beta, *, scale=None, initial_state=None, output_final_state=False,
                       cu_seqlens=None, state_v_first=False, gate_mode="precomputed", A_log=None, dt_bias=None,
                       lower_bound=-5.0, beta_mode="precomputed", beta_scale=1.0,
                       use_qk_l2norm_in_kernel=False, output_norm=None):
    B, T, HK, K = q.shape
    HV = v.shape[2]
    q, k = q.to(F64), k.to(F64)
    if use_qk_l2norm_in_kernel:
        q, k = l2norm(q), l2norm(k)
    gd = gate_log_decay(g, gate_mode, A_log, dt_bias, lower_bound)
    if gd.dim() == 3:
        gd = gd.unsqueeze(-1).expand(B, T, HV, K)
    bt = beta_value(beta, beta_mode, beta_scale)
    fw = chunked_forward(q, k, v, gd, bt, scale=scale, initial_state=initial_state, cu_seqlens=cu_seqlens,
                         state_v_first=state_v_first)
    o = fw["o"].reshape(B, T, HV, -1)
    if output_norm is not None:
        o = gated_rmsnorm(o, output_norm.get("weight"), output_norm["gate"], output_norm.get("act", "silu"),
                          output_norm.get("eps", 1e-6))
    ht = None
    if output_final_state:
        ht = fw["ht"].transpose(-1, -2).contiguous() if state_v_first else fw["ht"]
    return o, ht


def rel_err(a, b):
    """(max|a-b| / max|b|, mean|a-b| / mean|b|) in float64: the reference's metric (tests/kda_common.py:40-44)."""
    a, b = a.detach().double(), b.detach().double()
    d = (a - b).abs()
    return ((d.max() / b.abs().max().clamp_min(1e-300)).item(), (d.mean() / b.abs().mean().clamp_min(1e-300)).item())

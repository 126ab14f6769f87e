"""One Python wrapper per kernel entry point: allocate the outputs with torch, fill the parameter struct, launch on
the current CUDA stream.  Same division of labour as the reference's kernel wrappers (e.g.
mogan_kda/ops/kimi_delta_rule/chunk/hopper/kkt_solve_kda.py:546-623): the kernels never allocate.

Every function here requires CUDA tensors; there is no CPU path.
"""
import torch

from . import _lib
from ._lib import STRUCTS
from .index import Layout

_DT = {torch.float32: _lib.MKDA_F32, torch.bfloat16: _lib.MKDA_BF16, torch.float16: _lib.MKDA_F16}
GATE_MODES = {"precomputed": _lib.MKDA_GATE_PRECOMPUTED, "eda": _lib.MKDA_GATE_EDA, "kimi": _lib.MKDA_GATE_KIMI,
              "gdn": _lib.MKDA_GATE_GDN}
ACTS = {"silu": _lib.MKDA_ACT_SILU, "swish": _lib.MKDA_ACT_SILU, "sigmoid": _lib.MKDA_ACT_SIGMOID}


def _dt(t):
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}; expected float32, bfloat16 or float16") from None


def _ptr(t, dtype=None):
    if t is None:
        return None
    if not t.is_cuda:
        raise RuntimeError("mogankda_b200 kernels need CUDA tensors (there is no CPU fallback)")
    if not t.is_contiguous():
        raise RuntimeError("kernel operands must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"expected {dtype}, got {t.dtype}")
    if t.data_ptr() % 16:
        raise RuntimeError("kernel operands must be 16-byte aligned (the kernels use 16-byte vector loads and bulk copies); "
                           "pass inputs through ops.aligned()")
    return t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _layout_struct(lay: Layout, HK, HV, segments=True):
    L = STRUCTS["MkdaLayout"]()
    L.TT, L.NC, L.HK, L.HV = lay.TT, lay.NC, HK, HV
    L.chunk_start, L.chunk_len = _ptr(lay.chunk_start), _ptr(lay.chunk_len)
    if segments:
        L.NS, L.seg_chunk_off = lay.NS, _ptr(lay.seg_chunk_off)
    else:
        L.NS, L.seg_chunk_off = lay.N, _ptr(lay.seq_chunk_off)
    return L


def aligned(t):
    """``t`` made contiguous and 16-byte aligned: a contiguous view at an odd storage offset (a slice of a flat parameter
    buffer, say) is copied.  The caller keeps the result alive until its launch is enqueued."""
    if t is None:
        return None
    t = t.contiguous()
    return t if t.data_ptr() % 16 == 0 else t.clone()


def _f32(t):
    return None if t is None else aligned(t.float())


def gate_cumsum_fwd(lay, x, mode, A_log, dt_bias, lower_bound, HV, beta_raw=None, beta_sigmoid=False, beta_scale=1.0):
    """x [B,T,HV,128] or [B,T,HV] -> (g_c fp32 [TT,HV,128], beta_e fp32 [TT,HV] or None)."""
    scalar = x.dim() == 3
    p = STRUCTS["MkdaGateFwd"]()
    p.L = _layout_struct(lay, 1, HV)
    alloc = torch.empty if lay.covers_all else torch.zeros
    g_c = alloc(lay.TT, HV, 128, dtype=torch.float32, device=x.device)
    p.x, p.x_dtype, p.scalar_gate = _ptr(x), _dt(x), int(scalar)
    A_log, dt_bias = _f32(A_log), _f32(dt_bias)
    p.A_log, p.dt_bias = _ptr(A_log), _ptr(dt_bias)
    p.mode = GATE_MODES[mode]
    p.lower_bound = float("-inf") if lower_bound is None else float(lower_bound)
    if mode in ("eda", "kimi") and lower_bound is None:
        raise ValueError(f"gate_mode={mode!r} needs lower_bound")
    if mode == "gdn" and lower_bound is None:
        p.lower_bound = -3.0e38
    beta_e = None
    if beta_raw is not None:
        beta_e = alloc(lay.TT, HV, dtype=torch.float32, device=x.device)
        p.beta_raw, p.beta_dtype = _ptr(beta_raw), _dt(beta_raw)
        p.beta_sigmoid, p.beta_scale, p.beta_out = int(beta_sigmoid), float(beta_scale), _ptr(beta_e)
    p.g_c = _ptr(g_c)
    _lib.call("mkda_gate_cumsum_fwd", p, _stream())
    return g_c, beta_e


def reduce_partials(part, rows, cols, group=1):
    out = torch.empty(cols // group, dtype=torch.float32, device=part.device)
    p = STRUCTS["MkdaReduce"]()
    p.rows, p.cols, p.group = rows, cols, group
    setattr(p, "in", _ptr(part, torch.float32))
    p.out = _ptr(out)
    _lib.call("mkda_reduce_partials", p, _stream())
    return out


def gate_bwd(lay, x, dgp, mode, A_log, dt_bias, lower_bound, HV, want_bias, want_alog):
    """-> (dx [like x], ddt_bias flat fp32 or None, dA_log fp32 [HV] or None)."""
    scalar = x.dim() == 3
    p = STRUCTS["MkdaGateBwd"]()
    p.L = _layout_struct(lay, 1, HV)
    dx = (torch.empty_like if lay.covers_all else torch.zeros_like)(x)
    p.x, p.x_dtype, p.scalar_gate = _ptr(x), _dt(x), int(scalar)
    A_log, dt_bias = _f32(A_log), _f32(dt_bias)
    p.A_log, p.dt_bias = _ptr(A_log), _ptr(dt_bias)
    p.mode = GATE_MODES[mode]
    p.lower_bound = -3.0e38 if lower_bound is None else float(lower_bound)
    p.dgp, p.dx, p.dx_dtype = _ptr(dgp, torch.float32), _ptr(dx), _dt(dx)
    width = HV if scalar else HV * 128
    rows = max(1, min(lay.NC, 256))
    p.part_rows = rows
    part_b = part_a = None
    if mode != "precomputed":
        if want_bias:
            part_b = torch.empty(rows, width, dtype=torch.float32, device=x.device)
            p.part_bias = _ptr(part_b)
        if want_alog:
            part_a = torch.empty(rows, width, dtype=torch.float32, device=x.device)
            p.part_alog = _ptr(part_a)
    _lib.call("mkda_gate_bwd", p, _stream())
    d_bias = reduce_partials(part_b, rows, width) if part_b is not None else None
    d_alog = reduce_partials(part_a, rows, width, 1 if scalar else 128) if part_a is not None else None
    return dx, d_bias, d_alog


def l2norm_rstd(x, eps=1e-6):
    """x [..., 128] -> rstd fp32 [rows]."""
    rows = x.numel() // 128
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    p = STRUCTS["MkdaL2Norm"]()
    p.x, p.dtype, p.rows, p.eps, p.rstd = _ptr(x), _dt(x), rows, eps, _ptr(rstd)
    _lib.call("mkda_l2norm_rstd", p, _stream())
    return rstd


def intra_fwd(lay, q, k, v, q_rstd, k_rstd, g_c, beta_e, scale, HK, HV, scalar_gate=False):
    dev = q.device
    A = torch.empty(lay.NC, HV, 32, 128, dtype=torch.float32, device=q.device)       # quarter tiles per (chunk, head)
    Aqk = torch.empty(lay.NC, HV, 32, 128, dtype=torch.float32, device=q.device)
    tile = lambda: torch.empty(lay.NC, HV, 64, 128, dtype=torch.float32, device=dev)      # noqa: E731  (32 KB per chunk, head)
    nw, u, kbar, qs = tile(), tile(), tile(), tile()          # nw^T and u^T chunk tiles; kbar and scale q 2^g row tiles
    gl = torch.empty(lay.NC, HV, 128, dtype=torch.float32, device=dev)
    p = STRUCTS["MkdaIntraFwd"]()
    p.L = _layout_struct(lay, HK, HV)
    p.q, p.k, p.v, p.qkv_dtype = _ptr(q), _ptr(k), _ptr(v), _dt(q)
    p.q_rstd, p.k_rstd = _ptr(q_rstd), _ptr(k_rstd)
    p.g_c, p.beta, p.scale = _ptr(g_c, torch.float32), _ptr(beta_e, torch.float32), scale
    p.scalar_gate = int(scalar_gate)
    p.A, p.Aqk, p.nw, p.u = _ptr(A), _ptr(Aqk), _ptr(nw), _ptr(u)
    p.kbar, p.qs, p.gl = _ptr(kbar), _ptr(qs), _ptr(gl)
    _lib.call("mkda_intra_fwd", p, _stream())
    return A, Aqk, nw, u, kbar, qs, gl


def warmup_chunks(lay, gl, HK, HV, threshold):
    """Warm-up truncation table of the segment pre-passes for a decay threshold in natural-log units (the reference's
    default is -10).  Returns int32 (warm_start [NS,HV], warm_end [NS,HV]); see ``MkdaWarmup`` in include/mkda.h."""
    dev = gl.device
    ws = torch.empty(lay.NS, HV, dtype=torch.int32, device=dev)
    we = torch.empty(lay.NS, HV, dtype=torch.int32, device=dev)
    p = STRUCTS["MkdaWarmup"]()
    p.L = _layout_struct(lay, HK, HV)
    p.gl, p.threshold_log2, p.warm_start, p.warm_end = _ptr(gl), float(threshold) * 1.4426950408889634, _ptr(ws), _ptr(we)
    _lib.call("mkda_warmup_chunks", p, _stream())
    return ws, we


def recur_fwd(lay, nw, u, kbar, gl, HK, HV, *, h0=None, seg_h0=None, state_v_first=False, store_h=True,
              store_vd=True, want_ht=True, want_transition=False, segments=True, warm_start=None):
    """Runs the serial state pass over the layout's segments (or whole sequences with ``segments=False``).
    ``warm_start`` (from ``warmup_chunks``) shortens a pass from zero.
    Returns (h [NC,HV] state tiles or None, Vd [NC,HV] chunk tiles or None, ht [NS,HV,128,128] or None, mt or None)."""
    dev = nw.device
    NS = lay.NS if segments else lay.N
    p = STRUCTS["MkdaRecurFwd"]()
    p.L = _layout_struct(lay, HK, HV, segments)
    p.nw, p.u, p.kbar, p.gl = _ptr(nw), _ptr(u), _ptr(kbar), _ptr(gl)
    p.h0, p.seg_h0, p.state_v_first = _ptr(h0, torch.float32), _ptr(seg_h0, torch.int32), int(state_v_first)
    h = torch.empty(lay.NC, HV, 128, 128, dtype=torch.float32, device=dev) if store_h else None
    Vd = torch.empty(lay.NC, HV, 64, 128, dtype=torch.float32, device=dev) if store_vd else None    # chunk tiles
    ht = torch.empty(NS, HV, 128, 128, dtype=torch.float32, device=dev) if want_ht else None
    mt = torch.empty(NS, HV, 128, 128, dtype=torch.float32, device=dev) if want_transition else None
    p.h, p.Vd, p.ht, p.want_transition, p.mt = _ptr(h), _ptr(Vd), _ptr(ht), int(want_transition), _ptr(mt)
    if warm_start is not None:
        if h0 is not None or store_h or store_vd or not segments:
            raise ValueError("warm_start applies to a pass from zero that stores nothing per chunk")
        p.warm_start = _ptr(warm_start, torch.int32)
    _lib.call("mkda_recur_fwd", p, _stream())
    return h, Vd, ht, mt


def out_fwd(lay, qs, Aqk, Vd, h, HK, HV, out_dtype, norm=None, keep_raw=False):
    """norm = None or dict(weight, gate, act, eps).  Returns (out [TT,HV,128], o_raw fp32 or None)."""
    dev = qs.device
    alloc = torch.empty if lay.covers_all else torch.zeros
    out = alloc(lay.TT, HV, 128, dtype=out_dtype, device=dev)
    o_raw = alloc(lay.TT, HV, 128, dtype=torch.float32, device=dev) if keep_raw else None
    p = STRUCTS["MkdaOutFwd"]()
    p.L = _layout_struct(lay, HK, HV)
    p.qs, p.Aqk, p.Vd, p.h = _ptr(qs), _ptr(Aqk), _ptr(Vd), _ptr(h)
    if norm is not None:
        w, gate = aligned(norm.get("weight")), aligned(norm["gate"])
        p.has_norm = 1
        if w is not None:
            p.norm_w, p.norm_w_dtype = _ptr(w), _dt(w)
        p.gate, p.gate_dtype = _ptr(gate), _dt(gate)
        p.act, p.eps = ACTS[norm.get("act", "silu")], float(norm.get("eps", 1e-6))
    p.o_raw, p.out, p.out_dtype = _ptr(o_raw), _ptr(out), _dt(out)
    _lib.call("mkda_out_fwd", p, _stream())
    return out, o_raw


def epilogue_bwd(dy, o_raw, weight, gate, act, eps):
    """-> (do fp32 [rows,128], dgate [like gate], dweight fp32 [128] or None)."""
    weight, gate = aligned(weight), aligned(gate)
    rows = o_raw.numel() // 128
    dev = o_raw.device
    d_o = torch.empty(rows, 128, dtype=torch.float32, device=dev)
    dgate = torch.empty_like(gate)
    nblk = min((rows + 63) // 64, _lib.MKDA_EPILOGUE_MAX_PART_ROWS)
    part = torch.empty(nblk, 128, dtype=torch.float32, device=dev) if weight is not None else None
    p = STRUCTS["MkdaEpilogueBwd"]()
    p.rows = rows
    p.dy, p.dy_dtype, p.o_raw = _ptr(dy), _dt(dy), _ptr(o_raw, torch.float32)
    if weight is not None:
        p.norm_w, p.norm_w_dtype = _ptr(weight), _dt(weight)
    p.gate, p.gate_dtype, p.act, p.eps = _ptr(gate), _dt(gate), ACTS[act], float(eps)
    p.d_o, p.dgate, p.dgate_dtype, p.part_w = _ptr(d_o), _ptr(dgate), _dt(dgate), _ptr(part)
    _lib.call("mkda_epilogue_bwd", p, _stream())
    dw = reduce_partials(part, nblk, 128) if part is not None else None
    return d_o, dgate, dw


def rows_strides(t):
    """(row stride, column stride) in elements if ``t`` [..., 128] can be addressed as rows x 128 with one stride per axis
    (contiguous tensors, and broadcast views such as the gradient autograd produces for ``o.sum()``), else None."""
    st, sz = t.stride(), t.shape
    row = None
    for d in range(t.dim() - 2, -1, -1):          # collapse the leading dims from the inside out
        if sz[d] == 1:
            continue
        if row is None:
            row, span = st[d], st[d] * sz[d]
        elif st[d] == span:
            span = st[d] * sz[d]
        else:
            return None
    row = 0 if row is None else row
    col = st[-1]
    if row < 0 or col < 0 or (col == 1 and row % 8) or t.storage_offset() * t.element_size() % 16:
        return None
    return row, col


def epilogue_bwd_tiles(lay, dy, o_raw, weight, gate, act, eps, HV):
    """Gated RMSNorm backward addressed through the chunk tables.  ``dy`` is read through its strides (see
    ``rows_strides``); anything else is made contiguous first.  -> (dO_t row tiles [NC,HV], dgate [like gate], dweight fp32
    [128] or None)."""
    weight, gate = aligned(weight), aligned(gate)
    dev = o_raw.device
    strides = rows_strides(dy)
    if strides is None:
        dy, strides = aligned(dy), (128, 1)
    dO_t = torch.empty(lay.NC, HV, 64, 128, dtype=torch.float32, device=dev)
    dgate = (torch.empty_like if lay.covers_all else torch.zeros_like)(gate)
    nblk = min(lay.NC * HV, _lib.MKDA_EPILOGUE_MAX_PART_ROWS)
    part = torch.empty(nblk, 128, dtype=torch.float32, device=dev) if weight is not None else None
    p = STRUCTS["MkdaEpilogueBwdTiles"]()
    p.L = _layout_struct(lay, 1, HV)
    if not dy.is_cuda:
        raise RuntimeError("mogankda_b200 kernels need CUDA tensors (there is no CPU fallback)")
    p.dy, p.dy_dtype, p.o_raw = dy.data_ptr(), _dt(dy), _ptr(o_raw, torch.float32)
    p.dy_row_stride, p.dy_col_stride = strides
    if weight is not None:
        p.norm_w, p.norm_w_dtype = _ptr(weight), _dt(weight)
    p.gate, p.gate_dtype, p.act, p.eps = _ptr(gate), _dt(gate), ACTS[act], float(eps)
    p.dO_t, p.dgate, p.dgate_dtype, p.part_rows, p.part_w = _ptr(dO_t), _ptr(dgate), _dt(dgate), nblk, _ptr(part)
    _lib.call("mkda_epilogue_bwd_tiles", p, _stream())
    dw = reduce_partials(part, nblk, 128) if part is not None else None
    return dO_t, dgate, dw


def bwd_dh(lay, d_o, kbar, qs, gl, Aqk, nw, HK, HV, *, dht=None, seg_dht=None,
           state_v_first=False, want_dh0=True, segments=True, store=True, dO_in_t=None, warm_end=None):
    """Reverse state chain.  dO comes either as rows ``d_o`` [TT,HV,128] or as the row tiles ``dO_in_t`` of
    ``epilogue_bwd_tiles``.  With ``store`` the per-chunk results leave as tiles for ``bwd_chunk``: dh (state tiles), dVd^T
    (chunk tiles) and, for row input, the staged dO (row tiles); a pre-pass that only wants the segment-level gradient
    passes ``store=False``.  Returns (dh, dVd_t, dO_t, dh0) with dO_t = ``dO_in_t`` when that was given."""
    dev = nw.device
    NS = lay.NS if segments else lay.N
    p = STRUCTS["MkdaBwdDh"]()
    p.L = _layout_struct(lay, HK, HV, segments)
    if dO_in_t is not None:
        p.dO_in_t = _ptr(dO_in_t, torch.float32)
    else:
        p.d_o, p.do_dtype = _ptr(d_o), _dt(d_o)
    p.kbar, p.qs, p.gl, p.Aqk, p.nw = _ptr(kbar), _ptr(qs), _ptr(gl), _ptr(Aqk), _ptr(nw)
    p.dht, p.seg_dht, p.state_v_first = _ptr(dht, torch.float32), _ptr(seg_dht, torch.int32), int(state_v_first)
    dh = dVd_t = None
    dO_t = dO_in_t
    if store:
        dh = torch.empty(lay.NC, HV, 128, 128, dtype=torch.float32, device=dev)
        dVd_t = torch.empty(lay.NC, HV, 64, 128, dtype=torch.float32, device=dev)
        if dO_in_t is None:
            dO_t = torch.empty(lay.NC, HV, 64, 128, dtype=torch.float32, device=dev)
    dh0 = torch.empty(NS, HV, 128, 128, dtype=torch.float32, device=dev) if want_dh0 else None
    p.dh, p.dVd_t, p.dO_t, p.dh0 = _ptr(dh), _ptr(dVd_t), _ptr(None if dO_in_t is not None else dO_t), _ptr(dh0)
    if warm_end is not None:
        if dht is not None or store or not segments:
            raise ValueError("warm_end applies to a reverse pass from zero that stores nothing per chunk")
        p.warm_end = _ptr(warm_end, torch.int32)
    _lib.call("mkda_bwd_dh", p, _stream())
    return dh, dVd_t, dO_t, dh0


def bwd_chunk(lay, q, k, v, q_rstd, k_rstd, g_c, beta_e, A, h, dh, Vd, dO_t, dVd_t, scale, HK, HV,
              beta_raw, beta_sigmoid, beta_scale, scalar_gate=False):
    """Every gradient local to a (chunk, v-head), in one kernel.  Returns (dq_v, dk_v, dgp, dbeta, dv); dq_v / dk_v are
    fp32 [64][128] tiles per (chunk, q/k head), already summed over the v-heads of the head, dgp per (chunk, v-head)."""
    dev = q.device
    alloc = torch.empty if lay.covers_all else torch.zeros
    z = lambda H: torch.empty(lay.NC, H, 64, 128, dtype=torch.float32, device=dev)      # noqa: E731  (fp32 [64][128] tiles)
    dq_v, dk_v, dgp = z(HK), z(HK), z(HV)
    dbeta = alloc(lay.TT, HV, dtype=beta_raw.dtype, device=dev)
    dv = alloc(lay.TT, HV, 128, dtype=v.dtype, device=dev)
    p = STRUCTS["MkdaBwdChunk"]()
    p.L = _layout_struct(lay, HK, HV)
    p.q, p.k, p.v, p.qkv_dtype, p.q_rstd, p.k_rstd = _ptr(q), _ptr(k), _ptr(v), _dt(q), _ptr(q_rstd), _ptr(k_rstd)
    p.g_c, p.beta = _ptr(g_c, torch.float32), _ptr(beta_e, torch.float32)
    p.A, p.h, p.dh, p.Vd, p.dO_t, p.dVd_t = _ptr(A), _ptr(h), _ptr(dh), _ptr(Vd), _ptr(dO_t), _ptr(dVd_t)
    p.scale, p.scalar_gate = scale, int(scalar_gate)
    p.beta_raw, p.beta_dtype = _ptr(beta_raw), _dt(beta_raw)
    p.beta_sigmoid, p.beta_scale = int(beta_sigmoid), float(beta_scale)
    p.dq_v, p.dk_v, p.dgp, p.dbeta, p.dbeta_dtype = _ptr(dq_v), _ptr(dk_v), _ptr(dgp), _ptr(dbeta), _dt(dbeta)
    p.dv = _ptr(dv)
    _lib.call("mkda_bwd_chunk", p, _stream())
    return dq_v, dk_v, dgp, dbeta, dv


def qk_grad_finish(lay, dq_v, dk_v, q, k, q_rstd, k_rstd, HK, HV):
    """dq_v, dk_v: fp32 [NC,HK,64,128] tiles (summed over the v-heads of each q/k head) -> gradients w.r.t. the raw q and
    k, [TT,HK,128] in their dtype."""
    if tuple(dq_v.shape[:2]) != (lay.NC, HK) or tuple(dk_v.shape[:2]) != (lay.NC, HK):
        raise ValueError("qk_grad_finish takes one tile per (chunk, q/k head)")
    alloc = torch.empty if lay.covers_all else torch.zeros
    dq = alloc(lay.TT, HK, 128, dtype=q.dtype, device=q.device)
    dk = alloc(lay.TT, HK, 128, dtype=k.dtype, device=k.device)
    p = STRUCTS["MkdaQkGrad"]()
    p.L = _layout_struct(lay, HK, HV)
    p.dq_v, p.dk_v = _ptr(dq_v, torch.float32), _ptr(dk_v, torch.float32)
    p.q, p.k, p.x_dtype, p.q_rstd, p.k_rstd = _ptr(q), _ptr(k), _dt(q), _ptr(q_rstd), _ptr(k_rstd)
    p.dq, p.dk = _ptr(dq), _ptr(dk)
    _lib.call("mkda_qk_grad_finish", p, _stream())
    return dq, dk


def state_combine(grp_seg_off, NG, NS, HV, hs, ms, carry=None, reverse=False, want_out=True, want_in=True):
    """-> (s_in [NS,HV,128,128] or None, s_out [NG,HV,128,128] or None); all in [K,V] orientation.
    ``hs=None`` folds the transitions alone (with ``carry`` = identity this composes them)."""
    dev = ms.device
    s_in = torch.empty(NS, HV, 128, 128, dtype=torch.float32, device=dev) if want_in else None
    s_out = torch.empty(NG, HV, 128, 128, dtype=torch.float32, device=dev) if want_out else None
    p = STRUCTS["MkdaCombine"]()
    p.NG, p.HV, p.grp_seg_off = NG, HV, _ptr(grp_seg_off, torch.int32)
    p.hs, p.ms, p.carry, p.reverse = _ptr(hs, torch.float32), _ptr(ms, torch.float32), _ptr(carry, torch.float32), int(reverse)
    p.s_in, p.s_out = _ptr(s_in), _ptr(s_out)
    _lib.call("mkda_state_combine", p, _stream())
    return s_in, s_out

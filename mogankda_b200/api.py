"""Public API: ``chunk_kda``, ``chunk_delta_rule``, ``chunk_gated_delta_rule``.

Same names, keyword surface, shapes, dtypes and error behaviour as the reference entry points
(mogan_kda/ops/kimi_delta_rule/chunk/__init__.py:297-355 and
mogan_kda/ops/gated_delta_rule/chunk/__init__.py:313-469); the work is done by the sm_100a kernels of libmkda.

Differences that are extensions, not changes of meaning:
  * q / k / v may also be float32 (the reference kernels take bf16 / fp16 only); outputs follow the input dtype.
  * context parallelism exists for the per-channel gate as well (``cp_context`` from ``mogankda_b200.cp``).
  * a scalar gate [B,T,HV] goes through the same kernels with the decay broadcast over the key channels.
  * ``warmup_threshold`` (natural-log units, e.g. -10.0; default None = exact): warm-up truncation of the segment
    pre-passes.  The reference applies it inside its intra-card context parallelism with a fixed -10
    (mogan_kda/ops/gated_delta_rule/chunk/cp/preprocess.py:121-139); here it is an explicit choice because it is an
    approximation (relative error e^threshold in the states handed between segments).
"""
import torch

from . import ops
from .index import get_layout

CHUNK_SIZE = 64
# When the segment chooser (index.wants_segments) decides to cut, sequences are cut into segments of exactly this many
# chunks whose serial recurrences run concurrently (state + transition pre-pass, prefix combine, main pass).  A constant,
# so that a prefix of a sequence is always cut exactly like the same tokens inside the longer sequence.
AUTO_SEGMENT_CHUNKS = 32


class _DeltaRuleFunction(torch.autograd.Function):
    """forward: gate + cumsum (+beta) -> L2 statistics -> WY preparation -> state pass -> output (+epilogue).
    backward: epilogue -> reverse state chain -> WY / state gradients -> intra-chunk gradients -> gate / L2 / GVA."""

    @staticmethod
    def forward(ctx, q, k, v, x, beta, A_log, dt_bias, initial_state, ep_w, ep_gate, cfg):
        B, T, HK, K = q.shape
        HV = v.shape[2]
        dev = q.device
        lay = get_layout(B, T, cfg["cu_seqlens"], dev, cfg["seg_chunks"], HV if cfg["seg_auto"] else 0,
                         2.5 if cfg["warmup"] is None else 1.25)
        cp = cfg["cp_context"]
        scale = cfg["scale"]
        q_rstd = k_rstd = None
        if cfg["l2"]:
            q_rstd, k_rstd = ops.l2norm_rstd(q), ops.l2norm_rstd(k)
        g_c, beta_e = ops.gate_cumsum_fwd(lay, x, cfg["gate_mode"], A_log, dt_bias, cfg["lower_bound"], HV,
                                          beta_raw=beta, beta_sigmoid=cfg["beta_mode"] == "sigmoid",
                                          beta_scale=cfg["beta_scale"])
        A, Aqk, nw, u, kbar, qs, gl = ops.intra_fwd(lay, q, k, v, q_rstd, k_rstd, g_c, beta_e, scale, HK, HV,
                                                    scalar_gate=x.dim() == 3)
        vf = cfg["state_v_first"]
        need_ht = cfg["output_final_state"]
        ms = m_first = warm_end = None
        if lay.segmented or cp is not None:
            # pre-pass from zero: per-segment (state, transition); then the true entering state of every segment
            warm_start = None
            if cfg["warmup"] is not None:
                warm_start, warm_end = ops.warmup_chunks(lay, gl, HK, HV, cfg["warmup"])
            _, _, hs, ms = ops.recur_fwd(lay, nw, u, kbar, gl, HK, HV, store_h=False, store_vd=False,
                                         want_transition=True, warm_start=warm_start)
            carry = None
            if initial_state is not None:
                carry = initial_state.transpose(-1, -2).contiguous() if vf else initial_state
            if cp is not None:
                carry, m_first = cp.forward_carry(hs, ms, carry, lay, HV)
            s_in, _ = ops.state_combine(lay.grp_seg_off, lay.NG, lay.NS, HV, hs, ms, carry=carry, want_out=False)
            h, Vd, ht_seg, _ = ops.recur_fwd(lay, nw, u, kbar, gl, HK, HV, h0=s_in, state_v_first=False,
                                             want_ht=need_ht)
            ht = None
            if need_ht:
                ht = ht_seg.index_select(0, torch.nonzero(lay.seg_last >= 0).flatten())
                if vf:
                    ht = ht.transpose(-1, -2).contiguous()
        else:
            h, Vd, ht, _ = ops.recur_fwd(lay, nw, u, kbar, gl, HK, HV, h0=initial_state, state_v_first=vf,
                                         want_ht=need_ht)
        norm = None
        if cfg["has_ep"]:
            norm = dict(weight=ep_w, gate=ep_gate, act=cfg["ep_act"], eps=cfg["ep_eps"])
        need_bwd = any(ctx.needs_input_grad[:10])
        out_dtype = torch.float32 if cfg["has_ep"] else q.dtype
        out, o_raw = ops.out_fwd(lay, qs, Aqk, Vd, h, HK, HV, out_dtype, norm=norm,
                                 keep_raw=cfg["has_ep"] and need_bwd)
        if need_bwd:
            ctx.save_for_backward(q, k, v, x, beta, A_log, dt_bias, initial_state, ep_w, ep_gate, q_rstd, k_rstd,
                                  g_c, beta_e, A, Aqk, nw, h, o_raw, ms, kbar, qs, gl, Vd, m_first, warm_end)
        ctx.cfg, ctx.lay, ctx.dims = cfg, lay, (B, T, HK, HV)
        ctx.set_materialize_grads(False)
        return out.view(B, T, HV, 128), ht

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dy, dht):
        (q, k, v, x, beta, A_log, dt_bias, initial_state, ep_w, ep_gate, q_rstd, k_rstd, g_c, beta_e, A, Aqk, nw, h,
         o_raw, ms, kbar, qs, gl, Vd, m_first, warm_end) = ctx.saved_tensors
        cfg, lay = ctx.cfg, ctx.lay
        B, T, HK, HV = ctx.dims
        scale, vf, cp = cfg["scale"], cfg["state_v_first"], cfg["cp_context"]
        if dy is None:
            dy = torch.zeros(B, T, HV, 128, dtype=torch.float32 if cfg["has_ep"] else q.dtype, device=q.device)
        if not cfg["has_ep"]:
            dy = ops.aligned(dy)      # with the epilogue, dy is read through its strides (a broadcast gradient is not copied)
        dw = dgate = d_o = dO_in = None
        if cfg["has_ep"]:      # dO leaves the epilogue backward in the tile form the tensor-core kernels fetch
            dO_in, dgate, dw = ops.epilogue_bwd_tiles(lay, dy, o_raw, ep_w, ep_gate, cfg["ep_act"], cfg["ep_eps"], HV)
            if dw is not None:
                dw = dw.to(ep_w.dtype)
        else:
            d_o = dy
        if dht is not None:
            dht = ops.aligned(dht.float())
        need_dh0 = initial_state is not None and ctx.needs_input_grad[7]
        if lay.segmented or cp is not None:
            # pre-pass from zero: only the gradient entering each segment is wanted, nothing per chunk is stored
            _, _, _, dloc = ops.bwd_dh(lay, d_o, kbar, qs, gl, Aqk, nw, HK, HV, store=False, dO_in_t=dO_in,
                                       warm_end=warm_end)
            carry = None
            if dht is not None:
                carry = dht.transpose(-1, -2).contiguous() if vf else dht
            if cp is not None:
                carry = cp.backward_carry(dloc, ms, carry, lay, HV, m_first)
            g_in, dh0 = ops.state_combine(lay.grp_seg_off, lay.NG, lay.NS, HV, dloc, ms, carry=carry, reverse=True,
                                          want_out=need_dh0 or cp is not None)
            dh, dVd_t, dO_t, _ = ops.bwd_dh(lay, d_o, kbar, qs, gl, Aqk, nw, HK, HV, dht=g_in, want_dh0=False,
                                            dO_in_t=dO_in)
            if cp is not None:
                dh0 = cp.finish_backward(dh0)
            if dh0 is not None and vf:
                dh0 = dh0.transpose(-1, -2).contiguous()
        else:
            dh, dVd_t, dO_t, dh0 = ops.bwd_dh(lay, d_o, kbar, qs, gl, Aqk, nw, HK, HV, dht=dht,
                                              state_v_first=vf, want_dh0=need_dh0, dO_in_t=dO_in)
        dq_v, dk_v, dgp, dbeta, dv = ops.bwd_chunk(lay, q, k, v, q_rstd, k_rstd, g_c, beta_e, A, h, dh, Vd, dO_t, dVd_t,
                                                   scale, HK, HV, beta, cfg["beta_mode"] == "sigmoid", cfg["beta_scale"],
                                                   scalar_gate=x.dim() == 3)
        dx, d_bias, d_alog = ops.gate_bwd(lay, x, dgp, cfg["gate_mode"], A_log, dt_bias, cfg["lower_bound"], HV,
                                          want_bias=dt_bias is not None and ctx.needs_input_grad[6],
                                          want_alog=A_log is not None and ctx.needs_input_grad[5])
        dq, dk = ops.qk_grad_finish(lay, dq_v, dk_v, q, k, q_rstd, k_rstd, HK, HV)
        dq, dk = dq.view_as(q), dk.view_as(k)
        dv = dv.view(B, T, HV, 128)
        if d_alog is not None:
            d_alog = d_alog.view_as(A_log).to(A_log.dtype)
        if d_bias is not None:
            d_bias = d_bias.view_as(dt_bias).to(dt_bias.dtype)
        if not need_dh0:
            dh0 = None
        return (dq, dk, dv, dx, dbeta.view_as(beta), d_alog, d_bias, dh0, dw, dgate, None)


def _check_common(q, k, v, g, beta, initial_state, cu_seqlens):
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise RuntimeError("mogankda_b200 runs on CUDA tensors only (no CPU fallback)")
    assert q.dtype == k.dtype == v.dtype, "q, k, v must share a dtype"
    assert q.dtype in (torch.bfloat16, torch.float16, torch.float32), "q, k, v must be bfloat16, float16 or float32"
    assert q.shape == k.shape and q.dim() == 4 and v.dim() == 4, "q, k [B,T,HK,K]; v [B,T,HV,V]"
    assert q.shape[-1] == v.shape[-1] == 128, "head dims must be 128"
    assert v.shape[:2] == q.shape[:2], "q and v disagree on [B,T]"
    assert v.shape[2] % q.shape[2] == 0, "GVA needs HV % HK == 0"
    assert g.shape[:3] == v.shape[:3] and (g.dim() == 3 or (g.dim() == 4 and g.shape[3] == 128)), \
        "g must be [B,T,HV] or [B,T,HV,128]"
    assert beta.shape == v.shape[:3], "beta must be [B,T,HV]"
    if cu_seqlens is not None:
        if q.shape[0] != 1:
            raise ValueError(f"The batch size is expected to be 1 rather than {q.shape[0]} when using `cu_seqlens`.")
        n = cu_seqlens.numel() - 1
    else:
        n = q.shape[0]
    if initial_state is not None:
        assert initial_state.dtype == torch.float32, "initial_state must be float32"
        if initial_state.shape[0] != n:
            raise ValueError(f"The number of initial states is expected to be equal to the number of input "
                             f"sequences, i.e., {n} rather than {initial_state.shape[0]}.")
        assert tuple(initial_state.shape[1:]) == (v.shape[2], 128, 128), "initial_state must be [N,HV,128,128]"


def chunk_delta_rule(q, k, v, g, beta, *, scale=None, initial_state=None, output_final_state=False, cu_seqlens=None,
                     state_v_first=False, gate_mode="precomputed", A_log=None, dt_bias=None, lower_bound=-5.0,
                     beta_mode="precomputed", beta_scale=1.0, use_qk_l2norm_in_kernel=False, output_norm=None,
                     auto_cp=True, cp_context=None, warmup_threshold=None):
    """Unified delta rule (mogan_kda/ops/kimi_delta_rule/chunk/__init__.py:297-349).

    q, k [B,T,HK,128]; v [B,T,HV,128]; g [B,T,HV,128] per-channel or [B,T,HV] scalar gate input (raw pre-activation
    unless ``gate_mode="precomputed"``, then the natural-log per-token decay, contract g >= -5); beta [B,T,HV].
    Returns ``(o, final_state)``: o in q.dtype, or float32 when ``output_norm`` is given.
    """
    if cp_context is not None and getattr(cp_context, "cu_seqlens", None) is not None:
        cu_seqlens = cp_context.cu_seqlens      # the context's local boundaries replace the argument (reference :87-120)
    _check_common(q, k, v, g, beta, initial_state, cu_seqlens)
    if gate_mode not in ops.GATE_MODES:
        raise ValueError(f"unknown gate_mode {gate_mode!r}")
    if beta_mode not in ("precomputed", "sigmoid"):
        raise ValueError(f"unknown beta_mode {beta_mode!r}")
    if gate_mode == "gdn":
        assert A_log is not None, "gate_mode='gdn' needs A_log"
        if lower_bound is None and g.dim() == 4:
            lower_bound = -5.0          # the per-channel kernels rely on g >= -5 (reference :338-339)
    if gate_mode == "eda":
        assert A_log is not None and lower_bound is not None, "gate_mode='eda' needs A_log and lower_bound"
    if gate_mode == "kimi":
        assert lower_bound is not None, "gate_mode='kimi' needs lower_bound"
    ep = output_norm
    if ep is not None and ep.get("act", "silu") not in ops.ACTS:
        raise ValueError(f"unknown act {ep.get('act')!r}")
    if cp_context is not None and q.shape[0] != 1:
        raise ValueError("inter-card CP requires B==1 (varlen).")
    if warmup_threshold is not None and not float(warmup_threshold) < 0.0:
        raise ValueError("warmup_threshold must be negative (natural-log units, e.g. -10.0) or None")
    B, T = q.shape[:2]
    cfg = dict(scale=float(q.shape[-1] ** -0.5 if scale is None else scale), output_final_state=output_final_state,
               cu_seqlens=cu_seqlens, state_v_first=state_v_first, gate_mode=gate_mode, lower_bound=lower_bound,
               beta_mode=beta_mode, beta_scale=float(beta_scale), l2=use_qk_l2norm_in_kernel, has_ep=ep is not None,
               ep_act=None if ep is None else ep.get("act", "silu"),
               ep_eps=None if ep is None else ep.get("eps", 1e-6),
               seg_chunks=AUTO_SEGMENT_CHUNKS if (cp_context is not None or auto_cp) else 0,
               seg_auto=cp_context is None,          # without CP the chooser in index.wants_segments decides
               cp_context=cp_context, warmup=None if warmup_threshold is None else float(warmup_threshold))
    ep_gate = None if ep is None else ep["gate"]
    ep_w = None if ep is None else ep.get("weight")
    # contiguous and 16-byte aligned operands (a contiguous view at an odd storage offset is copied): what the kernels'
    # vector loads and bulk copies need; the small parameter tensors are realigned where they are used
    al = ops.aligned
    return _DeltaRuleFunction.apply(al(q), al(k), al(v), al(g), al(beta), A_log, dt_bias, al(initial_state), ep_w,
                                    al(ep_gate), cfg)


def chunk_kda(q, k, v, g, beta, **kwargs):
    """Kimi Delta Attention: ``chunk_delta_rule`` restricted to a per-channel gate g [B,T,HV,128]
    (mogan_kda/ops/kimi_delta_rule/chunk/__init__.py:352-355)."""
    assert g.dim() == 4, "chunk_kda needs a per-channel gate g [B, T, HV, K]; use chunk_gated_delta_rule for scalar gates"
    return chunk_delta_rule(q, k, v, g, beta, **kwargs)


def chunk_gated_delta_rule(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                           use_qk_l2norm_in_kernel=False, cu_seqlens=None, head_first=False, state_v_first=False,
                           auto_cp=True, enable_fwd_cp_cache=True, cp_context=None, force_intra_cp=False,
                           warmup_threshold=None):
    """Scalar-gate delta rule (mogan_kda/ops/gated_delta_rule/chunk/__init__.py:313-469).  g [B,T,HV] is the per-token
    natural-log decay, beta [B,T,HV] the effective beta."""
    assert q.dtype == k.dtype == v.dtype
    assert not head_first, "head_first=True is not supported."
    assert v.shape[2] % k.shape[2] == 0, "num_qk_heads must be divisible to num_v_heads."
    assert g.dim() == 3, "chunk_gated_delta_rule takes a scalar gate g [B, T, HV]"
    return chunk_delta_rule(q, k, v, g, beta, scale=scale, initial_state=initial_state,
                            output_final_state=output_final_state, cu_seqlens=cu_seqlens,
                            state_v_first=state_v_first, use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel,
                            auto_cp=auto_cp or force_intra_cp, cp_context=cp_context, warmup_threshold=warmup_threshold)

"""``fla.ops.kda.chunk_kda``-style call surface on top of :func:`mogankda_b200.chunk_kda`.

Existing callers of flash-linear-attention's KDA op can switch by changing the import.  The keyword mapping is the one
the reference documents for its own compatibility wrapper (tests/ref_kda.py:189-218):

  * ``use_gate_in_kernel=False``  -> ``gate_mode="precomputed"`` (g is the per-token natural-log decay);
    ``True`` with a ``lower_bound`` -> ``"kimi"`` (``lower_bound * sigmoid(exp(A_log) (g + dt_bias))``, A_log optional);
    ``True`` without one           -> ``"gdn"``  (``-exp(A_log) softplus(g + dt_bias)``, clamped at -5 as the kernels need).
  * ``use_beta_sigmoid_in_kernel`` -> ``beta_mode="sigmoid"``, scaled by 2 when ``allow_neg_eigval``.
  * ``safe_gate`` only picks a kernel variant in FLA; it does not change the math and is accepted and ignored.
  * Arguments with no counterpart (``cp_context`` of FLA's own type, ``use_graph``, ``max_num_seqs``, ``cu_seqlens_cpu``,
    ``disable_recompute``, ``return_intermediate_states``, a ``chunk_size`` other than 64) raise ``NotImplementedError``
    when set to a non-default value.
"""
from .api import chunk_kda as _chunk_kda

__all__ = ["chunk_kda"]


def chunk_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
              use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False, A_log=None, dt_bias=None, safe_gate=False,
              lower_bound=None, cu_seqlens=None, use_beta_sigmoid_in_kernel=False, allow_neg_eigval=False,
              state_v_first=False, **unsupported):
    for name, val in unsupported.items():
        if val not in (None, False, 64):
            raise NotImplementedError(f"chunk_kda argument {name!r} is not supported")
    mode, kw = "precomputed", {}
    if use_gate_in_kernel:
        mode = "kimi" if lower_bound is not None else "gdn"
        kw = dict(A_log=A_log, dt_bias=dt_bias)
    if lower_bound is not None:
        kw["lower_bound"] = lower_bound
    return _chunk_kda(q, k, v, g, beta, scale=scale, initial_state=initial_state, output_final_state=output_final_state,
                      cu_seqlens=cu_seqlens, state_v_first=state_v_first, gate_mode=mode,
                      beta_mode="sigmoid" if use_beta_sigmoid_in_kernel else "precomputed",
                      beta_scale=2.0 if allow_neg_eigval else 1.0, use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel, **kw)

"""B200-native chunked Kimi Delta Attention / gated delta rule (drop-in for ``mogan_kda``'s chunk API).

    from mogankda_b200 import chunk_kda, chunk_delta_rule, chunk_gated_delta_rule

The kernels live in ``libmkda.so`` (hand-written CUDA for sm_100a, C ABI declared in ``include/mkda.h``); build it with
``python -m mogankda_b200.build``.  There is no CPU or library fallback: calling the API without the built library or
with CPU tensors raises.
"""
from .api import chunk_delta_rule, chunk_gated_delta_rule, chunk_kda  # noqa: F401

__all__ = ["chunk_kda", "chunk_delta_rule", "chunk_gated_delta_rule"]

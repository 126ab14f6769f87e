"""B200-native chunked Kimi Delta Attention / gated delta rule (drop-in for ``mogan_kda``'s chunk API).

    from mogankda_b200 import chunk_kda, chunk_delta_rule, chunk_gated_delta_rule

The kernels live in ``libmkda.so`` (hand-written CUDA for sm_100a, C ABI declared in ``include/mkda.h``); build it with
``python -m mogankda_b200.build``.  There is no CPU or library fallback: calling the API without the built library or
with CPU tensors raises.

Every wait inside a kernel is bounded; ``device_status()`` (synchronises) tells whether one has expired since the last
``device_status_clear()``: poll it where the host synchronises anyway, e.g. at the end of a step.
"""
from ._lib import device_status, device_status_clear  # noqa: F401
from .api import chunk_delta_rule, chunk_gated_delta_rule, chunk_kda  # noqa: F401

__all__ = ["chunk_kda", "chunk_delta_rule", "chunk_gated_delta_rule", "device_status", "device_status_clear"]

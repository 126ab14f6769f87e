"""Chunk / segment tables (host logic).

Mirrors what ``prepare_chunk_indices`` / ``prepare_chunk_offsets`` give the reference kernels
(mogan_kda/utils/index.py:93-116): chunks never straddle a sequence and are numbered sequence-major.  On top of
that a sequence can be cut into *segments* of a fixed number of chunks; the serial recurrences then run per segment
and the segments are stitched by the state-combine kernel (the same mechanism carries context parallelism across
GPUs).  The segment length never depends on the sequence length, so a prefix of a sequence is segmented exactly
like the full sequence (bitwise prefix invariance).
"""
from dataclasses import dataclass, field

import torch

CHUNK = 64


@dataclass
class Layout:
    B: int
    T: int
    N: int                      # sequences
    NC: int                     # chunks
    NS: int                     # segments
    NG: int                     # groups of segments (= sequences)
    chunk_start: torch.Tensor   # int32 [NC]
    chunk_len: torch.Tensor     # int32 [NC]
    seg_chunk_off: torch.Tensor  # int32 [NS+1]
    grp_seg_off: torch.Tensor   # int32 [N+1]
    seq_chunk_off: torch.Tensor  # int32 [N+1]  (segments == sequences view)
    seg_first: torch.Tensor     # int32 [NS]: sequence id if the segment opens its sequence, else -1
    seg_last: torch.Tensor      # int32 [NS]: sequence id if the segment closes its sequence, else -1
    segmented: bool
    covers_all: bool            # every token of [0, B*T) belongs to a sequence
    host: dict = field(default_factory=dict)

    @property
    def TT(self):
        return self.B * self.T


def build_tables(B, T, cu, seg_chunks=0):
    """Pure-python tables.  ``cu`` is a list of ints or None; ``seg_chunks`` = chunks per segment (0 = no cut)."""
    if cu is None:
        bounds = [(b * T, b * T + T) for b in range(B)]
    else:
        if B != 1:
            raise ValueError("cu_seqlens requires B == 1")
        if len(cu) < 1 or cu[0] != 0 or any(cu[i + 1] < cu[i] for i in range(len(cu) - 1)) or cu[-1] > T:
            raise ValueError("cu_seqlens must start at 0, be non-decreasing and end within T")
        bounds = list(zip(cu[:-1], cu[1:]))
    start, length, seq_off = [], [], [0]
    seg_off, grp_off, seg_first, seg_last = [0], [0], [], []
    for n, (s, e) in enumerate(bounds):
        nc = -(-(e - s) // CHUNK)
        for i in range(nc):
            start.append(s + i * CHUNK)
            length.append(min(CHUNK, e - s - i * CHUNK))
        base = seq_off[-1]
        seq_off.append(base + nc)
        step = seg_chunks if seg_chunks and seg_chunks > 0 else max(nc, 1)
        cuts = list(range(0, nc, step)) if nc else [0]
        for j, c0 in enumerate(cuts):
            seg_off.append(base + min(c0 + step, nc))
            seg_first.append(n if j == 0 else -1)
            seg_last.append(n if j == len(cuts) - 1 else -1)
        grp_off.append(len(seg_off) - 1)
    covered = sum(e - s for s, e in bounds)
    return dict(chunk_start=start, chunk_len=length, seq_chunk_off=seq_off, seg_chunk_off=seg_off,
                grp_seg_off=grp_off, seg_first=seg_first, seg_last=seg_last, N=len(bounds),
                covers_all=covered == B * T)


def _sm_count(device=None):
    """SMs of the device the kernels will run on (the library asks the runtime in the same way for its persistent
    grids); 148 (B200) when no device is visible, so that the host logic stays testable on CPU."""
    if torch.cuda.is_available():
        return torch.cuda.get_device_properties(device if device is not None else torch.cuda.current_device()).multi_processor_count
    return 148


def wants_segments(chunks_per_seq, HV, seg_chunks, sm_count=None, cost_ratio=2.5):
    """Segment-parallelism chooser: should sequences be cut into segments of ``seg_chunks`` chunks?

    The serial kernels run one CTA per (sequence or segment, v-head), one chunk step after another.  Uncut, their time is
    set by the longest sequence (critical path) unless there is so much work that the even share of all chunk steps over
    the SMs is longer still.  Cutting spreads the steps evenly but adds the state + transition pre-pass in the forward
    direction and a second pass in the backward direction, about 2.5 x the serial work over a layer step, plus the prefix
    combine.  So: cut when the critical path is longer than 2.5 even shares (``cost_ratio``; 1.25 when the caller allows
    warm-up truncation, which shortens the two extra passes to a few chunks wherever the gate decays).  Decided from the
    lengths alone (host), never from data; it plays the role of the reference's intra-card CP decision
    (mogan_kda/ops/gated_delta_rule/chunk/cp/context.py:252-283, cp/autocp/decision.py:54-123)."""
    longest = max(chunks_per_seq, default=0)
    if seg_chunks <= 0 or longest <= seg_chunks:
        return False
    even_share = sum(chunks_per_seq) * HV / (sm_count or _sm_count())
    return longest > cost_ratio * even_share


# Entries: (static key, the cu_seqlens tensor itself, its version counter, layout).  The entry keeps the tensor alive
# and is matched by identity, as the reference's ``tensor_cache`` does (mogan_kda/utils/index.py:33-85): a fresh
# ``cu_seqlens`` that happens to land at the address of a freed one (the caching allocator hands blocks back in that
# way every step) can never hit an old entry, and an in-place edit changes the version.
_cache = []
_CACHE_MAX = 16


def get_layout(B, T, cu_seqlens, device, seg_chunks=0, auto_heads=0, cost_ratio=2.5):
    """Device tables, cached on (shape, identity + version of ``cu_seqlens``, segment policy) like the reference's
    ``tensor_cache`` (mogan_kda/utils/index.py:19-90).  A cache miss reads ``cu_seqlens`` back to the host.
    ``auto_heads`` > 0 lets ``wants_segments`` decide, for that many v-heads, whether ``seg_chunks`` is applied."""
    key = (B, T, str(device), seg_chunks, auto_heads, cost_ratio)
    ver = None if cu_seqlens is None else cu_seqlens._version
    for i, (k, ref, v, lay) in enumerate(_cache):
        if k == key and ref is cu_seqlens and v == ver:
            if i != len(_cache) - 1:
                _cache.append(_cache.pop(i))          # most recently used last
            return lay
    cu = None if cu_seqlens is None else [int(x) for x in cu_seqlens.tolist()]
    if auto_heads > 0:
        lens = [T] * B if cu is None else [e - s for s, e in zip(cu[:-1], cu[1:])]
        if not wants_segments([-(-n // CHUNK) for n in lens], auto_heads, seg_chunks, _sm_count(device) if str(device) != "cpu" else None,
                              cost_ratio):
            seg_chunks = 0
    tb = build_tables(B, T, cu, seg_chunks)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=device)      # noqa: E731
    lay = Layout(B=B, T=T, N=tb["N"], NC=len(tb["chunk_start"]), NS=len(tb["seg_first"]), NG=tb["N"],
                 chunk_start=i32(tb["chunk_start"]), chunk_len=i32(tb["chunk_len"]),
                 seg_chunk_off=i32(tb["seg_chunk_off"]), grp_seg_off=i32(tb["grp_seg_off"]),
                 seq_chunk_off=i32(tb["seq_chunk_off"]), seg_first=i32(tb["seg_first"]), seg_last=i32(tb["seg_last"]),
                 segmented=len(tb["seg_first"]) != tb["N"], covers_all=tb["covers_all"], host=tb)
    if len(_cache) >= _CACHE_MAX:
        _cache.pop(0)
    _cache.append((key, cu_seqlens, ver, lay))
    return lay

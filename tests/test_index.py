"""CPU: chunk / segment tables (host logic) against the oracle's table and hand-checked cases."""
import pytest

from mogankda_b200.index import build_tables
from oracle import kda_oracle as orc

VARLEN = [0, 1, 98, 354, 504, 704]          # lengths 1, 97, 256, 150, 200 (the reference's standard ragged layout)


@pytest.mark.parametrize("B,T,cu", [(2, 300, None), (1, 704, VARLEN), (1, 64, None), (1, 65, None), (3, 1, None)])
def test_chunks_match_oracle(B, T, cu):
    import torch
    tb = build_tables(B, T, cu)
    ref = orc.chunk_table(B, T, None if cu is None else torch.tensor(cu))
    assert tb["chunk_start"] == ref["start"] and tb["chunk_len"] == ref["length"]
    assert tb["seq_chunk_off"] == ref["seq_off"]
    assert tb["seg_chunk_off"] == ref["seq_off"]          # no cutting: segments are the sequences
    assert tb["covers_all"]


def test_segments_have_fixed_length_and_cover_each_sequence():
    tb = build_tables(1, 10000, [0, 100, 5000, 10000], seg_chunks=32)
    # doc 0: 2 chunks -> 1 segment; doc 1: 77 chunks -> 3 segments; doc 2: 79 chunks -> 3 segments
    assert tb["grp_seg_off"] == [0, 1, 4, 7]
    so = tb["seg_chunk_off"]
    assert so == [0, 2, 34, 66, 79, 111, 143, 158]
    assert tb["seg_first"] == [0, 1, -1, -1, 2, -1, -1]
    assert tb["seg_last"] == [0, -1, -1, 1, -1, -1, 2]
    # a prefix of doc 1 is cut at the same places
    tp = build_tables(1, 4000, [0, 100, 4000], seg_chunks=32)
    assert tp["seg_chunk_off"] == [0, 2, 34, 63] and tp["seg_chunk_off"][:3] == so[:3]


def test_padding_tokens_and_empty_sequences():
    tb = build_tables(1, 200, [0, 50, 50, 130])
    assert not tb["covers_all"]
    assert tb["seq_chunk_off"] == [0, 1, 1, 3]
    assert tb["seg_chunk_off"] == [0, 1, 1, 3]
    assert tb["chunk_len"] == [50, 64, 16]


def test_bad_cu_seqlens():
    with pytest.raises(ValueError):
        build_tables(2, 100, [0, 100])
    with pytest.raises(ValueError):
        build_tables(1, 100, [0, 120])
    with pytest.raises(ValueError):
        build_tables(1, 100, [0, 60, 40])


def test_segment_chooser():
    from mogankda_b200.index import wants_segments
    # nothing longer than a segment: never cut
    assert not wants_segments([8, 20, 32], 32, 32, sm_count=148)
    # one long sequence, few heads: the GPU cannot be filled without cutting
    assert wants_segments([1024], 32, 32, sm_count=148)
    # many documents of similar length fill the GPU on their own
    assert not wants_segments([40] * 100, 32, 32, sm_count=148)
    # a packed batch dominated by one document: its chain is far longer than the even share
    assert wants_segments([940] + [4] * 34, 32, 32, sm_count=148)
    # the same long document among enough other work is left alone
    assert not wants_segments([100] + [30] * 300, 32, 32, sm_count=148)
    assert not wants_segments([], 32, 32, sm_count=148) and not wants_segments([1000], 32, 0, sm_count=148)
    # four 256-chunk sequences x 16 heads leave SMs idle, but cutting would cost more than it spreads
    assert not wants_segments([256] * 4, 16, 32, sm_count=148)
    # ... unless warm-up truncation makes the extra passes short (the caller then passes the lower cost ratio)
    assert wants_segments([256] * 4, 16, 32, sm_count=148, cost_ratio=1.25)
    assert not wants_segments([40] * 100, 32, 32, sm_count=148, cost_ratio=1.25)


def test_layout_cache_is_keyed_on_tensor_identity_not_on_its_address():
    """A training loop builds a fresh ``cu_seqlens`` every step and the allocator usually hands back the block of the one
    just freed: same address, same shape, version 0, different boundaries.  The cached tables must not be reused."""
    import torch
    from mogankda_b200 import index
    a = torch.tensor([0, 100, 256], dtype=torch.int32)
    la = index.get_layout(1, 256, a, "cpu")
    assert index.get_layout(1, 256, a, "cpu") is la                    # same tensor object: a hit
    ptr = a.data_ptr()
    del a
    fresh = [torch.tensor([0, 30, 256], dtype=torch.int32) for _ in range(4)]      # one of them may reuse the block
    for b in fresh:
        lb = index.get_layout(1, 256, b, "cpu")
        assert lb is not la and lb.chunk_len.tolist()[0] == 30
    assert any(e[1] is not None and e[1].data_ptr() == ptr for e in index._cache)  # the entry keeps its tensor alive
    c = fresh[0]
    c[1] = 64                                                           # in-place edit: the version counter moves
    assert index.get_layout(1, 256, c, "cpu").chunk_len.tolist()[0] == 64

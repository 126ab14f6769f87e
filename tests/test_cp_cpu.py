"""CPU, world_size 2 over gloo: the host logic of cross-GPU context parallelism (rank-level fold, all-gather, prefix
fold in rank order) with the combine kernel replaced by a torch restatement of its contract."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HV, D = 2, 8


def combine_ref(grp_seg_off, NG, NS, HV_, hs, ms, carry=None, reverse=False, want_out=True, want_in=True):
    """Contract of mkda_state_combine: X enters segment s (stored in s_in[s]) and leaves as M_s X + H_s (forward) or
    M_s^T X + H_s (reverse, segments walked from the last to the first)."""
    off = [int(x) for x in grp_seg_off.tolist()]
    s_in = torch.zeros(NS, HV_, D, D, dtype=ms.dtype)
    s_out = torch.zeros(NG, HV_, D, D, dtype=ms.dtype)
    for g in range(NG):
        X = torch.zeros(HV_, D, D, dtype=ms.dtype) if carry is None else carry[g].clone()
        order = range(off[g], off[g + 1])
        for s in (reversed(order) if reverse else order):
            s_in[s] = X
            M = ms[s].transpose(-1, -2) if reverse else ms[s]
            X = M @ X + (0 if hs is None else hs[s])
        s_out[g] = X
    return (s_in if want_in else None), (s_out if want_out else None)


class FakeLayout:
    def __init__(self, ns):
        self.NG, self.NS = 1, ns
        self.grp_seg_off = torch.tensor([0, ns], dtype=torch.int32)


def _worker(rank, world, port, seg_counts):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mogankda_b200 import cp as cpmod, ops
        ops.state_combine = combine_ref
        g = torch.Generator().manual_seed(7)
        total = sum(seg_counts)
        H = torch.randn(total, HV, D, D, generator=g, dtype=torch.float64)
        M = torch.randn(total, HV, D, D, generator=g, dtype=torch.float64) * 0.3
        Dl = torch.randn(total, HV, D, D, generator=g, dtype=torch.float64)
        h0 = torch.randn(1, HV, D, D, generator=g, dtype=torch.float64)
        dht = torch.randn(1, HV, D, D, generator=g, dtype=torch.float64)
        lo = sum(seg_counts[:rank])
        hi = lo + seg_counts[rank]
        ctx = cpmod.ContextParallel(dist.group.WORLD)
        lay = FakeLayout(seg_counts[rank])
        got, m_first = ctx.forward_carry(H[lo:hi].contiguous(), M[lo:hi].contiguous(), h0 if rank == 0 else None, lay, HV)
        # a second layer runs its forward pass on the SAME context before the first one's backward pass: the first
        # layer's transition must come back from its own saved value, not from whatever the context saw last
        ctx.forward_carry(H[lo:hi].flip(0).contiguous(), (M[lo:hi] * 0.5).contiguous(), None, lay, HV)
        X = h0[0].clone()
        for s in range(lo):
            X = M[s] @ X + H[s]
        torch.testing.assert_close(got[0], X, rtol=1e-10, atol=1e-10)
        gotb = ctx.backward_carry(Dl[lo:hi].contiguous(), M[lo:hi].contiguous(), dht if rank == world - 1 else None, lay, HV,
                                  m_first)
        G = dht[0].clone()
        for s in reversed(range(hi, total)):
            G = M[s].transpose(-1, -2) @ G + Dl[s]
        torch.testing.assert_close(gotb[0], G, rtol=1e-10, atol=1e-10)
        dist.barrier()          # every rank reaches its asserts before anyone leaves (a failing rank cannot hang peers)
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("seg_counts", [(3, 2), (1, 4)])
def test_context_parallel_prefix_fold_two_ranks(seg_counts):
    mp.spawn(_worker, args=(2, _free_port(), seg_counts), nprocs=2, join=True)


class PackedLayout:
    def __init__(self, groups):
        self.NG, self.NS = len(groups), sum(groups)
        off = [0]
        for n in groups:
            off.append(off[-1] + n)
        self.grp_seg_off = torch.tensor(off, dtype=torch.int32)


def _packed_worker(rank, world, port):
    """Three sequences over two ranks: A (2 segments) on rank 0, B cut into 1 + 2 segments across the boundary, C
    (1 segment) on rank 1."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mogankda_b200 import cp as cpmod, ops
        ops.state_combine = combine_ref
        g = torch.Generator().manual_seed(11)
        rnd = lambda *s: torch.randn(*s, HV, D, D, generator=g, dtype=torch.float64)      # noqa: E731
        H, M, Dl = rnd(6), rnd(6) * 0.3, rnd(6)          # segments: A0 A1 B0 | B1 B2 C0
        h0, dht = rnd(3), rnd(3)                         # per global sequence A, B, C
        fold = lambda X, segs: [X := M[s] @ X + H[s] for s in segs][-1]                    # noqa: E731
        foldb = lambda G, segs: [G := M[s].transpose(-1, -2) @ G + Dl[s] for s in reversed(segs)][-1]   # noqa: E731
        if rank == 0:
            ctx = cpmod.ContextParallel(dist.group.WORLD, pre_num_ranks=0, post_num_ranks=1)
            lay, lo, hi = PackedLayout([2, 1]), 0, 3
            got, mf = ctx.forward_carry(H[lo:hi].contiguous(), M[lo:hi].contiguous(), h0[:2].clone(), lay, HV)
            torch.testing.assert_close(got, h0[:2])
            gb = ctx.backward_carry(Dl[lo:hi].contiguous(), M[lo:hi].contiguous(), dht[:2].clone(), lay, HV, mf)
            torch.testing.assert_close(gb[0], dht[0])
            torch.testing.assert_close(gb[1], foldb(dht[1].clone(), [3, 4]), rtol=1e-10, atol=1e-10)
            d = torch.ones(2, HV, D, D, dtype=torch.float64)
            assert ctx.finish_backward(d) is d
        else:
            ctx = cpmod.ContextParallel(dist.group.WORLD, pre_num_ranks=1, post_num_ranks=0)
            lay, lo, hi = PackedLayout([2, 1]), 3, 6
            junk = torch.cat([torch.full_like(h0[:1], 7.0), h0[2:3]])      # row 0 belongs to rank 0 and must be ignored
            got, mf = ctx.forward_carry(H[lo:hi].contiguous(), M[lo:hi].contiguous(), junk, lay, HV)
            torch.testing.assert_close(got[0], fold(h0[1].clone(), [2]), rtol=1e-10, atol=1e-10)
            torch.testing.assert_close(got[1], h0[2])
            gb = ctx.backward_carry(Dl[lo:hi].contiguous(), M[lo:hi].contiguous(), dht[1:].clone(), lay, HV, mf)
            torch.testing.assert_close(gb, dht[1:])
            d = ctx.finish_backward(torch.ones(2, HV, D, D, dtype=torch.float64))
            assert float(d[0].abs().sum()) == 0 and float(d[1].min()) == 1
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_context_parallel_packed_batch_two_ranks():
    mp.spawn(_packed_worker, args=(2, _free_port()), nprocs=2, join=True)


@pytest.mark.parametrize("cu,world", [([0, 300, 1200, 1400, 2048], 4), ([0, 2048], 4), ([0, 512, 1024, 2048], 4),
                                      ([0, 5, 6, 100, 101, 128], 2), ([0, 64, 192], 3)])
def test_partition_tokens_against_brute_force(cu, world):
    """Every field of the equal-token split, derived token by token."""
    from mogankda_b200.cp import partition_tokens
    total = cu[-1]
    part = total // world
    seq_of = [next(i for i in range(len(cu) - 1) if cu[i] <= t < cu[i + 1]) for t in range(total)]
    rank_of = [t // part for t in range(total)]
    for r in range(world):
        got = partition_tokens(torch.tensor(cu), world, r)
        toks = [t for t in range(total) if rank_of[t] == r]
        assert (got["rank_start"], got["rank_end"]) == (toks[0], toks[-1] + 1)
        bounds = [0] + [i + 1 for i in range(part) if i == part - 1 or seq_of[toks[i]] != seq_of[toks[i + 1]]]
        assert got["cu_seqlens"] == bounds
        f, l = seq_of[toks[0]], seq_of[toks[-1]]
        ranks_f = {rank_of[t] for t in range(cu[f], cu[f + 1])}
        ranks_l = {rank_of[t] for t in range(cu[l], cu[l + 1])}
        assert got["pre_num_ranks"] == r - min(ranks_f) and got["post_num_ranks"] == max(ranks_l) - r
        assert got["is_first_rank"] == (min(ranks_f) == r) and got["is_last_rank"] == (max(ranks_l) == r)
        assert got["pre_num_conv_tokens"] == toks[0] - cu[f]
    with pytest.raises(AssertionError):
        partition_tokens([0, 10, 60 * world + 1], world, 0)


# ---------------------------------------------------------------------------------------------------------------
# failure detection, injected on the host: no GPU is involved, nothing faults or hangs
# ---------------------------------------------------------------------------------------------------------------
def _failing_worker(rank, world, port, result):
    """Rank 1 raises before the all-gather.  Rank 0 must come out of the collective with an exception within the
    group's short timeout instead of waiting for ever; it reports what it saw through ``result``."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    from mogankda_b200 import cp as cpmod, ops
    ops.state_combine = combine_ref
    ctx = cpmod.ContextParallel(dist.group.WORLD)
    if rank == 1:
        os._exit(0)                      # the rank is gone before it joins the collective (no destroy, no barrier)
    g = torch.Generator().manual_seed(3)
    H = torch.randn(2, HV, D, D, generator=g, dtype=torch.float64)
    M = torch.randn(2, HV, D, D, generator=g, dtype=torch.float64)
    try:
        ctx.forward_carry(H, M, None, FakeLayout(2), HV)
        result.put("no error")
    except Exception as e:               # noqa: BLE001  (gloo reports a lost peer as RuntimeError / DistBackendError)
        result.put(type(e).__name__)


def test_a_rank_that_leaves_before_the_exchange_gives_its_peer_an_error_not_a_hang():
    ctxmp = mp.get_context("spawn")
    result = ctxmp.Queue()
    procs = [ctxmp.Process(target=_failing_worker, args=(r, 2, port, result)) for port in [_free_port()] for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=90)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()
    assert not alive, "a rank hung in the collective after its peer had left"
    assert result.get(timeout=5) != "no error"


def test_cp_argument_errors_follow_the_reference():
    """Token count not divisible by the world size, ranks outside the group, B != 1: the documented errors
    (mogan_kda/ops/gated_delta_rule/chunk/cp/context.py:202-205)."""
    from mogankda_b200 import cp as cpmod

    class Comm:
        rank, world = 1, 2

    with pytest.raises(AssertionError, match="divisible by world_size"):
        cpmod.partition_tokens([0, 100, 129], 2, 0)
    with pytest.raises(ValueError, match="outside the group"):
        cpmod.ContextParallel(comm=Comm(), pre_num_ranks=2)
    with pytest.raises(ValueError, match="outside the group"):
        cpmod.ContextParallel(comm=Comm(), post_num_ranks=1)
    with pytest.raises(AssertionError, match="divisible by world_size"):
        cpmod.build_cp_context(torch.tensor([0, 7, 13]), comm=Comm())

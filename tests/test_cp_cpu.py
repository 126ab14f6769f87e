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


def _worker(rank, world, port, seg_counts, fail_rank):
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
        if rank == fail_rank:
            with pytest.raises(ValueError):
                bad = FakeLayout(seg_counts[rank])
                bad.NG = 2
                ctx.forward_carry(H[lo:hi], M[lo:hi], h0, bad, HV)
        got = ctx.forward_carry(H[lo:hi].contiguous(), M[lo:hi].contiguous(), h0 if rank == 0 else None, lay, HV)
        X = h0[0].clone()
        for s in range(lo):
            X = M[s] @ X + H[s]
        torch.testing.assert_close(got[0], X, rtol=1e-10, atol=1e-10)
        gotb = ctx.backward_carry(Dl[lo:hi].contiguous(), M[lo:hi].contiguous(), dht if rank == world - 1 else None, lay, HV)
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
    mp.spawn(_worker, args=(2, _free_port(), seg_counts, 1), nprocs=2, join=True)

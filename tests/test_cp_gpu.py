"""GPU: context parallelism end to end.  The ranks are emulated one after the other in a single process (record /
replay of the all-gather, see ReplayComm): no kernel ever waits on another kernel.  The NCCL path itself is exercised by
``bench.py --workload longdoc`` under torchrun."""
import os
import pytest
import torch

import mogankda_b200 as mk
from mogankda_b200.cp import ContextParallel
from oracle import kda_oracle as orc
from tests.common import check, make_inputs

pytestmark = pytest.mark.gpu


class ReplayComm:
    """Emulates W ranks in one process without concurrency.  What a rank contributes to each all-gather depends only on
    its own slice (rank-level state / transition / state-gradient pairs), so the ranks are run twice: the first pass
    records every contribution (and hands back zeros), the second replays the complete gathers."""

    def __init__(self, world):
        self.world, self.rec, self.replay = world, {}, False

    def view(self, rank):
        outer = self

        class _V:
            world = outer.world

            def __init__(self):
                self.rank, self.calls = rank, 0

            def all_gather(self, flat_out, flat_in):
                key = self.calls
                self.calls += 1
                if not outer.replay:
                    outer.rec[(rank, key)] = flat_in.clone()
                    flat_out.zero_()
                else:
                    flat_out.copy_(torch.cat([outer.rec[(r, key)] for r in range(outer.world)]))
        return _V()


def _problem(T, seed=31, dtype=torch.float32):
    lv, do, dht, opts, _ = make_inputs(B=1, T=T, HK=1, HV=2, dtype=dtype, gate="kimi", epi=None, seed=seed)
    return lv, do, dht, opts


def _slice(lv, a, b):
    return {n: (t[:, a:b].contiguous() if t.dim() >= 3 and t.shape[0] == 1 and t.shape[1] > 128 else t) for n, t in lv.items()}


def _run_rank(ctx, lv, do, dht, opts, rank, world, a, b, out, **extra):
    if True:
        x = {n: t.clone().requires_grad_(True) for n, t in _slice(lv, a, b).items()}
        o, ht = mk.chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], gate_mode="kimi", A_log=x["A_log"],
                             dt_bias=x["dt_bias"], beta_mode="sigmoid", beta_scale=2.0, use_qk_l2norm_in_kernel=True,
                             initial_state=x["h0"], output_final_state=True, cp_context=ctx, **extra)
        loss = (o.double() * do[:, a:b].double()).sum()
        if rank == world - 1:
            loss = loss + (ht.double() * dht.double()).sum()
        names = ("q", "k", "v", "g", "beta", "h0")
        grads = torch.autograd.grad(loss, [x[n] for n in names], allow_unused=True)
        out[rank] = dict(o=o.detach(), ht=ht.detach(), **{"d" + n: g for n, g in zip(names, grads)})


@pytest.mark.parametrize("world,T,warmup", [(2, 640, None), (3, 64 * 45, None), (3, 64 * 45, -10.0)])
def test_context_parallel_matches_global_oracle(world, T, warmup):
    """``warmup`` = -10: the segment pre-passes are truncated where the decay allows (the reference's intra-card default);
    the result must stay inside the same tolerance against the exact global oracle."""
    lv, do, dht, opts = _problem(T)
    ref = {}
    x = {n: t.double().clone().requires_grad_(True) for n, t in lv.items()}
    o, ht = orc.chunked_delta_rule(x["q"], x["k"], x["v"], x["g"], x["beta"], gate_mode="kimi", A_log=x["A_log"],
                                   dt_bias=x["dt_bias"], beta_mode="sigmoid", beta_scale=2.0, use_qk_l2norm_in_kernel=True,
                                   initial_state=x["h0"], output_final_state=True)
    names = ("q", "k", "v", "g", "beta", "h0")
    grads = torch.autograd.grad((o * do.double()).sum() + (ht * dht.double()).sum(), [x[n] for n in names])
    ref = dict(o=o, ht=ht, **{"d" + n: g for n, g in zip(names, grads)})
    per = (T // 64 // world) * 64
    bounds = [(r * per, T if r == world - 1 else (r + 1) * per) for r in range(world)]
    comm, out = ReplayComm(world), [None] * world
    for replay in (False, True):
        comm.replay = replay
        for r, (a, b) in enumerate(bounds):
            _run_rank(ContextParallel(comm=comm.view(r)), lv, do, dht, opts, r, world, a, b, out, warmup_threshold=warmup)
    for r, (a, b) in enumerate(bounds):
        check(f"o[{r}]", out[r]["o"], ref["o"][:, a:b])
        for n in ("dq", "dk", "dv", "dg", "dbeta"):
            check(f"{n}[{r}]", out[r][n], ref[n][:, a:b])
    check("ht", out[-1]["ht"], ref["ht"])
    check("dh0", out[0]["dh0"], ref["dh0"])


def test_packed_batch_split_over_ranks_matches_global_oracle():
    """Four sequences in 2048 tokens over four emulated ranks: one sequence spans three ranks, one rank holds the tail of a
    sequence, a whole sequence and the head of the next.  Initial / final states and their gradients have one row per
    local sequence; rows of sequences that started on an earlier rank are ignored / zero."""
    from mogankda_b200.cp import build_cp_context, partition_tokens
    cu, world = [0, 300, 1200, 1400, 2048], 4
    lv, do, dht, opts, _ = make_inputs(B=1, T=cu[-1], HK=1, HV=2, cu=cu, dtype=torch.float32, gate="kimi", epi=None, seed=5)
    kw = dict(gate_mode="kimi", beta_mode="sigmoid", beta_scale=2.0, use_qk_l2norm_in_kernel=True, output_final_state=True)
    names = ("q", "k", "v", "g", "beta", "h0")
    x = {n: t.double().clone().requires_grad_(True) for n, t in lv.items()}
    o, ht = orc.chunked_delta_rule(x["q"], x["k"], x["v"], x["g"], x["beta"], A_log=x["A_log"], dt_bias=x["dt_bias"],
                                   initial_state=x["h0"], cu_seqlens=opts["cu_seqlens"], **kw)
    grads = torch.autograd.grad((o * do.double()).sum() + (ht * dht.double()).sum(), [x[n] for n in names])
    ref = dict(o=o, ht=ht, **{"d" + n: g for n, g in zip(names, grads)})

    parts = [partition_tokens(cu, world, r) for r in range(world)]
    seqs = []                                          # global sequence ids of every rank's local sequences
    for p in parts:
        ids = [i for i in range(len(cu) - 1) if cu[i] < p["rank_end"] and cu[i + 1] > p["rank_start"]]
        assert len(ids) == len(p["cu_seqlens"]) - 1
        seqs.append(ids)
    comm, out = ReplayComm(world), [None] * world
    cu_dev = torch.tensor(cu, dtype=torch.int32, device="cuda")
    for replay in (False, True):
        comm.replay = replay
        for r, p in enumerate(parts):
            a, b, ids = p["rank_start"], p["rank_end"], seqs[r]
            ctx = build_cp_context(cu_dev, comm=comm.view(r), conv1d_kernel_size=4)
            assert ctx.pre_num_ranks == p["pre_num_ranks"] and ctx.cu_seqlens.tolist() == p["cu_seqlens"]
            assert ctx.conv_halo_tokens == min(3, p["pre_num_conv_tokens"])
            loc = {n: t.clone().requires_grad_(True) for n, t in _slice(lv, a, b).items()}
            h0 = lv["h0"][ids].clone()
            if not p["is_first_rank"]:
                h0[0] = 123.0                          # not this rank's input: must not matter
            h0.requires_grad_(True)
            o, ht = mk.chunk_kda(loc["q"], loc["k"], loc["v"], loc["g"], loc["beta"], A_log=loc["A_log"],
                                 dt_bias=loc["dt_bias"], initial_state=h0, cp_context=ctx, **kw)
            dht_loc = dht[ids].clone()
            if not p["is_last_rank"]:
                dht_loc[-1] = 0                        # the sequence ends on a later rank: its final state is not here
            loss = (o.double() * do[:, a:b].double()).sum() + (ht.double() * dht_loc.double()).sum()
            g = torch.autograd.grad(loss, [loc[n] for n in names[:5]] + [h0])
            out[r] = dict(o=o.detach(), ht=ht.detach(), **{"d" + n: t for n, t in zip(names, g)})
    for r, p in enumerate(parts):
        a, b, ids = p["rank_start"], p["rank_end"], seqs[r]
        check(f"o[{r}]", out[r]["o"], ref["o"][:, a:b])
        for n in ("dq", "dk", "dv", "dg", "dbeta"):
            check(f"{n}[{r}]", out[r][n], ref[n][:, a:b])
        for j, s in enumerate(ids):
            if cu[s + 1] <= b:                         # the sequence ends here: this rank reports its final state
                check(f"ht[{r}][{j}]", out[r]["ht"][j], ref["ht"][s])
            if cu[s] >= a:                             # it starts here: this rank owns the gradient of its initial state
                check(f"dh0[{r}][{j}]", out[r]["dh0"][j], ref["dh0"][s])
            else:
                assert float(out[r]["dh0"][j].abs().max()) == 0.0


def test_two_layers_share_one_context():
    """A model passes ONE context to every layer, and all forward passes run before the first backward pass.  Each
    layer's backward exchange must use that layer's own transition, so two different problems pushed through the same
    context object, then differentiated together, must each match their own global oracle."""
    world, T = 2, 640
    probs = [_problem(T, seed=41), _problem(T, seed=43)]
    names = ("q", "k", "v", "g", "beta")
    kw = dict(gate_mode="kimi", beta_mode="sigmoid", beta_scale=2.0, use_qk_l2norm_in_kernel=True)
    refs = []
    for lv, do, _, _ in probs:
        x = {n: t.double().clone().requires_grad_(True) for n, t in lv.items()}
        o, _ = orc.chunked_delta_rule(x["q"], x["k"], x["v"], x["g"], x["beta"], A_log=x["A_log"], dt_bias=x["dt_bias"], **kw)
        grads = torch.autograd.grad((o * do.double()).sum(), [x[n] for n in names])
        refs.append(dict(o=o, **{"d" + n: g for n, g in zip(names, grads)}))
    per = T // world
    comm, out = ReplayComm(world), {}
    for replay in (False, True):
        comm.replay = replay
        for r in range(world):
            a, b = r * per, (r + 1) * per
            ctx = ContextParallel(comm=comm.view(r))            # one context for both layers of this rank
            xs, loss = [], 0.0
            for lv, do, _, _ in probs:
                x = {n: t.clone().requires_grad_(True) for n, t in _slice(lv, a, b).items()}
                o, _ = mk.chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], A_log=x["A_log"], dt_bias=x["dt_bias"],
                                    cp_context=ctx, **kw)
                loss = loss + (o.double() * do[:, a:b].double()).sum()
                xs.append((x, o))
            grads = torch.autograd.grad(loss, [x[n] for x, _ in xs for n in names])
            for i, (x, o) in enumerate(xs):
                out[(r, i)] = dict(o=o.detach(), **{"d" + n: grads[i * len(names) + j] for j, n in enumerate(names)})
    for r in range(world):
        a, b = r * per, (r + 1) * per
        for i in range(2):
            for n in ("o", "dq", "dk", "dv", "dg", "dbeta"):
                check(f"layer {i} {n}[{r}]", out[(r, i)][n], refs[i][n][:, a:b])

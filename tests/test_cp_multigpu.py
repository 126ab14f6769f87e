"""GPU, 2+ devices: context parallelism over NCCL with one process per GPU, checked against the single-GPU result of the
same document.  Skipped on a single-GPU box (the single-process emulation in test_cp_gpu.py covers the logic there)."""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu

CHILD = textwrap.dedent("""
    import os, sys, torch, torch.distributed as dist
    sys.path.insert(0, os.environ["MKDA_ROOT"])
    import mogankda_b200 as mk
    from mogankda_b200.cp import ContextParallel
    from oracle import kda_oracle as orc
    from tests.common import make_inputs
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl")
    T = 64 * 40 * world
    lv, do, dht, opts, _ = make_inputs(B=1, T=T, HK=1, HV=2, dtype=torch.bfloat16, gate="kimi", epi=None, seed=5, device="cuda")
    kw = dict(gate_mode="kimi", beta_mode="sigmoid", beta_scale=2.0, use_qk_l2norm_in_kernel=True, output_final_state=True)
    names = ("q", "k", "v", "g", "beta")

    def run(a, b, ctx):
        x = {n: (t[:, a:b].contiguous() if n in names else t).clone().requires_grad_(True) for n, t in lv.items()}
        o, ht = mk.chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], A_log=x["A_log"], dt_bias=x["dt_bias"],
                             initial_state=x["h0"], cp_context=ctx, **kw)
        loss = (o.double() * do[:, a:b].double()).sum()
        if ctx is None or rank == world - 1:
            loss = loss + (ht.double() * dht.double()).sum()
        g = torch.autograd.grad(loss, [x[n] for n in names])
        return o.detach(), ht.detach(), [t.detach() for t in g]

    per = T // world
    o, ht, g = run(rank * per, (rank + 1) * per, ContextParallel(dist.group.WORLD))
    o_ref, ht_ref, g_ref = run(0, T, None)                      # every rank also runs the whole document alone
    sl = slice(rank * per, (rank + 1) * per)
    worst = 0.0
    for name, a, b in [("o", o, o_ref[:, sl])] + [("d" + n, x, y[:, sl]) for n, x, y in zip(names, g, g_ref)]:
        mx, mn = orc.rel_err(a.float(), b.float())
        worst = max(worst, mx)
        assert mx <= 2e-3 + 2.0 ** -8 and mn <= 2e-3 + 1.6e-3, (rank, name, mx, mn)
    if rank == world - 1:
        mx, mn = orc.rel_err(ht, ht_ref)
        assert mx <= 2e-3 and mn <= 2e-3, ("ht", mx, mn)

    # the same tokens as a packed batch of three sequences, the middle one crossing the rank boundary
    from mogankda_b200.cp import build_cp_context
    cu = torch.tensor([0, 700, T - 1120, T], dtype=torch.int32, device="cuda")

    def run_packed(a, b, ctx):
        x = {n: t[:, a:b].contiguous().clone().requires_grad_(True) for n, t in lv.items() if n in names}
        o, _ = mk.chunk_kda(x["q"], x["k"], x["v"], x["g"], x["beta"], A_log=lv["A_log"], dt_bias=lv["dt_bias"],
                            cu_seqlens=None if ctx is not None else cu, cp_context=ctx, **dict(kw, output_final_state=False))
        g = torch.autograd.grad((o.double() * do[:, a:b].double()).sum(), [x[n] for n in names])
        return o.detach(), [t.detach() for t in g]

    ctx = build_cp_context(cu, group=dist.group.WORLD)
    assert ctx.pre_num_ranks == rank and ctx.num_seqs == 2
    o, g = run_packed(rank * per, (rank + 1) * per, ctx)
    o_ref, g_ref = run_packed(0, T, None)
    for name, a, b in [("o", o, o_ref[:, sl])] + [("d" + n, x, y[:, sl]) for n, x, y in zip(names, g, g_ref)]:
        mx, mn = orc.rel_err(a.float(), b.float())
        worst = max(worst, mx)
        assert mx <= 2e-3 + 2.0 ** -8 and mn <= 2e-3 + 1.6e-3, (rank, "packed " + name, mx, mn)
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank} ok worst {worst:.2e}")
""")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_context_parallel_over_nccl_matches_single_gpu(tmp_path):
    world = 2
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "cp_child.py"
    script.write_text(CHILD)
    env = dict(os.environ, MKDA_ROOT=root, MASTER_ADDR="127.0.0.1", MASTER_PORT="29577", WORLD_SIZE=str(world))
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r} ok" in out, out[-2000:]

#!/usr/bin/env python
"""Benchmark of one KDA / GDN layer forward + backward through the public API.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload packed|1b|longdoc|gdn] [--impl reference]

Default workload = the configuration the headline metric is quoted on: 8 rows x 8192 tokens of packed short documents
(lognormal lengths, median 500, sigma 1.0, cut at row boundaries) per GPU, HK=16 / HV=32 / D=128, bf16 q/k/v, eda
gate + sigmoid beta (x2) + in-kernel L2 + silu gated-RMSNorm epilogue, loss = o.sum().  Data is synthetic and seeded;
no dataset is involved.  With N > 1 (launched by torchrun) every rank runs its own packed batch (weak scaling, no
collective on the data path); ``--workload longdoc`` instead shards ONE document across the ranks with context
parallelism (one NCCL all-gather of per-rank (state, transition) pairs per pass).

One JSON line is printed by rank 0.  ``value`` is measured with inputs resident in HBM; ``e2e`` is the same metric
with pinned host inputs copied in and the loss read back inside the timed region.  ``roofline`` describes the kernel
that took the largest share of the timed region, timed with CUDA events on the launching stream.
``--impl reference`` times the CPU restatement of the reference's torch oracle (tests/ref_kda.py of the reference) on
the host cores on a bounded sample of the same workload.
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HK, HV, D = 16, 32, 128


# ----------------------------------------------------------------------------------------------------------
# synthetic workloads
# ----------------------------------------------------------------------------------------------------------
def packed_cu(rows=8, row_len=8192, median=500.0, sigma=1.0, seed=0):
    g = torch.Generator().manual_seed(seed)
    cu = [0]
    for r in range(rows):
        end = (r + 1) * row_len
        while cu[-1] < end:
            n = int(math.exp(math.log(median) + sigma * torch.randn((), generator=g).item()))
            cu.append(min(cu[-1] + max(n, 1), end))
    return cu


def make_workload(name, rank, device, pin=False, tokens=65536):
    """Returns (host tensors dict, options dict, description).  ``tokens``: length of this rank's slice of the long
    document (``longdoc`` only)."""
    g = torch.Generator().manual_seed(rank)
    r = lambda *s: torch.randn(*s, generator=g)                               # noqa: E731
    if name in ("packed", "1b"):
        if name == "packed":
            hk, hv, cu = HK, HV, packed_cu(seed=rank)
            T = cu[-1]
        else:
            hk, hv, cu, T = 8, 16, [0, 3000, 5000, 8192], 8192
        t = dict(q=r(1, T, hk, D).bfloat16(), k=r(1, T, hk, D).bfloat16(), v=r(1, T, hv, D).bfloat16(),
                 g=r(1, T, hv, D), beta=r(1, T, hv), ep_gate=r(1, T, hv, D).bfloat16(),
                 A_log=torch.zeros(hv), dt_bias=torch.zeros(hv, D), ep_w=torch.ones(D),
                 cu=torch.tensor(cu, dtype=torch.int32))
        opts = dict(gate_mode="eda", lower_bound=-5.0, beta_mode="sigmoid", beta_scale=2.0, l2=True, epi="silu")
        desc = (f"packed short documents: {len(cu) - 1} docs in 8x8192 tokens, lognormal(median 500, sigma 1.0)"
                if name == "packed" else "1B shape: T=8192, docs 3000/2000/3192")
        dims = dict(tokens=T, HK=hk, HV=hv, docs=len(cu) - 1)
    elif name == "longdoc":
        T = tokens
        t = dict(q=r(1, T, HK, D).bfloat16(), k=r(1, T, HK, D).bfloat16(), v=r(1, T, HV, D).bfloat16(),
                 g=r(1, T, HV, D), beta=r(1, T, HV), A_log=r(HV) * 0.1, dt_bias=r(HV, D) * 0.1)
        opts = dict(gate_mode="kimi", lower_bound=-5.0, beta_mode="sigmoid", beta_scale=1.0, l2=True, epi=None)
        desc, dims = f"one document, {T} tokens of it on this GPU, kimi gate", dict(tokens=T, HK=HK, HV=HV, docs=1)
    elif name == "gdn":
        B, T, H = 4, 16384, 16
        A_log, x = r(H) * 0.1, r(B, T, H)
        gdec = torch.clamp(-A_log.exp() * torch.nn.functional.softplus(x), min=-5.0)
        # q / k are L2-normalised before the call, as in the reference's own scalar-gate benchmark
        # (benchmark/bench_gated_delta_rule.py:200-209): with raw N(0,1) keys (|k|^2 ~ 128) the delta rule diverges
        # within a few dozen tokens in any arithmetic
        nrm = lambda x: torch.nn.functional.normalize(x, dim=-1).bfloat16()       # noqa: E731
        t = dict(q=nrm(r(B, T, H, D)), k=nrm(r(B, T, H, D)), v=r(B, T, H, D).bfloat16(), g=gdec,
                 beta=torch.sigmoid(r(B, T, H)), h0=r(B, H, D, D) * 0.02)
        opts = dict(gate_mode="precomputed", beta_mode="precomputed", beta_scale=1.0, l2=False, epi=None, gdn=True)
        desc, dims = "scalar gate, B=4 x T=16384, H=16, L2-normalised q / k, [V,K] initial state", dict(tokens=B * T, HK=H, HV=H, docs=B)
    else:
        raise SystemExit(f"unknown workload {name}")
    if pin:
        t = {n: x.pin_memory() for n, x in t.items()}
    return t, opts, desc, dims


GRAD_LEAVES = ("q", "k", "v", "g", "beta", "A_log", "dt_bias", "ep_w", "ep_gate", "h0")
# natural-log decay below which the segment pre-passes may be truncated: the value the reference uses inside its intra-card
# context parallelism (mogan_kda/ops/gated_delta_rule/chunk/blackwell/cp_fwd.py:81-115).  Only the "*_truncated" figures
# of the extra records use it; every headline number is exact.
WARMUP_THRESHOLD = -10.0


def layer_step(mk, dev, opts, cp=None):
    """One forward + backward of the layer on device tensors ``dev``; returns the loss tensor."""
    lv = {n: (x.detach().requires_grad_(True) if n in GRAD_LEAVES and x.is_floating_point() else x) for n, x in dev.items()}
    if opts.get("gdn"):
        o, ht = mk.chunk_gated_delta_rule(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], initial_state=lv["h0"],
                                          output_final_state=True, state_v_first=True,
                                          warmup_threshold=opts.get("warmup"))
        loss = o.float().sum() + ht.sum()
    else:
        norm = None
        if opts["epi"]:
            norm = dict(weight=lv["ep_w"], gate=lv["ep_gate"], act=opts["epi"], eps=1e-6)
        o, _ = mk.chunk_kda(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], cu_seqlens=lv.get("cu"),
                            gate_mode=opts["gate_mode"], A_log=lv.get("A_log"), dt_bias=lv.get("dt_bias"),
                            lower_bound=opts["lower_bound"], beta_mode=opts["beta_mode"], beta_scale=opts["beta_scale"],
                            use_qk_l2norm_in_kernel=opts["l2"], output_norm=norm, cp_context=cp,
                            warmup_threshold=opts.get("warmup"))
        loss = o.float().sum()
    loss.backward()
    return loss


# ----------------------------------------------------------------------------------------------------------
# roofline bookkeeping: algorithmic FLOPs per token per v-head of each contraction kernel (full tiles, no
# precision-split or recompute multipliers, no triangular discount) and algorithmic bytes of the streaming kernels.
# ----------------------------------------------------------------------------------------------------------
C_, K_, V_ = 64, 128, 128
F_CK, F_KV, F_CC = 2 * C_ * K_, 2 * K_ * V_, 2 * C_ * C_
KERNEL_FLOPS = {                      # per token per v-head
    "mkda_intra_fwd": 3 * F_CK,                       # Gamma, Q K^T, A (beta [k~ | v]) counted as one C x C x (K|V) product pair
    "mkda_recur_fwd": 2 * F_KV,                       # nw S, kbar^T Vd
    "mkda_out_fwd": F_KV + F_CK,                      # q~ S, Aqk Vd
    "mkda_bwd_dh": F_CK + 3 * F_KV,                   # Aqk^T dO, kbar dS', q~^T dO, nw^T dVd
    # k~ S, dO Vd^T, A^T dVd, dVd W^T, two C^3 products (Vd comes from the forward pass); dO S^T, dX S^T, Vd dS'^T; row / column
    # terms through Gamma and Q K^T
    "mkda_bwd_chunk": 4 * F_KV + 7 * F_CK + 2 * F_CC,
}
# Algorithmic bytes per token per v-head: each kernel's own tensor I/O at the default workload (bf16 q/k/v/gate,
# fp32 intermediates, HV = 2 HK), every operand counted once.
KERNEL_BYTES = {
    "mkda_gate_cumsum_fwd": 1024, "mkda_l2norm_rstd": 128, "mkda_intra_fwd": 3592, "mkda_recur_fwd": 3080,
    "mkda_out_fwd": 3584, "mkda_epilogue_bwd_tiles": 2048, "mkda_epilogue_bwd": 2048, "mkda_bwd_dh": 3848,
    "mkda_bwd_chunk": 6152, "mkda_gate_bwd": 1536, "mkda_qk_grad_finish": 1024,      # dq / dk tiles are per q/k head: 512 B per v-head
}
def load_kernel_traffic(path=os.path.join(ROOT, "profiles", "counters_per_kernel_1b_shape.md")):
    """DRAM traffic per token per v-head of every kernel, read from the committed ncu summary (its table has the columns
    `entry point`, `pass` and `B/token-head` = (dram read + write per launch) / token-heads of the captured case; traffic grows in
    proportion to tokens x heads).  Rows of the pre-pass of a serial kernel are skipped; several launches of one entry point
    are averaged.  Returns {} when the file is missing."""
    out, cols = {}, None
    if not os.path.exists(path):
        return out
    acc = {}
    for line in open(path):
        cells = [c.strip() for c in line.strip().strip("|").split("|")]
        if "entry point" in cells and "B/token-head" in cells:
            cols = {name: i for i, name in enumerate(cells)}
            continue
        if cols is None or len(cells) < len(cols) or not cells[0].startswith("`mkda_"):
            continue
        if cells[cols["pass"]] != "main":
            continue
        try:
            acc.setdefault(cells[0].strip("`"), []).append(float(cells[cols["B/token-head"]]))
        except ValueError:
            continue
    return {k: sum(v) / len(v) for k, v in acc.items()}


KERNEL_TRAFFIC = load_kernel_traffic()


class LaunchRecorder:
    """Wraps the C-ABI call so that every kernel launch is counted and bracketed by CUDA events on its stream."""

    def __init__(self, lib_module):
        self.lib, self.orig, self.events, self.count, self.timing = lib_module, lib_module.call, [], 0, False

    def __enter__(self):
        def call(name, params, stream):
            self.count += 1
            if not self.timing:
                return self.orig(name, params, stream)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            self.orig(name, params, stream)
            e1.record()
            self.events.append((name, e0, e1))
        self.lib.call = call
        return self

    def __exit__(self, *exc):
        self.lib.call = self.orig

    def totals(self):
        out = {}
        for name, e0, e1 in self.events:
            ms, n = out.get(name, (0.0, 0))
            out[name] = (ms + e0.elapsed_time(e1), n + 1)
        return out


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.proc, self.path = gpu_index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.idx), "-lms", "100"], stdout=open(self.path, "w"),
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for nm, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        os.unlink(self.path)
        if not sm:
            return None
        busy = sorted(sm)[len(sm) // 2:]
        return dict(sm_mhz=statistics.median(busy), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))


def time_workload(mk, name, rank, world, device, steps=5, warmup=3, cp=None, tokens=65536, truncated=False):
    """Short device-timed run of another workload (same timing rules as the headline: warm-up, barrier + synchronise on
    both sides, CUDA events, max over ranks).  Returns (ms per step, tokens per step on this rank); with ``truncated``
    the same inputs are timed a second time with warm-up truncation of the segment pre-passes at the reference's
    threshold, and ms per step is the pair (exact, truncated)."""
    import torch.distributed as dist
    host, opts, _, dims = make_workload(name, rank, device, tokens=tokens)
    dev = {n: x.to(device) for n, x in host.items()}

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    out = []
    for thr in ((None, WARMUP_THRESHOLD) if truncated else (None,)):
        o = dict(opts, warmup=thr)
        for _ in range(warmup):
            layer_step(mk, dev, o, cp)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            layer_step(mk, dev, o, cp)
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1) / steps], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out.append(float(t.item()))
    del dev
    return (tuple(out) if truncated else out[0]), dims["tokens"]


def bind_to_gpu_numa_node(index):
    """Best effort: run this process on the host cores of the NUMA node the GPU hangs off, so that the pinned buffers
    allocated afterwards are on that node.  Returns the node or None."""
    try:
        pr = torch.cuda.get_device_properties(index)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        node = int(open(f"/sys/bus/pci/devices/{bdf}/numa_node").read())
        if node < 0:
            return None
        cpus = []
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            a, _, b = part.partition("-")
            cpus += list(range(int(a), int(b or a) + 1))
        os.sched_setaffinity(0, set(cpus) & os.sched_getaffinity(0) or os.sched_getaffinity(0))
        return node
    except Exception:                                       # noqa: BLE001  (no sysfs, no permission: leave the placement alone)
        return None


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm=p["hbm_gbs"], tensor=p["bf16_tflops_sustained"], source="measured")
    return dict(hbm=6650.0, tensor=1400.0, source="fallback")


def cpu_baseline(seconds=12.0):
    """The CPU restatement of the reference's torch oracle on benchmark config 1 (T=256, HK2/HV4, fp32, precomputed
    gate), forward + backward, all host threads."""
    from oracle import kda_oracle as orc
    torch.manual_seed(0)
    B, T, hk, hv = 1, 256, 2, 4
    q = torch.nn.functional.normalize(torch.randn(B, T, hk, D), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(B, T, hk, D), dim=-1)
    v, g, beta = torch.randn(B, T, hv, D), -0.5 * torch.rand(B, T, hv, D), torch.sigmoid(torch.randn(B, T, hv))
    times = []
    t_end = time.time() + seconds
    while len(times) < 2 or (time.time() < t_end and len(times) < 20):
        lv = [x.clone().requires_grad_(True) for x in (q, k, v, g, beta)]
        t0 = time.time()
        o, _ = orc.recurrent_delta_rule(*lv, output_final_state=True)
        o.sum().backward()
        times.append(time.time() - t0)
    med = statistics.median(times[1:])
    return dict(value=T / med / 1e6, unit="Mtok/s", cores=torch.get_num_threads(), kind="port",
                sample=f"config 1 (B=1,T=256,HK=2,HV=4,D=128 fp32, token-by-token fp64 recurrence + autograd), median of {len(times) - 1} runs after 1 warm-up")


def reference_function():
    """The reference's own CPU implementation of the path: ``ref_chunk_delta_rule`` of its ``tests/ref_kda.py`` (pure torch,
    fp64), imported by path from the checkout named by the environment variable MOGANKDA_REFERENCE_ROOT.  Without that
    checkout (the usual case on a GPU box) the restatement in ``oracle/`` is timed instead.  Returns (fn, kind)."""
    root = os.environ.get("MOGANKDA_REFERENCE_ROOT", "")
    path = os.path.join(root, "tests", "ref_kda.py")
    if root and os.path.exists(path):
        import importlib.util
        spec = importlib.util.spec_from_file_location("ref_kda", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod.ref_chunk_delta_rule, "reference"
    from oracle import kda_oracle as orc
    return orc.recurrent_delta_rule, "port"


def reference_arm(args, world, rank):
    """CPU arm: the reference's torch oracle (or its restatement, see ``reference_function``) on a bounded sample (the
    first 128 tokens of every batch row) of the workload's shape (default: HK16/HV32/D128, eda gate, sigmoid beta x2, L2,
    silu epilogue), all host threads."""
    if rank != 0:
        return
    fn, kind = reference_function()
    torch.set_num_threads(os.cpu_count() or 1)
    t, opts, desc, dims = make_workload(args.workload if args.workload != "longdoc" else "packed", 0, "cpu")
    T = 128
    cut = {n: (x[:, :T].contiguous() if x.dim() >= 3 else x) for n, x in t.items()}

    def step():
        lv = {n: (x.float().requires_grad_(True) if x.is_floating_point() else x) for n, x in cut.items()}
        if opts.get("gdn"):
            o, _ = fn(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], initial_state=lv["h0"],
                      state_v_first=True, output_final_state=True)
        else:
            norm = dict(weight=lv["ep_w"], gate=lv["ep_gate"], act=opts["epi"]) if opts["epi"] else None
            o, _ = fn(lv["q"], lv["k"], lv["v"], lv["g"], lv["beta"], gate_mode=opts["gate_mode"],
                      A_log=lv.get("A_log"), dt_bias=lv.get("dt_bias"), lower_bound=-5.0,
                      beta_mode=opts["beta_mode"], beta_scale=opts["beta_scale"],
                      use_qk_l2norm_in_kernel=opts["l2"], output_norm=norm)
        o.sum().backward()

    ntok = cut["q"].shape[0] * T
    for _ in range(min(args.warmup, 1)):
        step()
    t0 = time.time()
    for _ in range(args.steps):
        step()
    dt = (time.time() - t0) / args.steps
    val = ntok / dt / 1e6
    sample = (f"first {T} tokens of every batch row of the workload, full head count, token-by-token fp64 recurrence + autograd"
              + (" (the reference's tests/ref_kda.py)" if kind == "reference" else " (restatement of the reference's tests/ref_kda.py)"))
    print(json.dumps({
        "impl": "reference", "metric": "KDA fwd+bwd Mtok/s per layer", "value": val, "unit": "Mtok/s",
        "n_gpus": world, "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {desc}", **dims, "D": D, "parallelism": "host cores (rank 0)",
                   "sample_tokens": ntok},
        "cpu_baseline": dict(value=val, unit="Mtok/s", cores=torch.get_num_threads(), kind=kind, sample=sample),
        "e2e": {"value": val, "unit": "Mtok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="packed")
    ap.add_argument("--impl", default="mogankda_b200")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the short runs of the other workloads")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        args.steps = min(args.steps, 5)
        return reference_arm(args, world, rank)
    args.warmup = max(args.warmup, 3)

    import torch.distributed as dist
    import mogankda_b200 as mk
    from mogankda_b200 import _lib
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    cp = None
    if args.workload == "longdoc" and world > 1:
        from mogankda_b200.cp import ContextParallel
        cp = ContextParallel(dist.group.WORLD)

    numa_node = bind_to_gpu_numa_node(local)
    host, opts, desc, dims = make_workload(args.workload, rank, device, pin=True)
    dev = {n: x.to(device) for n, x in host.items()}
    tokens_per_step = dims["tokens"]
    h2d = sum(x.numel() * x.element_size() for x in host.values())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with LaunchRecorder(_lib) as rec:
        for _ in range(args.warmup):
            layer_step(mk, dev, opts, cp)
        barrier()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        rec.count, rec.timing = 0, True
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            layer_step(mk, dev, opts, cp)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        launches = rec.count
        rec.timing = False
        per_kernel = rec.totals()
        # end to end: pinned host inputs in, loss out, every step.  As in a training loop with a prefetching loader the
        # next step's inputs travel on a second stream while the current step computes; all K copies and K loss
        # read-backs are inside the timed region (the first copy has nothing to hide behind).
        copy_stream = torch.cuda.Stream()

        def upload():
            with torch.cuda.stream(copy_stream):
                t = {n: x.to(device, non_blocking=True) for n, x in host.items()}
                ev = torch.cuda.Event()
                ev.record(copy_stream)
            return t, ev

        def e2e_steps(n):
            nxt = upload()
            for i in range(n):
                cur, ev = nxt
                torch.cuda.current_stream().wait_event(ev)
                if i + 1 < n:
                    nxt = upload()
                loss = layer_step(mk, cur, opts, cp)
                for x in cur.values():
                    x.record_stream(torch.cuda.current_stream())
                loss.item()

        e2e_steps(2)
        barrier()
        # the plain pinned-host -> device copy rate of the same buffers, all ranks at once, for attribution of `e2e`
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        for _ in range(3):
            tmp = {n: x.to(device, non_blocking=True) for n, x in host.items()}
        c1.record()
        barrier()
        ms_copy = c0.elapsed_time(c1) / 3
        del tmp
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        e2e_steps(args.steps)
        f1.record()
        barrier()
        ms_e2e = f0.elapsed_time(f1)
        clocks = sampler.stop() if rank == 0 else None
        if _lib.device_status() != 0:
            raise SystemExit("a bounded wait inside a tensor-core kernel expired: the run is invalid")

    tms = torch.tensor([ms, ms_e2e, ms_copy], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms, ms_e2e, ms_copy = tms.tolist()
    del dev, host
    torch.cuda.empty_cache()

    # further workloads in the same record (short runs; every rank takes part, rank 0 reports)
    extra = {}
    if args.workload == "packed" and not args.no_extra:
        if world == 1:
            other = {}
            for name in ("1b", "longdoc", "gdn"):
                # timed exactly and with warm-up truncation (which also lets the chooser cut the few long chains of gdn)
                (t_ms, t_tr), ntok = time_workload(mk, name, rank, world, device, truncated=True)
                other[name] = dict(ms_per_step=round(t_ms, 4), mtok_s=round(ntok / t_ms / 1e3, 4), tokens=ntok)
                if t_tr is not None:
                    other[name].update(ms_per_step_truncated=round(t_tr, 4), warmup_threshold=WARMUP_THRESHOLD)
            extra["other_workloads"] = other
        else:
            from mogankda_b200.cp import ContextParallel
            ctx = ContextParallel(dist.group.WORLD)
            cpk = {}
            for mode, per_rank in (("weak", 65536), ("strong", 65536 // world)):
                (t1, t1_tr), _ = time_workload(mk, "longdoc", rank, world, device, tokens=per_rank,
                                               truncated=True)                                     # every GPU alone, no exchange
                (tw, tw_tr), _ = time_workload(mk, "longdoc", rank, world, device, cp=ctx, tokens=per_rank,
                                               truncated=True)                                     # one document over all ranks
                tot = per_rank * world
                if mode == "weak":          # per-GPU work fixed: the CP step against the same slice as a stand-alone document
                    eff, eff_tr = t1 / tw, t1_tr / tw_tr
                else:                       # total work fixed at 65536 tokens: against W times the one-GPU rate on the whole document
                    (t_full, t_full_tr), _ = time_workload(mk, "longdoc", rank, world, device, tokens=tot, truncated=True)
                    eff, eff_tr = t_full / (world * tw), t_full_tr / (world * tw_tr)
                    cpk[mode + "_ms_1gpu_whole_document"] = round(t_full, 4)
                    cpk[mode + "_ms_1gpu_whole_document_truncated"] = round(t_full_tr, 4)
                cpk[mode] = dict(tokens_total=tot, tokens_per_rank=per_rank, ms_per_step=round(tw, 4),
                                 mtok_s=round(tot / tw / 1e3, 4), ms_1gpu_same_tokens_per_rank=round(t1, 4),
                                 efficiency=round(eff, 4), ms_per_step_truncated=round(tw_tr, 4),
                                 ms_1gpu_same_tokens_per_rank_truncated=round(t1_tr, 4),
                                 efficiency_truncated=round(eff_tr, 4), warmup_threshold=WARMUP_THRESHOLD)
            extra["cp"] = cpk
    if rank == 0:
        peaks = measured_peaks()
        total_tokens = tokens_per_step * world * args.steps
        value = total_tokens / (ms * 1e-3) / 1e6
        top = max(per_kernel.items(), key=lambda kv: kv[1][0])
        name, (kms, n) = top
        per_launch_s = kms / n * 1e-3
        units = tokens_per_step * dims["HV"]
        # the roofline that bounds the kernel is the one with the larger time floor for its algorithmic work
        t_hbm = KERNEL_BYTES.get(name, 0) * units / (peaks["hbm"] * 1e9)
        t_tc = KERNEL_FLOPS.get(name, 0) * units / (peaks["tensor"] * 1e12)
        traffic = KERNEL_TRAFFIC[name] * units if name in KERNEL_TRAFFIC else None
        if t_tc > t_hbm:
            ach = KERNEL_FLOPS[name] * units / per_launch_s / 1e12
            roof = dict(kernel=name, bound="tensor", achieved=ach, peak=peaks["tensor"], unit="TFLOP/s", frac=ach / peaks["tensor"])
        else:
            ach = KERNEL_BYTES.get(name, 0) * units / per_launch_s / 1e9
            roof = dict(kernel=name, bound="hbm", achieved=ach, peak=peaks["hbm"], unit="GB/s", frac=ach / peaks["hbm"])
        roof.update(traffic=traffic, peak_source=peaks["source"] + " (sustained bf16 / copy)", share_of_step=kms / ms,
                    launch_ms=per_launch_s * 1e3, alg_flops_per_launch=KERNEL_FLOPS.get(name, 0) * units,
                    alg_bytes_per_launch=KERNEL_BYTES.get(name, 0) * units)
        line = {
            "metric": "KDA fwd+bwd Mtok/s per layer", "value": value, "unit": "Mtok/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16x3", "data": "synthetic",
            "config": {"workload": f"{args.workload}: {desc}", **dims, "D": D,
                       "parallelism": ("cp%d" % world) if cp is not None else ("dp%d" % world),
                       "l2": "per-step working set (> 10 GB of inputs and intermediates) exceeds the 126 MB L2"},
            "e2e": {"value": total_tokens / (ms_e2e * 1e-3) / 1e6, "unit": "Mtok/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4, "ms_per_step": ms_e2e / args.steps,
                    "plain_h2d_copy_ms": round(ms_copy, 3), "plain_h2d_copy_gbs": round(h2d / ms_copy / 1e6, 2),
                    "host_numa_node": numa_node},
            "gpu_launches": launches, "roofline": roof, "clocks": clocks,
            "kernels_ms_per_step": {k: round(v[0] / args.steps, 4) for k, v in sorted(per_kernel.items(), key=lambda kv: -kv[1][0])},
        }
        line.update(extra)
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline()
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

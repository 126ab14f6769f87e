"""GPU: every C-ABI kernel on its own, fed the oracle's fp64 intermediates (rounded to fp32) so that one kernel's error
is isolated -- the same scheme as the reference's per-kernel tests (tests/test_kda_bwd_kernels.py:26-29)."""
import pytest
import torch

from mogankda_b200 import ops
from mogankda_b200.index import get_layout
from oracle import kda_oracle as orc
from tests.common import (VARLEN_CU, make_inputs, pack_chunk_tiles, pack_quarter_tiles, pack_plain_tiles, pack_row_tiles, pack_state_tiles, row_tiles_dense,
                          scaled_operands, unpack_chunk_tiles, unpack_plain_tiles, unpack_quarter_tiles, unpack_row_tiles,
                          unpack_state_tiles)

pytestmark = pytest.mark.gpu
KTOL = 1e-3          # per-kernel bar (the compensated bf16 hi/lo products measure ~1e-5)


def _err(name, got, ref, tol=KTOL):
    assert got.shape == ref.shape, (name, got.shape, ref.shape)
    mx, mn = orc.rel_err(got, ref.to(got.device))
    assert mx <= tol and mn <= tol, f"{name}: max_rel {mx:.3e} mean_rel {mn:.3e}"


@pytest.fixture(scope="module", params=["varlen-f32", "dense-bf16"])
def world(request):
    if request.param == "varlen-f32":
        kw = dict(cu=VARLEN_CU, T=704, dtype=torch.float32, gate="eda", seed=21)
    else:
        kw = dict(B=2, T=300, dtype=torch.bfloat16, gate="kimi", seed=22)
    lv, do, dht, opts, _ = make_inputs(HK=2, HV=4, **kw)
    B, T = lv["q"].shape[:2]
    cu = opts["cu_seqlens"]
    qn, kn = orc.l2norm(lv["q"]), orc.l2norm(lv["k"])
    gd = orc.gate_log_decay(lv["g"], opts["gate_mode"], lv["A_log"], lv["dt_bias"], -5.0)
    be = orc.beta_value(lv["beta"], "sigmoid", 2.0)
    bw = orc.chunked_backward(qn, kn, lv["v"], gd, be, do, dht=dht, initial_state=lv["h0"], cu_seqlens=cu)
    lay = get_layout(B, T, cu, lv["q"].device)
    f32 = lambda t: t.float().contiguous()                            # noqa: E731
    w = dict(lv=lv, do=do.reshape(B * T, 4, 128), dht=dht, opts=opts, bw=bw, fw=bw["fwd"], lay=lay, TT=B * T, f32=f32,
             be=f32(be.reshape(B * T, 4)), scale=128 ** -0.5)
    w["q_rstd"], w["k_rstd"] = ops.l2norm_rstd(lv["q"]), ops.l2norm_rstd(lv["k"])
    # the state kernels' scaled operands (reference values, then in the hand-over formats)
    kbar, qs, gl = scaled_operands(qn.reshape(B * T, 2, 128), kn.reshape(B * T, 2, 128), w["fw"]["g_c"], lay, w["scale"])
    w.update(kbar=kbar, qs=qs, gl=gl, kbar_t=pack_row_tiles(kbar, lay), qs_t=pack_row_tiles(qs, lay), gl_t=f32(gl))
    return w


def test_gate_cumsum_and_beta(world):
    lv, o = world["lv"], world["opts"]
    g_c, beta_e = ops.gate_cumsum_fwd(world["lay"], lv["g"], o["gate_mode"], lv["A_log"], lv["dt_bias"], -5.0, 4,
                                      beta_raw=lv["beta"], beta_sigmoid=True, beta_scale=2.0)
    _err("g_c", g_c, world["fw"]["g_c"], 2e-5)
    _err("beta", beta_e, world["be"], 2e-6)


def test_l2norm_statistics(world):
    q = world["lv"]["q"]
    _err("rstd", world["q_rstd"], torch.rsqrt((q.double() ** 2).sum(-1) + 1e-6).reshape(-1), 2e-6)


def test_intra_fwd(world):
    lv, fw, f32 = world["lv"], world["fw"], world["f32"]
    A, Aqk, nw, u, kbar, qs, gl = ops.intra_fwd(world["lay"], lv["q"], lv["k"], lv["v"], world["q_rstd"], world["k_rstd"],
                                                f32(fw["g_c"]), world["be"], world["scale"], 2, 4)
    _err("kbar", unpack_row_tiles(kbar, world["lay"], world["TT"]), world["kbar"])
    _err("qs", unpack_row_tiles(qs, world["lay"], world["TT"]), world["qs"])
    _err("gl", gl, world["gl"])
    nw = unpack_chunk_tiles(nw, world["lay"], world["TT"])
    u = unpack_chunk_tiles(u, world["lay"], world["TT"])
    A, Aqk = unpack_quarter_tiles(A, world["lay"], world["TT"]), unpack_quarter_tiles(Aqk, world["lay"], world["TT"])
    for n, t in dict(A=A, Aqk=Aqk, nw=nw, u=u).items():
        _err(n, t, fw[n])
    idx = torch.arange(64, device="cuda")
    lay = world["lay"]
    for c in range(lay.NC):                       # exactly zero above the diagonal (reference: test_kkt_solve_kda.py:115-118)
        s, n = int(lay.chunk_start[c]), int(lay.chunk_len[c])
        rows = idx[:n, None]
        assert (A[s:s + n][:, :, :].permute(0, 2, 1)[(idx[None, :] > rows)[:, :, None].expand(n, 64, 4)] == 0).all()
        assert (Aqk[s:s + n].permute(0, 2, 1)[(idx[None, :] > rows)[:, :, None].expand(n, 64, 4)] == 0).all()


def test_recurrence_and_output(world):
    lv, fw, f32, lay = world["lv"], world["fw"], world["f32"], world["lay"]
    h, Vd, ht, _ = ops.recur_fwd(lay, pack_chunk_tiles(f32(fw["nw"]), lay), pack_chunk_tiles(f32(fw["u"]), lay), world["kbar_t"], world["gl_t"],
                                 2, 4, h0=lv["h0"])
    _err("h", unpack_state_tiles(h), fw["h"]); _err("Vd", unpack_chunk_tiles(Vd, lay, world["TT"]), fw["Vd"])
    _err("ht", ht, fw["ht"])
    o, _ = ops.out_fwd(lay, world["qs_t"], pack_quarter_tiles(f32(fw["Aqk"]), lay), pack_chunk_tiles(f32(fw["Vd"]), lay),
                       pack_state_tiles(f32(fw["h"])), 2, 4, torch.float32)
    _err("o", o, fw["o"])


def test_transition_matrix_reproduces_the_state_pass(world):
    """State leaving a segment = transition @ state entering + state reached from zero (what the prefix combine uses)."""
    lv, fw, f32, lay = world["lv"], world["fw"], world["f32"], world["lay"]
    args = (lay, pack_chunk_tiles(f32(fw["nw"]), lay), pack_chunk_tiles(f32(fw["u"]), lay), world["kbar_t"], world["gl_t"], 2, 4)
    _, _, hs, ms = ops.recur_fwd(*args, store_h=False, store_vd=False, want_transition=True)
    _, _, ht, _ = ops.recur_fwd(*args, h0=lv["h0"], store_h=False, store_vd=False)
    _err("M h0 + h", ms.double() @ lv["h0"].double() + hs.double(), ht)
    s_in, s_out = ops.state_combine(lay.grp_seg_off, lay.NG, lay.NS, 4, hs, ms, carry=lv["h0"])
    assert torch.equal(s_in, lv["h0"])
    _err("combine", s_out, fw["ht"])


def test_bwd_dh(world):
    lv, fw, bw, f32, lay = world["lv"], world["fw"], world["bw"], world["f32"], world["lay"]
    dh, dVd_t, dO_t, dh0 = ops.bwd_dh(lay, world["do"], world["kbar_t"], world["qs_t"], world["gl_t"],
                                      pack_quarter_tiles(f32(fw["Aqk"]), lay), pack_chunk_tiles(f32(fw["nw"]), lay), 2, 4,
                                      dht=world["dht"])
    _err("dh", unpack_state_tiles(dh), bw["dh"]); _err("dh0", dh0, bw["dh0"])
    _err("dVd", unpack_chunk_tiles(dVd_t, lay, world["TT"]), bw["dVd"])
    # the staged dO leaves as it was split for the products: hi + lo reproduces the fp32 input to 2^-16
    _err("dO", unpack_row_tiles(dO_t, lay, world["TT"]), world["do"], 2e-5)
    # dO given as the row tiles of the chunked epilogue backward: same results, the tile is handed through
    dh2, dVd2, dO2, dh02 = ops.bwd_dh(lay, None, world["kbar_t"], world["qs_t"], world["gl_t"],
                                      pack_quarter_tiles(f32(fw["Aqk"]), lay), pack_chunk_tiles(f32(fw["nw"]), lay), 2, 4,
                                      dht=world["dht"], dO_in_t=dO_t)
    assert dO2 is dO_t and torch.equal(dh2, dh) and torch.equal(dVd2, dVd_t) and torch.equal(dh02, dh0)
    # a pre-pass that stores nothing still returns the segment-level gradient
    _, _, _, dh0b = ops.bwd_dh(lay, world["do"], world["kbar_t"], world["qs_t"], world["gl_t"],
                               pack_quarter_tiles(f32(fw["Aqk"]), lay), pack_chunk_tiles(f32(fw["nw"]), lay), 2, 4,
                               dht=world["dht"], store=False)
    assert torch.equal(dh0, dh0b)


def test_bwd_chunk_gate_and_finish(world):
    lv, fw, bw, f32, lay, o = world["lv"], world["fw"], world["bw"], world["f32"], world["lay"], world["opts"]
    t_q, t_k, t_g, t_b, t_v = ops.bwd_chunk(lay, lv["q"], lv["k"], lv["v"], world["q_rstd"], world["k_rstd"], f32(fw["g_c"]),
                                           world["be"], pack_quarter_tiles(f32(fw["A"]), lay), pack_state_tiles(f32(fw["h"])),
                                           pack_state_tiles(f32(bw["dh"])), pack_chunk_tiles(f32(fw["Vd"]), lay),
                                           pack_row_tiles(world["do"], lay), pack_chunk_tiles(f32(bw["dVd"]), lay),
                                           world["scale"], 2, 4, lv["beta"], False, 1.0)
    _err("dv", t_v, bw["dX"].reshape(t_v.shape), KTOL if t_v.dtype == torch.float32 else 2.0 ** -8)
    TT = world["TT"]
    # dq / dk leave summed over the two v-heads of each q/k head
    _err("dq_v", unpack_plain_tiles(t_q, lay, TT), bw["dq_v"].reshape(TT, 2, 2, 128).sum(2))
    _err("dk_v", unpack_plain_tiles(t_k, lay, TT), bw["dk_v"].reshape(TT, 2, 2, 128).sum(2))
    _err("dgp", unpack_plain_tiles(t_g, lay, TT), bw["dgp"])
    _err("dbeta", t_b, bw["dbeta"].reshape(world["TT"], 4))
    # gate backward (reverse cumsum folded in) against autograd of the oracle's gate
    x = lv["g"].double().requires_grad_(True)
    A = lv["A_log"].double().requires_grad_(True)
    b = lv["dt_bias"].double().requires_grad_(True)
    gd = orc.gate_log_decay(x, o["gate_mode"], A, b, -5.0)
    rx, rA, rb = torch.autograd.grad((gd * bw["dg"]).sum(), [x, A, b])
    dx, d_bias, d_alog = ops.gate_bwd(lay, lv["g"], pack_plain_tiles(f32(bw["dgp"]), lay), o["gate_mode"], lv["A_log"], lv["dt_bias"], -5.0, 4,
                                      True, True)
    _err("dx", dx, rx, 2e-4); _err("ddt_bias", d_bias.view_as(rb), rb, 5e-4); _err("dA_log", d_alog, rA, 5e-4)
    # GVA sum + L2-norm backward against autograd of the oracle's l2norm
    qd = lv["q"].double().requires_grad_(True)
    B, T = lv["q"].shape[:2]
    up = bw["dq_v"].reshape(B, T, 2, 2, 128).sum(3)
    (rq,) = torch.autograd.grad((orc.l2norm(qd) * up).sum(), [qd])
    dq, _ = ops.qk_grad_finish(lay, pack_plain_tiles(f32(up.reshape(B * T, 2, 128)), lay),
                               pack_plain_tiles(f32(bw["dk_v"].reshape(B * T, 2, 2, 128).sum(2)), lay), lv["q"],
                               lv["k"], world["q_rstd"], world["k_rstd"], 2, 4)
    tol = 1e-5 if lv["q"].dtype == torch.float32 else 2.0 ** -8
    _err("dq", dq.view_as(rq), rq, tol)


def test_epilogue_backward(world):
    lv, fw, f32 = world["lv"], world["fw"], world["f32"]
    o = fw["o"].clone().requires_grad_(True)
    w = lv["ep_w"].double().requires_grad_(True)
    z = lv["ep_gate"].double().reshape(-1, 4, 128).requires_grad_(True)
    dy = world["do"]
    for act in ("silu", "sigmoid"):
        y = orc.gated_rmsnorm(o, w, z, act)
        ro, rw, rz = torch.autograd.grad((y * dy.double()).sum(), [o, w, z])
        d_o, dgate, dw = ops.epilogue_bwd(dy.contiguous(), f32(fw["o"]), lv["ep_w"], lv["ep_gate"], act, 1e-6)
        _err("do", d_o.view_as(ro), ro, 1e-5); _err("dw", dw, rw, 1e-5)
        _err("dgate", dgate.reshape(rz.shape), rz, 1e-5 if dgate.dtype == torch.float32 else 2.0 ** -8)
        # the chunk-structured variant: dO as row tiles (hi + lo reproduces fp32 to 2^-16), same dgate and dw
        lay = world["lay"]
        dO_t, dgate2, dw2 = ops.epilogue_bwd_tiles(lay, dy.contiguous(), f32(fw["o"]), lv["ep_w"], lv["ep_gate"], act, 1e-6, 4)
        _err("do (tiles)", unpack_row_tiles(dO_t, lay, world["TT"]), ro.reshape(world["TT"], 4, 128), 2e-5)
        dense = row_tiles_dense(dO_t, lay)
        for c, n in enumerate(lay.chunk_len.tolist()):                     # rows past the end of a chunk are exact zeros
            assert float(dense[c, :, n:].abs().sum()) == 0.0
        _err("dw (tiles)", dw2, rw, 1e-5)
        _err("dgate (tiles)", dgate2.reshape(rz.shape), rz, 1e-5 if dgate2.dtype == torch.float32 else 2.0 ** -8)
        # dy is read through its strides: a broadcast gradient (what autograd hands over for o.sum()) and a column-strided one
        # give bit for bit what their contiguous copies give
        wide = torch.randn(world["TT"], 4, 256, device="cuda")
        for view in (torch.full((), 0.75, device="cuda").expand(world["TT"], 4, 128), wide[..., ::2],
                     torch.randn(world["TT"], 4, 1, device="cuda").expand(world["TT"], 4, 128)):
            assert not view.is_contiguous() and ops.rows_strides(view) is not None
            a = ops.epilogue_bwd_tiles(lay, view, f32(fw["o"]), lv["ep_w"], lv["ep_gate"], act, 1e-6, 4)
            b = ops.epilogue_bwd_tiles(lay, view.contiguous(), f32(fw["o"]), lv["ep_w"], lv["ep_gate"], act, 1e-6, 4)
            assert all(torch.equal(x, y) for x, y in zip(a, b))


@pytest.mark.parametrize("mode", [0, 1, 2, 3])
@pytest.mark.parametrize("N,K", [(64, 64), (64, 128), (128, 64), (128, 128)])
def test_tensor_core_plumbing_in_isolation(mode, N, K):
    """mkda_selftest_umma: D = A B^T through the same tile layout, descriptors and three-product bf16 split the kernels
    use, with the operands staged K-major or MN-major (mode bits); the error must be at the 2^-16 level of the split."""
    from mogankda_b200 import _lib
    torch.manual_seed(7 + mode)
    A, B = torch.randn(128, K, device="cuda"), torch.randn(N, K, device="cuda")
    D = torch.zeros(128, N, device="cuda")
    p = _lib.STRUCTS["MkdaSelfTest"]()
    p.A, p.B, p.D, p.N, p.K, p.mode = A.data_ptr(), B.data_ptr(), D.data_ptr(), N, K, mode
    _lib.call("mkda_selftest_umma", p, torch.cuda.current_stream().cuda_stream)
    ref = A.double() @ B.double().T
    err = ((D.double() - ref).abs().max() / ref.abs().max()).item()
    assert err < 5e-5, err

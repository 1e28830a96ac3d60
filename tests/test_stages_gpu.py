"""Parity of the stand-alone forward stages (the reference's low-level operators) with the CPU oracle, through the C ABI.

Each operator receives the oracle's (bf16-rounded) inputs of its own stage, so errors do not compound along the chain, and is
held to max-abs-err / RMS(ref) <= 5e-3 on top of the bf16 rounding of the stored result (the reference's own bars are looser:
kkt max_abs 5e-3, solve_tri residual 2e-2 for bf16, w/u 0.1; test files cited in oracle/stages.py).  The chain test runs the
six stages back to back through their bf16 intermediates, like the reference chain, and is held to the reference's own
end-to-end pass rule."""
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from oracle import stages
from _util import assert_close

pytestmark = pytest.mark.gpu
C = 64
TOL = 5e-3
G = Path(__file__).resolve().parent / "golden"


def _bf(t):
    return t.bfloat16()


def _case(B, T, HK, HV, seed, cu=None):
    """Oracle tensors of every stage for one seeded problem (head-first)."""
    inp = oracle.make_gdn_inputs(B=B, T=T, HK=HK, HV=HV, K=128, V=128, seed=seed, dtype=torch.bfloat16)
    hf = lambda t: t.transpose(1, 2).contiguous()  # noqa: E731
    q, k, v = hf(inp["q"]), hf(inp["k"]), hf(inp["v"])
    g_raw, beta = hf(inp["g"].float()), hf(inp["beta"])
    N = B if cu is None else len(cu) - 1
    h0 = 0.1 * torch.randn(N, HV, 128, 128, generator=torch.Generator().manual_seed(seed + 1))
    d = dict(q=q, k=k, v=v, g_raw=g_raw, beta=beta, h0=h0)
    d["gam"] = stages.chunk_local_cumsum_ref(g_raw, C, cu_seqlens=cu).float()
    d["A"] = stages.chunk_scaled_dot_kkt_ref(k, d["gam"], beta, C, cu)
    d["X"] = stages.solve_tri_ref(d["A"].float(), C, cu)
    Xb = _bf(d["X"])
    d["w"], d["u"] = stages.recompute_w_u_ref(k, v, beta, Xb, d["gam"], C, cu)
    wb, ub = _bf(d["w"]), _bf(d["u"])
    d["h"], d["v_new"], d["ht"] = stages.chunk_fwd_h_ref(k, wb, ub, d["gam"], C, initial_state=h0, cu_seqlens=cu)
    d["o"] = stages.chunk_fwd_o_ref(q, k, _bf(d["v_new"]), _bf(d["h"]), d["gam"], 128 ** -0.5, C, cu)
    d["d_o"] = hf(inp["do"])
    d["dht"] = 0.1 * torch.randn(N, HV, 128, 128, generator=torch.Generator().manual_seed(seed + 2))
    d["dv_local"] = stages.chunk_bwd_dv_local_ref(q, k, d["d_o"], d["gam"], 128 ** -0.5, C, cu)
    d["dh"], d["dh0"], d["dv2"] = stages.chunk_bwd_dhu_ref(q, k, wb, d["d_o"], _bf(d["dv_local"]), d["gam"], 128 ** -0.5, C, dht=d["dht"],
                                                           cu_seqlens=cu)
    d["dq"], d["dk"], d["dw"], d["dg"] = stages.chunk_bwd_dqkwg_ref(q, k, _bf(d["v_new"]), d["gam"], _bf(d["h"]), d["d_o"], _bf(d["dh"]),
                                                                    _bf(d["dv2"]), 128 ** -0.5, C, cu)
    d["wy"] = stages.prepare_wy_repr_bwd_ref(k, v, beta, Xb, _bf(d["dw"]), _bf(d["dv2"]), d["gam"], C, cu)
    return d


# the third case packs an empty sequence, a one-token sequence and ragged tails
CASES = [(1, 160, 1, 2, None), (2, 256, 2, 4, None), (1, 300, 2, 2, [0, 70, 70, 71, 200, 300]), (3, 64, 1, 1, None)]


@pytest.fixture(scope="module", params=range(len(CASES)), ids=lambda i: f"case{i}")
def case(request):
    B, T, HK, HV, cu = CASES[request.param]
    return _case(B, T, HK, HV, 40 + request.param, cu), cu


def test_chunk_local_cumsum(case):
    from fla_b200.ops import chunk_local_cumsum
    d, cu = case
    g = d["g_raw"].cuda()
    out = chunk_local_cumsum(g, C, cu_seqlens=cu)
    assert_close("gam", out, d["gam"], 1e-6)
    rev = chunk_local_cumsum(g, C, cu_seqlens=cu, reverse=True, scale=0.5)
    assert_close("reverse", rev, stages.chunk_local_cumsum_ref(d["g_raw"], C, True, 0.5, cu), 1e-6)
    # sequence-first input, bf16 in and out
    gs = g.transpose(1, 2).contiguous().bfloat16()
    o2 = chunk_local_cumsum(gs, C, cu_seqlens=cu, head_first=False, output_dtype="same")
    assert o2.dtype == torch.bfloat16 and o2.shape == gs.shape
    assert_close("seq-first", o2.transpose(1, 2), stages.chunk_local_cumsum_ref(gs.float().cpu().transpose(1, 2), C, cu_seqlens=cu), 1e-6,
                 stored_bf16=True)


def test_chunk_local_cumsum_per_channel():
    from fla_b200.ops import chunk_local_cumsum
    g = torch.nn.functional.logsigmoid(torch.randn(2, 3, 150, 128, generator=torch.Generator().manual_seed(3))) / 16
    out = chunk_local_cumsum(g.cuda(), C, scale=1.4426950408889634)
    assert_close("gk", out, stages.chunk_local_cumsum_ref(g, C, scale=1.4426950408889634), 1e-6)


@pytest.mark.parametrize("mode", ["raw", "softplus", "safe"])
@pytest.mark.parametrize("cu", [None, [0, 40, 150]])
def test_kda_gate_cumsum(mode, cu):
    """aclnnKdaGateCumsum semantics (kda/chunk_kda_fwd/docs/api.md:103-115; golden
    tests/atk/chunk_kda_fwd/executor_chunk_kda_fwd.py:316-343)."""
    import math
    from fla_b200.ops import kda_gate_cumsum
    g_ = torch.Generator().manual_seed(17)
    B, T, HV, K = (2, 150, 3, 128) if cu is None else (1, 150, 3, 128)
    g = torch.randn(B, T, HV, K, generator=g_).bfloat16()
    A_log = 0.5 * torch.randn(HV, generator=g_)
    dt_bias = 0.5 * torch.randn(HV * K, generator=g_)
    gf = g.double()
    if mode == "raw":
        gate, kw = gf, {}
    else:
        raw = gf + dt_bias.double().view(1, 1, HV, K)
        eig = A_log.double().exp().view(1, 1, HV, 1)
        gate = -4.0 * torch.sigmoid(eig * raw) if mode == "safe" else -eig * torch.nn.functional.softplus(raw)
        kw = dict(A_log=A_log.cuda(), dt_bias=dt_bias.cuda(), use_gate_in_kernel=True, safe_gate=mode == "safe", lower_bound=-4.0)
    ref = stages.chunk_local_cumsum_ref(gate.transpose(1, 2), C, scale=1.0 / math.log(2.0), cu_seqlens=cu).transpose(1, 2)
    out = kda_gate_cumsum(g.cuda(), C, cu_seqlens=cu, **kw)
    assert out.dtype == torch.float32 and out.shape == g.shape
    assert_close("gk", out, ref, 1e-5)


def test_chunk_scaled_dot_kkt(case):
    from fla_b200.ops import chunk_scaled_dot_kkt
    d, cu = case
    A = chunk_scaled_dot_kkt(d["k"].cuda(), d["gam"].cuda(), d["beta"].cuda(), cu_seqlens=cu)
    assert A.dtype == torch.float32
    assert_close("A", A, d["A"], 1e-5)
    upper = torch.triu(torch.ones(C, C, dtype=torch.bool))
    T = A.shape[2]
    if cu is None and T % C == 0:
        assert (A.cpu().reshape(A.shape[0], A.shape[1], T // C, C, C)[..., upper] == 0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_solve_tri(case, dtype):
    from fla_b200.ops import solve_tri
    d, cu = case
    A = d["A"].to(dtype)
    ref = stages.solve_tri_ref(A.float(), C, cu)
    X = solve_tri(A.cuda(), cu_seqlens=cu, layout="bnsd")
    assert X.dtype == dtype
    assert_close("X", X, ref, 1e-5, stored_bf16=dtype != torch.float32)
    Xs = solve_tri(A.transpose(1, 2).contiguous().cuda(), cu_seqlens=cu, layout="bsnd")
    assert torch.equal(Xs.transpose(1, 2), X)


def test_recompute_w_u(case):
    from fla_b200.ops import recompute_w_u_fwd
    d, cu = case
    w, u = recompute_w_u_fwd(d["k"].cuda(), d["v"].cuda(), d["beta"].cuda(), _bf(d["X"]).cuda(), C, g=d["gam"].cuda(), cu_seqlens=cu)
    assert_close("w", w, d["w"], TOL, stored_bf16=True)
    assert_close("u", u, d["u"], TOL, stored_bf16=True)


def test_chunk_fwd_h(case):
    from fla_b200.ops import chunk_gated_delta_rule_fwd_h
    d, cu = case
    h, v_new, ht = chunk_gated_delta_rule_fwd_h(d["k"].cuda(), _bf(d["w"]).cuda(), _bf(d["u"]).cuda(), d["gam"].cuda(),
                                                initial_state=d["h0"].cuda(), output_final_state=True, chunk_size=C, cu_seqlens=cu)
    assert_close("h", h, d["h"], TOL, stored_bf16=True)
    assert_close("v_new", v_new, d["v_new"], TOL, stored_bf16=True)
    assert_close("ht", ht, d["ht"], TOL)
    h2, v2, none = chunk_gated_delta_rule_fwd_h(d["k"].cuda(), _bf(d["w"]).cuda(), _bf(d["u"]).cuda(), d["gam"].cuda(), cu_seqlens=cu)
    assert none is None and (h2[:, :, 0] == 0).all()
    # state_v_first: the same states with their last two dims swapped
    h3, v3, ht3 = chunk_gated_delta_rule_fwd_h(d["k"].cuda(), _bf(d["w"]).cuda(), _bf(d["u"]).cuda(), d["gam"].cuda(),
                                               initial_state=d["h0"].transpose(-1, -2).contiguous().cuda(), output_final_state=True,
                                               chunk_size=C, cu_seqlens=cu, state_v_first=True)
    assert torch.equal(h3, h.transpose(-1, -2)) and torch.equal(ht3, ht.transpose(-1, -2)) and torch.equal(v3, v_new)


def test_chunk_fwd_o(case):
    from fla_b200.ops import chunk_fwd_o
    d, cu = case
    o = chunk_fwd_o(d["q"].cuda(), d["k"].cuda(), _bf(d["v_new"]).cuda(), _bf(d["h"]).cuda(), 128 ** -0.5, g=d["gam"].cuda(), cu_seqlens=cu)
    assert_close("o", o, d["o"], TOL, stored_bf16=True)


def test_chunk_bwd_dv_local(case):
    from fla_b200.ops import chunk_bwd_dv_local
    d, cu = case
    dv = chunk_bwd_dv_local(d["q"].cuda(), d["k"].cuda(), d["d_o"].cuda(), d["gam"].cuda(), 128 ** -0.5, C, cu_seqlens=cu)
    assert_close("dv_local", dv, d["dv_local"], TOL, stored_bf16=True)


def test_chunk_bwd_dhu(case):
    from fla_b200.ops import chunk_gated_delta_rule_bwd_dhu
    d, cu = case
    args = (d["q"].cuda(), d["k"].cuda(), _bf(d["w"]).cuda(), d["d_o"].cuda(), _bf(d["dv_local"]).cuda(), 128 ** -0.5, C)
    dh, dh0, dv2 = chunk_gated_delta_rule_bwd_dhu(*args, g=d["gam"].cuda(), h0=d["h0"].cuda(), dht=d["dht"].cuda(), cu_seqlens=cu)
    assert_close("dh", dh, d["dh"], TOL, stored_bf16=True)
    assert_close("dv2", dv2, d["dv2"], TOL, stored_bf16=True)
    assert_close("dh0", dh0, d["dh0"], TOL)
    dh_b, none, _ = chunk_gated_delta_rule_bwd_dhu(*args, g=d["gam"].cuda(), cu_seqlens=cu)
    assert none is None
    last = -1 if cu is None else None
    if last is not None:
        assert (dh_b[:, :, last] == 0).all()     # without dht the gradient of the last chunk's end state is zero


def test_chunk_bwd_dqkwg(case):
    from fla_b200.ops import chunk_bwd_dqkwg
    d, cu = case
    dq, dk, dw, dg = chunk_bwd_dqkwg(d["q"].cuda(), d["k"].cuda(), _bf(d["v_new"]).cuda(), d["gam"].cuda(), _bf(d["h"]).cuda(),
                                     d["d_o"].cuda(), _bf(d["dh"]).cuda(), _bf(d["dv2"]).cuda(), C, cu_seqlens=cu, w=_bf(d["w"]).cuda(),
                                     scale=128 ** -0.5)
    assert_close("dq", dq, d["dq"], TOL, stored_bf16=True)
    assert_close("dk", dk, d["dk"], TOL, stored_bf16=True)
    assert_close("dw", dw, d["dw"], TOL, stored_bf16=True)
    assert_close("dg", dg, d["dg"], TOL)


def _wy_args(d):
    return (d["k"].cuda(), d["v"].cuda(), d["beta"].cuda(), _bf(d["X"]).cuda())


def test_prepare_wy_repr_bwd_fused_and_split(case):
    from fla_b200.ops import prepare_wy_repr_bwd, prepare_wy_repr_bwd_da, prepare_wy_repr_bwd_full
    d, cu = case
    dA_ref, dk_ref, dv_ref, db_ref, dg_ref = d["wy"]
    k, v, beta, X = _wy_args(d)
    dw, du, g = _bf(d["dw"]).cuda(), _bf(d["dv2"]).cuda(), d["gam"].cuda()
    dk, dv, dbeta, dg = prepare_wy_repr_bwd(k, v, beta, X, dw, du, g, C, cu_seqlens=cu)
    assert_close("dk", dk, dk_ref, TOL, stored_bf16=True)
    assert_close("dv", dv, dv_ref, TOL, stored_bf16=True)
    assert_close("dbeta", dbeta, db_ref, TOL, stored_bf16=True)
    assert_close("dg", dg, dg_ref, TOL)
    # the two-step form: dA, then the rest from a given (bf16-rounded) dA
    X32 = _bf(d["X"]).cuda()
    dA = prepare_wy_repr_bwd_da(k, v, beta, X32, dw, du, g, chunk_size=C, cu_seqlens=cu)
    assert dA.dtype == X32.dtype
    assert_close("dA", dA, dA_ref, TOL, stored_bf16=True)
    dk2, dv2, db2, dg2 = prepare_wy_repr_bwd_full(k, v, beta, X, _bf(dA_ref).cuda(), dw, du, g, C, cu_seqlens=cu)
    ref2 = stages.prepare_wy_repr_bwd_ref(d["k"], d["v"], d["beta"], _bf(d["X"]), _bf(d["dw"]), _bf(d["dv2"]), d["gam"], C, cu,
                                          dA=_bf(dA_ref))
    assert_close("dk (from dA)", dk2, ref2[1], TOL, stored_bf16=True)
    assert_close("dv (from dA)", dv2, ref2[2], TOL, stored_bf16=True)
    assert_close("dbeta (from dA)", db2, ref2[3], TOL, stored_bf16=True)
    assert_close("dg (from dA)", dg2, ref2[4], TOL)


def test_stage_chain_matches_fused_operator():
    """Running the six stages one after the other gives the fused operator's output (and the oracle's)."""
    from fla_b200 import ops
    inp = oracle.make_gdn_inputs(B=2, T=200, HK=2, HV=4, K=128, V=128, seed=9, dtype=torch.bfloat16)
    q, k, v, g, beta, h0 = (inp[n].cuda() for n in ("q", "k", "v", "g", "beta", "h0"))
    hf = lambda t: t.transpose(1, 2)  # noqa: E731  (views: the stages take strides)
    gam = ops.chunk_local_cumsum(g.float(), C, head_first=False)
    A = ops.chunk_scaled_dot_kkt(hf(k), hf(gam), hf(beta))
    X = ops.solve_tri(A.bfloat16(), layout="bnsd")
    w, u = ops.recompute_w_u_fwd(hf(k), hf(v), hf(beta), X, C, g=hf(gam))
    h, v_new, ht = ops.chunk_gated_delta_rule_fwd_h(hf(k), w, u, hf(gam), initial_state=h0, output_final_state=True)
    o = ops.chunk_fwd_o(hf(q), hf(k), v_new, h, 128 ** -0.5, g=hf(gam))
    o_f, ht_f = ops.chunk_gated_delta_rule(q, k, v, g, beta, initial_state=h0, output_final_state=True)
    ref = oracle.gdn_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], initial_state=inp["h0"])
    # the reference's own end-to-end pass rule for o (examples/flash_gated_delta_rule.py:1738-1761,1894-1901):
    # finite, allclose(rtol = atol = 5e-3), cosine >= 0.999 -- the chain's bf16 intermediates (X above all) set the error
    for name, got, want in (("o vs oracle", o.transpose(1, 2).float().cpu(), ref["o"].float()),
                            ("ht vs oracle", ht.cpu(), ref["ht"].float()),
                            ("o vs fused", o.transpose(1, 2).float().cpu(), o_f.float().cpu())):
        assert torch.isfinite(got).all(), name
        assert torch.allclose(got, want, rtol=5e-3, atol=5e-3), f"{name}: max abs err {(got - want).abs().max().item():.3e}"
        cos = torch.nn.functional.cosine_similarity(got.flatten().double(), want.flatten().double(), dim=0).item()
        assert cos >= 0.999, f"{name}: cosine {cos}"


def test_backward_stage_chain_matches_autograd_oracle():
    """The reference's backward chain (examples/flash_gated_delta_rule.py:884-1023) run operator by operator:
    w,u -> fwd_h -> dv_local -> bwd_dhu -> dqkwg -> prepare_wy_repr_bwd, dk and dg summed, dg reverse-cumsummed;
    checked with the reference's end-to-end pass rule (:1738-1761,1894-1901) against autograd through the recurrence."""
    from fla_b200 import ops
    inp = oracle.make_gdn_inputs(B=2, T=192, HK=2, HV=4, K=128, V=128, seed=13, dtype=torch.bfloat16)
    q, k, v, g, beta, h0, do = (inp[n].cuda() for n in ("q", "k", "v", "g", "beta", "h0", "do"))
    hf = lambda t: t.transpose(1, 2)  # noqa: E731
    scale = 128 ** -0.5
    gam = ops.chunk_local_cumsum(g.float(), C, head_first=False)
    A = ops.chunk_scaled_dot_kkt(hf(k), hf(gam), hf(beta))
    X = ops.solve_tri(A, layout="bnsd", output_dtype=torch.bfloat16)
    w, u = ops.recompute_w_u_fwd(hf(k), hf(v), hf(beta), X, C, g=hf(gam))
    h, v_new, _ = ops.chunk_gated_delta_rule_fwd_h(hf(k), w, u, hf(gam), initial_state=h0)
    dv = ops.chunk_bwd_dv_local(hf(q), hf(k), hf(do), hf(gam), scale, C)
    dh, dh0, dv2 = ops.chunk_gated_delta_rule_bwd_dhu(hf(q), hf(k), w, hf(do), dv, scale, C, g=hf(gam), h0=h0)
    dq, dk, dw, dg = ops.chunk_bwd_dqkwg(hf(q), hf(k), v_new, hf(gam), h, hf(do), dh, dv2, C, w=w, scale=scale)
    dk2, dv_f, dbeta, dg2 = ops.prepare_wy_repr_bwd(hf(k), hf(v), hf(beta), X, dw, dv2, hf(gam), C)
    dk = dk.float() + dk2.float()
    dg = ops.chunk_local_cumsum((dg.float() + dg2.float()).contiguous(), C, reverse=True)
    ref = oracle.gdn_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], initial_state=inp["h0"], do=inp["do"])
    checks = (("dq", hf(dq), ref["dq"], 8e-3, 0.999), ("dk", hf(dk), ref["dk"], 8e-3, 0.999), ("dv", hf(dv_f), ref["dv"], 8e-3, 0.999),
              ("dbeta", hf(dbeta), ref["dbeta"], 2e-2, 0.99), ("dg", hf(dg), ref["dg"], 2e-2, 0.99), ("dh0", dh0, ref["dh0"], 8e-3, 0.999))
    for name, got, want, tol, cos_min in checks:
        got, want = got.float().cpu(), want.float()
        assert torch.isfinite(got).all(), name
        assert torch.allclose(got, want, rtol=tol, atol=tol), f"{name}: max abs err {(got - want).abs().max().item():.3e}"
        cos = torch.nn.functional.cosine_similarity(got.flatten().double(), want.flatten().double(), dim=0).item()
        assert cos >= cos_min, f"{name}: cosine {cos}"


def test_stage_goldens_from_the_reference():
    """The committed vectors produced by the reference's own goldens, replayed through the CUDA operators."""
    from fla_b200 import ops
    fx = {k: torch.from_numpy(v) for k, v in np.load(G / "stages_golden.npz").items()}
    for tag, cu in (("fix", None), ("var", [0, 70, 160])):
        gam = ops.chunk_local_cumsum(fx["g_raw"].cuda(), C, cu_seqlens=cu)
        assert_close("gam", gam, fx[f"{tag}_gam"], 1e-6)
        k, q, v, beta = (fx[n].bfloat16().cuda() for n in ("k", "q", "v", "beta"))
        gam = fx[f"{tag}_gam"].cuda()
        assert_close("A", ops.chunk_scaled_dot_kkt(k, gam, beta, cu_seqlens=cu), fx[f"{tag}_A"], 1e-5)
        assert_close("X", ops.solve_tri(fx[f"{tag}_A"].cuda(), cu_seqlens=cu, layout="bnsd"), fx[f"{tag}_X"], 1e-5)
        w, u = ops.recompute_w_u_fwd(k, v, beta, fx[f"{tag}_X"].bfloat16().cuda(), C, g=gam, cu_seqlens=cu)
        assert_close("w", w, fx[f"{tag}_w"], TOL, stored_bf16=True)
        assert_close("u", u, fx[f"{tag}_u"], TOL, stored_bf16=True)
        h, v_new, _ = ops.chunk_gated_delta_rule_fwd_h(k, fx[f"{tag}_w"].bfloat16().cuda(), fx[f"{tag}_u"].bfloat16().cuda(), gam, cu_seqlens=cu)
        assert_close("h", h, fx[f"{tag}_h"], TOL, stored_bf16=True)
        assert_close("v_new", v_new, fx[f"{tag}_v_new"], TOL, stored_bf16=True)
        o = ops.chunk_fwd_o(q, k, fx[f"{tag}_v_new"].bfloat16().cuda(), fx[f"{tag}_h"].bfloat16().cuda(), 128 ** -0.5, g=gam, cu_seqlens=cu)
        # this golden is itself rounded to bf16 and, in its fixed-length branch, rounds the gate to fp16 before the exponential
        assert_close("o", o, fx[f"{tag}_o"], 2e-2, stored_bf16=True)
        d_o = fx["d_o"].bfloat16().cuda()
        dv = ops.chunk_bwd_dv_local(q, k, d_o, gam, 128 ** -0.5, C, cu_seqlens=cu)
        assert_close("dv_local", dv, fx[f"{tag}_dv_local"], TOL, stored_bf16=True)
        N = 1 if cu is None else len(cu) - 1
        dh, dh0, dv2 = ops.chunk_gated_delta_rule_bwd_dhu(q, k, fx[f"{tag}_w"].bfloat16().cuda(), d_o, fx[f"{tag}_dv_local"].bfloat16().cuda(),
                                                          128 ** -0.5, C, g=gam, h0=torch.zeros(N, 2, 128, 128).cuda(), cu_seqlens=cu)
        assert_close("dh", dh, fx[f"{tag}_dh"], TOL, stored_bf16=True)
        assert_close("dh0", dh0, fx[f"{tag}_dh0"], TOL)
        assert_close("dv2", dv2, fx[f"{tag}_dv2"], TOL, stored_bf16=True)

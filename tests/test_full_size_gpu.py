"""Size-independent properties at the benchmark's full sizes (the oracle is too slow there): chaining two half
sequences through the state reproduces one pass bit for bit (forward and backward), a batch row does not depend on
its neighbours, the causal prefix of the output matches the oracle on that prefix, outputs are linear in v / dO,
and the identity taps of the conv copy their input."""
import pytest
import torch
import torch.nn.functional as F

import oracle
from _util import assert_close

pytestmark = pytest.mark.gpu


def _gdn_inputs(B, T, HK, HV, seed, dev="cuda"):
    g_ = torch.Generator(device=dev).manual_seed(seed)
    rn = lambda *s: torch.randn(*s, device=dev, generator=g_)  # noqa: E731
    return dict(q=F.normalize(rn(B, T, HK, 128), dim=-1).bfloat16(), k=F.normalize(rn(B, T, HK, 128), dim=-1).bfloat16(),
                v=rn(B, T, HV, 128).bfloat16(), g=F.logsigmoid(rn(B, T, HV)).bfloat16(),
                beta=torch.sigmoid(rn(B, T, HV)).bfloat16(), h0=0.1 * rn(B, HV, 128, 128),
                do=rn(B, T, HV, 128).bfloat16(), dht=0.1 * rn(B, HV, 128, 128))


def test_gdn_config2_chained_halves_and_batch_rows_are_bit_identical():
    from fla_b200.ops import chunk_gated_delta_rule_fwd_bwd as fb
    B, T, HK, HV = 8, 4096, 16, 32
    d = _gdn_inputs(B, T, HK, HV, seed=2002)
    o, ht, gr = fb(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], initial_state=d["h0"], dht=d["dht"])
    h = T // 2
    a = {n: d[n][:, :h] for n in ("q", "k", "v", "g", "beta", "do")}
    b = {n: d[n][:, h:] for n in ("q", "k", "v", "g", "beta", "do")}
    # forward chain first (its middle state feeds the second half), backward chain in reverse
    o1, hm, _ = fb(a["q"], a["k"], a["v"], a["g"], a["beta"], a["do"], initial_state=d["h0"], dht=torch.zeros_like(d["dht"]))
    o2, ht2, g2 = fb(b["q"], b["k"], b["v"], b["g"], b["beta"], b["do"], initial_state=hm, dht=d["dht"])
    _, _, g1 = fb(a["q"], a["k"], a["v"], a["g"], a["beta"], a["do"], initial_state=d["h0"], dht=g2[5])
    assert torch.equal(torch.cat([o1, o2], 1), o) and torch.equal(ht2, ht)
    for i, name in enumerate(("dq", "dk", "dv", "dg", "dbeta")):
        assert torch.equal(torch.cat([g1[i], g2[i]], 1), gr[i]), name
    assert torch.equal(g1[5], gr[5])        # dh0
    # one batch row on its own
    r = 5
    one = {n: d[n][r:r + 1] for n in d}
    o_r, ht_r, g_r = fb(one["q"], one["k"], one["v"], one["g"], one["beta"], one["do"], initial_state=one["h0"], dht=one["dht"])
    assert torch.equal(o_r, o[r:r + 1]) and torch.equal(ht_r, ht[r:r + 1])
    for i in range(6):
        assert torch.equal(g_r[i], gr[i][r:r + 1])


def test_gdn_config2_prefix_matches_oracle_and_is_linear_in_v():
    from fla_b200.ops import chunk_gated_delta_rule
    B, T, HK, HV = 8, 4096, 16, 32
    d = _gdn_inputs(B, T, HK, HV, seed=2003)
    with torch.no_grad():
        o, _ = chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"], output_dtype=torch.float32)
        # causality: the first 512 output tokens of one GVA group only see the first 512 inputs
        r, hk, P = 3, 7, 512
        hv = slice(2 * hk, 2 * hk + 2)
        ref = oracle.gdn_reference_fwd_bwd(d["q"][r:r + 1, :P, hk:hk + 1].cpu(), d["k"][r:r + 1, :P, hk:hk + 1].cpu(),
                                           d["v"][r:r + 1, :P, hv].cpu(), d["g"][r:r + 1, :P, hv].cpu(),
                                           d["beta"][r:r + 1, :P, hv].cpu(), initial_state=d["h0"][r:r + 1, hv].cpu(),
                                           dtype=torch.float64)
        assert_close("o prefix", o[r:r + 1, :P, hv], ref["o"], 5e-3)
        # linearity in v with a zero initial state: o(v1 + v2) = o(v1) + o(v2)
        v2 = torch.randn_like(d["v"].float()).bfloat16()
        vs = (d["v"].float() + v2.float()).bfloat16()
        v1 = (vs.float() - v2.float()).bfloat16()          # v1 + v2 == vs exactly in most entries; use the rounded triple
        oa, _ = chunk_gated_delta_rule(d["q"], d["k"], v1, d["g"], d["beta"], output_dtype=torch.float32)
        ob, _ = chunk_gated_delta_rule(d["q"], d["k"], v2, d["g"], d["beta"], output_dtype=torch.float32)
        oc, _ = chunk_gated_delta_rule(d["q"], d["k"], (v1.float() + v2.float()).bfloat16(), d["g"], d["beta"],
                                       output_dtype=torch.float32)
        exact = (v1.float() + v2.float()).bfloat16().float() == v1.float() + v2.float()
        assert exact.float().mean() > 0.5
        lin = (oa + ob - oc)
        # tokens whose v rows were summed exactly dominate; compare in the RMS sense over the whole tensor
        assert lin.pow(2).mean().sqrt() <= 1e-2 * oc.pow(2).mean().sqrt()


def test_kda_config3_chained_halves_are_bit_identical():
    from fla_b200.ops import chunk_kda
    B, T, H = 4, 8192, 32
    g_ = torch.Generator(device="cuda").manual_seed(2004)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g_)  # noqa: E731
    q, k = F.normalize(rn(B, T, H, 128), dim=-1).bfloat16(), F.normalize(rn(B, T, H, 128), dim=-1).bfloat16()
    v, g = rn(B, T, H, 128).bfloat16(), (F.logsigmoid(rn(B, T, H, 128)) / 16).bfloat16()
    beta = torch.sigmoid(rn(B, T, H)).bfloat16()
    with torch.no_grad():
        o, ht = chunk_kda(q, k, v, g, beta, output_final_state=True)
        h = T // 2
        o1, hm = chunk_kda(q[:, :h], k[:, :h], v[:, :h], g[:, :h], beta[:, :h], output_final_state=True)
        o2, ht2 = chunk_kda(q[:, h:], k[:, h:], v[:, h:], g[:, h:], beta[:, h:], initial_state=hm, output_final_state=True)
    assert torch.equal(torch.cat([o1, o2], 1), o) and torch.equal(ht2, ht)
    assert torch.isfinite(o.float()).all()


def test_decode_config4_subsample_matches_oracle_and_null_update_keeps_the_state():
    from fla_b200.ops import fused_recurrent_gated_delta_rule
    N, HK, HV = 256, 16, 32
    inp = oracle.make_decode_inputs(N, HK, HV, seed=2005)
    dev = {n: t.cuda() for n, t in inp.items()}
    q, k, v = (dev[n].view(N, 1, -1, 128) for n in ("q", "k", "v"))
    g, beta = dev["g"].view(N, 1, HV), dev["beta"].view(N, 1, HV)
    o, ht = fused_recurrent_gated_delta_rule(q, k, v, g=g, beta=beta, initial_state=dev["state"], output_final_state=True)
    sel = torch.arange(0, N, 37)
    asl = torch.tensor([0] + [1] * len(sel), dtype=torch.int32)
    idx = torch.arange(len(sel), dtype=torch.int32)
    ref_o, ref_s = oracle.recurrent_gated_delta_rule_golden(
        inp["q"][sel], inp["k"][sel], inp["v"][sel], inp["state"][sel].transpose(-1, -2).contiguous(), inp["beta"][sel],
        128 ** -0.5, asl, idx, g=inp["g"][sel].float(), dtype=torch.float64, out_dtype=torch.float64,
        state_out_dtype=torch.float64)
    assert_close("o", o[sel.cuda()].view(len(sel), HV, 128), ref_o, 5e-3, stored_bf16=True)
    assert_close("state", ht[sel.cuda()], ref_s.transpose(-1, -2), 1e-5)
    # beta = 0 and g = 0: the delta vanishes and the decay is one, so the state pool must come back bit for bit
    o0, h0 = fused_recurrent_gated_delta_rule(q, k, v, g=torch.zeros_like(g), beta=torch.zeros_like(beta),
                                              initial_state=dev["state"], output_final_state=True)
    assert torch.equal(h0, dev["state"])


def test_conv_config1_identity_taps_copy_the_input_and_states_chain():
    from fla_b200.ops import causal_conv1d
    B, T, D, W = 8, 4096, 8192, 4
    g_ = torch.Generator(device="cuda").manual_seed(2006)
    x = torch.randn(B, T, D, device="cuda", generator=g_).bfloat16()
    w = torch.zeros(D, W, device="cuda", dtype=torch.bfloat16)
    w[:, W - 1] = 1
    y, _ = causal_conv1d(x, w)
    assert torch.equal(y, x)
    w[:, W - 1] = 0
    w[:, 0] = 1                                  # pure delay by W - 1 tokens
    y, _ = causal_conv1d(x, w)
    assert torch.equal(y[:, W - 1:], x[:, :T - (W - 1)]) and not y[:, :W - 1].any()
    # two halves chained through the conv state reproduce one pass bit for bit
    wr = (0.5 * torch.randn(D, W, device="cuda", generator=g_)).bfloat16()
    yf, sf = causal_conv1d(x, wr, activation="silu", output_final_state=True)
    y1, s1 = causal_conv1d(x[:, :T // 2], wr, activation="silu", output_final_state=True)
    y2, s2 = causal_conv1d(x[:, T // 2:], wr, activation="silu", initial_state=s1, output_final_state=True)
    assert torch.equal(torch.cat([y1, y2], 1), yf) and torch.equal(s2, sf)


def test_gdn_long_sequence_65536_tokens_prefix_and_chaining():
    """The reference's smoke shape B=1, T=65536 (ci/example_st_cases.json:124-339): the first 4096 output tokens equal a run
    over those tokens alone bit for bit (causality at a length where 32-bit element offsets would overflow), and the
    sequence chained in two halves reproduces the single pass."""
    from fla_b200.ops import chunk_gated_delta_rule
    B, T, HK, HV = 1, 65536, 16, 32
    d = _gdn_inputs(B, T, HK, HV, seed=2010)
    with torch.no_grad():
        o, ht = chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"], output_final_state=True)
        assert torch.isfinite(o.float()).all() and torch.isfinite(ht).all()
        P = 4096
        o_p, _ = chunk_gated_delta_rule(d["q"][:, :P], d["k"][:, :P], d["v"][:, :P], d["g"][:, :P], d["beta"][:, :P],
                                        initial_state=d["h0"], output_final_state=True)
        assert torch.equal(o_p, o[:, :P])
        h = T // 2
        o1, hm = chunk_gated_delta_rule(d["q"][:, :h], d["k"][:, :h], d["v"][:, :h], d["g"][:, :h], d["beta"][:, :h],
                                        initial_state=d["h0"], output_final_state=True)
        o2, ht2 = chunk_gated_delta_rule(d["q"][:, h:], d["k"][:, h:], d["v"][:, h:], d["g"][:, h:], d["beta"][:, h:],
                                         initial_state=hm, output_final_state=True)
        assert torch.equal(torch.cat([o1, o2], 1), o) and torch.equal(ht2, ht)

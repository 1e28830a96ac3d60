"""Pins the CPU oracle to the reference: replays fixtures produced by the reference's own CPU
functions (tests/golden/make_golden.py) through oracle/ and requires agreement to fp32 round-off."""
from pathlib import Path

import numpy as np
import torch

import oracle

G = Path(__file__).resolve().parent / "golden"


def _load(name):
    return {k: torch.from_numpy(v) for k, v in np.load(G / name).items()}


def _close(a, b, tol=2e-5):
    assert a.shape == b.shape, (a.shape, b.shape)
    err = (a.double() - b.double()).abs().max().item()
    assert err <= tol * max(1.0, b.abs().max().item()), err


def test_gdn_naive_forward_and_autograd_match_reference():
    f = _load("gdn_naive.npz")
    r = oracle.gdn_reference_fwd_bwd(f["q"], f["k"], f["v"], f["g"], f["beta"], do=f["do"], dtype=torch.float32)
    for name in ("o", "dq", "dk", "dv", "dg", "dbeta"):
        _close(r[name], f[name])
    # zero initial state == the reference's implicit start
    h0 = torch.zeros(f["q"].shape[0], f["q"].shape[2], f["q"].shape[3], f["v"].shape[3])
    r0 = oracle.gdn_reference_fwd_bwd(f["q"], f["k"], f["v"], f["g"], f["beta"], initial_state=h0)
    _close(r0["o"], f["o"])


def test_gdn_chunked_restatement_matches_reference():
    f = _load("gdn_naive.npz")
    for C in (64, 32):
        c = oracle.chunk_gated_delta_rule_restated(f["q"], f["k"], f["v"], f["g"], f["beta"], chunk_size=C)
        _close(c["o"].float(), f["o"])


def test_gdn_final_state_consistent_with_split_sequence():
    # the extension (initial_state / final state) is pinned by composition: running [0,T1) then
    # [T1,T) from the returned state must equal the reference's single pass.
    f = _load("gdn_naive.npz")
    T1 = 37
    a = oracle.gdn_reference_fwd_bwd(f["q"][:, :T1], f["k"][:, :T1], f["v"][:, :T1], f["g"][:, :T1], f["beta"][:, :T1])
    b = oracle.gdn_reference_fwd_bwd(f["q"][:, T1:], f["k"][:, T1:], f["v"][:, T1:], f["g"][:, T1:], f["beta"][:, T1:],
                                     initial_state=a["ht"])
    _close(torch.cat([a["o"], b["o"]], 1), f["o"])


def test_decode_golden_matches_reference():
    f = _load("decode_golden.npz")
    args = [f["query"].bfloat16(), f["key"].bfloat16(), f["value"].bfloat16(), f["state"].bfloat16(),
            f["beta"].bfloat16(), float(f["scale"]), f["actual_seq_lengths"], f["ssm_state_indices"]]
    out, st = oracle.recurrent_gated_delta_rule_golden(*args, num_accepted_tokens=f["num_accepted_tokens"], g=f["g"])
    _close(out.float(), f["out_acc"], 1e-6)
    _close(st.float(), f["state_acc"], 1e-6)
    out, st = oracle.recurrent_gated_delta_rule_golden(*args, g=f["g"])
    _close(out.float(), f["out"], 1e-6)
    _close(st.float(), f["state_out"], 1e-6)


def test_conv_goldens_match_reference():
    f = _load("conv_golden.npz")
    y0, fs0 = oracle.causal_conv1d_ref(f["x"], f["w"], f["b"], None, True, "silu")
    _close(y0, f["y0"]); _close(fs0, f["fs0"])
    y1, fs1 = oracle.causal_conv1d_ref(f["x"], f["w"], None, f["init"], True, None)
    _close(y1, f["y1"]); _close(fs1, f["fs1"])
    y2, fs2 = oracle.causal_conv1d_ref(f["xs"], f["w"], f["b"], None, True, "silu")
    _close(y2, f["y2"]); _close(fs2, f["fs2"])
    st = f["init"].clone()
    yu = oracle.causal_conv1d_update_ref(f["xu"], st, f["w"], f["b"], "silu")
    _close(yu, f["yu"]); _close(st, f["st_after"])
    st = f["st_spec"].clone()
    ysp = oracle.causal_conv1d_update_spec_ref(f["xsp"], st, f["w"], f["b"], f["accepted"], "silu")
    _close(ysp, f["ysp"]); _close(st, f["st_spec_after"])


def test_kda_naive_matches_reference():
    f = _load("kda_naive.npz")
    rep = f["v"].shape[2] // f["q"].shape[2]
    q = f["q"].repeat_interleave(rep, dim=2)
    k = f["k"].repeat_interleave(rep, dim=2)
    o, ht = oracle.naive_recurrent_kda(q, k, f["v"], f["g"], f["beta"], scale=q.shape[-1] ** -0.5,
                                       initial_state=f["h0"].transpose(-1, -2))
    _close(o, f["o"])
    _close(ht.transpose(-1, -2), f["ht"])


def test_conv_backward_golden_matches_reference():
    f = _load("conv_bwd_golden.npz")
    for name, act, init, dht in (("plain", 0, None, None), ("silu_state", 1, f["init"], f["dht"])):
        dx, dw, db, dh0 = oracle.causal_conv1d_bwd_ref(f["x"], f["w"], f["dy"], None, init, dht, act)
        for n, got in (("dx", dx), ("dw", dw), ("db", db)):
            torch.testing.assert_close(got.float(), f[f"{name}_{n}"], rtol=2e-5, atol=2e-5)
        if init is not None:
            torch.testing.assert_close(dh0.float(), f[f"{name}_dh0"], rtol=2e-5, atol=2e-5)


def test_kda_bwd_intra_matches_reference_golden():
    f = _load("kda_bwd_intra_golden.npz")
    out = oracle.chunk_kda_bwd_intra_ref(f["q"], f["k"], f["gk"], f["beta"], f["d_aqk"], f["d_akk"], f["dq"], f["dk"], f["db"], f["dg"])
    for name, got in zip(("dq_out", "dk_out", "db_out", "dg_out"), out):
        _close(got.float(), f[name], 2e-5)


def test_fast_gelu_matches_reference_golden_and_autograd():
    f = _load("fast_gelu_golden.npz")
    torch.testing.assert_close(oracle.fast_gelu_ref(f["x"]).float(), f["y"], rtol=1e-6, atol=1e-6)
    # the golden casts back to the input dtype (bf16 for the second case)
    torch.testing.assert_close(oracle.fast_gelu_ref(f["xb"]).bfloat16().float(), f["yb"], rtol=0, atol=0)
    x = f["x"].double().requires_grad_(True)
    dy = torch.randn(x.shape, dtype=torch.float64, generator=torch.Generator().manual_seed(3))
    (x / (1 + torch.exp(-1.702 * x)) * dy).sum().backward()
    torch.testing.assert_close(oracle.fast_gelu_bwd_ref(dy, x.detach()), x.grad, rtol=1e-12, atol=1e-12)


def test_kda_chunked_forward_golden_pins_the_score_blocks_and_the_recurrence():
    """The reference's chunked chunk_kda_fwd golden (float64, packed GVA case with an initial state): its Aqk / Akk / gk
    pin the oracle's score-block restatement, and its output / final state pin the naive recurrence with an initial
    state on every sequence of the packed batch."""
    f = _load("kda_chunk_fwd_golden.npz")
    cu = [int(x) for x in f["cu"]]
    scale = float(f["scale"])
    aqk, akk, gk = oracle.kda_chunk_score_blocks_ref(f["q"], f["k"], f["g"], f["beta"], scale, cu)
    for name, got, ref in (("gk", gk, f["gk"]), ("Aqk", aqk, f["aqk"]), ("Akk", akk, f["akk"])):
        err = (got - ref.double()).abs().max().item() / ref.double().pow(2).mean().sqrt().item()
        assert err < 2e-6, (name, err)                       # the fixture is stored in float32
    for i, (bos, eos) in enumerate(zip(cu[:-1], cu[1:])):
        q = f["q"][:, bos:eos].double().repeat_interleave(2, dim=2)
        k = f["k"][:, bos:eos].double().repeat_interleave(2, dim=2)
        o, ht = oracle.naive_recurrent_kda(q, k, f["v"][:, bos:eos], f["g"][:, bos:eos], f["beta"][:, bos:eos], scale=scale,
                                           initial_state=f["h0"][i:i + 1].double(), dtype=torch.float64)
        for name, got, ref in (("o", o, f["o"][:, bos:eos]), ("ht", ht, f["final_state"][i:i + 1])):
            err = (got - ref.double()).abs().max().item() / ref.double().pow(2).mean().sqrt().item()
            assert err < 2e-6, (name, i, err)


def test_kda_chunked_forward_golden_pins_the_intermediates():
    """w, u, qg, kg, v_new, h, o and the final state of the reference's chunked golden (the same fixture, chunk size 64) pin the
    oracle's restatement of its chunk loop, which the GPU tests then run at chunk size 128 as well."""
    f = _load("kda_chunk_fwd_golden.npz")
    cu = [int(x) for x in f["cu"]]
    got = oracle.kda_chunk_intermediates_ref(f["q"], f["k"], f["v"], f["g"], f["beta"], float(f["scale"]), initial_state=f["h0"],
                                             cu_seqlens=cu, chunk_size=64)
    for name in ("w", "u", "qg", "kg", "v_new", "final_state"):
        ref = f[name].double()
        err = (got[name] - ref).abs().max().item() / ref.pow(2).mean().sqrt().item()
        assert err < 2e-6, (name, err)
    ref = f["h"].double().squeeze(0)
    assert (got["h"] - ref).abs().max().item() / ref.pow(2).mean().sqrt().item() < 2e-6
    ref = f["o"].double().permute(0, 2, 1, 3)
    assert (got["o"] - ref).abs().max().item() / ref.pow(2).mean().sqrt().item() < 2e-6

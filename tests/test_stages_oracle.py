"""Pins the per-operator stage oracle (oracle/stages.py) to the reference: replays the fixture that
tests/golden/make_golden.py produced by running the reference's own golden of each low-level operator."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import stages

G = Path(__file__).resolve().parent / "golden"
C = 64


@pytest.fixture(scope="module")
def fx():
    return {k: torch.from_numpy(v) for k, v in np.load(G / "stages_golden.npz").items()}


def _close(got, ref, tol):
    assert got.shape == ref.shape, (got.shape, ref.shape)
    err = (got.double() - ref.double()).abs().max().item()
    assert err <= tol * max(1.0, ref.abs().max().item()), err


@pytest.mark.parametrize("tag,cu", [("fix", None), ("var", [0, 70, 160])])
def test_stage_oracle_matches_reference_goldens(fx, tag, cu):
    bf = lambda t: t.bfloat16().float()  # noqa: E731
    gam = stages.chunk_local_cumsum_ref(fx["g_raw"], C, cu_seqlens=cu)
    _close(gam, fx[f"{tag}_gam"], 1e-6)
    _close(stages.chunk_local_cumsum_ref(fx["g_raw"], C, reverse=True, scale=0.5, cu_seqlens=cu), fx[f"{tag}_rev"], 1e-6)
    gam = fx[f"{tag}_gam"]
    _close(stages.chunk_scaled_dot_kkt_ref(fx["k"], gam, fx["beta"], C, cu), fx[f"{tag}_A"], 2e-6)
    _close(stages.solve_tri_ref(fx[f"{tag}_A"], C, cu), fx[f"{tag}_X"], 2e-5)
    Xb = bf(fx[f"{tag}_X"])
    w, u = stages.recompute_w_u_ref(fx["k"], fx["v"], fx["beta"], Xb, gam, C, cu)
    _close(w, fx[f"{tag}_w"], 2e-6)
    _close(u, fx[f"{tag}_u"], 2e-6)
    h, v_new, _ = stages.chunk_fwd_h_ref(fx["k"], bf(fx[f"{tag}_w"]), bf(fx[f"{tag}_u"]), gam, C, cu_seqlens=cu)
    _close(h, fx[f"{tag}_h"], 2e-6)
    _close(v_new, fx[f"{tag}_v_new"], 2e-6)
    o = stages.chunk_fwd_o_ref(fx["q"], fx["k"], bf(fx[f"{tag}_v_new"]), bf(fx[f"{tag}_h"]), gam, 128 ** -0.5, C, cu)
    _close(o, fx[f"{tag}_o"], 2.0 ** -8)   # the reference golden returns bf16
    scale = 128 ** -0.5
    _close(stages.chunk_bwd_dv_local_ref(fx["q"], fx["k"], fx["d_o"], gam, scale, C, cu), fx[f"{tag}_dv_local"], 2e-6)
    dh, dh0, dv2 = stages.chunk_bwd_dhu_ref(fx["q"], fx["k"], bf(fx[f"{tag}_w"]), fx["d_o"], bf(fx[f"{tag}_dv_local"]), gam, scale, C,
                                            cu_seqlens=cu)
    _close(dh, fx[f"{tag}_dh"], 2e-6)
    _close(dh0, fx[f"{tag}_dh0"], 2e-6)
    _close(dv2, fx[f"{tag}_dv2"], 2e-6)
    dq, dk, dw, dg = stages.chunk_bwd_dqkwg_ref(fx["q"], fx["k"], bf(fx[f"{tag}_v_new"]), gam, bf(fx[f"{tag}_h"]), fx["d_o"],
                                                bf(fx[f"{tag}_dh"]), bf(fx[f"{tag}_dv2"]), scale, C, cu)
    for name, got in (("dq", dq), ("dk", dk), ("dw", dw), ("dg", dg)):
        _close(got, fx[f"{tag}_{name}"], 2e-6)
    dwb, dub = bf(fx[f"{tag}_dw"]), bf(fx[f"{tag}_dv2"])
    wy = stages.prepare_wy_repr_bwd_ref(fx["k"], fx["v"], fx["beta"], Xb, dwb, dub, gam, C, cu)
    for name, got in zip(("wy_dA", "wy_dk", "wy_dv", "wy_dbeta", "wy_dg"), wy):
        _close(got, fx[f"{tag}_{name}"], 1e-5)     # these goldens round intermediates to the inputs' dtype (fp32 here)


def test_stage_chain_reproduces_the_recurrence():
    """cumsum -> kkt -> solve_tri -> w,u -> fwd_h -> fwd_o in fp64 equals the naive recurrence."""
    import oracle
    inp = oracle.make_gdn_inputs(B=1, T=150, HK=1, HV=2, K=128, V=128, seed=5, dtype=torch.float32)
    q, k, v, g, beta = (inp[n].double() for n in ("q", "k", "v", "g", "beta"))
    hf = lambda t: t.transpose(1, 2).contiguous()  # noqa: E731
    gam = stages.chunk_local_cumsum_ref(hf(g), C)
    A = stages.chunk_scaled_dot_kkt_ref(hf(k), gam, hf(beta), C)
    X = stages.solve_tri_ref(A, C)
    w, u = stages.recompute_w_u_ref(hf(k), hf(v), hf(beta), X, gam, C)
    h, v_new, ht = stages.chunk_fwd_h_ref(hf(k), w, u, gam, C, initial_state=inp["h0"])
    o = stages.chunk_fwd_o_ref(hf(q), hf(k), v_new, h, gam, 128 ** -0.5, C)
    kk, qq = (t.repeat_interleave(2, dim=2) for t in (k, q))
    o_ref, ht_ref = oracle.naive_recurrent_gated_delta_rule(qq, kk, v, beta, g, scale=128 ** -0.5, initial_state=inp["h0"],
                                                            dtype=torch.float64)
    _close(o.transpose(1, 2), o_ref, 1e-9)
    _close(ht, ht_ref, 1e-9)

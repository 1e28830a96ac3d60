"""Parity of the chunked KDA forward with the naive per-channel-gate recurrence (oracle/kda.py)."""
import math

import pytest
import torch
import torch.nn.functional as F

import oracle
from _util import assert_close

pytestmark = pytest.mark.gpu
TOL = 5e-3


def _run(B, T, HK, HV, seed, h0=False, cu=None, gate_scale=1.0, out_dtype=torch.float32, **kw):
    from fla_b200.ops import chunk_kda
    inp = oracle.make_kda_inputs(B, T, HK, HV, seed=seed, with_grad=False)
    inp["g"] = (inp["g"].float() * gate_scale).bfloat16()
    N = B if cu is None else len(cu) - 1
    if h0:
        inp["h0"] = (0.1 * torch.randn(N, HV, 128, 128, generator=torch.Generator().manual_seed(seed))).float()
    if cu is None:
        ref = oracle.kda_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], initial_state=inp["h0"],
                                           dtype=torch.float64)
    else:
        os_, hs = [], []
        for i in range(N):
            sl = slice(cu[i], cu[i + 1])
            r = oracle.kda_reference_fwd_bwd(inp["q"][:, sl], inp["k"][:, sl], inp["v"][:, sl], inp["g"][:, sl],
                                             inp["beta"][:, sl], dtype=torch.float64,
                                             initial_state=None if inp["h0"] is None else inp["h0"][i:i + 1])
            os_.append(r["o"]); hs.append(r["ht"])
        ref = {"o": torch.cat(os_, 1), "ht": torch.cat(hs, 0)}
    d = {n: (t.cuda() if t is not None else None) for n, t in inp.items()}
    with torch.no_grad():
        o, ht = chunk_kda(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"], output_final_state=True,
                          output_dtype=out_dtype, cu_seqlens=None if cu is None else torch.tensor(cu, dtype=torch.int32),
                          **kw)
    torch.cuda.synchronize()
    return o, ht, ref


@pytest.mark.parametrize("B,T,HK,HV", [(1, 64, 1, 1), (1, 128, 1, 2), (2, 256, 2, 2), (1, 512, 2, 4)])
def test_kda_forward_fp32_output(B, T, HK, HV):
    o, ht, ref = _run(B, T, HK, HV, seed=3000 + T, h0=(T != 64))
    assert_close("o", o, ref["o"], TOL)
    assert_close("final_state", ht, ref["ht"], TOL)


@pytest.mark.parametrize("T", [1, 31, 65, 100])
def test_kda_forward_ragged_lengths(T):
    o, ht, ref = _run(1, T, 1, 1, seed=50 + T, h0=True)
    assert_close("o", o, ref["o"], TOL)
    assert_close("final_state", ht, ref["ht"], TOL)


def test_kda_forward_strong_gates_bf16_output():
    # 16x stronger decay (per-channel logsigmoid without the 1/16): exercises the anchored scaling
    o, ht, ref = _run(1, 256, 2, 2, seed=9, gate_scale=16.0, out_dtype=torch.bfloat16)
    assert_close("o", o, ref["o"], TOL, stored_bf16=True)
    assert_close("final_state", ht, ref["ht"], TOL)


def test_kda_forward_varlen_packed():
    cu = [0, 70, 71, 199, 263, 300]
    o, ht, ref = _run(1, 300, 2, 2, seed=12, cu=cu, h0=True)
    assert_close("o", o, ref["o"], TOL)
    assert_close("final_state", ht, ref["ht"], TOL)


def test_kda_gate_in_kernel_and_cumsum_output():
    from fla_b200.ops import chunk_kda
    B, T, HK, HV = 1, 192, 1, 2
    inp = oracle.make_kda_inputs(B, T, HK, HV, seed=77, with_grad=False)
    gen = torch.Generator().manual_seed(5)
    raw = torch.randn(B, T, HV, 128, generator=gen).bfloat16()
    A_log = torch.randn(HV, generator=gen) * 0.3 - 2.0
    dt_bias = torch.randn(HV, 128, generator=gen) * 0.1
    gate = -torch.exp(A_log.double())[None, None, :, None] * F.softplus(raw.double() + dt_bias.double()[None, None])
    ref = oracle.kda_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], gate, inp["beta"], dtype=torch.float64)
    d = {n: (t.cuda() if t is not None else None) for n, t in inp.items()}
    with torch.no_grad():
        o, ht, gk = chunk_kda(d["q"], d["k"], d["v"], raw.cuda(), d["beta"], output_final_state=True,
                              use_gate_in_kernel=True, A_log=A_log.cuda(), dt_bias=dt_bias.cuda(),
                              return_gate_cumsum=True, output_dtype=torch.float32)
    assert_close("o", o, ref["o"], TOL)
    gk_ref = gate.view(B, T // 64, 64, HV, 128).cumsum(2).view(B, T, HV, 128)
    assert_close("gk", gk, gk_ref, 1e-4)
    # safe gate: lower_bound * sigmoid(exp(A_log) (g + dt_bias))
    lb = -5.0
    gate2 = lb * torch.sigmoid(torch.exp(A_log.double())[None, None, :, None] * (raw.double() + dt_bias.double()[None, None]))
    ref2 = oracle.kda_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], gate2, inp["beta"], dtype=torch.float64)
    with torch.no_grad():
        o2, _ = chunk_kda(d["q"], d["k"], d["v"], raw.cuda(), d["beta"], use_gate_in_kernel=True, safe_gate=True,
                          lower_bound=lb, A_log=A_log.cuda(), dt_bias=dt_bias.cuda(), output_dtype=torch.float32)
    assert_close("o_safe_gate", o2, ref2["o"], TOL)

"""Parity of the chunked GDN forward with the naive fp32/fp64 recurrent oracle (through the C ABI).

Bar: max-abs-err / RMS(ref) <= 5e-3 for o (checked on fp32 output; the bf16 output additionally gets
the half-ulp allowance of its final rounding) and for the fp32 final state.
"""
import pytest
import torch

import oracle
from _util import assert_close, rel_err

pytestmark = pytest.mark.gpu
TOL = 5e-3


def _run(B, T, HK, HV, seed, h0=True, cu=None, out_dtype=torch.float32):
    from fla_b200.ops import chunk_gated_delta_rule
    inp = oracle.make_gdn_inputs(B, T, HK, HV, seed=seed, h0_scale=0.1 if h0 else 0.0, with_grad=False)
    N = B if cu is None else len(cu) - 1
    if h0 and cu is not None:
        inp["h0"] = (0.1 * torch.randn(N, HV, 128, 128, generator=torch.Generator().manual_seed(seed))).float()
    ref = oracle.gdn_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], initial_state=inp["h0"],
                                       dtype=torch.float64, cu_seqlens=cu)
    d = {n: (t.cuda() if t is not None else None) for n, t in inp.items()}
    o, ht = chunk_gated_delta_rule(d["q"], d["k"], d["v"], d["g"], d["beta"], initial_state=d["h0"],
                                   output_final_state=True, output_dtype=out_dtype,
                                   cu_seqlens=None if cu is None else torch.tensor(cu, dtype=torch.int32))
    torch.cuda.synchronize()
    return o, ht, ref


@pytest.mark.parametrize("B,T,HK,HV", [(1, 64, 1, 1), (1, 128, 1, 2), (2, 256, 2, 4), (1, 1024, 2, 2)])
def test_forward_fp32_output(B, T, HK, HV):
    o, ht, ref = _run(B, T, HK, HV, seed=1000 + T)
    assert_close("o", o, ref["o"], TOL)
    assert_close("final_state", ht, ref["ht"], TOL)


@pytest.mark.parametrize("T", [1, 15, 63, 65, 127, 200])
def test_forward_ragged_lengths(T):
    o, ht, ref = _run(1, T, 1, 2, seed=7 + T)
    assert_close("o", o, ref["o"], TOL)
    assert_close("final_state", ht, ref["ht"], TOL)


def test_forward_bf16_output_and_zero_state():
    o, ht, ref = _run(2, 192, 2, 4, seed=5, h0=False, out_dtype=torch.bfloat16)
    assert o.dtype == torch.bfloat16
    assert_close("o", o, ref["o"], TOL, stored_bf16=True)
    assert_close("final_state", ht, ref["ht"], TOL)


def test_forward_varlen_packed():
    cu = [0, 70, 71, 199, 263, 300]
    o, ht, ref = _run(1, 300, 2, 4, seed=11, cu=cu)
    assert_close("o", o, ref["o"], TOL)
    assert_close("final_state", ht, ref["ht"], TOL)


def test_forward_is_deterministic():
    o1, h1, _ = _run(1, 256, 2, 4, seed=3)
    o2, h2, _ = _run(1, 256, 2, 4, seed=3)
    assert torch.equal(o1, o2) and torch.equal(h1, h2)


def test_head_first_and_reference_entry_are_views_of_the_same_operator():
    """`head_first=True` and the reference's composed entry `flash_gated_delta_rule` ([B,H,T,D] tokens) give bit-identical
    results to the sequence-first call, forward and backward."""
    from fla_b200.ops import chunk_gated_delta_rule, flash_gated_delta_rule
    inp = oracle.make_gdn_inputs(B=2, T=130, HK=2, HV=4, K=128, V=128, seed=77, dtype=torch.bfloat16)
    q, k, v, g, beta, h0, do = (inp[n].cuda() for n in ("q", "k", "v", "g", "beta", "h0", "do"))
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
    o, ht = chunk_gated_delta_rule(*leaves, g, beta, initial_state=h0, output_final_state=True)
    (o.float() * do.float()).sum().backward()
    hf = [t.transpose(1, 2).contiguous() for t in (q, k, v)]
    o1, ht1 = chunk_gated_delta_rule(*hf, g.transpose(1, 2).contiguous(), beta.transpose(1, 2).contiguous(), initial_state=h0,
                                     output_final_state=True, head_first=True)
    assert torch.equal(o1.transpose(1, 2), o) and torch.equal(ht1, ht)
    leaves2 = [t.clone().requires_grad_(True) for t in hf]
    o2, ht2 = flash_gated_delta_rule(*leaves2, g, beta, initial_state=h0, output_final_state=True)
    assert tuple(o2.shape) == tuple(o.shape) and torch.equal(o2, o) and torch.equal(ht2, ht)
    (o2.float() * do.float()).sum().backward()
    for a, b in zip(leaves, leaves2):
        assert torch.equal(b.grad.transpose(1, 2), a.grad)
    with pytest.raises(ValueError, match="does not support float32"):
        flash_gated_delta_rule(*(t.float() for t in hf), g, beta)


def test_reference_chunk_sizes_give_the_same_function():
    """The reference tiles for chunk sizes 16 .. 128; the blocking does not change o or the final state, so the operator
    accepts them (and keeps its own tiling) and still meets the oracle."""
    from fla_b200.ops import chunk_gated_delta_rule
    inp = oracle.make_gdn_inputs(B=1, T=300, HK=1, HV=2, K=128, V=128, seed=91, dtype=torch.bfloat16, with_grad=False)
    ref = oracle.gdn_reference_fwd_bwd(inp["q"], inp["k"], inp["v"], inp["g"], inp["beta"], initial_state=inp["h0"],
                                       dtype=torch.float64)
    q, k, v, g, beta, h0 = (inp[n].cuda() for n in ("q", "k", "v", "g", "beta", "h0"))
    o64, h64 = chunk_gated_delta_rule(q, k, v, g, beta, initial_state=h0, output_final_state=True, chunk_size=64)
    o128, h128 = chunk_gated_delta_rule(q, k, v, g, beta, initial_state=h0, output_final_state=True, chunk_size=128)
    assert torch.equal(o64, o128) and torch.equal(h64, h128)
    assert_close("o", o128, ref["o"], 5e-3, stored_bf16=True)
    assert_close("ht", h128, ref["ht"], 5e-3)
    with pytest.raises(NotImplementedError):
        chunk_gated_delta_rule(q, k, v, g, beta, chunk_size=48)

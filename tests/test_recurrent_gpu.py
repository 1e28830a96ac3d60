"""Parity of the fused-recurrent decode kernel with the CPU oracle (through the C ABI)."""
import numpy as np
import pytest
import torch

import oracle
from _util import assert_close

pytestmark = pytest.mark.gpu


def _oracle_decode(inp, N, tps, vfirst_state=None):
    q, k, v, g, beta, state = (inp[n] for n in ("q", "k", "v", "g", "beta", "state"))
    T = q.shape[0]
    asl = torch.tensor([0] + [tps] * N, dtype=torch.int32)
    idx = torch.arange(N, dtype=torch.int32).repeat_interleave(tps)
    st_vk = state.transpose(-1, -2).contiguous()
    out, st = oracle.recurrent_gated_delta_rule_golden(q, k, v, st_vk, beta, q.shape[-1] ** -0.5, asl, idx, g=g.float(),
                                                       dtype=torch.float64, out_dtype=torch.float64,
                                                       state_out_dtype=torch.float64)
    return out, st.transpose(-1, -2)


@pytest.mark.parametrize("N,HK,HV,K,V,tps", [(4, 2, 4, 128, 128, 1), (3, 2, 2, 64, 64, 3), (2, 1, 2, 64, 128, 2),
                                             (2, 2, 4, 128, 64, 1), (3, 2, 4, 128, 256, 2), (2, 1, 2, 64, 256, 1)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_fused_recurrent_matches_oracle(N, HK, HV, K, V, tps, out_dtype):
    from fla_b200.ops import fused_recurrent_gated_delta_rule
    inp = oracle.make_decode_inputs(N, HK, HV, K, V, seed=5, tokens_per_seq=tps)
    ref_o, ref_s = _oracle_decode(inp, N, tps)
    dev = {n: t.cuda() for n, t in inp.items()}
    q, k, v = (dev[n].view(N, tps, -1, dev[n].shape[-1]) for n in ("q", "k", "v"))
    g, beta = dev["g"].view(N, tps, HV), dev["beta"].view(N, tps, HV)
    o, ht = fused_recurrent_gated_delta_rule(q, k, v, g=g, beta=beta, initial_state=dev["state"],
                                             output_final_state=True)
    assert o.dtype == torch.bfloat16
    assert_close("o", o.view(N * tps, HV, V), ref_o, 5e-3, stored_bf16=True)
    assert_close("final_state", ht, ref_s, 1e-5)
    # the pool variant updates the state in place and bumps its version counter
    pool = dev["state"].clone()
    ver = pool._version
    o2, ht2 = fused_recurrent_gated_delta_rule(q, k, v, g=g, beta=beta, initial_state=pool, inplace_final_state=True)
    assert ht2 is pool and pool._version > ver
    assert torch.equal(pool, ht) and torch.equal(o2, o)


def test_fused_recurrent_v_first_and_bf16_state():
    from fla_b200.ops import fused_recurrent_gated_delta_rule
    N, HK, HV, K, V = 3, 2, 4, 128, 128
    inp = oracle.make_decode_inputs(N, HK, HV, K, V, seed=6)
    ref_o, ref_s = _oracle_decode(inp, N, 1)
    dev = {n: t.cuda() for n, t in inp.items()}
    q, k, v = (dev[n].view(N, 1, -1, 128) for n in ("q", "k", "v"))
    st_vk = dev["state"].transpose(-1, -2).contiguous()
    o, ht = fused_recurrent_gated_delta_rule(q, k, v, g=dev["g"].view(N, 1, HV), beta=dev["beta"].view(N, 1, HV),
                                             initial_state=st_vk, output_final_state=True, transpose_state_layout=True)
    assert_close("o", o.view(N, HV, V), ref_o, 5e-3, stored_bf16=True)
    assert_close("final_state", ht.transpose(-1, -2), ref_s, 1e-5)


def test_reference_surface_state_pool_with_indices_and_accepted_tokens():
    """Same scenario as the reference's own accuracy test: shuffled state slots, 2 tokens per sequence,
    start state chosen by num_accepted_tokens, per-token state write-back, skipped prefix token."""
    from fla_b200.ops import recurrent_gated_delta_rule
    torch.manual_seed(42)
    bs, mtp, nk, nv, dk, dv = 3, 2, 2, 4, 64, 64
    asl = torch.cat([torch.tensor([1], dtype=torch.int32), torch.full((bs,), mtp, dtype=torch.int32)])
    t = int(asl.sum())
    state = torch.rand((t, nv, dv, dk))
    query = torch.nn.functional.normalize(torch.rand((t, nk, dk)), p=2, dim=-1).bfloat16()
    key = torch.nn.functional.normalize(torch.rand((t, nk, dk)), p=2, dim=-1).bfloat16()
    value = torch.rand((t, nv, dv)).bfloat16()
    beta = torch.rand((t, nv)).bfloat16()
    g = -torch.rand((t, nv))
    ssm = torch.randperm(t).to(torch.int32)
    acc = torch.tensor([1, 2, 1], dtype=torch.int32)
    for accepted in (None, acc):
        ref_o, ref_s = oracle.recurrent_gated_delta_rule_golden(query, key, value, state, beta, dk ** -0.5, asl, ssm,
                                                                num_accepted_tokens=accepted, g=g, dtype=torch.float64,
                                                                out_dtype=torch.float64, state_out_dtype=torch.float64)
        pool = state.clone().cuda()
        out = recurrent_gated_delta_rule(query.cuda(), key.cuda(), value.cuda(), pool, beta=beta.cuda(),
                                         scale=dk ** -0.5, actual_seq_lengths=asl.cuda(), ssm_state_indices=ssm.cuda(),
                                         num_accepted_tokens=None if accepted is None else accepted.cuda(), g=g.cuda())
        # token 0 is the skipped prefix: the oracle leaves its output at zero and so must not be compared
        assert_close("attn_out", out[1:], ref_o[1:], 5e-3, stored_bf16=True)
        assert_close("state", pool, ref_s, 1e-5)


def test_l2norm_in_kernel_and_no_gate():
    from fla_b200.ops import fused_recurrent_gated_delta_rule
    N, HK, HV = 2, 2, 4
    inp = oracle.make_decode_inputs(N, HK, HV, seed=9)
    inp["q"] = (inp["q"].float() * 3).bfloat16()
    inp["k"] = (inp["k"].float() * 0.5).bfloat16()
    qn = torch.nn.functional.normalize(inp["q"].double(), dim=-1)
    kn = torch.nn.functional.normalize(inp["k"].double(), dim=-1)
    asl = torch.tensor([0] + [1] * N, dtype=torch.int32)
    idx = torch.arange(N, dtype=torch.int32)
    ref_o, ref_s = oracle.recurrent_gated_delta_rule_golden(qn, kn, inp["v"], inp["state"].transpose(-1, -2), inp["beta"],
                                                            128 ** -0.5, asl, idx, g=torch.zeros(N, HV),
                                                            dtype=torch.float64, out_dtype=torch.float64,
                                                            state_out_dtype=torch.float64)
    dev = {n: t.cuda() for n, t in inp.items()}
    o, ht = fused_recurrent_gated_delta_rule(dev["q"].view(N, 1, HK, 128), dev["k"].view(N, 1, HK, 128),
                                             dev["v"].view(N, 1, HV, 128), g=None, beta=dev["beta"].view(N, 1, HV),
                                             initial_state=dev["state"], output_final_state=True,
                                             use_qk_l2norm_in_kernel=True)
    assert_close("o", o.view(N, HV, 128), ref_o, 5e-3, stored_bf16=True)
    assert_close("state", ht, ref_s.transpose(-1, -2), 2e-5)


def test_argument_errors_are_reported_not_launched():
    from fla_b200.ops import fused_recurrent_gated_delta_rule
    q = torch.zeros(1, 1, 2, 128, dtype=torch.bfloat16, device="cuda")
    v = torch.zeros(1, 1, 3, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        fused_recurrent_gated_delta_rule(q, q, v)                     # HV not a multiple of HK
    v = torch.zeros(1, 1, 2, 96, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="status=2"):
        fused_recurrent_gated_delta_rule(q, q, v)                     # unsupported V
    with pytest.raises(TypeError):
        fused_recurrent_gated_delta_rule(q.float(), q, v)
    with pytest.raises(RuntimeError, match="CUDA device"):
        fused_recurrent_gated_delta_rule(q.cpu(), q.cpu(), v.cpu())

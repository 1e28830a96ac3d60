"""Parity of the recurrent KDA step (per-key-channel gate) with the naive recurrence of the reference's executor
(tests/atk/recurrent_kda/executor_recurrent_kda.py:63-83, restated in oracle/kda.py), through the C ABI."""
import pytest
import torch
import torch.nn.functional as F

import oracle
from _util import assert_close

pytestmark = pytest.mark.gpu


def _inputs(B, T, H, HV, seed, K=128, V=128):
    g_ = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, H, K, generator=g_).bfloat16()
    k = F.normalize(torch.randn(B, T, H, K, generator=g_), dim=-1).bfloat16()
    v = torch.randn(B, T, HV, V, generator=g_).bfloat16()
    g = F.logsigmoid(torch.randn(B, T, HV, K, generator=g_)) / 4
    beta = torch.rand(B, T, HV, generator=g_) * 0.8 + 0.1
    state = 0.1 * torch.randn(B, HV, K, V, generator=g_)
    return q, k, v, g, beta, state


def _ref(q, k, v, gate, beta, state, scale):
    rep = v.shape[2] // q.shape[2]
    return oracle.naive_recurrent_kda(q.double().repeat_interleave(rep, 2), k.double().repeat_interleave(rep, 2), v.double(),
                                      gate.double(), beta.double(), scale=scale, initial_state=state.double(),
                                      dtype=torch.float64)


@pytest.mark.parametrize("B,T,H,HV", [(3, 1, 2, 4), (2, 4, 2, 2), (1, 8, 1, 2)])
@pytest.mark.parametrize("v_first", [False, True])
def test_recurrent_kda_matches_recurrence(B, T, H, HV, v_first):
    from fla_b200.ops import recurrent_kda
    q, k, v, g, beta, state = _inputs(B, T, H, HV, seed=11 + T)
    scale = 128 ** -0.5
    ref_o, ref_s = _ref(q, k, v, g, beta, state, scale)
    pool = (state.transpose(-1, -2) if v_first else state).contiguous().cuda()
    o, ht = recurrent_kda(q.cuda(), k.cuda(), v.cuda(), g.cuda(), beta.cuda(), pool, output_final_state=True,
                          inplace_final_state=True, state_v_first=v_first)
    assert ht is pool
    assert_close("o", o, ref_o, 5e-3, stored_bf16=True)
    assert_close("state", ht.transpose(-1, -2) if v_first else ht, ref_s, 1e-5)


@pytest.mark.parametrize("v_first", [False, True])
def test_recurrent_kda_value_dim_256(v_first):
    """K = 128, V = 256 (the reference accepts V up to 256): each state is updated by two CTAs of 128 value channels."""
    from fla_b200.ops import recurrent_kda
    B, T, H, HV = 2, 3, 2, 4
    q, k, v, g, beta, state = _inputs(B, T, H, HV, seed=41, V=256)
    scale = 128 ** -0.5
    ref_o, ref_s = _ref(q, k, v, g, beta, state, scale)
    pool = (state.transpose(-1, -2) if v_first else state).contiguous().cuda()
    o, ht = recurrent_kda(q.cuda(), k.cuda(), v.cuda(), g.cuda(), beta.cuda(), pool, output_final_state=True,
                          inplace_final_state=True, state_v_first=v_first)
    assert_close("o", o, ref_o, 5e-3, stored_bf16=True)
    assert_close("state", ht.transpose(-1, -2) if v_first else ht, ref_s, 1e-5)


def test_recurrent_kda_gate_beta_activations_and_l2norm():
    from fla_b200.ops import recurrent_kda
    B, T, H, HV = 2, 3, 2, 4
    q, k, v, _, _, state = _inputs(B, T, H, HV, seed=31)
    g_ = torch.Generator().manual_seed(32)
    raw = torch.randn(B, T, HV, 128, generator=g_)
    braw = torch.randn(B, T, HV, generator=g_)
    A_log = torch.randn(HV, generator=g_) * 0.3 - 1.0
    dt_bias = torch.randn(HV, 128, generator=g_) * 0.1
    qn, kn = F.normalize(q.double(), dim=-1), F.normalize(k.double(), dim=-1)
    eig = torch.exp(A_log.double())[None, None, :, None]
    for safe in (False, True):
        gate = (-4.0 * torch.sigmoid(eig * (raw.double() + dt_bias.double())) if safe
                else -eig * F.softplus(raw.double() + dt_bias.double()))
        beta = 2 * torch.sigmoid(braw.double())
        ref_o, ref_s = _ref(qn, kn, v, gate, beta, state, 0.1)
        o, ht = recurrent_kda(q.cuda(), k.cuda(), v.cuda(), raw.cuda(), braw.cuda(), state.cuda(), A_log=A_log.cuda(),
                              dt_bias=dt_bias.cuda(), scale=0.1, output_final_state=True, inplace_final_state=False,
                              use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, use_beta_sigmoid_in_kernel=True,
                              allow_neg_eigval=True, safe_gate=safe, lower_bound=-4.0 if safe else None)
        assert_close("o", o, ref_o, 5e-3, stored_bf16=True)
        assert_close("state", ht, ref_s, 2e-5)


def test_recurrent_kda_tnd_varlen_with_state_indices():
    from fla_b200.ops import recurrent_kda
    lens = [3, 1, 4]
    T, H, HV = sum(lens), 2, 2
    q, k, v, g, beta, _ = _inputs(1, T, H, HV, seed=41)
    g_ = torch.Generator().manual_seed(42)
    pool = 0.1 * torch.randn(16, HV, 128, 128, generator=g_)
    cu = torch.tensor([0, 3, 4, 8], dtype=torch.int32)
    # speculative indices [seq_num, max_step]; sequence 0 restarts from its 2nd slot (2 accepted tokens)
    idx2d = torch.tensor([[5, 6, 7, 0], [9, 0, 0, 0], [1, 2, 3, 4]], dtype=torch.int32)
    accepted = torch.tensor([2, 1, 1], dtype=torch.int32)
    ref_pool = pool.double().clone()
    outs = []
    for n, L in enumerate(lens):
        sl = slice(int(cu[n]), int(cu[n + 1]))
        st = ref_pool[idx2d[n, accepted[n] - 1]][None]
        for s in range(L):
            t = sl.start + s
            o_t, st = _ref(q[:, t:t + 1], k[:, t:t + 1], v[:, t:t + 1], g[:, t:t + 1], beta[:, t:t + 1], st[0][None].float().double(),
                           128 ** -0.5)
            outs.append(o_t)
            ref_pool[idx2d[n, s]] = st[0]
    ref_o = torch.cat(outs, 1)[0]
    pool_d = pool.cuda()
    o, _ = recurrent_kda(q[0].cuda(), k[0].cuda(), v[0].cuda(), g[0].cuda(), beta[0].cuda(), pool_d, cu_seqlens=cu.cuda(),
                         ssm_state_indices=idx2d.cuda(), num_accepted_tokens=accepted.cuda(), layout="TND")
    assert_close("o", o, ref_o, 5e-3, stored_bf16=True)
    assert_close("pool", pool_d, ref_pool, 1e-5)


def test_fused_recurrent_with_scalar_and_channel_gates():
    from fla_b200.ops import fused_recurrent_gated_delta_rule
    B, T, H, HV = 2, 2, 2, 4
    q, k, v, gk, beta, state = _inputs(B, T, H, HV, seed=51)
    g = F.logsigmoid(torch.randn(B, T, HV, generator=torch.Generator().manual_seed(52)))
    ref_o, ref_s = _ref(q, k, v, gk + g[..., None], beta, state, 128 ** -0.5)
    o, ht = fused_recurrent_gated_delta_rule(q.cuda(), k.cuda(), v.cuda(), g=g.cuda(), gk=gk.cuda(), beta=beta.cuda(),
                                             initial_state=state.cuda(), output_final_state=True)
    assert_close("o", o, ref_o, 5e-3, stored_bf16=True)
    assert_close("state", ht, ref_s, 1e-5)

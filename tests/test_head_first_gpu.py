"""Head-first batches (`[B,H,T,D]` storage, the layout of the reference's composed entry,
examples/flash_gated_delta_rule.py:1126-1228) run on the caller's memory: the batch is folded into the head
dimension as a strided view, nothing is copied, and the results are those of the sequence-first call bit for bit."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _inputs(B, T, HK, HV, V, seed):
    g_ = torch.Generator(device="cuda").manual_seed(seed)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g_)
    q = F.normalize(rn(B, HK, T, 128), dim=-1).bfloat16()
    k = F.normalize(rn(B, HK, T, 128), dim=-1).bfloat16()
    v = rn(B, HV, T, V).bfloat16()
    g = F.logsigmoid(rn(B, T, HV))
    beta = torch.sigmoid(rn(B, T, HV))
    h0 = 0.1 * rn(B, HV, 128, V)
    return q, k, v, g, beta, h0


@pytest.mark.parametrize("B,T,HK,HV,V", [(3, 200, 2, 4, 128), (2, 129, 2, 2, 256)])
def test_fold_is_a_view_and_matches_sequence_first(B, T, HK, HV, V):
    from fla_b200.ops import chunk_gated_delta_rule, flash_gated_delta_rule
    from fla_b200.ops.gdn import _as_rows, _fold_batch, _fold_plan
    q, k, v, g, beta, h0 = _inputs(B, T, HK, HV, V, 7)
    # the views the operator hands to the kernels share the caller's storage
    views = _fold_plan(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), None)
    assert views is not None
    for t, f in zip((q, k, v), views):
        assert f.data_ptr() == t.data_ptr() and _as_rows(f) is f and f.shape[0] == 1 and f.shape[2] == B * t.shape[1]
        b, h, tok = B - 1, t.shape[1] - 1, T // 2
        assert torch.equal(f[0, tok, b * t.shape[1] + h], t[b, h, tok])
    assert _fold_batch(q.transpose(1, 2)[:, :, :1]) is None or HK == 1   # a head slice of head-first storage does not fold

    leaves = [x.clone().requires_grad_(True) for x in (q, k, v, g, beta, h0)]
    o, ht = flash_gated_delta_rule(*leaves[:5], initial_state=leaves[5], output_final_state=True)
    assert o.shape == (B, T, HV, V) and ht.shape == (B, HV, 128, V)
    g_ = torch.Generator(device="cuda").manual_seed(11)
    do = torch.randn(B, T, HV, V, device="cuda", generator=g_).bfloat16()
    dht = 0.1 * torch.randn(B, HV, 128, V, device="cuda", generator=g_)
    torch.autograd.backward([o, ht], [do, dht])

    ref = [x.clone() for x in (q, k, v, g, beta, h0)]
    ref[:3] = [x.transpose(1, 2).contiguous() for x in ref[:3]]       # sequence-first copies
    ref = [x.requires_grad_(True) for x in ref]
    o2, ht2 = chunk_gated_delta_rule(*ref[:5], initial_state=ref[5], output_final_state=True)
    torch.autograd.backward([o2, ht2], [do, dht])
    assert torch.equal(o, o2) and torch.equal(ht, ht2)
    for name, a, b in zip(("dq", "dk", "dv"), leaves[:3], ref[:3]):
        assert torch.equal(a.grad, b.grad.transpose(1, 2)), name
    for name, a, b in zip(("dg", "dbeta", "dh0"), leaves[3:], ref[3:]):
        assert torch.equal(a.grad, b.grad), name


def test_head_first_flag_of_chunk_gated_delta_rule():
    from fla_b200.ops import chunk_gated_delta_rule
    B, T, HK, HV, V = 2, 96, 2, 4, 128
    q, k, v, g, beta, h0 = _inputs(B, T, HK, HV, V, 3)
    o, ht = chunk_gated_delta_rule(q, k, v, g.transpose(1, 2), beta.transpose(1, 2), initial_state=h0, output_final_state=True,
                                   head_first=True)
    o2, ht2 = chunk_gated_delta_rule(q.transpose(1, 2).contiguous(), k.transpose(1, 2).contiguous(), v.transpose(1, 2).contiguous(),
                                     g, beta, initial_state=h0, output_final_state=True)
    assert o.shape == (B, HV, T, V)
    assert torch.equal(o.transpose(1, 2), o2) and torch.equal(ht, ht2)

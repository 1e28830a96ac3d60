"""The Gated-DeltaNet block (fla_b200.modules) against the same block written with the CPU oracle in fp64, and its
decode step against its prefill (reference block: examples/flash_gated_delta_rule.py:1249-1365)."""
import pytest
import torch
import torch.nn.functional as F

import oracle
from _util import assert_close

pytestmark = pytest.mark.gpu


class _RoundBf16(torch.autograd.Function):
    """Round to bf16 where the bf16 module stores a tensor; straight-through gradient."""

    @staticmethod
    def forward(ctx, t):
        return t.float().bfloat16().double()

    @staticmethod
    def backward(ctx, g):
        return g


def _oracle_block(blk, x, dy):
    """fp64 autograd through the block's definition with the naive recurrence; parameters taken from `blk` (CPU copies);
    tensors the bf16 module materialises (projection outputs, conv output, normalised q/k, o) are rounded likewise."""
    P = {n: p.detach().double().cpu().requires_grad_(True) for n, p in blk.named_parameters()}
    xd = x.double().cpu()
    rb = _RoundBf16.apply
    lin = lambda name, t: rb(t @ P[name + ".weight"].t())   # noqa: E731
    mixed = lin("in_proj_qkv", xd)
    B, T, C = mixed.shape
    W = P["conv_weight"].shape[1]
    xe = torch.cat([torch.zeros(B, W - 1, C, dtype=torch.float64), mixed], 1)
    mixed = rb(F.silu(sum(P["conv_weight"][:, j] * xe[:, j:j + T, :] for j in range(W))))
    kd, D, HK, HV = blk.key_dim, blk.D, blk.HK, blk.HV
    q = rb(F.normalize(mixed[..., :kd].unflatten(-1, (HK, D)), dim=-1))
    k = rb(F.normalize(mixed[..., kd:2 * kd].unflatten(-1, (HK, D)), dim=-1))
    v = mixed[..., 2 * kd:].unflatten(-1, (HV, D))
    beta = rb(lin("in_proj_b", xd).sigmoid())
    g = -P["A_log"].exp() * F.softplus(lin("in_proj_a", xd) + P["dt_bias"])
    rep = HV // HK
    o, _ = oracle.naive_recurrent_gated_delta_rule(q.repeat_interleave(rep, 2), k.repeat_interleave(rep, 2), v, beta, g,
                                                   scale=D ** -0.5, dtype=torch.float64)
    o = rb(o)
    z = lin("in_proj_z", xd).unflatten(-1, (HV, D))
    y = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + blk.norm.eps) * P["norm.weight"] * F.silu(z)
    out = lin("out_proj", rb(y).flatten(-2))
    (out * dy.double().cpu()).sum().backward()
    return out.detach(), {n: p.grad for n, p in P.items()}


def _make(hidden=256, HV=4, HK=2):
    from fla_b200.modules import GatedDeltaNetBlock
    torch.manual_seed(3)
    return GatedDeltaNetBlock(hidden, num_value_heads=HV, num_key_heads=HK).cuda().bfloat16()


def test_block_forward_backward_matches_oracle_block():
    blk = _make()
    g_ = torch.Generator().manual_seed(5)
    x = torch.randn(2, 192, 256, generator=g_).bfloat16()
    dy = torch.randn(2, 192, 256, generator=g_).bfloat16()
    ref_out, ref_grads = _oracle_block(blk, x, dy)
    xg = x.cuda().requires_grad_(True)
    out = blk(xg)
    (out.float() * dy.cuda().float()).sum().backward()
    assert_close("out", out, ref_out, 2e-2, stored_bf16=True)
    # parameter gradients of a bf16 module (bf16 GEMMs in the projections' backward): direction and size
    for n, p in blk.named_parameters():
        assert p.grad is not None, n
        a, b = p.grad.double().cpu().flatten(), ref_grads[n].flatten()
        cos = torch.dot(a, b) / (a.norm() * b.norm())
        assert cos > 0.995, (n, cos.item())
        assert abs(a.norm() / b.norm() - 1) < 0.03, (n, (a.norm() / b.norm()).item())


def test_block_decode_step_continues_the_prefill():
    blk = _make()
    g_ = torch.Generator().manual_seed(6)
    x = torch.randn(3, 65, 256, generator=g_).bfloat16().cuda()
    with torch.no_grad():
        full = blk(x)
        _, caches = blk(x[:, :64], return_caches=True)
        last = blk.step(x[:, 64], caches)
    assert_close("decode", last, full[:, 64], 3e-2, stored_bf16=True)

"""Oracle parity at the benchmark's own sizes.

The full-size launch of each training configuration (GDN: B=8, T=4096, HK=16, HV=32; KDA: B=4, T=8192, H=32) is
run once on the GPU; (batch row, q/k head) slices are independent recurrences, so one slice - every token of
one batch row for one q/k head and the value heads that share it - is cut out of the full-size results and
compared with the naive fp64 recurrence and its autograd gradients on the same slice of the inputs
(the reference's own harness, examples/flash_gated_delta_rule.py:1574-1631,1738-1761, at the full length).
Tolerance: max-abs-error / RMS(reference) <= 5e-3 on fp32 outputs and gradients; the bf16-stored results of the
same launch are held to the same bar plus half a bf16 ulp of the reference value (the store's own rounding).
"""
import pytest
import torch
import torch.nn.functional as F

import oracle
from _util import assert_close

pytestmark = pytest.mark.gpu

TOL = 5e-3


def _gdn_inputs(B, T, HK, HV, seed):
    g_ = torch.Generator(device="cuda").manual_seed(seed)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g_)  # noqa: E731
    return dict(q=F.normalize(rn(B, T, HK, 128), dim=-1).bfloat16(), k=F.normalize(rn(B, T, HK, 128), dim=-1).bfloat16(),
                v=rn(B, T, HV, 128).bfloat16(), g=F.logsigmoid(rn(B, T, HV)).bfloat16(),
                beta=torch.sigmoid(rn(B, T, HV)).bfloat16(), h0=0.1 * rn(B, HV, 128, 128),
                do=rn(B, T, HV, 128).bfloat16(), dht=0.1 * rn(B, HV, 128, 128))


def test_gdn_config2_slice_matches_the_fp64_recurrence_at_full_length():
    from fla_b200.ops import chunk_gated_delta_rule_fwd_bwd as fb
    B, T, HK, HV = 8, 4096, 16, 32
    d = _gdn_inputs(B, T, HK, HV, seed=4002)
    r, hk = 6, 11
    hv = slice(2 * hk, 2 * hk + 2)
    o32, ht, g32 = fb(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], initial_state=d["h0"], dht=d["dht"],
                      output_dtype=torch.float32, grad_dtype=torch.float32)
    o16, _, g16 = fb(d["q"], d["k"], d["v"], d["g"], d["beta"], d["do"], initial_state=d["h0"], dht=d["dht"])
    cut = lambda t, heads: t[r:r + 1, :, heads].cpu()  # noqa: E731
    ref = oracle.gdn_reference_fwd_bwd(cut(d["q"], slice(hk, hk + 1)), cut(d["k"], slice(hk, hk + 1)), cut(d["v"], hv),
                                       cut(d["g"], hv), cut(d["beta"], hv), initial_state=d["h0"][r:r + 1, hv].cpu(),
                                       do=cut(d["do"], hv), dht=d["dht"][r:r + 1, hv].cpu(), dtype=torch.float64)
    qk = slice(hk, hk + 1)
    for got32, got16 in ((dict(o=o32, dq=g32[0], dk=g32[1], dv=g32[2], dg=g32[3], dbeta=g32[4]),
                          dict(o=o16, dq=g16[0], dk=g16[1], dv=g16[2], dg=g16[3], dbeta=g16[4])),):
        for name in ("o", "dq", "dk", "dv", "dg", "dbeta"):
            heads = qk if name in ("dq", "dk") else hv
            assert_close(name + " (fp32 out)", cut(got32[name], heads), ref[name], TOL)
            assert_close(name + " (bf16 out)", cut(got16[name], heads), ref[name], TOL, stored_bf16=True)
    assert_close("ht", ht[r:r + 1, hv], ref["ht"], TOL)
    assert_close("dh0", g32[5][r:r + 1, hv], ref["dh0"], TOL)


def test_kda_config3_slice_matches_the_fp64_recurrence_at_full_length():
    from fla_b200.ops import chunk_kda_fwd_bwd
    B, T, H = 4, 8192, 32
    g_ = torch.Generator(device="cuda").manual_seed(4003)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g_)  # noqa: E731
    q, k = F.normalize(rn(B, T, H, 128), dim=-1).bfloat16(), F.normalize(rn(B, T, H, 128), dim=-1).bfloat16()
    v, g = rn(B, T, H, 128).bfloat16(), (F.logsigmoid(rn(B, T, H, 128)) / 16).bfloat16()
    beta, do = torch.sigmoid(rn(B, T, H)).bfloat16(), rn(B, T, H, 128).bfloat16()
    r, h = 2, 19
    hs = slice(h, h + 1)
    o32, ht, g32 = chunk_kda_fwd_bwd(q, k, v, g, beta, do, output_dtype=torch.float32, grad_dtype=torch.float32)
    cut = lambda t: t[r:r + 1, :, hs].cpu()  # noqa: E731
    ref = oracle.kda_reference_fwd_bwd(cut(q), cut(k), cut(v), cut(g), cut(beta), do=cut(do), dtype=torch.float64)
    got = dict(o=o32, dq=g32[0], dk=g32[1], dv=g32[2], dg=g32[3], dbeta=g32[4])
    for name in ("o", "dq", "dk", "dv", "dg", "dbeta"):
        assert_close(name, cut(got[name]), ref[name], TOL)
    assert_close("ht", ht[r:r + 1, hs], ref["ht"], TOL)
    del o32, g32
    o16, _, g16 = chunk_kda_fwd_bwd(q, k, v, g, beta, do)
    got = dict(o=o16, dq=g16[0], dk=g16[1], dv=g16[2], dg=g16[3], dbeta=g16[4])
    for name in ("o", "dq", "dk", "dv", "dg", "dbeta"):
        assert_close(name + " (bf16 out)", cut(got[name]), ref[name], TOL, stored_bf16=True)

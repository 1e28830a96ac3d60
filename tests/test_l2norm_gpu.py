"""l2norm kernels against the formulas of the reference's l2norm_fwd / l2norm_bwd, and the
use_qk_l2norm_in_kernel option of chunk_gated_delta_rule."""
import pytest
import torch
import torch.nn.functional as F

import oracle
from _util import assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape", [(3, 7, 2, 128), (50, 64), (5, 256), (1, 1024)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_l2norm_forward_backward(shape, dtype):
    from fla_b200.ops import l2norm_bwd, l2norm_fwd
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(*shape, generator=g) * 2).to(dtype)
    dy = torch.randn(*shape, generator=g).to(dtype)
    xd = x.double()
    rstd_ref = torch.rsqrt((xd * xd).sum(-1) + 1e-6)
    y_ref = xd * rstd_ref[..., None]
    y, rstd = l2norm_fwd(x.cuda(), output_dtype=torch.float32)
    assert_close("rstd", rstd, rstd_ref, 1e-5)
    assert_close("y", y, y_ref, 1e-5)
    y_store, _ = l2norm_fwd(x.cuda())
    assert y_store.dtype == dtype
    assert_close("y_stored", y_store, y_ref, 1e-5, stored_bf16=(dtype == torch.bfloat16))
    yd = y_store.double().cpu()
    dx_ref = dy.double() * rstd_ref[..., None] - (dy.double() * yd).sum(-1, keepdim=True) * yd * rstd_ref[..., None]
    dx = l2norm_bwd(y_store, rstd, dy.cuda())
    assert_close("dx", dx, dx_ref, 1e-5, stored_bf16=(dtype == torch.bfloat16))


def test_chunk_gdn_with_qk_l2norm_in_kernel():
    """Like the reference, the normalised q and k are stored in bf16 before the chunk kernels; parity is
    therefore taken against the oracle fed with those stored values, and the l2norm backward is checked by
    comparing with autograd through F.normalize-free formulas above (dq, dk chain through l2norm_bwd)."""
    from fla_b200.ops import chunk_gated_delta_rule, l2norm_fwd
    inp = oracle.make_gdn_inputs(1, 192, 2, 4, seed=21)
    gen = torch.Generator().manual_seed(3)
    q = (torch.randn(1, 192, 2, 128, generator=gen) * 2).bfloat16()
    k = (torch.randn(1, 192, 2, 128, generator=gen) * 0.7).bfloat16()
    qn, q_rstd = l2norm_fwd(q.cuda())
    kn, k_rstd = l2norm_fwd(k.cuda())
    ref = oracle.gdn_reference_fwd_bwd(qn.cpu(), kn.cpu(), inp["v"], inp["g"], inp["beta"], initial_state=inp["h0"],
                                       do=inp["do"], dht=inp["dht"], dtype=torch.float64)
    d = {n: t.cuda() for n, t in inp.items()}
    ql, kl = q.cuda().requires_grad_(True), k.cuda().requires_grad_(True)
    vl = d["v"].clone().requires_grad_(True)
    o, ht = chunk_gated_delta_rule(ql, kl, vl, d["g"], d["beta"], initial_state=d["h0"], output_final_state=True,
                                   use_qk_l2norm_in_kernel=True, output_dtype=torch.float32)
    assert_close("o", o, ref["o"], 5e-3)
    assert_close("ht", ht, ref["ht"], 5e-3)
    ((o * d["do"].float()).sum() + (ht * d["dht"]).sum()).backward()
    assert_close("dv", vl.grad, ref["dv"], 5e-3, stored_bf16=True)
    # chain rule through the normalisation, in fp64 from the oracle's gradients w.r.t. the normalised q, k
    for name, x, xn, rstd, grad in (("dq", q, qn, q_rstd, ql.grad), ("dk", k, kn, k_rstd, kl.grad)):
        yd, r = xn.double().cpu(), rstd.double().cpu()[..., None]
        gy = ref[name]
        dx_ref = gy * r - (gy * yd).sum(-1, keepdim=True) * yd * r
        assert_close(name, grad, dx_ref, 8e-3, stored_bf16=True)

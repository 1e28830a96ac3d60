"""The sequence-first operator names of the reference's second package (fla_npu.ops.triton) against the CPU oracle."""
import pytest
import torch
import torch.nn.functional as F

import oracle
from _util import assert_close

pytestmark = pytest.mark.gpu


def _inputs(B, T, HK, HV, seed):
    g_ = torch.Generator().manual_seed(seed)
    k = F.normalize(torch.randn(B, T, HK, 128, generator=g_), dim=-1).bfloat16()
    g = F.logsigmoid(torch.randn(B, T, HV, generator=g_))
    beta = torch.sigmoid(torch.randn(B, T, HV, generator=g_))
    return k, g, beta


@pytest.mark.parametrize("cu", [None, [0, 70, 71, 200, 300]])
def test_cumsum_kkt_solve_chain_sequence_first(cu):
    from fla_b200.ops import upstream as up
    B, T, HK, HV = (2, 200, 2, 4) if cu is None else (1, 300, 1, 2)
    k, g, beta = _inputs(B, T, HK, HV, seed=5)
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32)
    st = oracle.stages
    # oracle works head-first
    g_ref = st.chunk_local_cumsum_ref(g.transpose(1, 2), 64, cu_seqlens=cu)
    gc = up.chunk_local_cumsum(g.cuda(), 64, cu_seqlens=cu_t)
    assert gc.shape == g.shape and gc.dtype == torch.float32
    assert_close("cumsum", gc.transpose(1, 2), g_ref, 1e-5)
    gr = up.chunk_local_cumsum(g.cuda(), 64, reverse=True, cu_seqlens=cu_t, head_first=False)
    assert_close("reverse cumsum", gr.transpose(1, 2), st.chunk_local_cumsum_ref(g.transpose(1, 2), 64, cu_seqlens=cu, reverse=True), 1e-5)
    A_ref = st.chunk_scaled_dot_kkt_ref(k.transpose(1, 2), g_ref, beta.transpose(1, 2), 64, cu_seqlens=cu)
    # the reference function takes k head-first ([B,HK,T,K]) next to sequence-first g / beta
    A = up.chunk_scaled_dot_kkt_fwd(k.transpose(1, 2).contiguous().cuda(), g=gc, beta=beta.cuda(), cu_seqlens=cu_t, chunk_size=64)
    with pytest.raises(ValueError, match=r"expected k \[B, Hk, T, K\]"):
        up.chunk_scaled_dot_kkt_fwd(k.cuda(), g=gc, beta=beta.cuda(), cu_seqlens=cu_t, chunk_size=64)
    assert tuple(A.shape) == (B, T, HV, 64) and A.dtype == torch.float32
    assert_close("A", A.transpose(1, 2), A_ref, 5e-3)
    X_ref = st.solve_tri_ref(A_ref.float(), 64, cu_seqlens=cu)
    X = up.solve_tril(A, cu_seqlens=cu_t, output_dtype=torch.float32)
    assert tuple(X.shape) == (B, T, HV, 64)
    assert_close("X", X.transpose(1, 2), X_ref, 5e-3)


def test_l2norm_function_and_module():
    from fla_b200.ops import upstream as up
    x = torch.randn(3, 50, 4, 128, generator=torch.Generator().manual_seed(9)).bfloat16()
    dy = torch.randn(3, 50, 4, 128, generator=torch.Generator().manual_seed(10)).bfloat16()
    xr = x.double().requires_grad_(True)
    yr = xr * torch.rsqrt((xr * xr).sum(-1, keepdim=True) + 1e-6)
    (yr * dy.double()).sum().backward()
    xd = x.cuda().requires_grad_(True)
    y = up.L2Norm()(xd)
    (y.float() * dy.cuda().float()).sum().backward()
    assert y.dtype == torch.bfloat16 and xd.grad.dtype == torch.bfloat16
    assert_close("y", y, yr.detach(), 5e-3, stored_bf16=True)
    assert_close("dx", xd.grad, xr.grad, 5e-3, stored_bf16=True)
    assert torch.equal(up.l2norm(x.cuda()), y.detach())
    assert set(up.__all__) >= {"chunk_local_cumsum", "chunk_scaled_dot_kkt_fwd", "l2norm", "solve_tril", "input_guard",
                               "autocast_custom_fwd", "autocast_custom_bwd"}

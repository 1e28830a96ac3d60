"""Parity of the causal_conv1d backward with the CPU oracle (autograd through the definition, pinned to the
reference's hand-written golden by tests/test_oracle_golden.py), through the C ABI."""
import pytest
import torch

import oracle
from _util import assert_close

pytestmark = pytest.mark.gpu
TOL = 5e-3


def _inputs(B, T, D, W, seed):
    g_ = torch.Generator().manual_seed(seed)
    x = torch.randn(B, T, D, generator=g_).bfloat16()
    w = (0.5 * torch.randn(D, W, generator=g_)).bfloat16()
    b = (0.1 * torch.randn(D, generator=g_)).bfloat16()
    dy = torch.randn(B, T, D, generator=g_).bfloat16()
    init = torch.randn(B, D, W - 1, generator=g_).bfloat16()
    dht = torch.randn(B, D, W - 1, generator=g_).bfloat16()
    return x, w, b, dy, init, dht


def _ref(x, w, b, dy, init, dht, act):
    """oracle in the reference layouts ([W,D] weights, [B,W,D] states with row 0 unused) -> this package's layouts"""
    B, _, D = x.shape
    W = w.shape[1]
    to_ref = lambda s: None if s is None else torch.cat([torch.zeros(s.shape[0], 1, D), s.float().transpose(1, 2)], 1)  # noqa: E731
    dx, dw, db, dh0 = oracle.causal_conv1d_bwd_ref(x, w.t(), dy, b, to_ref(init), to_ref(dht), act)
    return dx, dw.t(), db, dh0[:, 1:, :].transpose(1, 2)


@pytest.mark.parametrize("B,T,D,W", [(2, 300, 64, 4), (1, 257, 1032, 3), (3, 70, 128, 2), (2, 513, 2048, 4)])
@pytest.mark.parametrize("act", [None, "silu"])
def test_conv_backward_matches_oracle(B, T, D, W, act):
    from fla_b200.ops import causal_conv1d_bwd
    x, w, b, dy, init, dht = _inputs(B, T, D, W, seed=7 + T)
    ref = _ref(x, w, b, dy, init, dht, 1 if act else 0)
    dx, dw, db, dh0 = causal_conv1d_bwd(x.cuda(), w.cuda(), dy.cuda(), b.cuda(), init.cuda(), dht.cuda(), act)
    torch.cuda.synchronize()
    assert_close("dx", dx, ref[0], TOL, stored_bf16=True)
    assert_close("dw", dw, ref[1], 1e-4)
    assert_close("db", db, ref[2], 1e-4)
    assert_close("dh0", dh0, ref[3], 1e-4)


def test_conv_backward_without_states_and_bias():
    from fla_b200.ops import causal_conv1d_bwd
    x, w, _, dy, _, _ = _inputs(2, 130, 256, 4, seed=3)
    ref = _ref(x, w, None, dy, None, None, 1)
    dx, dw, db, dh0 = causal_conv1d_bwd(x.cuda(), w.cuda(), dy.cuda(), activation="silu")
    assert dh0 is None
    assert_close("dx", dx, ref[0], TOL, stored_bf16=True)
    assert_close("dw", dw, ref[1], 1e-4)
    assert_close("db", db, ref[2], 1e-4)


def test_conv_backward_varlen_packed():
    from fla_b200.ops import causal_conv1d_bwd
    cu = [0, 5, 5, 270, 271, 600]
    N, T, D, W = len(cu) - 1, cu[-1], 128, 4
    x, w, b, dy, _, _ = _inputs(1, T, D, W, seed=9)
    g_ = torch.Generator().manual_seed(10)
    init = torch.randn(N, D, W - 1, generator=g_).bfloat16()
    dht = torch.randn(N, D, W - 1, generator=g_).bfloat16()
    dxs, dws, dbs, dh0s = [], 0, 0, []
    for n in range(N):
        sl = slice(cu[n], cu[n + 1])
        if sl.stop - sl.start < W - 1:       # shorter than the state: compare only sequences the reference defines
            dht[n] = 0
        if sl.stop == sl.start:
            dh0s.append(torch.zeros(1, D, W - 1, dtype=torch.float64))
            continue
        r = _ref(x[:, sl], w, b, dy[:, sl], init[n:n + 1], dht[n:n + 1], 1)
        dxs.append(r[0]); dws = dws + r[1]; dbs = dbs + r[2]; dh0s.append(r[3])
    dx, dw, db, dh0 = causal_conv1d_bwd(x.cuda(), w.cuda(), dy.cuda(), b.cuda(), init.cuda(), dht.cuda(), "silu",
                                        cu_seqlens=torch.tensor(cu, dtype=torch.int32))
    assert_close("dx", dx, torch.cat(dxs, 1), TOL, stored_bf16=True)
    assert_close("dw", dw, dws, 1e-4)
    assert_close("db", db, dbs, 1e-4)
    assert_close("dh0", dh0, torch.cat(dh0s, 0), 1e-4)


def test_causal_conv1d_is_differentiable_and_reference_signature():
    from fla_b200.ops import causal_conv1d, npu_causal_conv1d_bwd
    B, T, D, W = 2, 140, 256, 4
    x, w, b, dy, init, dht = _inputs(B, T, D, W, seed=21)
    ref = _ref(x, w, b, dy, init, dht, 1)
    leaves = [t.cuda().requires_grad_(True) for t in (x, w, b, init)]
    y, final = causal_conv1d(leaves[0], leaves[1], leaves[2], initial_state=leaves[3], output_final_state=True,
                             activation="silu")
    ((y.float() * dy.cuda().float()).sum() + (final.float() * dht.cuda().float()).sum()).backward()
    assert_close("dx", leaves[0].grad, ref[0], TOL, stored_bf16=True)
    assert_close("dw", leaves[1].grad, ref[1], TOL, stored_bf16=True)
    assert_close("db", leaves[2].grad, ref[2], TOL, stored_bf16=True)
    assert_close("dh0", leaves[3].grad, ref[3], TOL, stored_bf16=True)
    # the reference's low-level signature: [W,D] weights, [B,W,D] states, pre-activation y
    x32 = x.float()
    xe = torch.cat([init.float().transpose(1, 2), x32], 1)
    pre = sum(w.float()[:, j] * xe[:, j:j + T, :] for j in range(W)).bfloat16()       # no bias in this signature
    ref2 = _ref(x, w, None, dy, init, dht, 1)
    st = lambda s: torch.cat([torch.zeros(B, 1, D), s.float().transpose(1, 2)], 1).bfloat16().cuda()  # noqa: E731
    dx, dw, db, dh0 = npu_causal_conv1d_bwd(x.cuda(), pre.cuda(), w.t().contiguous().cuda(), dy.cuda(), st(init), st(dht),
                                            activation=1)
    assert dw.shape == (W, D) and dh0.shape == (B, W, D)
    assert_close("dx", dx, ref2[0], 2e-2, stored_bf16=True)        # y arrives rounded to bf16
    assert_close("dw", dw.t(), ref2[1], 2e-2, stored_bf16=True)
    assert_close("dh0", dh0[:, 1:, :].transpose(1, 2), ref2[3], 2e-2, stored_bf16=True)

"""Parity of causal_conv1d forward / update with the CPU oracle (through the C ABI)."""
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from _util import assert_close

pytestmark = pytest.mark.gpu
TOL = 5e-3


def _ref_fwd(x, w, b, init, act):
    # oracle works channel-first in fp64 on the bf16-rounded inputs
    y, fs = oracle.causal_conv1d_ref(x.double().transpose(1, 2), w.double(), None if b is None else b.double(),
                                     None if init is None else init.double(), True, act)
    return y.transpose(1, 2), fs


@pytest.mark.parametrize("B,T,D,W", [(2, 100, 256, 4), (1, 5, 64, 3), (3, 2, 128, 4), (2, 64, 1024, 2), (1, 1, 8, 4)])
@pytest.mark.parametrize("act", [None, "silu"])
@pytest.mark.parametrize("with_init", [False, True])
def test_prefill_matches_oracle(B, T, D, W, act, with_init):
    from fla_b200.ops import causal_conv1d
    inp = oracle.make_conv_inputs(B, T, D, W, seed=3, with_state=with_init)
    init = inp.get("state")
    ref_y, ref_fs = _ref_fwd(inp["x"], inp["weight"], inp["bias"], init, act)
    y, fs = causal_conv1d(inp["x"].cuda(), inp["weight"].cuda(), inp["bias"].cuda(),
                          initial_state=None if init is None else init.cuda(), output_final_state=True, activation=act)
    assert_close("y", y, ref_y, TOL, stored_bf16=True)
    assert torch.equal(fs.cpu().float(), ref_fs.float()), "final state must be the exact last W-1 inputs"


def test_prefill_residual_weight_layout_and_no_bias():
    from fla_b200.ops import causal_conv1d
    inp = oracle.make_conv_inputs(2, 70, 128, 4, seed=4)
    res = torch.randn(2, 70, 128).bfloat16()
    ref_y, _ = _ref_fwd(inp["x"], inp["weight"], None, None, "silu")
    ref_y = ref_y + res.double()
    w_wd = inp["weight"].t().contiguous().cuda()      # reference layout [W,D], passed as a transposed view
    y, fs = causal_conv1d(inp["x"].cuda(), w_wd.t(), None, residual=res.cuda(), activation="silu")
    assert fs is None
    assert_close("y", y, ref_y, TOL, stored_bf16=True)


def test_prefill_varlen_with_initial_states():
    from fla_b200.ops import causal_conv1d
    D, W = 128, 4
    lens = [1, 70, 2, 64, 3, 129]
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    inp = oracle.make_conv_inputs(1, int(cu[-1]), D, W, seed=8)
    init = torch.randn(len(lens), D, W - 1).bfloat16()
    ys, fss = [], []
    for i, L in enumerate(lens):
        xs = inp["x"][:, int(cu[i]):int(cu[i + 1])]
        y_i, fs_i = _ref_fwd(xs, inp["weight"], inp["bias"], init[i:i + 1], "silu")
        ys.append(y_i); fss.append(fs_i)
    y, fs = causal_conv1d(inp["x"].cuda(), inp["weight"].cuda(), inp["bias"].cuda(), initial_state=init.cuda(),
                          output_final_state=True, activation="silu", cu_seqlens=cu.cuda())
    assert_close("y", y, torch.cat(ys, 1), TOL, stored_bf16=True)
    assert torch.equal(fs.cpu().float(), torch.cat(fss, 0).float())


@pytest.mark.parametrize("layout", ["taps_contiguous", "channels_contiguous", "strided"])
@pytest.mark.parametrize("W", [2, 3, 4])
def test_update_single_token(layout, W):
    from fla_b200.ops import causal_conv1d_update
    N, D = 5, 256
    inp = oracle.make_conv_inputs(N, 1, D, W, seed=12, with_state=True)
    x = inp["x"][:, 0]
    st_ref = inp["state"].double().clone()
    ref = oracle.causal_conv1d_update_ref(x.double(), st_ref, inp["weight"].double(), inp["bias"].double(), "silu")
    if layout == "taps_contiguous":
        cache = inp["state"].cuda().contiguous()                       # [N,D,W-1]
    elif layout == "channels_contiguous":
        cache = inp["state"].transpose(1, 2).contiguous().cuda().transpose(1, 2)   # memory [N,W-1,D]
    else:
        big = torch.zeros(N, D, W + 2, dtype=torch.bfloat16, device="cuda")
        cache = big[:, :, 1:W]
        cache.copy_(inp["state"].cuda())
    ver = cache._version
    y = causal_conv1d_update(x.cuda(), cache, weight=inp["weight"].cuda(), bias=inp["bias"].cuda(), activation="silu")
    assert cache._version > ver
    assert_close("y", y, ref, TOL, stored_bf16=True)
    assert torch.equal(cache.cpu().float(), st_ref.float())


def test_update_cache_indices_and_pad_slot():
    from fla_b200.ops import causal_conv1d_update
    N, D, W, slots = 4, 128, 4, 9
    inp = oracle.make_conv_inputs(slots, 1, D, W, seed=13, with_state=True)
    x = inp["x"][:N, 0]
    idx = torch.tensor([7, -1, 2, 5], dtype=torch.int32)
    pool = inp["state"].cuda().clone()
    before = pool.clone()
    y = causal_conv1d_update(x.cuda(), pool, weight=inp["weight"].cuda(), bias=None, activation=None,
                             cache_indices=idx.cuda(), pad_slot_id=-1)
    for n, s in enumerate(idx.tolist()):
        if s < 0:
            continue
        st = inp["state"][s:s + 1].double().clone()
        ref = oracle.causal_conv1d_update_ref(x[n:n + 1].double(), st, inp["weight"].double(), None, None)
        assert_close(f"y[{n}]", y[n:n + 1], ref, TOL, stored_bf16=True)
        assert torch.equal(pool[s].cpu().float(), st[0].float())
    untouched = [s for s in range(slots) if s not in (7, 2, 5)]
    assert torch.equal(pool[untouched], before[untouched])


def test_update_multi_token_and_speculative_window():
    from fla_b200.ops import causal_conv1d_update
    N, D, W, T = 3, 64, 4, 3
    g = torch.Generator().manual_seed(21)
    w = (0.5 * torch.randn(D, W, generator=g)).bfloat16()
    b = (0.1 * torch.randn(D, generator=g)).bfloat16()
    x = torch.randn(N, D, T, generator=g).bfloat16()               # oracle layout (batch, dim, seqlen)
    st = torch.randn(N, D, W - 1 + T - 1, generator=g).bfloat16()
    acc = torch.tensor([1, 3, 2], dtype=torch.int32)
    st_ref = st.double().clone()
    ref = oracle.causal_conv1d_update_spec_ref(x.double(), st_ref, w.double(), b.double(), acc, "silu")
    pool = st.cuda().clone()
    y = causal_conv1d_update(x.transpose(1, 2).contiguous().cuda(), pool, weight=w.cuda(), bias=b.cuda(),
                             activation="silu", num_accepted_tokens=acc.cuda())
    assert_close("y_spec", y, ref.transpose(1, 2), TOL, stored_bf16=True)
    assert torch.equal(pool.cpu().float(), st_ref.float())
    # plain multi-token update: state is the last S entries of (state, x)
    st_ref = st.double().clone()
    ref = oracle.causal_conv1d_update_ref(x.double(), st_ref, w.double(), b.double(), None)
    pool = st.cuda().clone()
    y = causal_conv1d_update(x.transpose(1, 2).contiguous().cuda(), pool, weight=w.cuda(), bias=b.cuda())
    assert_close("y_multi", y, ref.transpose(1, 2), TOL, stored_bf16=True)
    assert torch.equal(pool.cpu().float(), st_ref.float())


def test_reference_known_answer_vectors():
    """The arange/128 known-answer inputs of the reference's unit tests, through the reference signature."""
    from fla_b200.ops import npu_causal_conv1d
    f = {k: torch.from_numpy(v) for k, v in np.load(Path(__file__).parent / "golden" / "conv_golden.npz").items()}
    D = 16
    x = f["x"].transpose(1, 2).contiguous().bfloat16()          # [B,T,D]
    w_op = f["w"].t().contiguous().bfloat16()                    # [W,D]
    bias = f["b"].bfloat16()
    ref_y, ref_fs = oracle.causal_conv1d_ref(x.double().transpose(1, 2), w_op.double().t(), bias.double(), None, True, "silu")
    conv_states = torch.zeros(2, 3, D, dtype=torch.bfloat16, device="cuda")
    y = npu_causal_conv1d(x.cuda(), w_op.cuda(), bias.cuda(), conv_states, activation_mode=1, run_mode=0)
    assert_close("y", y, ref_y.transpose(1, 2), TOL, stored_bf16=True)
    assert torch.equal(conv_states.cpu().float(), ref_fs.transpose(1, 2).float())
    # decode step on the same state pool
    xu = f["xu"].bfloat16()
    st_ref = ref_fs.double().clone()
    ref_u = oracle.causal_conv1d_update_ref(xu.double(), st_ref, w_op.double().t(), bias.double(), "silu")
    yu = npu_causal_conv1d(xu.cuda(), w_op.cuda(), bias.cuda(), conv_states, activation_mode=1, run_mode=1)
    assert_close("y_update", yu, ref_u, TOL, stored_bf16=True)
    assert torch.equal(conv_states.cpu().float(), st_ref.transpose(1, 2).float())


@pytest.mark.parametrize("packed", [False, True])
def test_prefill_head_first_output(packed):
    """`head_num` of the reference operator (_aclnn_ctypes.py:939-948): the prefill output is written head-first,
    `[B, head_num, T, D // head_num]`; bit-identical to the `[B, T, D]` output re-laid on the host."""
    from fla_b200.ops import npu_causal_conv1d
    B, T, D, W, H = (1, 150, 512, 4, 4) if packed else (2, 70, 256, 3, 8)
    inp = oracle.make_conv_inputs(B, T, D, W, seed=21)
    x = inp["x"].cuda()
    w_wd = inp["weight"].t().contiguous().cuda()
    kw = dict(activation_mode=1)
    if packed:
        x = x[0]
        kw["query_start_loc"] = [0, 40, 41, 150]
    y_plain = npu_causal_conv1d(x, w_wd, inp["bias"].cuda(), **kw)
    y_heads = npu_causal_conv1d(x, w_wd, inp["bias"].cuda(), head_num=H, **kw)
    if packed:
        assert y_heads.shape == (H, T, D // H)
        assert torch.equal(y_heads, y_plain.view(T, H, D // H).permute(1, 0, 2))
    else:
        assert y_heads.shape == (B, H, T, D // H)
        assert torch.equal(y_heads, y_plain.view(B, T, H, D // H).permute(0, 2, 1, 3))

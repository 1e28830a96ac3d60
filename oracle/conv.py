"""causal_conv1d oracle (test infrastructure only).

Follows the reference's CPU goldens (torch_custom/fla_npu/test/test_npu_causal_conv1d.py:25-151),
which use channel-first tensors: x (batch, dim, seqlen), weight (dim, width),
conv_state (batch, dim, state_len).  y[t] = act(bias + sum_j w[j] x[t - (W-1) + j]).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def causal_conv1d_ref(x, weight, bias=None, initial_states=None, return_final_states=False, activation="silu"):
    """Prefill golden (test_npu_causal_conv1d.py:25-54).  Returns (out, final_states or None)."""
    dtype_in = x.dtype
    x = x.to(weight.dtype)
    seqlen = x.shape[-1]
    dim, width = weight.shape
    if initial_states is None:
        out = F.conv1d(x, weight.unsqueeze(1), bias, padding=width - 1, groups=dim)
    else:
        x = torch.cat([initial_states.to(weight.dtype), x], dim=-1)
        out = F.conv1d(x, weight.unsqueeze(1), bias, padding=0, groups=dim)
    out = out[..., :seqlen]
    final_states = None
    if return_final_states:
        final_states = F.pad(x, (width - 1 - x.shape[-1], 0)).to(dtype_in)
    out = (out if activation is None else F.silu(out)).to(dtype=dtype_in)
    return out, final_states


def causal_conv1d_update_ref(x, conv_state, weight, bias=None, activation=None):
    """Decode golden without circular cache (test_npu_causal_conv1d.py:57-91); conv_state updated in place."""
    dtype_in = x.dtype
    unsqueeze = x.dim() == 2
    if unsqueeze:
        x = x.unsqueeze(-1)
    batch, dim, seqlen = x.shape
    state_len = conv_state.shape[-1]
    x_new = torch.cat([conv_state, x], dim=-1).to(weight.dtype)
    conv_state.copy_(x_new[:, :, -state_len:])
    out = F.conv1d(x_new, weight.unsqueeze(1), bias, padding=0, groups=dim)[:, :, -seqlen:]
    if unsqueeze:
        out = out.squeeze(-1)
    return (out if activation is None else F.silu(out)).to(dtype=dtype_in)


def causal_conv1d_update_spec_ref(x, conv_state, weight, bias=None, num_accepted_tokens=None, activation=None):
    """Speculative-decode golden (test_npu_causal_conv1d.py:94-151): history window starts at accepted-1."""
    dtype_in = x.dtype
    x = x.to(weight.dtype)
    conv_state_f = conv_state.to(weight.dtype)
    num_accepted_tokens = torch.as_tensor(num_accepted_tokens, dtype=torch.long)
    batch, dim, seqlen = x.shape
    width = weight.shape[1]
    keep = width - 2
    out = torch.empty_like(x)
    for s in range(batch):
        offset = int(num_accepted_tokens[s]) - 1
        hist = conv_state_f[s:s + 1, :, offset:offset + width - 1]
        x_cat = torch.cat([hist, x[s:s + 1]], dim=-1)
        y = F.conv1d(x_cat, weight.unsqueeze(1), bias, padding=0, groups=dim)[..., :seqlen]
        out[s:s + 1] = y if activation is None else F.silu(y)
        if keep > 0:
            conv_state_f[s, :, :keep] = conv_state_f[s, :, offset + 1:offset + 1 + keep].clone()
        conv_state_f[s, :, keep:keep + seqlen] = x[s]
    conv_state.copy_(conv_state_f.to(conv_state.dtype))
    return out.to(dtype=dtype_in)


def causal_conv1d_bwd_ref(x, weight, dy, bias=None, initial_state=None, dht=None, activation=0, dtype=torch.float64):
    """Gradients of the prefill conv by autograd through its definition, in the reference operator's layouts
    (golden torch_custom/fla_npu/test/test_npu_causal_conv1d_bwd.py:33-127, which writes the same sums out by hand):
    x, dy `[B,T,D]`; weight `[W,D]`; initial_state / dht `[B,W,D]` whose rows 1..W-1 are the W-1 stored inputs.
    Returns dx `[B,T,D]`, dw `[W,D]`, db `[D]`, dh0 `[B,W,D]` (row 0 zero) in `dtype`."""
    B, T, D = x.shape
    W = weight.shape[0]
    xf = x.to(dtype).clone().requires_grad_(True)
    wf = weight.to(dtype).clone().requires_grad_(True)
    bf = (torch.zeros(D) if bias is None else bias).to(dtype).clone().requires_grad_(True)
    init = (torch.zeros(B, W, D) if initial_state is None else initial_state).to(dtype).clone().requires_grad_(True)
    xe = torch.cat([init[:, 1:, :], xf], dim=1)                       # [B, W-1+T, D]
    pre = bf + sum(wf[j] * xe[:, j:j + T, :] for j in range(W))
    out = F.silu(pre) if activation else pre
    loss = (out * dy.to(dtype)).sum()
    if dht is not None:
        loss = loss + (xe[:, T:, :] * dht.to(dtype)[:, 1:, :]).sum()   # final state = the last W-1 inputs
    loss.backward()
    return xf.grad, wf.grad, bf.grad, init.grad

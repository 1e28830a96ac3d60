"""causal_conv1d forward / decode update.

`causal_conv1d` and `causal_conv1d_update` use the `[B,T,D]` surface the reference's composed entry
exposes (examples/flash_gated_delta_rule.py:422-443: x, weight `[D,W]`, bias, residual, initial_state,
activation, cu_seqlens, output_final_state).  States are `[N,D,W-1]` (the last W-1 inputs);
`npu_causal_conv1d` below keeps the reference low-level operator's signature and its
`[W,D]` weight / `[N,W-1,D]` state layouts (…/ops/ascendc/_aclnn_ctypes.py:951-985).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _runtime as rt
from ._structs import CausalConv1dBwdArgs, CausalConv1dFwdArgs, CausalConv1dUpdateArgs


def _act(activation) -> int:
    if activation in (None, 0, False):
        return 0
    if activation in ("silu", "swish", 1, True):
        return 1
    raise NotImplementedError(f"activation must be None, 'silu' or 'swish', got {activation!r}")


def causal_conv1d_bwd(x, weight, dy, bias=None, initial_state=None, dht=None, activation=None, cu_seqlens=None,
                      y_pre=None, need_dh0=None):
    """Gradients of :func:`causal_conv1d` (layouts as there).  Returns ``(dx, dw [D,W] f32, db [D] f32, dh0 | None)``.
    The pre-activation is recomputed from x (and bias) unless ``y_pre`` holds it."""
    B, T, D = x.shape
    W = weight.shape[1]
    if x.stride(-1) != 1:
        x = x.contiguous()
    dy = dy.contiguous() if dy.stride(-1) != 1 or dy.dtype != x.dtype else dy
    if dy.dtype != x.dtype:
        dy = dy.to(x.dtype)
    cu = None
    N = B
    if cu_seqlens is not None:
        cu = cu_seqlens.to(device=x.device, dtype=torch.int32)
        N = cu.numel() - 1
    dx = torch.empty_like(x)
    dw = torch.empty((D, W), dtype=torch.float32, device=x.device)
    db = torch.empty((D,), dtype=torch.float32, device=x.device)
    want_dh0 = (initial_state is not None) if need_dh0 is None else need_dh0
    dh0 = torch.zeros((N, D, W - 1), dtype=torch.float32, device=x.device) if want_dh0 else None
    a = CausalConv1dBwdArgs()
    a.x, a.weight, a.bias, a.dy, a.y_pre = rt.desc(x), rt.desc(weight), rt.desc(bias), rt.desc(dy), rt.desc(y_pre)
    a.initial_state, a.dht = rt.desc(initial_state), rt.desc(dht)
    a.dx, a.dw, a.db, a.dh0, a.cu_seqlens = rt.desc(dx), rt.desc(dw), rt.desc(db), rt.desc(dh0), rt.desc(cu)
    a.activation_silu = _act(activation)
    rt.call("causal_conv1d_bwd", a, [x, weight, bias, dy, y_pre, initial_state, dht, dx, dw, db, dh0, cu])
    return dx, dw, db, dh0


class CausalConv1dFunction(torch.autograd.Function):
    """Autograd glue of :func:`causal_conv1d` (the reference wires its operator the same way,
    examples/flash_gated_delta_rule.py:323-419): saves the inputs, the backward recomputes the pre-activation."""

    @staticmethod
    def forward(ctx, x, weight, bias, residual, initial_state, output_final_state, activation, cu_seqlens):
        y, final = _causal_conv1d_fwd(x, weight, bias, residual, initial_state, output_final_state, activation, cu_seqlens)
        ctx.save_for_backward(x, weight, bias, initial_state, cu_seqlens)
        ctx.activation, ctx.has_residual = activation, residual is not None
        return y, final

    @staticmethod
    def backward(ctx, dy, dfinal):
        x, weight, bias, initial_state, cu = ctx.saved_tensors
        dht = None if dfinal is None else dfinal.to(x.dtype)
        dx, dw, db, dh0 = causal_conv1d_bwd(x, weight, dy, bias, initial_state, dht, ctx.activation, cu)
        return (dx, dw.to(weight.dtype), None if bias is None else db.to(bias.dtype), dy if ctx.has_residual else None,
                None if dh0 is None else dh0.to(initial_state.dtype), None, None, None)


def causal_conv1d(x, weight=None, bias=None, residual=None, initial_state=None, output_final_state=False,
                  activation=None, cu_seqlens=None):
    """x `[B,T,D]` bf16; weight `[D,W]`; initial_state / final_state `[N,D,W-1]`.
    Returns ``(y [B,T,D], final_state | None)``; differentiable in x, weight, bias, residual and initial_state."""
    if weight is None:
        raise RuntimeError("causal_conv1d: weight is required")
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (x, weight, bias, residual, initial_state)):
        return CausalConv1dFunction.apply(x, weight, bias, residual, initial_state, output_final_state, activation, cu_seqlens)
    return _causal_conv1d_fwd(x, weight, bias, residual, initial_state, output_final_state, activation, cu_seqlens)


def _causal_conv1d_fwd(x, weight=None, bias=None, residual=None, initial_state=None, output_final_state=False,
                       activation=None, cu_seqlens=None, head_num=0):
    """`head_num` > 0: y comes out head-first, `[B, head_num, T, D // head_num]`, written in that layout by the kernel."""
    op = "causal_conv1d"
    if x.dim() != 3:
        raise RuntimeError(f"{op}: x must be [B,T,D], got {tuple(x.shape)}")
    if weight is None:
        raise RuntimeError(f"{op}: weight is required")
    B, T, D = x.shape
    W = weight.shape[1]
    if x.stride(-1) != 1:
        x = x.contiguous()
    cu = None
    N = B
    if cu_seqlens is not None:
        cu = cu_seqlens.to(device=x.device, dtype=torch.int32)
        N = cu.numel() - 1
    head_num = int(head_num)
    if head_num > 0:
        if D % head_num or (D // head_num) % 8:
            raise RuntimeError(f"{op}: head_num={head_num} must divide D={D} into heads of a multiple of 8 channels")
        y = torch.empty((B, head_num, T, D // head_num), dtype=x.dtype, device=x.device)
    else:
        y = torch.empty_like(x)
    final = torch.empty((N, D, W - 1), dtype=x.dtype, device=x.device) if output_final_state else None
    a = CausalConv1dFwdArgs()
    a.x, a.weight, a.bias, a.residual = rt.desc(x), rt.desc(weight), rt.desc(bias), rt.desc(residual)
    a.initial_state, a.y, a.final_state, a.cu_seqlens = rt.desc(initial_state), rt.desc(y), rt.desc(final), rt.desc(cu)
    a.activation_silu = _act(activation)
    rt.call("causal_conv1d_fwd", a, [x, weight, bias, residual, initial_state, y, final, cu])
    return y, final


def causal_conv1d_update(x, cache, residual=None, weight=None, bias=None, activation=None, cache_indices=None,
                         num_accepted_tokens=None, pad_slot_id=-1):
    """Decode step.  x `[N,D]` or `[N,T,D]`; cache `[slots,D,S]` (S >= W-1), updated in place.
    Returns y with the shape of x."""
    op = "causal_conv1d_update"
    if weight is None:
        raise RuntimeError(f"{op}: weight is required")
    rt.reject_requires_grad(op, cache=cache)
    squeeze = x.dim() == 2
    x3 = x.unsqueeze(1) if squeeze else x
    r3 = None if residual is None else (residual.unsqueeze(1) if squeeze else residual)
    y3 = torch.empty_like(x3)
    a = CausalConv1dUpdateArgs()
    a.x, a.weight, a.bias, a.residual = rt.desc(x3), rt.desc(weight), rt.desc(bias), rt.desc(r3)
    a.conv_state, a.y = rt.desc(cache), rt.desc(y3)
    a.cache_indices, a.num_accepted_tokens = rt.desc(cache_indices), rt.desc(num_accepted_tokens)
    a.activation_silu, a.pad_slot_id = _act(activation), int(pad_slot_id)
    rt.call("causal_conv1d_update", a, [x3, weight, bias, r3, cache, y3, cache_indices, num_accepted_tokens])
    rt.mark_mutated(cache)
    return y3.squeeze(1) if squeeze else y3


def npu_causal_conv1d(x, weight, bias=None, conv_states=None, *, query_start_loc=None, cache_indices=None,
                      initial_state_mode=None, num_accepted_tokens=None, activation_mode=0, pad_slot_id=-1,
                      run_mode=0, head_num=0):
    """Reference low-level signature.  x `[B,T,D]` / `[T,D]` (varlen with query_start_loc) for run_mode 0,
    `[N,D]` / `[N,T,D]` for run_mode 1; weight `[W,D]`; conv_states `[slots,S,D]` updated in place.
    `head_num` > 0 (prefill only, …/_aclnn_ctypes.py:939-948): the output is `[B, head_num, T, D // head_num]`."""
    op = "npu_causal_conv1d"
    head_num = int(head_num)
    if head_num and int(run_mode) == 1:
        head_num = 0    # the reference re-lays the output only in prefill mode (_infer_causal_conv1d_y)
    w_dw = weight.transpose(0, 1)                                   # [D,W] view of the [W,D] tensor
    st = None if conv_states is None else conv_states.transpose(1, 2)  # [slots,D,S] view
    dev = x.device

    def as_i32(v):
        if v is None:
            return None
        return v.to(device=dev, dtype=torch.int32) if isinstance(v, torch.Tensor) else torch.tensor(
            list(v), dtype=torch.int32, device=dev)

    if int(run_mode) == 1:
        return causal_conv1d_update(x, st, weight=w_dw, bias=bias, activation=int(activation_mode),
                                    cache_indices=as_i32(cache_indices),
                                    num_accepted_tokens=as_i32(num_accepted_tokens), pad_slot_id=pad_slot_id)
    W = weight.shape[0]
    varlen = x.dim() == 2
    x3 = x.unsqueeze(0) if varlen else x
    cu = as_i32(query_start_loc) if varlen else None
    N = (cu.numel() - 1) if varlen else x3.shape[0]
    init = None
    idx = as_i32(cache_indices)
    if st is not None:
        rt.reject_requires_grad(op, conv_states=conv_states)
        if st.shape[2] != W - 1:
            raise RuntimeError(f"{op}: prefill expects conv_states with state_len == W-1")
        if initial_state_mode is not None:
            sel = st if idx is None else st[idx.long()]
            mode = as_i32(initial_state_mode).bool()
            init = torch.where(mode[:, None, None], sel, torch.zeros_like(sel))
    if head_num:   # prefill output as [B, head_num, T, D / head_num] ([head_num, T, D / head_num] for packed input)
        y, final = _causal_conv1d_fwd(x3, w_dw, bias, None, init, st is not None, int(activation_mode), cu, head_num=head_num)
    else:
        y, final = causal_conv1d(x3, w_dw, bias, None, init, st is not None, int(activation_mode), cu)
    if st is not None:
        if idx is None:
            st[:N].copy_(final)
        else:
            keep = idx != pad_slot_id
            st[idx[keep].long()] = final[keep]
        rt.mark_mutated(conv_states)
    return y.squeeze(0) if varlen else y   # packed input with head_num: [head_num, T, D / head_num]


def npu_causal_conv1d_bwd(x, y, weight, dy, initial_state=None, dht=None, *, query_start_loc=None, activation=0,
                          input_layout="BSND"):
    """Reference low-level signature (…/ops/ascendc/_aclnn_ctypes.py:988-1037): x, dy `[B,T,D]` (or `[T,D]` with
    ``query_start_loc``), y the forward's pre-activation, weight `[W,D]`, initial_state / dht `[B,W,D]` whose rows
    1..W-1 hold the W-1 stored inputs.  Returns ``(dx, dw [W,D], db [D], dh0 [B,W,D])`` in the dtype of x."""
    op = "npu_causal_conv1d_bwd"
    if input_layout not in ("BSND", "NTD", "TND"):
        raise NotImplementedError(f"{op}: input_layout {input_layout!r} is not provided")
    varlen = x.dim() == 2
    if varlen and query_start_loc is None:
        raise RuntimeError(f"{op}: query_start_loc is required for {input_layout} input.")
    W, D = weight.shape
    x3, dy3 = (t.unsqueeze(0) if varlen else t for t in (x, dy))
    y3 = None if y is None else (y.unsqueeze(0) if varlen else y)
    cu = None
    if varlen:
        cu = query_start_loc if isinstance(query_start_loc, torch.Tensor) else torch.tensor(list(query_start_loc))
        cu = cu.to(device=x.device, dtype=torch.int32)
    to_mine = lambda s: None if s is None else s[:, 1:, :].transpose(1, 2)   # noqa: E731  [B,W,D] -> [B,D,W-1] view
    dx, dw, db, dh0 = causal_conv1d_bwd(x3, weight.transpose(0, 1), dy3, None, to_mine(initial_state), to_mine(dht),
                                        int(activation), cu, y_pre=y3 if int(activation) else None, need_dh0=True)
    N = dh0.shape[0]
    dh0_ref = torch.zeros((N, W, D), dtype=x.dtype, device=x.device)
    if initial_state is not None:
        dh0_ref[:, 1:, :] = dh0.transpose(1, 2).to(x.dtype)
    return (dx.squeeze(0) if varlen else dx), dw.transpose(0, 1).to(x.dtype), db.to(x.dtype), dh0_ref

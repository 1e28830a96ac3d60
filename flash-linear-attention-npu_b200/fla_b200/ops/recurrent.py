"""Fused-recurrent gated delta rule (decode).  Two entry points over one CUDA kernel:

* :func:`fused_recurrent_gated_delta_rule` - the `[B,T,H,D]` surface with `initial_state` /
  `final_state` of shape `[N,HV,K,V]` (upstream ``fla.ops`` naming, which the reference targets).
* :func:`recurrent_gated_delta_rule` - the reference's in-place state-pool operator
  (torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:654-846), same argument names.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import _runtime as rt
from ._structs import RecurrentGdnArgs

_OP = "recurrent_gdn"


def _activation_ok(name, t):
    if t.dtype != torch.bfloat16:
        raise TypeError(f"{name} dtype must be torch.bfloat16, got {t.dtype}")


def fused_recurrent_gated_delta_rule(q, k, v, g=None, beta=None, scale=None, initial_state=None,
                                     output_final_state=False, use_qk_l2norm_in_kernel=False, cu_seqlens=None,
                                     transpose_state_layout=False, inplace_final_state=False):
    """q,k `[B,T,HK,K]`, v `[B,T,HV,V]` bf16; g, beta `[B,T,HV]`; initial_state `[N,HV,K,V]` fp32|bf16
    (`[N,HV,V,K]` with ``transpose_state_layout``).  Returns ``(o [B,T,HV,V], final_state | None)``.

    With ``inplace_final_state`` the final state overwrites ``initial_state`` (serving pools) and that
    same tensor is returned.  With ``cu_seqlens`` (int32/int64 `[N+1]`) B must be 1.
    """
    op = "fused_recurrent_gated_delta_rule"
    for n, t in (("q", q), ("k", k), ("v", v)):
        _activation_ok(f"{op}: {n}", t)
    if q.dim() != 4 or q.shape != k.shape or v.dim() != 4:
        raise RuntimeError(f"{op}: q/k must be [B,T,HK,K] and v [B,T,HV,V]")
    B, T, HK, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    if HV % HK:
        raise RuntimeError(f"{op}: HV={HV} must be a multiple of HK={HK}")
    scale = K ** -0.5 if scale is None else float(scale)
    if not math.isfinite(scale):
        raise ValueError(f"{op}: scale must be finite, got {scale}")
    if cu_seqlens is not None:
        if B != 1:
            raise RuntimeError(f"{op}: cu_seqlens requires batch size 1")
        cu = cu_seqlens.to(device=q.device, dtype=torch.int32)
        N = cu.numel() - 1
    else:
        cu, N = None, B
    sshape = (N, HV, V, K) if transpose_state_layout else (N, HV, K, V)
    if initial_state is None:
        state_in = torch.zeros(sshape, dtype=torch.float32, device=q.device)
    else:
        if tuple(initial_state.shape) != sshape:
            raise RuntimeError(f"{op}: initial_state shape must be {sshape}, got {tuple(initial_state.shape)}")
        state_in = initial_state if initial_state.is_contiguous() else initial_state.contiguous()
    if inplace_final_state:
        rt.reject_requires_grad(op, initial_state=initial_state)
        state_out = state_in
    elif output_final_state:
        state_out = torch.empty_like(state_in)
    else:
        state_out = torch.empty_like(state_in)  # the kernel always streams the state back; discard it
    out = torch.empty_like(v)
    q3, k3, v3, o3 = (x.reshape(B * T, x.shape[2], x.shape[3]) for x in (q, k, v, out))
    g2 = None if g is None else g.reshape(B * T, HV)
    b2 = None if beta is None else beta.reshape(B * T, HV)
    a = RecurrentGdnArgs()
    a.q, a.k, a.v, a.g, a.beta = rt.desc(q3), rt.desc(k3), rt.desc(v3), rt.desc(g2), rt.desc(b2)
    a.state_in, a.state_out, a.out = rt.desc(state_in), rt.desc(state_out), rt.desc(o3)
    a.cu_seqlens = rt.desc(cu)
    a.scale, a.tokens_per_seq = scale, T
    a.state_v_first, a.use_qk_l2norm = int(transpose_state_layout), int(use_qk_l2norm_in_kernel)
    rt.call(_OP, a, [q3, k3, v3, g2, b2, state_in, state_out, o3, cu])
    if inplace_final_state and initial_state is not None:
        rt.mark_mutated(state_out)
    return out, (state_out if (output_final_state or inplace_final_state) else None)


def recurrent_gated_delta_rule(query, key, value, state, *, beta, scale=1.0, actual_seq_lengths, ssm_state_indices,
                               num_accepted_tokens=None, g=None, gk=None):
    """Reference operator surface: run recurrent GDN and update ``state`` in place.

    query/key `[T,Nk,Dk]`, value `[T,Nv,Dv]`, beta `[T,Nv]` bf16; g `[T,Nv]` fp32; state
    `[blocks,Nv,Dv,Dk]` bf16|fp32 (V-first); ``actual_seq_lengths`` int32 `[B+1]` whose entry 0 is a
    skipped prefix length and entries 1.. are per-sequence token counts; ``ssm_state_indices`` int32 `[T]`.
    Returns the attention output `[T,Nv,Dv]` (bf16).
    """
    op = "recurrent_gated_delta_rule"
    if g is None and gk is None:
        raise RuntimeError(f"{op}: either g or gk must be provided.")
    if gk is not None:
        raise NotImplementedError(f"{op}: gk (per-channel decay) is not supported by this operator; "
                                  "the reference documents it as not supported yet as well")
    for n, t in (("query", query), ("key", key), ("value", value), ("beta", beta)):
        _activation_ok(f"{op}: {n}", t)
    if state.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError(f"{op}: state dtype must be bfloat16 or float32, got {state.dtype}")
    if actual_seq_lengths.dtype != torch.int32 or ssm_state_indices.dtype != torch.int32:
        raise TypeError(f"{op}: actual_seq_lengths and ssm_state_indices must be int32")
    if query.dim() != 3 or query.shape != key.shape or value.dim() != 3 or state.dim() != 4:
        raise RuntimeError(f"{op}: expected query/key [T,Nk,Dk], value [T,Nv,Dv], state [blocks,Nv,Dv,Dk]")
    T, Nk, Dk = query.shape
    Nv, Dv = value.shape[1], value.shape[2]
    if tuple(state.shape[1:]) != (Nv, Dv, Dk):
        raise RuntimeError(f"{op}: state shape must be (blocks, {Nv}, {Dv}, {Dk}), got {tuple(state.shape)}")
    if Nv % Nk:
        raise RuntimeError(f"{op}: Nv must be an integer multiple of Nk, got Nv={Nv}, Nk={Nk}.")
    if actual_seq_lengths.numel() < 2:
        raise RuntimeError(f"{op}: actual_seq_lengths must contain the prefix entry and at least one sequence length.")
    scale = float(scale)
    if not math.isfinite(scale):
        raise ValueError(f"{op}: scale must be finite, got {scale}.")
    rt.reject_requires_grad(op, state=state)
    cu = torch.cumsum(actual_seq_lengths.to(torch.int32), 0, dtype=torch.int32)   # [prefix, prefix+l1, ...]
    out = torch.empty_like(value)
    a = RecurrentGdnArgs()
    a.q, a.k, a.v, a.g, a.beta = rt.desc(query), rt.desc(key), rt.desc(value), rt.desc(g), rt.desc(beta)
    a.state_in = a.state_out = rt.desc(state)
    a.out = rt.desc(out)
    a.cu_seqlens, a.state_indices = rt.desc(cu), rt.desc(ssm_state_indices)
    a.num_accepted_tokens = rt.desc(num_accepted_tokens)
    a.scale, a.tokens_per_seq, a.state_v_first, a.use_qk_l2norm = scale, 0, 1, 0
    rt.call(_OP, a, [query, key, value, g, beta, state, out, cu, ssm_state_indices, num_accepted_tokens])
    rt.mark_mutated(state)
    return out

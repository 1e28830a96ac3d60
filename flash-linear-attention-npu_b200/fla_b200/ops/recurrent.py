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
    # fp16 activations are read exactly by the decode kernel (fp32 arithmetic on CUDA cores); q, k, v share one dtype
    if t.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"{name} dtype must be torch.bfloat16 or torch.float16, got {t.dtype}")


def _gate_f16_to_f32(t, op):
    """fp16 gate tensors (g, beta, gk) as fp32, through the library's conversion kernel; others unchanged."""
    if t is None or t.dtype != torch.float16:
        return t
    from ._convert import convert
    shape = t.shape
    return convert(t.reshape(-1, shape[-1]), torch.float32, op).view(shape)


def fused_recurrent_gated_delta_rule(q, k, v, g=None, beta=None, scale=None, initial_state=None,
                                     output_final_state=False, use_qk_l2norm_in_kernel=False, cu_seqlens=None,
                                     transpose_state_layout=False, inplace_final_state=False, gk=None):
    """q,k `[B,T,HK,K]`, v `[B,T,HV,V]` bf16; g, beta `[B,T,HV]`; gk `[B,T,HV,K]` (per-key-channel log decay, optional);
    initial_state `[N,HV,K,V]` fp32|bf16 (`[N,HV,V,K]` with ``transpose_state_layout``).
    Returns ``(o [B,T,HV,V], final_state | None)``.

    With ``inplace_final_state`` the final state overwrites ``initial_state`` (serving pools) and that
    same tensor is returned.  With ``cu_seqlens`` (int32/int64 `[N+1]`) B must be 1.
    """
    op = "fused_recurrent_gated_delta_rule"
    for n, t in (("q", q), ("k", k), ("v", v)):
        _activation_ok(f"{op}: {n}", t)
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError(f"{op}: q, k, v must share one dtype, got {q.dtype}, {k.dtype}, {v.dtype}")
    g, beta, gk = (_gate_f16_to_f32(x, op) for x in (g, beta, gk))
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
        if inplace_final_state and not initial_state.is_contiguous():
            # a copy would receive the update and leave the caller's state pool as it was
            raise RuntimeError(f"{op}: inplace_final_state=True needs a contiguous initial_state, got strides {initial_state.stride()}")
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
    gk3 = None
    if gk is not None:
        if tuple(gk.shape) != (B, T, HV, K):
            raise RuntimeError(f"{op}: gk must be {(B, T, HV, K)}, got {tuple(gk.shape)}")
        gk3 = gk.reshape(B * T, HV, K)
    a = RecurrentGdnArgs()
    a.q, a.k, a.v, a.g, a.beta = rt.desc(q3), rt.desc(k3), rt.desc(v3), rt.desc(g2), rt.desc(b2)
    a.state_in, a.state_out, a.out = rt.desc(state_in), rt.desc(state_out), rt.desc(o3)
    a.cu_seqlens, a.gk = rt.desc(cu), rt.desc(gk3)
    a.scale, a.tokens_per_seq = scale, T
    a.state_v_first, a.use_qk_l2norm = int(transpose_state_layout), int(use_qk_l2norm_in_kernel)
    rt.call(_OP, a, [q3, k3, v3, g2, b2, state_in, state_out, o3, cu, gk3])
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
    if not (query.dtype == key.dtype == value.dtype):
        raise TypeError(f"{op}: query, key, value must share one dtype, got {query.dtype}, {key.dtype}, {value.dtype}")
    beta, g = _gate_f16_to_f32(beta, op), _gate_f16_to_f32(g, op)
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


def recurrent_kda(q, k, v, g, beta, initial_state=None, *, cu_seqlens=None, ssm_state_indices=None, A_log=None,
                  dt_bias=None, num_accepted_tokens=None, layout="BSND", scale=None, output_final_state=False,
                  inplace_final_state=True, use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False,
                  use_beta_sigmoid_in_kernel=False, allow_neg_eigval=False, safe_gate=False, lower_bound=None,
                  state_v_first=False):
    """Recurrent KDA step over a state pool, with the reference operator's argument names
    (npu_recurrent_kda, torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:1298-1503).

    BSND: q,k `[B,T,H,K]`, v `[B,T,HV,V]`, g `[B,T,HV,K]`, beta `[B,T,HV]`; TND: the same without the batch dim.
    ``initial_state`` `[state_capacity,HV,K,V]` (`[..,V,K]` with ``state_v_first``) fp32|bf16, updated in place when
    ``inplace_final_state``.  ``ssm_state_indices``: packed `[T]` (state after token t goes to block indices[t]) or
    speculative `[seq_num,max_step]` (token s of sequence n goes to block indices[n,s]); a sequence starts from the
    block of its first token, or of token ``num_accepted_tokens[n] - 1``.  Returns ``(out, final_state | None)``.
    """
    op = "recurrent_kda"
    if layout not in ("BSND", "TND"):
        raise RuntimeError(f"{op}: layout must be BSND or TND.")
    tnd = layout == "TND"
    rank = 3 if tnd else 4
    if any(x.dim() != rank for x in (q, k, v, g)) or beta.dim() != rank - 1:
        raise RuntimeError(f"{op}: layout/rank mismatch. TND expects q/k [T,H,K], v [T,HV,V], g [T,HV,K], beta [T,HV]; "
                           "BSND expects q/k [B,T,H,K], v [B,T,HV,V], g [B,T,HV,K], beta [B,T,HV].")
    if q.shape != k.shape:
        raise RuntimeError(f"{op}: q and k must have identical shape.")
    for n, t in (("q", q), ("k", k), ("v", v)):
        _activation_ok(f"{op}: {n}", t)
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError(f"{op}: q, k, v must share one dtype, got {q.dtype}, {k.dtype}, {v.dtype}")
    g, beta = _gate_f16_to_f32(g, op), _gate_f16_to_f32(beta, op)
    if tnd:
        q, k, v, g, beta = (x.unsqueeze(0) for x in (q, k, v, g, beta))
    B, T, H, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    if tuple(g.shape) != (B, T, HV, K) or tuple(beta.shape) != (B, T, HV) or tuple(v.shape[:2]) != (B, T):
        raise RuntimeError(f"{op}: v/g/beta shape mismatch.")
    if HV % H:
        raise RuntimeError(f"{op}: HV must be divisible by H.")
    if g.dtype not in (torch.bfloat16, torch.float32) or beta.dtype not in (torch.bfloat16, torch.float32):
        raise RuntimeError(f"{op}: g and beta must use BF16 or FP32.")
    dev = q.device
    total = B * T
    if cu_seqlens is None:
        seq_num = B
        cu = None if not tnd else torch.tensor([0, T], dtype=torch.int32, device=dev)
    else:
        if not isinstance(cu_seqlens, torch.Tensor) or cu_seqlens.dim() != 1 or cu_seqlens.numel() < 2:
            raise RuntimeError(f"{op}: cu_seqlens must be a 1D INT32 or INT64 tensor.")
        cu = cu_seqlens.to(device=dev, dtype=torch.int32)
        seq_num = cu.numel() - 1
    tail = (HV, V, K) if state_v_first else (HV, K, V)
    if initial_state is None:
        if inplace_final_state:
            raise RuntimeError(f"{op}: inplace_final_state=True requires initial_state.")
        state_in = torch.zeros((seq_num, *tail), dtype=torch.float32, device=dev)
    else:
        if initial_state.dtype not in (torch.float32, torch.bfloat16):
            raise RuntimeError(f"{op}: initial_state must use FP32 or BF16.")
        if initial_state.dim() != 4 or tuple(initial_state.shape[1:]) != tail:
            raise RuntimeError(f"{op}: initial_state must be [state_capacity,{','.join(map(str, tail))}].")
        state_in = initial_state if initial_state.is_contiguous() else initial_state.contiguous()
    idx = None
    if ssm_state_indices is not None:
        if ssm_state_indices.dim() == 1 and ssm_state_indices.shape[0] >= total:
            idx = ssm_state_indices[:total].to(device=dev, dtype=torch.int32).contiguous()
        elif ssm_state_indices.dim() == 2 and ssm_state_indices.shape[0] == seq_num and ssm_state_indices.shape[1] > 0:
            # speculative [seq_num, max_step]: token s of sequence n -> indices[n, s]
            bounds = cu if cu is not None else torch.arange(0, total + 1, T, dtype=torch.int32, device=dev)
            tok = torch.arange(total, device=dev)
            seq_of = torch.bucketize(tok, bounds[1:].long(), right=True).clamp_(max=seq_num - 1)
            step = (tok - bounds[:-1].long()[seq_of]).clamp_(0, ssm_state_indices.shape[1] - 1)
            idx = ssm_state_indices.to(dev)[seq_of, step].to(torch.int32).contiguous()
        else:
            raise RuntimeError(f"{op}: ssm_state_indices must be INT32/INT64 packed [T] or speculative [seq_num,max_step].")
    elif state_in.shape[0] != seq_num:
        raise RuntimeError(f"{op}: without ssm_state_indices, state_capacity must equal seq_num.")
    if num_accepted_tokens is not None:
        if idx is None:
            raise RuntimeError(f"{op}: num_accepted_tokens requires ssm_state_indices.")
        if tuple(num_accepted_tokens.shape) != (seq_num,):
            raise RuntimeError(f"{op}: num_accepted_tokens must be INT32/INT64 [seq_num].")
        num_accepted_tokens = num_accepted_tokens.to(device=dev, dtype=torch.int32)
    gate_mode = 0
    lower = -5.0 if lower_bound is None else float(lower_bound)
    if use_gate_in_kernel:
        if A_log is None or A_log.dtype != torch.float32 or tuple(A_log.shape) != (HV,):
            raise RuntimeError(f"{op}: A_log must be FP32 [HV] when use_gate_in_kernel=True.")
        if safe_gate and not -5.0 <= lower < 0.0:
            raise RuntimeError(f"{op}: lower_bound must be in [-5,0) when safe_gate=True.")
        if dt_bias is not None:
            if dt_bias.dtype != torch.float32 or tuple(dt_bias.shape) not in ((HV * K,), (HV, K)):
                raise RuntimeError(f"{op}: dt_bias must be FP32 [HV*K] or [HV,K].")
            dt_bias = dt_bias.reshape(HV, K).contiguous()
        gate_mode = 2 if safe_gate else 1
    elif safe_gate or A_log is not None or dt_bias is not None:
        raise RuntimeError(f"{op}: A_log, dt_bias and safe_gate require use_gate_in_kernel=True.")
    scale = K ** -0.5 if scale is None else float(scale)
    if inplace_final_state:
        rt.reject_requires_grad(op, initial_state=initial_state)
        state_out = state_in
    else:
        state_out = torch.empty_like(state_in)
    out = torch.empty_like(v)
    q3, k3, v3, o3 = (x.reshape(total, x.shape[2], x.shape[3]) for x in (q, k, v, out))
    gk3, b2 = g.reshape(total, HV, K), beta.reshape(total, HV)
    a = RecurrentGdnArgs()
    a.q, a.k, a.v, a.beta, a.gk = rt.desc(q3), rt.desc(k3), rt.desc(v3), rt.desc(b2), rt.desc(gk3)
    a.a_log, a.dt_bias = rt.desc(A_log if gate_mode else None), rt.desc(dt_bias if gate_mode else None)
    a.state_in, a.state_out, a.out = rt.desc(state_in), rt.desc(state_out), rt.desc(o3)
    a.cu_seqlens, a.state_indices, a.num_accepted_tokens = rt.desc(cu), rt.desc(idx), rt.desc(num_accepted_tokens)
    a.scale, a.lower_bound, a.tokens_per_seq = scale, lower, T
    a.state_v_first, a.use_qk_l2norm, a.gate_mode = int(state_v_first), int(use_qk_l2norm_in_kernel), gate_mode
    a.beta_mode = (2 if allow_neg_eigval else 1) if use_beta_sigmoid_in_kernel else 0
    rt.call(_OP, a, [q3, k3, v3, b2, gk3, A_log if gate_mode else None, dt_bias if gate_mode else None, state_in, state_out,
                     o3, cu, idx, num_accepted_tokens])
    if inplace_final_state and initial_state is not None:
        rt.mark_mutated(state_out)
    if tnd:
        out = out.squeeze(0)
    return out, (state_out if output_final_state else None)

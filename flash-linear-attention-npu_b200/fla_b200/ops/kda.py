"""Chunked Kimi Delta Attention (KDA) - `[B,T,H,D]` operator surface.

`chunk_kda` keeps the argument names of the reference's forward contract (npu_chunk_kda_fwd,
torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:1066-1265, BSND layout): q,k `[B,T,HK,K]`,
v `[B,T,HV,V]`, per-channel gate g `[B,T,HV,K]`, beta `[B,T,HV]`, optional in-kernel gate activation
(`use_gate_in_kernel` with `A_log`, `dt_bias`, `safe_gate` / `lower_bound`), `initial_state` / final state
`[N,HV,K,V]` fp32.  Forward only: the reference itself ships no KDA backward (it defers to a third-party
package), and this build has none yet, so tensors that require grad are refused instead of silently
producing a graph-less result.
"""
from __future__ import annotations

import torch

from .. import _runtime as rt
from ._structs import KdaChunkFwdArgs
from .gdn import CHUNK, _as_rows, _varlen_meta


def chunk_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
              use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False, use_beta_sigmoid_in_kernel=False,
              cu_seqlens=None, safe_gate=False, lower_bound=None, A_log=None, dt_bias=None,
              return_gate_cumsum=False, output_dtype=None):
    """Returns ``(o [B,T,HV,V], final_state [N,HV,K,V] | None)`` (plus the cumulative gate `[B,T,HV,K]` fp32
    when ``return_gate_cumsum``)."""
    op = "chunk_kda"
    if use_qk_l2norm_in_kernel or use_beta_sigmoid_in_kernel:
        raise NotImplementedError(f"{op}: in-kernel q/k L2 norm and beta sigmoid are not available yet")
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (q, k, v, g, beta, initial_state)):
        raise NotImplementedError(f"{op}: backward is not implemented; call under torch.no_grad() or detach the inputs")
    for name, t in (("q", q), ("k", k), ("v", v)):
        if t.dtype != torch.bfloat16:
            raise TypeError(f"{op}: {name} must be bfloat16, got {t.dtype}")
    if q.dim() != 4 or q.shape != k.shape or v.dim() != 4 or v.shape[:2] != q.shape[:2]:
        raise RuntimeError(f"{op}: expected q,k [B,T,HK,K] and v [B,T,HV,V]")
    B, T, HK, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    if K != 128 or V != 128:
        raise RuntimeError(f"{op}: this build supports K = V = 128, got K={K}, V={V}")
    if HV % HK:
        raise RuntimeError(f"{op}: HV={HV} must be a multiple of HK={HK}")
    if tuple(g.shape) != (B, T, HV, K) or tuple(beta.shape) != (B, T, HV):
        raise RuntimeError(f"{op}: g must be {(B, T, HV, K)} and beta {(B, T, HV)}")
    scale = K ** -0.5 if scale is None else float(scale)
    gate_mode = 0
    if use_gate_in_kernel:
        if A_log is None:
            raise RuntimeError(f"{op}: use_gate_in_kernel needs A_log")
        gate_mode = 2 if safe_gate else 1
        if safe_gate and lower_bound is None:
            raise RuntimeError(f"{op}: safe_gate needs lower_bound")
        A_log = A_log.float().contiguous()
        dt_bias = None if dt_bias is None else dt_bias.float().reshape(HV, K).contiguous()
    q, k, v, g, beta = (_as_rows(x) for x in (q, k, v, g, beta))
    dev = q.device
    cu = co = None
    N, max_len, total_chunks = B, T, B * ((T + CHUNK - 1) // CHUNK)
    if cu_seqlens is not None:
        if B != 1:
            raise RuntimeError(f"{op}: cu_seqlens requires batch size 1 (packed sequences)")
        cu, co, max_len, total_chunks, N, total = _varlen_meta(cu_seqlens, dev)
        if total != T:
            raise RuntimeError(f"{op}: cu_seqlens[-1]={total} must equal T={T}")
    if initial_state is not None:
        if tuple(initial_state.shape) != (N, HV, K, V):
            raise RuntimeError(f"{op}: initial_state must be {(N, HV, K, V)}, got {tuple(initial_state.shape)}")
        initial_state = initial_state.float().contiguous()
    o = torch.empty((B, T, HV, V), dtype=output_dtype or q.dtype, device=dev)
    ht = torch.empty((N, HV, K, V), dtype=torch.float32, device=dev) if output_final_state else None
    gk = torch.empty((B, T, HV, K), dtype=torch.float32, device=dev) if return_gate_cumsum else None
    a = KdaChunkFwdArgs()
    a.q, a.k, a.v, a.g, a.beta = rt.desc(q), rt.desc(k), rt.desc(v), rt.desc(g), rt.desc(beta)
    a.a_log, a.dt_bias = rt.desc(A_log if gate_mode else None), rt.desc(dt_bias if gate_mode else None)
    a.initial_state, a.o, a.final_state, a.gk = rt.desc(initial_state), rt.desc(o), rt.desc(ht), rt.desc(gk)
    a.cu_seqlens, a.chunk_offsets = rt.desc(cu), rt.desc(co)
    a.scale, a.lower_bound, a.gate_mode = scale, float(lower_bound or 0.0), gate_mode
    a.chunk_size, a.max_seqlen, a.total_chunks = CHUNK, int(max_len), int(total_chunks)
    rt.call("kda_chunk_fwd", a, [q, k, v, g, beta, initial_state, o, ht, gk, cu, co])
    if return_gate_cumsum:
        return o, ht, gk
    return o, ht

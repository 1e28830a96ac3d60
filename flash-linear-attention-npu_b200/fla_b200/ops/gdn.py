"""Chunked gated delta rule (GDN) - the `[B,T,H,D]` operator surface.

`chunk_gated_delta_rule` keeps the argument names and semantics of the reference's composed entry
`flash_gated_delta_rule` (examples/flash_gated_delta_rule.py:1126-1228): q,k `[B,T,HK,K]`,
v `[B,T,HV,V]`, g (log decay) and beta `[B,T,HV]`, `scale` defaulting to K^-0.5, `initial_state`
`[N,HV,K,V]`, `output_final_state`, optional in-kernel q/k L2 normalisation, packed variable-length
batches through `cu_seqlens`, and GVA (value head hv reads q/k head hv // (HV/HK)) without
materialising repeated q/k.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _runtime as rt
from ._structs import GdnChunkFwdArgs

CHUNK = 64


def _varlen_meta(cu_seqlens, device):
    """Host-side chunk bookkeeping for packed batches (the reference prepares the same
    (sequence, chunk) metadata on the host, examples/flash_gated_delta_rule.py:78-100)."""
    cu_host = [int(x) for x in (cu_seqlens.tolist() if isinstance(cu_seqlens, torch.Tensor) else cu_seqlens)]
    if len(cu_host) < 2 or cu_host[0] != 0 or any(b < a for a, b in zip(cu_host, cu_host[1:])):
        raise RuntimeError(f"cu_seqlens must start at 0 and be non-decreasing, got {cu_host}")
    lens = [b - a for a, b in zip(cu_host, cu_host[1:])]
    offs = [0]
    for L in lens:
        offs.append(offs[-1] + (L + CHUNK - 1) // CHUNK)
    cu = torch.tensor(cu_host, dtype=torch.int32, device=device)
    co = torch.tensor(offs, dtype=torch.int32, device=device)
    return cu, co, max(lens), offs[-1], len(lens), cu_host[-1]


def _as_rows(t):
    """The kernels address tokens by a flat row index: batch rows must sit back to back."""
    if t.stride(-1) != 1 or (t.shape[0] > 1 and t.stride(0) != t.shape[1] * t.stride(1)):
        return t.contiguous()
    return t


def gdn_chunk_fwd(q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens=None, save_for_backward=False,
                  output_dtype=None):
    """Launch the forward kernels.  Returns (o, final_state, saved) where saved holds gam, X and, when
    `save_for_backward`, the split per-chunk states and v_new that the backward kernels consume."""
    op = "chunk_gated_delta_rule"
    for name, t in (("q", q), ("k", k), ("v", v)):
        if t.dtype != torch.bfloat16:
            raise TypeError(f"{op}: {name} must be bfloat16 (fp32 inputs are rejected like in the reference), got {t.dtype}")
    if q.dim() != 4 or q.shape != k.shape or v.dim() != 4 or v.shape[:2] != q.shape[:2]:
        raise RuntimeError(f"{op}: expected q,k [B,T,HK,K] and v [B,T,HV,V], got {tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    B, T, HK, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    if K != 128 or V != 128:
        raise RuntimeError(f"{op}: this build supports K = V = 128, got K={K}, V={V}")
    if HV % HK:
        raise RuntimeError(f"{op}: HV={HV} must be a multiple of HK={HK}")
    if tuple(g.shape) != (B, T, HV) or tuple(beta.shape) != (B, T, HV):
        raise RuntimeError(f"{op}: g and beta must be [B,T,HV]={(B, T, HV)}, got {tuple(g.shape)}, {tuple(beta.shape)}")
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
    gam = torch.empty((B, T, HV), dtype=torch.float32, device=dev)
    x_inv = torch.empty((B, T, HV, CHUNK), dtype=torch.bfloat16, device=dev)
    s_hi = s_lo = vn_hi = vn_lo = None
    if save_for_backward:
        s_hi = torch.empty((total_chunks, HV, K, V), dtype=torch.bfloat16, device=dev)
        s_lo = torch.empty_like(s_hi)
        vn_hi = torch.empty((B, T, HV, V), dtype=torch.bfloat16, device=dev)
        vn_lo = torch.empty_like(vn_hi)
    a = GdnChunkFwdArgs()
    a.q, a.k, a.v, a.g, a.beta = rt.desc(q), rt.desc(k), rt.desc(v), rt.desc(g), rt.desc(beta)
    a.initial_state, a.o, a.final_state = rt.desc(initial_state), rt.desc(o), rt.desc(ht)
    a.gam, a.x_inv = rt.desc(gam), rt.desc(x_inv)
    a.s_hi, a.s_lo, a.vn_hi, a.vn_lo = rt.desc(s_hi), rt.desc(s_lo), rt.desc(vn_hi), rt.desc(vn_lo)
    a.cu_seqlens, a.chunk_offsets = rt.desc(cu), rt.desc(co)
    a.scale, a.chunk_size, a.max_seqlen, a.total_chunks = float(scale), CHUNK, int(max_len), int(total_chunks)
    rt.call("gdn_chunk_fwd", a, [q, k, v, g, beta, initial_state, o, ht, gam, x_inv, s_hi, s_lo, vn_hi, vn_lo, cu, co])
    saved = dict(gam=gam, x_inv=x_inv, s_hi=s_hi, s_lo=s_lo, vn_hi=vn_hi, vn_lo=vn_lo, cu=cu, co=co,
                 max_len=max_len, total_chunks=total_chunks, N=N)
    return o, ht, saved


def chunk_gated_delta_rule(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                           use_qk_l2norm_in_kernel=False, cu_seqlens=None, chunk_size=64, head_first=False,
                           output_dtype=None):
    """Returns ``(o [B,T,HV,V], final_state [N,HV,K,V] | None)``."""
    op = "chunk_gated_delta_rule"
    if head_first:
        raise NotImplementedError(f"{op}: head_first layouts are not provided; pass [B,T,H,D] tensors")
    if chunk_size != CHUNK:
        raise NotImplementedError(f"{op}: chunk_size must be {CHUNK}")
    if use_qk_l2norm_in_kernel:
        raise NotImplementedError(f"{op}: use_qk_l2norm_in_kernel is not available yet")
    scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
    o, ht, _ = gdn_chunk_fwd(q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens,
                             save_for_backward=False, output_dtype=output_dtype)
    return o, ht

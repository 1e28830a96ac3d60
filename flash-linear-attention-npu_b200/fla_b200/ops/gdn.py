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
from ._structs import GdnChunkBwdArgs, GdnChunkFwdArgs

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


def _fold_batch(t):
    """A `[B,T,H,D]` view of head-first memory (`[B,H,T,D]` storage: batch stride = H x head stride) seen as one sequence of
    B*H heads, `[1,T,B*H,D]`, on the same storage.  Every (batch row, head) pair is an independent recurrence, so the kernels
    run head-first batches through this view without a copy.  None when the strides do not allow it."""
    B, T, H, D = t.shape
    if t.stride(3) != 1 or t.stride(0) != H * t.stride(2):
        return None
    return t.as_strided((1, T, B * H, D), (B * t.stride(0), t.stride(1), t.stride(2), 1))


def _fold_plan(q, k, v, cu_seqlens):
    """Whether a fixed-length batch whose rows do not sit back to back (head-first storage) can run as one sequence of
    B*H heads instead of being copied: returns the folded (q, k, v) views or None."""
    if cu_seqlens is not None or q.shape[0] == 1 or all(_as_rows(t) is t for t in (q, k, v)):
        return None
    folded = tuple(_fold_batch(t) for t in (q, k, v))
    return None if any(f is None for f in folded) else folded


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
    if K != 128 or V not in (128, 256):
        raise RuntimeError(f"{op}: this build supports K = 128 and V = 128 or 256, got K={K}, V={V}")
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
    x_inv = torch.empty(total_chunks * HV * 8192, dtype=torch.bfloat16, device=dev)   # (I + A)^-1 per chunk: value + residual strips
    s_img = vn_img = p_img = None
    if save_for_backward:
        s_img = torch.empty(total_chunks * HV * (V // 64) * 16384, dtype=torch.bfloat16, device=dev)
        vn_img = torch.empty(total_chunks * HV * (V // 64) * 8192, dtype=torch.bfloat16, device=dev)
        p_img = torch.empty(total_chunks * HV * 8768, dtype=torch.bfloat16, device=dev)   # P tile (16 KB) + the chunk's factor record
    a = GdnChunkFwdArgs()
    a.q, a.k, a.v, a.g, a.beta = rt.desc(q), rt.desc(k), rt.desc(v), rt.desc(g), rt.desc(beta)
    a.initial_state, a.o, a.final_state = rt.desc(initial_state), rt.desc(o), rt.desc(ht)
    a.gam, a.x_inv = rt.desc(gam), rt.desc(x_inv)
    a.s_img, a.vn_img, a.p_img = rt.desc(s_img), rt.desc(vn_img), rt.desc(p_img)
    a.cu_seqlens, a.chunk_offsets = rt.desc(cu), rt.desc(co)
    a.scale, a.chunk_size, a.max_seqlen, a.total_chunks = float(scale), CHUNK, int(max_len), int(total_chunks)
    rt.call("gdn_chunk_fwd", a, [q, k, v, g, beta, initial_state, o, ht, gam, x_inv, s_img, vn_img, p_img, cu, co])
    saved = dict(gam=gam, x_inv=x_inv, s_img=s_img, vn_img=vn_img, p_img=p_img, cu=cu, co=co,
                 max_len=max_len, total_chunks=total_chunks, N=N)
    return o, ht, saved


def gdn_chunk_bwd(q, k, v, beta, saved, do, dht, scale, want_dh0, grad_dtype=None):
    """Launch the backward kernels on the tensors the forward saved.
    Returns (dq, dk, dv, dg, dbeta, dh0 | None); gradients are bf16 unless `grad_dtype` says fp32."""
    op = "chunk_gated_delta_rule_bwd"
    B, T, HK, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    dev = q.device
    if do.dtype != torch.bfloat16:
        from ._convert import convert
        do = convert(do, torch.bfloat16, op)
    do = _as_rows(do)
    if tuple(do.shape) != (B, T, HV, V):
        raise RuntimeError(f"{op}: do must be {(B, T, HV, V)}, got {tuple(do.shape)}")
    if saved["s_img"] is None:
        raise RuntimeError(f"{op}: the forward was not run with save_for_backward=True")
    N = saved["N"]
    if dht is not None:
        if tuple(dht.shape) != (N, HV, K, V):
            raise RuntimeError(f"{op}: dht must be {(N, HV, K, V)}, got {tuple(dht.shape)}")
        dht = dht.float().contiguous()
    gdt = grad_dtype or torch.bfloat16
    dq = torch.empty((B, T, HK, K), dtype=gdt, device=dev)
    dk = torch.empty_like(dq)
    dv = torch.empty((B, T, HV, V), dtype=gdt, device=dev)
    dg = torch.empty((B, T, HV), dtype=gdt, device=dev)
    dbeta = torch.empty_like(dg)
    dh0 = torch.empty((N, HV, K, V), dtype=torch.float32, device=dev) if want_dh0 else None
    a = GdnChunkBwdArgs()
    a.q, a.k, a.v, a.beta = rt.desc(q), rt.desc(k), rt.desc(v), rt.desc(beta)
    a.gam, a.x_inv, a.s_img, a.vn_img, a.p_img = (rt.desc(saved[n]) for n in ("gam", "x_inv", "s_img", "vn_img", "p_img"))
    a.d_o, a.dht = rt.desc(do), rt.desc(dht)
    a.dq, a.dk, a.dv, a.dg, a.dbeta, a.dh0 = (rt.desc(x) for x in (dq, dk, dv, dg, dbeta, dh0))
    a.cu_seqlens, a.chunk_offsets = rt.desc(saved["cu"]), rt.desc(saved["co"])
    a.scale, a.chunk_size = float(scale), CHUNK
    a.max_seqlen, a.total_chunks = int(saved["max_len"]), int(saved["total_chunks"])
    rt.call("gdn_chunk_bwd", a, [q, k, v, beta, saved["gam"], saved["x_inv"], saved["s_img"], saved["vn_img"], saved["p_img"], do, dht,
                                 dq, dk, dv, dg, dbeta, dh0, saved["cu"], saved["co"]])
    return dq, dk, dv, dg, dbeta, dh0


class ChunkGatedDeltaRuleFunction(torch.autograd.Function):
    """Autograd binding (the reference's ChunkGatedDeltaRuleFunction, examples/flash_gated_delta_rule.py:1026-1122).
    Saves q, k, v, beta, gam, X and the split per-chunk states / v_new instead of recomputing them."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens, output_dtype, qk_l2norm):
        need_grad = any(t is not None and t.requires_grad for t in (q, k, v, g, beta, initial_state))
        B, T, HK, HV = q.shape[0], q.shape[1], q.shape[2], v.shape[2]
        h0 = None if initial_state is None else initial_state.detach()
        folded = _fold_plan(q.detach(), k.detach(), v.detach(), cu_seqlens)
        ctx.fold = (B, HK, HV) if folded is not None else None
        if folded is not None:   # head-first storage: B*H heads of one sequence, gates re-laid to match (they are small)
            q_, k_, v_ = folded
            g_, b_ = (x.detach().permute(1, 0, 2).reshape(1, T, B * HV) for x in (g, beta))
            h0 = None if h0 is None else h0.reshape(1, B * HV, *h0.shape[2:])
        else:
            q_, k_, v_, g_, b_ = (_as_rows(x.detach()) for x in (q, k, v, g, beta))
        ctx.qk_l2norm = qk_l2norm
        if qk_l2norm:
            # q, k <- x * rsqrt(sum x^2 + 1e-6), stored in the input dtype like the reference's l2norm_fwd
            # (examples/flash_gated_delta_rule.py:1046-1050); rstd is kept for the backward
            from .l2norm import l2norm_fwd
            q_, q_rstd = l2norm_fwd(q_)
            k_, k_rstd = l2norm_fwd(k_)
        o, ht, saved = gdn_chunk_fwd(q_, k_, v_, g_, b_, scale, h0, output_final_state, cu_seqlens, save_for_backward=need_grad,
                                     output_dtype=output_dtype)
        if folded is not None:
            o = o.view(T, B, HV, o.shape[-1]).permute(1, 0, 2, 3)
            ht = None if ht is None else ht.view(B, HV, *ht.shape[2:])
        if need_grad:
            extra = (q_rstd, k_rstd) if qk_l2norm else ()
            ctx.save_for_backward(q_, k_, v_, b_, saved["gam"], saved["x_inv"], saved["s_img"], saved["vn_img"],
                                  saved["p_img"], *extra)
            ctx.meta = {kk: saved[kk] for kk in ("cu", "co", "max_len", "total_chunks", "N")}
            ctx.scale = scale
            ctx.has_h0 = initial_state is not None
            ctx.in_dtypes = (q.dtype, k.dtype, v.dtype, g.dtype, beta.dtype)
        return o, ht

    @staticmethod
    def backward(ctx, do, dht):
        q, k, v, beta, gam, x_inv, s_img, vn_img, p_img = ctx.saved_tensors[:9]
        saved = dict(ctx.meta, gam=gam, x_inv=x_inv, s_img=s_img, vn_img=vn_img, p_img=p_img)
        if ctx.fold is not None:
            B, HK, HV = ctx.fold
            T = do.shape[1]
            do = do.permute(1, 0, 2, 3).reshape(1, T, B * HV, do.shape[-1])   # a view when do has the strides of o
            dht = None if dht is None else dht.reshape(1, B * HV, *dht.shape[2:])
        dq, dk, dv, dg, dbeta, dh0 = gdn_chunk_bwd(q, k, v, beta, saved, do, dht, ctx.scale, ctx.has_h0,
                                                   grad_dtype=torch.float32 if (ctx.in_dtypes[3] == torch.float32 or ctx.qk_l2norm) else None)
        if ctx.qk_l2norm:
            from .l2norm import l2norm_bwd
            q_rstd, k_rstd = ctx.saved_tensors[9:11]
            dq = l2norm_bwd(q, q_rstd, dq)
            dk = l2norm_bwd(k, k_rstd, dk)
        if ctx.fold is not None:
            dq, dk = (x.view(T, B, HK, x.shape[-1]).permute(1, 0, 2, 3) for x in (dq, dk))
            dv = dv.view(T, B, HV, dv.shape[-1]).permute(1, 0, 2, 3)
            dg, dbeta = (x.view(T, B, HV).permute(1, 0, 2) for x in (dg, dbeta))
            dh0 = None if dh0 is None else dh0.view(B, HV, *dh0.shape[2:])
        dts = ctx.in_dtypes
        return (dq.to(dts[0]), dk.to(dts[1]), dv.to(dts[2]), dg.to(dts[3]), dbeta.to(dts[4]), None, dh0, None, None, None,
                None)


def chunk_gated_delta_rule_fwd_bwd(q, k, v, g, beta, do, scale=None, initial_state=None, dht=None, cu_seqlens=None,
                                   output_dtype=None, grad_dtype=None):
    """Forward and backward in one call without the autograd graph (what a training step costs).
    Returns (o, final_state, (dq, dk, dv, dg, dbeta, dh0))."""
    scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
    q, k, v, g, beta = (_as_rows(x) for x in (q, k, v, g, beta))
    o, ht, saved = gdn_chunk_fwd(q, k, v, g, beta, scale, initial_state, True, cu_seqlens, save_for_backward=True,
                                 output_dtype=output_dtype)
    grads = gdn_chunk_bwd(q, k, v, beta, saved, do, dht, scale, initial_state is not None, grad_dtype=grad_dtype)
    return o, ht, grads


chunk_gated_delta_rule_bwd = gdn_chunk_bwd


def chunk_gated_delta_rule(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                           use_qk_l2norm_in_kernel=False, cu_seqlens=None, chunk_size=64, head_first=False,
                           output_dtype=None):
    """Returns ``(o [B,T,HV,V], final_state [N,HV,K,V] | None)``; differentiable w.r.t. q, k, v, g, beta, initial_state."""
    op = "chunk_gated_delta_rule"
    if head_first:   # [B,H,T,D] tokens and [B,H,T] gates: the same operator on transposed views, output back in [B,H,T,V]
        o, ht = chunk_gated_delta_rule(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), g.transpose(1, 2), beta.transpose(1, 2),
                                       scale=scale, initial_state=initial_state, output_final_state=output_final_state,
                                       use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel, cu_seqlens=cu_seqlens, chunk_size=chunk_size,
                                       output_dtype=output_dtype)
        return o.transpose(1, 2), ht
    # chunk_size is the reference's blocking parameter: o, the final state and every gradient are the same function of
    # the inputs for any blocking, so the fused kernels keep their own 64-token tiling for the sizes the reference tiles for
    if int(chunk_size) not in (16, 32, 64, 128):
        raise NotImplementedError(f"{op}: chunk_size must be one of 16, 32, 64, 128, got {chunk_size}")
    scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
    if torch.float16 in (q.dtype, k.dtype, v.dtype):
        # fp16 tensors (the reference takes them, examples/flash_gated_delta_rule.py:1161-1162): the tensor-core products
        # run on bf16 operands, so q, k, v are rounded to bf16 by the library's conversion kernel, fp16 gates become fp32,
        # o is computed in fp32 and converted to fp16 once; the gradients come back through the same conversions
        if not (q.dtype == k.dtype == v.dtype):
            raise TypeError(f"{op}: q, k, v must share one dtype, got {q.dtype}, {k.dtype}, {v.dtype}")
        from ._convert import to_dtype
        q, k, v = (to_dtype(x, torch.bfloat16, op) for x in (q, k, v))
        g, beta = (to_dtype(x, torch.float32, op) if x.dtype == torch.float16 else x for x in (g, beta))
        o, ht = ChunkGatedDeltaRuleFunction.apply(q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens,
                                                  torch.float32, bool(use_qk_l2norm_in_kernel))
        return to_dtype(o, output_dtype or torch.float16, op), ht
    return ChunkGatedDeltaRuleFunction.apply(q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens,
                                             output_dtype, bool(use_qk_l2norm_in_kernel))


def flash_gated_delta_rule(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                           use_qk_l2norm_in_kernel=False, cu_seqlens=None, cu_seqlens_list=None, chunk_indices=None,
                           chunk_indices_list=None, chunk_size=64, head_first=False):
    """The reference's composed entry with its own layout and checks (examples/flash_gated_delta_rule.py:1126-1228):
    q, k `[B,H,T,K]`, v `[B,H,T,V]` (head-first), g, beta `[B,T,H]`; returns (o `[B,T,H,V]`, final_state `[N,H,K,V]` or None).
    The host-side chunk metadata arguments (`cu_seqlens_list`, `chunk_indices`, `chunk_indices_list`) are accepted and not
    needed: the chunk geometry follows from `cu_seqlens`.  GVA callers pass q, k with fewer heads than v."""
    del cu_seqlens_list, chunk_indices, chunk_indices_list
    if q.dtype != k.dtype or k.dtype != v.dtype:
        raise ValueError(f"q current type is {q.dtype}, k current type is {k.dtype}, v current type is {v.dtype}; they should be equal")
    if q.dtype == torch.float32:
        raise ValueError("ChunkGatedDeltaRuleFunction does not support float32. Please use float16/bfloat16.")
    if beta.ndim != 3 or g.ndim != 3:
        raise ValueError("g and beta must be rank-3 tensors with shape [B, T, H].")
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
        raise ValueError("q, k and v must be rank-4 tensors with shape [B, H, T, D].")
    if q.shape[:3] != k.shape[:3] or q.shape[0] != v.shape[0] or q.shape[2] != v.shape[2]:
        raise ValueError(f"q/k/v shape prefixes must match, got {q.shape}, {k.shape}, {v.shape}.")
    if g.shape != beta.shape:
        raise ValueError(f"g and beta shapes must match, got {g.shape} and {beta.shape}.")
    if g.shape[0] != v.shape[0] or g.shape[1] != v.shape[2] or g.shape[2] != v.shape[1]:
        raise ValueError(f"Expected q/k/v in [B, H, T, D] and g/beta in [B, T, H]; got q={tuple(q.shape)}, g={tuple(g.shape)}.")
    if head_first:
        import warnings
        warnings.warn("head_first is kept only for API compatibility. This entry always expects q/k/v as [B, H, T, D].", stacklevel=2)
    if chunk_size != 2 ** (int(chunk_size).bit_length() - 1):
        raise ValueError(f"chunk_size must be a power of 2, got {chunk_size}.")
    if cu_seqlens is not None and q.shape[0] != 1:
        raise ValueError(f"The batch size is expected to be 1 rather than {q.shape[0]} when using cu_seqlens. "
                         "Please flatten variable-length inputs before processing.")
    if cu_seqlens is not None and initial_state is not None and initial_state.shape[0] != len(cu_seqlens) - 1:
        raise ValueError("The number of initial states is expected to match the number of input sequences, "
                         f"got initial_state.shape[0]={initial_state.shape[0]} and sequences={len(cu_seqlens) - 1}.")
    return chunk_gated_delta_rule(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), g, beta, scale=scale,
                                  initial_state=initial_state, output_final_state=output_final_state,
                                  use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel, cu_seqlens=cu_seqlens, chunk_size=chunk_size)

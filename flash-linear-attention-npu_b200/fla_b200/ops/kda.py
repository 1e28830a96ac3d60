"""Chunked Kimi Delta Attention (KDA) - `[B,T,H,D]` operator surface.

`chunk_kda` keeps the argument names of the reference's forward contract (npu_chunk_kda_fwd,
torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:1066-1265, BSND layout): q,k `[B,T,HK,K]`,
v `[B,T,HV,V]`, per-channel gate g `[B,T,HV,K]`, beta `[B,T,HV]`, optional in-kernel gate activation
(`use_gate_in_kernel` with `A_log`, `dt_bias`, `safe_gate` / `lower_bound`), `initial_state` / final state
`[N,HV,K,V]` fp32.  The operator is differentiable in q, k, v, g, beta and initial_state: the reference ships
only the intra-chunk piece of the KDA backward (npu_chunk_kda_bwd_intra, `_aclnn_ctypes.py:1534-1783`) and defers the
rest to a third-party package; here `fla_b200_kda_chunk_bwd` returns the complete gradient of the recurrence in one
call, recomputing the forward from the inputs.  With `use_gate_in_kernel` and gradients enabled the gate activation
runs in PyTorch (so autograd differentiates it) and the kernels receive the activated log decay.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _runtime as rt
from .. import load_library
from ._structs import KdaChunkBwdArgs, KdaChunkFwdArgs
from .gdn import CHUNK, _as_rows, _varlen_meta


def _kda_forward(q, k, v, g, beta, scale, initial_state, output_final_state, gate_mode, A_log, dt_bias, lower_bound,
                 meta, return_gate_cumsum, output_dtype, keep_for_backward=False, scores=None):
    B, T, HK, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    cu, co, N, max_len, total_chunks = meta
    dev = q.device
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
    if scores is not None:   # (aqk, akk) as [B,T,HV,64] views, filled from the forward's score images
        a.aqk, a.akk = rt.desc(scores[0]), rt.desc(scores[1])
    saved = None
    if keep_for_backward:   # the reference's disable_recompute=True: keep the intermediates instead of recomputing them
        nbytes = ctypes.c_uint64(0)
        status = load_library().fla_b200_kda_chunk_saved_size(ctypes.byref(a), ctypes.byref(nbytes))
        if status:
            raise RuntimeError(f"kda_chunk_saved_size failed with status={status}")
        saved = torch.empty((nbytes.value + 1) // 2, dtype=torch.bfloat16, device=dev)
        a.saved = rt.desc(saved)
    rt.call("kda_chunk_fwd", a, [q, k, v, g, beta, initial_state, o, ht, gk, cu, co, saved] + list(scores or ()))
    if keep_for_backward:
        return o, ht, saved
    return o, ht, gk


def kda_chunk_bwd(q, k, v, g, beta, scale, initial_state, do, dht, meta, grad_dtype=None, saved=None):
    """Complete KDA chunk backward (g = per-channel log decay).  Returns dq, dk, dv, dg, dbeta, dh0.
    `saved` is the buffer a forward with ``keep_for_backward`` returned; without it the forward is recomputed."""
    B, T, HK, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    cu, co, N, max_len, total_chunks = meta
    dev = q.device
    gdt = grad_dtype or torch.float32
    dq = torch.empty((B, T, HK, K), dtype=gdt, device=dev)
    dk = torch.empty_like(dq)
    dv = torch.empty((B, T, HV, V), dtype=gdt, device=dev)
    dg = torch.empty((B, T, HV, K), dtype=gdt, device=dev)
    dbeta = torch.empty((B, T, HV), dtype=gdt, device=dev)
    dh0 = torch.empty((N, HV, K, V), dtype=torch.float32, device=dev) if initial_state is not None else None
    if do.dtype != torch.bfloat16:
        from ._convert import convert
        do = convert(do, torch.bfloat16, "chunk_kda_bwd")
    do = _as_rows(do)
    if dht is not None:
        dht = dht.float().contiguous()
    a = KdaChunkBwdArgs()
    a.q, a.k, a.v, a.g, a.beta = rt.desc(q), rt.desc(k), rt.desc(v), rt.desc(g), rt.desc(beta)
    a.initial_state, a.d_o, a.dht = rt.desc(initial_state), rt.desc(do), rt.desc(dht)
    a.dq, a.dk, a.dv, a.dg, a.dbeta, a.dh0 = (rt.desc(x) for x in (dq, dk, dv, dg, dbeta, dh0))
    a.cu_seqlens, a.chunk_offsets, a.saved = rt.desc(cu), rt.desc(co), rt.desc(saved)
    a.scale = scale
    a.chunk_size, a.max_seqlen, a.total_chunks = CHUNK, int(max_len), int(total_chunks)
    rt.call("kda_chunk_bwd", a, [q, k, v, g, beta, initial_state, do, dht, dq, dk, dv, dg, dbeta, dh0, cu, co, saved])
    return dq, dk, dv, dg, dbeta, dh0


class ChunkKdaFunction(torch.autograd.Function):
    """Autograd glue of `chunk_kda` (gate already activated): saves only the inputs, the backward recomputes."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, initial_state, scale, output_final_state, meta, output_dtype, disable_recompute,
                qk_l2norm=False):
        ctx.qk_l2norm = qk_l2norm
        rstd = ()
        if qk_l2norm:   # q, k <- x * rsqrt(sum x^2 + 1e-6) stored in the input dtype; rstd kept for the backward
            from .l2norm import l2norm_fwd
            q, q_rstd = l2norm_fwd(q)
            k, k_rstd = l2norm_fwd(k)
            rstd = (q_rstd, k_rstd)
        o, ht, saved = _kda_forward(q, k, v, g, beta, scale, initial_state, output_final_state, 0, None, None, None, meta,
                                    False, output_dtype, keep_for_backward=disable_recompute)
        ctx.save_for_backward(q, k, v, g, beta, initial_state, saved if disable_recompute else None, *rstd)
        ctx.scale, ctx.meta = scale, meta
        ctx.in_dtypes = (q.dtype, k.dtype, v.dtype, g.dtype, beta.dtype)
        return o, ht

    @staticmethod
    def backward(ctx, do, dht):
        q, k, v, g, beta, h0, saved = ctx.saved_tensors[:7]
        dq, dk, dv, dg, dbeta, dh0 = kda_chunk_bwd(q, k, v, g, beta, ctx.scale, h0, do.contiguous(), dht, ctx.meta,
                                                   saved=saved, grad_dtype=torch.float32 if ctx.qk_l2norm else None)
        if ctx.qk_l2norm:
            from .l2norm import l2norm_bwd
            q_rstd, k_rstd = ctx.saved_tensors[7:9]
            dq = l2norm_bwd(q, q_rstd, dq)
            dk = l2norm_bwd(k, k_rstd, dk)
        dts = ctx.in_dtypes
        return (dq.to(dts[0]), dk.to(dts[1]), dv.to(dts[2]), dg.to(dts[3]), dbeta.to(dts[4]), dh0,
                None, None, None, None, None, None)


def chunk_kda_fwd_bwd(q, k, v, g, beta, do, scale=None, initial_state=None, dht=None, output_dtype=None, grad_dtype=None,
                      disable_recompute=False):
    """Forward and backward in one call without the autograd graph (what a training step costs); g is the log decay.
    With ``disable_recompute`` the forward keeps its intermediates (about 265 KB per (chunk, head)) for the backward.
    Returns (o, final_state, (dq, dk, dv, dg, dbeta, dh0))."""
    B, T = q.shape[:2]
    scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
    q, k, v, g, beta = (_as_rows(x) for x in (q, k, v, g, beta))
    meta = (None, None, B, T, B * ((T + CHUNK - 1) // CHUNK))
    o, ht, saved = _kda_forward(q, k, v, g, beta, scale, initial_state, True, 0, None, None, None, meta, False, output_dtype,
                                keep_for_backward=disable_recompute)
    grads = kda_chunk_bwd(q, k, v, g, beta, scale, initial_state, do, dht, meta, grad_dtype=grad_dtype,
                          saved=saved if disable_recompute else None)
    return o, ht, grads


class _KdaGateFunction(torch.autograd.Function):
    """The activated gate as a tensor (`fla_b200_kda_gate_fwd`) with its gradient w.r.t. g, A_log and dt_bias
    (`fla_b200_kda_gate_bwd`): one pass each way."""

    @staticmethod
    def forward(ctx, g, A_log, dt_bias, mode, lower_bound):
        from ._structs import KdaGateArgs
        HV, K = g.shape[2], g.shape[3]
        g_ = _as_rows(g.detach())
        al = A_log.detach().float().reshape(HV).contiguous()
        db = None if dt_bias is None else dt_bias.detach().float().reshape(HV, K).contiguous()
        gate = torch.empty(g.shape, dtype=torch.float32, device=g.device)
        a = KdaGateArgs()
        a.g, a.a_log, a.dt_bias, a.gate = rt.desc(g_), rt.desc(al), rt.desc(db), rt.desc(gate)
        a.gate_mode, a.lower_bound = int(mode), float(lower_bound or 0.0)
        _single_phase("kda_gate_fwd", a, g.device)
        ctx.save_for_backward(g_, al, db)
        ctx.mode, ctx.lower_bound = int(mode), float(lower_bound or 0.0)
        ctx.shapes = (A_log.shape, A_log.dtype, None if dt_bias is None else (dt_bias.shape, dt_bias.dtype), g.dtype)
        return gate

    @staticmethod
    def backward(ctx, d_gate):
        from ._structs import KdaGateArgs
        g_, al, db = ctx.saved_tensors
        a_shape, a_dtype, b_meta, g_dtype = ctx.shapes
        HV, K = g_.shape[2], g_.shape[3]
        d_gate = _as_rows(d_gate.float())
        d_g = torch.empty(g_.shape, dtype=g_dtype, device=g_.device)
        d_al = torch.empty(HV, dtype=torch.float32, device=g_.device)
        d_db = None if db is None else torch.empty((HV, K), dtype=torch.float32, device=g_.device)
        a = KdaGateArgs()
        a.g, a.a_log, a.dt_bias = rt.desc(g_), rt.desc(al), rt.desc(db)
        a.d_gate, a.d_g, a.d_a_log, a.d_dt_bias = rt.desc(d_gate), rt.desc(d_g), rt.desc(d_al), rt.desc(d_db)
        a.gate_mode, a.lower_bound = ctx.mode, ctx.lower_bound
        rt.call("kda_gate_bwd", a, [g_, al, db, d_gate, d_g, d_al, d_db])
        return (d_g, d_al.reshape(a_shape).to(a_dtype), None if d_db is None else d_db.reshape(b_meta[0]).to(b_meta[1]), None, None)


def _single_phase(fn_name, args, dev):
    rt._check_arch(dev, fn_name)
    with torch.cuda.device(dev):
        status = getattr(load_library(), f"fla_b200_{fn_name}")(ctypes.byref(args),
                                                               ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    if status != 0:
        raise RuntimeError(f"{fn_name} failed with status={status}: {rt._STATUS_NAMES.get(status, '?')}")


def _gate_activation(g, A_log, dt_bias, safe_gate, lower_bound):
    """The gate activations of kda/chunk_kda_fwd/docs/api.md:103-115 as a tensor, differentiable w.r.t. g, A_log and dt_bias:
    the library's gate kernels, for the paths on which the activated gate has to exist (gradients required, or the forward's
    intermediates kept).  fp32 `[B,T,HV,K]`."""
    return _KdaGateFunction.apply(g, A_log, dt_bias, 2 if safe_gate else 1, lower_bound)


def chunk_kda(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
              use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False, use_beta_sigmoid_in_kernel=False,
              cu_seqlens=None, safe_gate=False, lower_bound=None, A_log=None, dt_bias=None,
              return_gate_cumsum=False, output_dtype=None, disable_recompute=False, export_scores=None,
              _return_saved=False):
    """Returns ``(o [B,T,HV,V], final_state [N,HV,K,V] | None)`` (plus the cumulative gate `[B,T,HV,K]` fp32
    when ``return_gate_cumsum``).  ``export_scores`` (inference only): a pair of `[B,T,HV,64]` views that receive the
    per-chunk blocks Aqk and Akk (what `npu_chunk_kda_fwd` returns).  ``_return_saved`` (inference only, used by
    `npu_chunk_kda_fwd`): also return the buffer of forward intermediates, the chunk metadata and the row-major inputs."""
    op = "chunk_kda"
    if use_beta_sigmoid_in_kernel:
        # beta arrives as logits.  It is a [B,T,HV] tensor, 1/128 of the gate's bytes: the activation (and, through autograd,
        # its gradient) is one elementwise pass in front of the kernels rather than a mode of them.
        beta = torch.sigmoid(beta.float())
    if torch.float16 in (q.dtype, k.dtype, v.dtype):
        # fp16 tensors (the reference's published 4-stage case is fp16, fla/ops/ascendc/kda/KDA_FORWARD_VALIDATION_REPORT.md:133-146):
        # q, k, v are rounded to the bf16 operands of the tensor-core products by the library's conversion kernel, fp16
        # gates become fp32, o is computed in fp32 and converted to fp16 once; gradients return through the same conversions
        if not (q.dtype == k.dtype == v.dtype):
            raise TypeError(f"{op}: q, k, v must share one dtype, got {q.dtype}, {k.dtype}, {v.dtype}")
        from ._convert import to_dtype
        q, k, v = (to_dtype(x, torch.bfloat16, op) for x in (q, k, v))
        g, beta = (to_dtype(x, torch.float32, op) if x.dtype == torch.float16 else x for x in (g, beta))
        if export_scores is not None and any(x.dtype == torch.float16 for x in export_scores):
            raise NotImplementedError(f"{op}: export_scores takes bf16 or fp32 views")
        res = chunk_kda(q, k, v, g, beta, scale=scale, initial_state=initial_state, output_final_state=output_final_state,
                        use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel, use_gate_in_kernel=use_gate_in_kernel,
                        use_beta_sigmoid_in_kernel=False, cu_seqlens=cu_seqlens, safe_gate=safe_gate, lower_bound=lower_bound,
                        A_log=A_log, dt_bias=dt_bias, return_gate_cumsum=return_gate_cumsum, output_dtype=torch.float32,
                        disable_recompute=disable_recompute, export_scores=export_scores, _return_saved=_return_saved)
        return (to_dtype(res[0], output_dtype or torch.float16, op),) + tuple(res[1:])
    for name, t in (("q", q), ("k", k), ("v", v)):
        if t.dtype != torch.bfloat16:
            raise TypeError(f"{op}: {name} must be bfloat16 or float16, got {t.dtype}")
    if q.dim() != 4 or q.shape != k.shape or v.dim() != 4 or v.shape[:2] != q.shape[:2]:
        raise RuntimeError(f"{op}: expected q,k [B,T,HK,K] and v [B,T,HV,V]")
    B, T, HK, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    if K != 128 or V not in (128, 256):
        raise RuntimeError(f"{op}: this build supports K = 128 and V = 128 or 256, got K={K}, V={V}")
    if HV % HK:
        raise RuntimeError(f"{op}: HV={HV} must be a multiple of HK={HK}")
    if tuple(g.shape) != (B, T, HV, K) or tuple(beta.shape) != (B, T, HV):
        raise RuntimeError(f"{op}: g must be {(B, T, HV, K)} and beta {(B, T, HV)}")
    scale = K ** -0.5 if scale is None else float(scale)
    needs_grad = torch.is_grad_enabled() and any(
        t is not None and t.requires_grad for t in (q, k, v, g, beta, initial_state, A_log, dt_bias))
    gate_mode = 0
    if use_gate_in_kernel:
        if A_log is None:
            raise RuntimeError(f"{op}: use_gate_in_kernel needs A_log")
        if safe_gate and lower_bound is None:
            raise RuntimeError(f"{op}: safe_gate needs lower_bound")
        if needs_grad or _return_saved:   # the kernels keep their intermediates only for gates given as they are
            g = _gate_activation(g, A_log, dt_bias, safe_gate, lower_bound)
        else:
            gate_mode = 2 if safe_gate else 1
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
    meta = (cu, co, N, max_len, total_chunks)
    if needs_grad:
        if return_gate_cumsum or export_scores is not None:
            raise NotImplementedError(f"{op}: return_gate_cumsum / export_scores are not available on the differentiable path")
        o, ht = ChunkKdaFunction.apply(q, k, v, g, beta, initial_state, scale, output_final_state, meta, output_dtype,
                                       bool(disable_recompute), bool(use_qk_l2norm_in_kernel))
        return o, ht
    if use_qk_l2norm_in_kernel:   # x * rsqrt(sum x^2 + 1e-6), stored in the input dtype (the l2norm kernels)
        from .l2norm import l2norm_fwd
        q, k = l2norm_fwd(q)[0], l2norm_fwd(k)[0]
    if _return_saved:
        o, ht, saved = _kda_forward(q, k, v, g, beta, scale, initial_state, output_final_state, 0, None, None, None, meta,
                                    False, output_dtype, keep_for_backward=True, scores=export_scores)
        return o, ht, saved, meta, (q, k, v, beta)
    o, ht, gk = _kda_forward(q, k, v, g, beta, scale, initial_state, output_final_state, gate_mode, A_log, dt_bias,
                             lower_bound, meta, return_gate_cumsum, output_dtype, scores=export_scores)
    if return_gate_cumsum:
        return o, ht, gk
    return o, ht


def kda_chunk_intermediates(q, k, v, beta, saved, meta, *, full, state_v_first=False, dtype=None):
    """w, u, qg, kg, v_new `[B,HV,T,.]` (when ``full``) and h `[B*NT | chunks, HV, K, V]` from the buffer a forward with
    ``keep_for_backward`` left (`fla_b200_kda_chunk_intermediates`): a chunk-parallel fp32 pass outside the hot path."""
    from ._structs import KdaIntermediatesArgs
    B, T, HK, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    cu, co, N, max_len, total_chunks = meta
    dev, dtype = q.device, dtype or q.dtype
    outs = {}
    if full:
        for name, d in (("w", K), ("u", V), ("qg", K), ("kg", K), ("v_new", V)):
            outs[name] = torch.zeros((B, HV, T, d), dtype=dtype, device=dev)
    hshape = (total_chunks, HV, V, K) if state_v_first else (total_chunks, HV, K, V)
    h = torch.empty(hshape, dtype=dtype, device=dev)
    a = KdaIntermediatesArgs()
    a.q, a.k, a.v, a.beta, a.saved = rt.desc(q), rt.desc(k), rt.desc(v), rt.desc(beta), rt.desc(saved)
    a.cu_seqlens, a.chunk_offsets = rt.desc(cu), rt.desc(co)
    for name, t in outs.items():
        setattr(a, name, rt.desc(t.transpose(1, 2)))
    a.h = rt.desc(h)
    a.max_seqlen, a.total_chunks, a.state_v_first = int(max_len), int(total_chunks), int(bool(state_v_first))
    lib = load_library()
    rt._check_arch(dev, "kda_chunk_intermediates")
    with torch.cuda.device(dev):
        status = lib.fla_b200_kda_chunk_intermediates(ctypes.byref(a), ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    if status != 0:
        raise RuntimeError(f"kda_chunk_intermediates failed with status={status}: {rt._STATUS_NAMES.get(status, '?')}")
    return outs, h


def _merge_score_blocks(q, k, beta, gk64, aqk64, akk64, scale, cu_seqlens, dtype, want_gk):
    """Aqk, Akk `[B,HV,T,128]` and gk `[B,HV,T,K]` of 128-token chunks from the 64-token blocks (`fla_b200_kda_merge_score_blocks`).
    q, k `[B,T,HK,K]`, beta `[B,T,HV]`, gk64 `[B,T,HV,K]` fp32 base 2, aqk64 / akk64 `[B,HV,T,64]` fp32."""
    from ._structs import KdaMergeBlocksArgs
    B, T, HK, K = q.shape
    HV = beta.shape[2]
    dev = q.device
    if q.dtype == torch.float16:   # the same rounded operands the forward kernels saw
        from ._convert import convert
        q, k = convert(q, torch.bfloat16), convert(k, torch.bfloat16)
    q, k, beta = _as_rows(q), _as_rows(k), _as_rows(beta)
    if beta.dtype not in (torch.float32, torch.bfloat16):
        beta = beta.float()
    cu = co = None
    max_len = T
    if cu_seqlens is not None:
        cu, co, max_len, _, _, _ = _varlen_meta(cu_seqlens, dev)
    aqk = torch.zeros((B, HV, T, 128), dtype=dtype, device=dev)
    akk = torch.zeros_like(aqk)
    gk = torch.empty((B, HV, T, K), dtype=torch.float32, device=dev) if want_gk else None
    a = KdaMergeBlocksArgs()
    a.q, a.k, a.beta, a.gk = rt.desc(q), rt.desc(k), rt.desc(beta), rt.desc(gk64.contiguous())
    a.aqk64, a.akk64 = rt.desc(aqk64.transpose(1, 2)), rt.desc(akk64.transpose(1, 2))
    a.cu_seqlens, a.chunk_offsets = rt.desc(cu), rt.desc(co)
    a.aqk, a.akk = rt.desc(aqk.transpose(1, 2)), rt.desc(akk.transpose(1, 2))
    a.gk_out = rt.desc(None if gk is None else gk.transpose(1, 2))
    a.scale, a.max_seqlen, a.gk_base2 = float(scale), int(max_len), 1
    _single_phase("kda_merge_score_blocks", a, dev)
    return aqk, akk, gk


def _merge_intermediates(k, beta, gk64, akk64, inter64, cu_seqlens, dtype):
    """w, u, qg, kg `[B,HV,T,.]` of 128-token chunks from the fp32 ones of the 64-token chunks (`fla_b200_kda_merge_intermediates`).
    k `[B,T,HK,K]`, beta `[B,T,HV]` (row-major), gk64 `[B,T,HV,K]` fp32 base 2, akk64 `[B,HV,T,64]` fp32."""
    from ._structs import KdaMergeInterArgs
    B, T, HK, K = k.shape
    HV = beta.shape[2]
    dev = k.device
    if beta.dtype not in (torch.float32, torch.bfloat16):
        beta = beta.float()
    cu = co = None
    max_len = T
    if cu_seqlens is not None:
        cu, co, max_len, _, _, _ = _varlen_meta(cu_seqlens, dev)
    out = {n: torch.zeros(inter64[n].shape, dtype=dtype, device=dev) for n in ("w", "u", "qg", "kg")}
    a = KdaMergeInterArgs()
    a.k, a.beta, a.gk, a.akk64 = rt.desc(k), rt.desc(beta), rt.desc(gk64.contiguous()), rt.desc(akk64.transpose(1, 2))
    a.w64, a.u64, a.qg64, a.kg64 = (rt.desc(inter64[n].transpose(1, 2)) for n in ("w", "u", "qg", "kg"))
    a.cu_seqlens, a.chunk_offsets = rt.desc(cu), rt.desc(co)
    a.w, a.u, a.qg, a.kg = (rt.desc(out[n].transpose(1, 2)) for n in ("w", "u", "qg", "kg"))
    a.max_seqlen, a.gk_base2 = int(max_len), 1
    _single_phase("kda_merge_intermediates", a, dev)
    return out


def npu_chunk_kda_fwd(q, k, v, g, beta, scale, chunk_size=64, *, layout="BSND", initial_state=None, output_final_state=False,
                      cu_seqlens=None, chunk_indices=None, safe_gate=False, lower_bound=None, use_gate_in_kernel=False,
                      A_log=None, dt_bias=None, disable_recompute=False, return_intermediate_states=False, state_v_first=False):
    """The reference's low-level KDA forward (torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:1066-1265) with its
    12-value return `(attn_out, final_state, gk, Aqk, Akk, w, u, qg, kg, v_new, h, initial_state)` and the visibility rule of
    `_kda_policy.py:15-37`: final_state when asked for, gk (base-2 chunk-local cumulative gate, head-first fp32) unless the gate
    is activated in the kernel, Aqk and Akk `[B,HV,T,64]` always.  The head-major intermediates never exist in the fused
    kernels; `disable_recompute=True` (w, u, qg, kg, v_new, h and gk) and `return_intermediate_states=True` (h) run a
    second, chunk-parallel pass over the forward's saved operand images that forms them (`kda_chunk_intermediates`), with
    the gate activated in front of the kernels when `use_gate_in_kernel` is set.  `chunk_size=128`: o and the states do not
    depend on the blocking; gk, Aqk, Akk `[B,HV,T,128]` are merged from the 64-token blocks (`fla_b200_kda_merge_score_blocks`)
    h keeps every second state, and w, u, qg, kg are merged from the fp32 ones of the halves (`fla_b200_kda_merge_intermediates`).
    `state_v_first=True` takes and returns the recurrent state as `[N,HV,V,K]`.  Layouts: "BSND" `[B,T,H,D]`, "BNSD" `[B,H,T,D]`, "TND" / "NTD" (3-D, packed, with `cu_seqlens`); `attn_out`
    comes back in the input's layout."""
    del chunk_indices
    op = "npu_chunk_kda_fwd"
    layout = str(layout)
    if layout not in {"BSND", "BNSD", "TND", "NTD"}:
        raise RuntimeError(f"{op}: layout must be uppercase and one of BSND, BNSD, TND, NTD.")
    if int(chunk_size) not in {64, 128}:
        raise RuntimeError(f"{op}: chunk_size must be 64 or 128.")
    big = int(chunk_size) == 128     # the kernels tile by 64 tokens: o and the states do not depend on the blocking, the score
    #                                  blocks and gk of 128-token chunks are merged from those of their two halves afterwards
    want_full = bool(disable_recompute)
    want_h = want_full or bool(return_intermediate_states)
    rank3 = layout in {"TND", "NTD"}

    def to_bsnd(t):
        if t is None:
            return None
        if rank3:
            t = t.unsqueeze(0)
        return t.transpose(1, 2) if layout in {"BNSD", "NTD"} else t

    qb, kb, vb, gb, bb = (to_bsnd(t) for t in (q, k, v, g, beta))
    B, T, HK, K = qb.shape
    HV = vb.shape[2]
    dev = q.device
    # fp16 callers: the score blocks leave the export kernel as fp32 and are converted once at the end
    aqk = torch.zeros((B, HV, T, CHUNK), dtype=torch.float32 if (big or q.dtype == torch.float16) else q.dtype, device=dev)
    akk = torch.zeros_like(aqk)
    gate_kw = {}
    if use_gate_in_kernel:
        gate_kw = dict(use_gate_in_kernel=True, safe_gate=safe_gate, lower_bound=lower_bound, A_log=A_log, dt_bias=dt_bias)
    # forward with the score blocks exported (chunk_kda's own checks and metadata apply)
    # state_v_first: the caller's states are `[N,HV,V,K]`; the kernels keep `[N,HV,K,V]` (a transposed copy of a small tensor)
    h0 = initial_state
    if state_v_first and initial_state is not None:
        if initial_state.dim() != 4 or initial_state.shape[-2] != vb.shape[-1] or initial_state.shape[-1] != K:
            raise RuntimeError(f"{op}: initial_state shape does not match state_v_first.")
        h0 = initial_state.transpose(-1, -2)
    inter, h = {}, None
    with torch.no_grad():
        if want_h:
            o, ht, saved, meta, rows_in = chunk_kda(qb, kb, vb, gb, bb, scale=scale, initial_state=h0,
                                                    output_final_state=output_final_state, cu_seqlens=cu_seqlens,
                                                    export_scores=(aqk.transpose(1, 2), akk.transpose(1, 2)), _return_saved=True,
                                                    **gate_kw)
            inter, h = kda_chunk_intermediates(*rows_in, saved, meta, full=want_full, state_v_first=state_v_first,
                                               dtype=torch.float32 if (big and want_full) else q.dtype)
            if big:   # the states at the starts of the 128-token chunks: every second 64-token chunk of each sequence
                bounds = [0, T] if cu_seqlens is None else [int(x) for x in cu_seqlens]
                first, idx = 0, []
                for _ in range(B if cu_seqlens is None else 1):
                    for bos, eos in zip(bounds[:-1], bounds[1:]):
                        n64 = (eos - bos + CHUNK - 1) // CHUNK
                        idx += list(range(first, first + n64, 2))
                        first += n64
                h = h.index_select(0, torch.tensor(idx, dtype=torch.int64, device=dev))
            h = h if rank3 else h.view(B, -1, *h.shape[1:])
        else:
            o, ht = chunk_kda(qb, kb, vb, gb, bb, scale=scale, initial_state=h0, output_final_state=output_final_state,
                              cu_seqlens=cu_seqlens, export_scores=(aqk.transpose(1, 2), akk.transpose(1, 2)), **gate_kw)
    gk_out = None
    if not use_gate_in_kernel or want_full or big:
        from .stages import kda_gate_cumsum
        gk64 = kda_gate_cumsum(gb, CHUNK, cu_seqlens=cu_seqlens, **{k_: v_ for k_, v_ in gate_kw.items()})          # [B,T,HV,K], base 2
        gk_out = gk64.permute(0, 2, 1, 3)                                                                             # [B,HV,T,K]
    if big:
        if want_full:   # w, u, qg, kg of the 128-token chunks from the fp32 ones of their halves; v_new and h only change dtype
            from ._convert import convert
            merged = _merge_intermediates(rows_in[1], rows_in[3], gk64, akk, inter, cu_seqlens, q.dtype)
            merged["v_new"] = convert(inter["v_new"], q.dtype, op)
            inter = merged
            h = convert(h.reshape(-1, *h.shape[-2:]), q.dtype, op).view(h.shape)
        aqk, akk, gk_out = _merge_score_blocks(qb, kb, bb, gk64, aqk, akk, scale, cu_seqlens, q.dtype,
                                               want_gk=not use_gate_in_kernel or want_full)
    if state_v_first and ht is not None:
        ht = ht.transpose(-1, -2).contiguous()
    if q.dtype == torch.float16 and not big:
        from ._convert import convert
        aqk, akk = convert(aqk, torch.float16, op), convert(akk, torch.float16, op)
    if layout in {"BNSD", "NTD"}:
        o = o.transpose(1, 2).contiguous()
    if rank3:
        o, aqk, akk = o.squeeze(0), aqk.squeeze(0), akk.squeeze(0)
        gk_out = None if gk_out is None else gk_out.squeeze(0)
        inter = {n: t.squeeze(0) for n, t in inter.items()}
    return (o, ht, gk_out, aqk, akk, inter.get("w"), inter.get("u"), inter.get("qg"), inter.get("kg"), inter.get("v_new"), h,
            initial_state)


"""Stage-by-stage operators of the chunked gated-delta-rule forward, with the names, argument order and head-first
`[B,H,T,D]` layouts of the reference's low-level surface (torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py):
`npu_chunk_local_cumsum` (:875-904), `npu_chunk_scaled_dot_kkt` (:907-936), `npu_solve_tri` (:1786-1800),
`npu_recompute_w_u_fwd` (:618-651), `npu_chunk_gated_delta_rule_fwd_h` (:552-615), `npu_chunk_fwd_o` (:517-549).

The fused `chunk_gated_delta_rule` never writes A, w, u or the per-chunk states to memory; these functions are for
call sites that run the reference's chain one operator at a time (examples/flash_gated_delta_rule.py:796-881).
Tensors are passed with their strides, so sequence-first tensors can be given as transposed views without a copy.
`cu_seqlens` is a host list (or tensor) of sequence boundaries as in the reference; `chunk_indices` is accepted and
ignored because the chunk geometry follows from `cu_seqlens`.
"""
from __future__ import annotations

import torch

from .. import _runtime as rt
from ._structs import ChunkKdaBwdIntraArgs, ChunkStageArgs
from .gdn import CHUNK, _varlen_meta

_DTYPES = {"float": torch.float32, "float32": torch.float32, "half": torch.float16, "float16": torch.float16,
           "bf16": torch.bfloat16, "bfloat16": torch.bfloat16}


def _stage_call(op, fields, tensors, ref, cu_seqlens, chunk_size, scale=1.0, reverse=False, gate_mode=0, lower_bound=0.0):
    if int(chunk_size) != CHUNK:
        raise NotImplementedError(f"{op}: this build supports chunk_size = {CHUNK}, got {chunk_size}")
    B, T = ref.shape[0], ref.shape[2]
    dev = ref.device
    cu = co = None
    max_len, total_chunks = T, B * ((T + CHUNK - 1) // CHUNK)
    if cu_seqlens is not None:
        if B != 1:
            raise RuntimeError(f"{op}: cu_seqlens requires batch size 1 (packed sequences)")
        cu, co, max_len, total_chunks, _n, total = _varlen_meta(cu_seqlens, dev)
        if total != T:
            raise RuntimeError(f"{op}: cu_seqlens[-1]={total} must equal T={T}")
    a = ChunkStageArgs()
    for name, t in fields.items():
        setattr(a, name, rt.desc(t))
    a.cu_seqlens, a.chunk_offsets = rt.desc(cu), rt.desc(co)
    a.scale, a.chunk_size, a.max_seqlen, a.total_chunks, a.reverse = float(scale), CHUNK, int(max_len), int(total_chunks), int(bool(reverse))
    a.gate_mode, a.lower_bound = int(gate_mode), float(lower_bound)
    rt.call(op, a, list(tensors) + [cu, co])
    return total_chunks


def _num_sequences(B, cu_seqlens):
    return B if cu_seqlens is None else len(cu_seqlens) - 1


def chunk_local_cumsum(g, chunk_size, *, cu_seqlens=None, chunk_indices_out=None, reverse=False, scale=1.0, head_first=True,
                       output_dtype="float32"):
    """Chunk-local (reverse) cumulative sum of the gate.  g `[B,H,T]` (or `[B,H,T,D]`) when `head_first`, else
    `[B,T,H]` / `[B,T,H,D]`; the result has g's shape and `output_dtype` ("same" keeps g's dtype)."""
    del chunk_indices_out
    if isinstance(output_dtype, torch.dtype) or output_dtype is None:
        out_dtype = output_dtype or torch.float32
    else:
        name = str(output_dtype).removeprefix("torch.").lower()
        if name in ("same", "input", "none"):
            out_dtype = g.dtype
        elif name in _DTYPES:
            out_dtype = _DTYPES[name]
        else:
            raise TypeError(f"Unsupported chunk_local_cumsum output_dtype: {output_dtype}.")
    if g.dim() not in (3, 4):
        raise RuntimeError(f"chunk_local_cumsum: g must be 3-D or 4-D, got {tuple(g.shape)}")
    out = torch.empty(g.shape, dtype=out_dtype, device=g.device)
    gv, ov = (g, out) if head_first else (g.transpose(1, 2), out.transpose(1, 2))
    _stage_call("chunk_local_cumsum", dict(g=gv, out0=ov), [g, out], gv, cu_seqlens, chunk_size, scale=scale, reverse=reverse)
    return out


def kda_gate_cumsum(g, chunk_size, *, A_log=None, dt_bias=None, cu_seqlens=None, use_gate_in_kernel=False, safe_gate=False,
                    lower_bound=None):
    """Per-channel gate activation and chunk-local cumulative sum in base 2: `gk = cumsum_chunk(gate) / ln 2` with
    gate = g, `-e^{A_log} softplus(g + dt_bias)` (`use_gate_in_kernel`) or `lower_bound sigmoid(e^{A_log} (g + dt_bias))`
    (`use_gate_in_kernel` and `safe_gate`).  g `[B,T,HV,K]` -> fp32 of the same shape."""
    if g.dim() != 4:
        raise RuntimeError(f"kda_gate_cumsum: g must be [B,T,HV,K], got {tuple(g.shape)}")
    HV, K = g.shape[2], g.shape[3]
    mode, al, db = 0, None, None
    if use_gate_in_kernel:
        if A_log is None:
            raise RuntimeError("kda_gate_cumsum: use_gate_in_kernel needs A_log")
        mode = 2 if safe_gate else 1
        al = A_log.float().reshape(HV).contiguous()
        db = None if dt_bias is None else dt_bias.float().reshape(HV, K).contiguous()
    out = torch.empty(g.shape, dtype=torch.float32, device=g.device)
    gv, ov = g.transpose(1, 2), out.transpose(1, 2)
    _stage_call("chunk_local_cumsum", dict(g=gv, out0=ov, q=al, k=db), [g, out, al, db], gv, cu_seqlens, chunk_size,
                scale=1.4426950408889634, gate_mode=mode, lower_bound=-5.0 if lower_bound is None else lower_bound)
    return out


def chunk_scaled_dot_kkt(k, g, beta, *, cu_seqlens=None, chunk_indices=None, chunk_size=64):
    """A `[B,HV,T,C]` fp32: `beta_i exp(clip(g_i - g_j, +-50)) k_i.k_j` below the diagonal of every chunk, else 0.
    k `[B,HK,T,K]` bf16, g (chunk-local cumulative gate) and beta `[B,HV,T]`."""
    del chunk_indices
    B, HK, T, K = k.shape
    HV = g.shape[1]
    out = torch.empty((B, HV, T, int(chunk_size)), dtype=torch.float32, device=k.device)
    _stage_call("chunk_scaled_dot_kkt", dict(k=k, g=g, beta=beta, out0=out), [k, g, beta, out], g, cu_seqlens, chunk_size)
    return out


def solve_tri(x, *, cu_seqlens=None, chunk_indices=None, layout="bsnd", output_dtype=None):
    """Per chunk `(I + strict_lower(x))^-1`.  x is `[B,T,H,C]` for layout "bsnd" and `[B,H,T,C]` for "bnsd"
    ("tnd" `[T,H,C]` and "ntd" `[H,T,C]` are the packed 3-D forms, used with `cu_seqlens`).  The result has x's dtype
    unless `output_dtype` (not in the reference's signature) asks for another, which saves the separate cast of A."""
    del chunk_indices
    lay = str(layout).lower()
    if lay in ("tnd", "ntd"):     # packed 3-D forms of the same two layouts
        if x.dim() != 3:
            raise RuntimeError(f"solve_tri: layout {layout!r} expects a 3-D tensor, got {tuple(x.shape)}")
        return solve_tri(x.unsqueeze(0), cu_seqlens=cu_seqlens, layout="bsnd" if lay == "tnd" else "bnsd",
                         output_dtype=output_dtype).squeeze(0)
    if lay not in ("bsnd", "bnsd"):
        raise NotImplementedError(f"solve_tri: layout {layout!r} is not supported (bsnd, bnsd, tnd, ntd)")
    if x.dim() != 4 or x.shape[-1] != CHUNK:
        raise NotImplementedError(f"solve_tri: x must be 4-D with a last dimension of {CHUNK}, got {tuple(x.shape)}")
    out = torch.empty(x.shape, dtype=output_dtype or x.dtype, device=x.device)
    xv, ov = (x, out) if lay == "bnsd" else (x.transpose(1, 2), out.transpose(1, 2))
    _stage_call("solve_tri", dict(A=xv, out0=ov), [x, out], xv, cu_seqlens, CHUNK)
    return out


def recompute_w_u_fwd(k, v, beta, A, chunk_size, *, g=None, gk=None, cu_seqlens=None, chunk_indices=None):
    """`w = A (k beta e^g)`, `u = A (v beta)` per chunk.  k `[B,HK,T,K]`, v `[B,HV,T,V]`, A `[B,HV,T,C]` bf16,
    beta and g `[B,HV,T]`.  Returns (w `[B,HV,T,K]`, u `[B,HV,T,V]`)."""
    del chunk_indices
    if gk is not None:
        raise NotImplementedError("recompute_w_u_fwd: per-channel gates (gk) are handled by the fused KDA operator")
    if g is None:
        raise RuntimeError("recompute_w_u_fwd: g is required")
    B, HV, T, V = v.shape
    w = torch.empty((B, HV, T, k.shape[3]), dtype=k.dtype, device=k.device)
    u = torch.empty_like(v)
    _stage_call("recompute_w_u_fwd", dict(k=k, v=v, beta=beta, A=A, g=g, out0=w, out1=u), [k, v, beta, A, g, w, u], v, cu_seqlens,
                chunk_size)
    return w, u


def chunk_gated_delta_rule_fwd_h(k, w, u, g=None, *, gk=None, initial_state=None, output_final_state=False, chunk_size=None,
                                 cu_seqlens=None, chunk_indices=None, state_v_first=False):
    """Sequential state pass: `h_c = S`, `v_new = u - w S`, `S <- e^{g_last} S + k^T (e^{g_last - g} v_new)`.
    Returns (h `[B,HV,NT,K,V]`, v_new `[B,HV,T,V]`, final_state `[N,HV,K,V]` fp32 or None).
    `state_v_first` (…/_aclnn_ctypes.py:564,581-586): initial_state, h and final_state have their last two dims swapped
    (`[.., V, K]`); the kernel works K-first, so the states are transposed on the way in and out (a copy each)."""
    del chunk_indices
    if gk is not None or g is None:
        raise NotImplementedError("chunk_gated_delta_rule_fwd_h: scalar gates (g) only; gk belongs to the fused KDA operator")
    if state_v_first:
        if initial_state is not None:
            if initial_state.dim() != 4 or initial_state.shape[2:] != (u.shape[3], k.shape[3]):
                raise RuntimeError("npu_chunk_gated_delta_rule_fwd_h: initial_state shape does not match state_v_first.")
            initial_state = initial_state.transpose(-1, -2)
        h, v_new, ht = chunk_gated_delta_rule_fwd_h(k, w, u, g, initial_state=initial_state, output_final_state=output_final_state,
                                                    chunk_size=chunk_size, cu_seqlens=cu_seqlens)
        return h.transpose(-1, -2).contiguous(), v_new, None if ht is None else ht.transpose(-1, -2).contiguous()
    chunk_size = CHUNK if chunk_size is None else int(chunk_size)
    B, HV, T, V = u.shape
    K = k.shape[3]
    N = _num_sequences(B, cu_seqlens)
    if cu_seqlens is None:
        NT = (T + CHUNK - 1) // CHUNK
    else:
        cu_host = [int(x) for x in (cu_seqlens.tolist() if isinstance(cu_seqlens, torch.Tensor) else cu_seqlens)]
        NT = sum((b - a + CHUNK - 1) // CHUNK for a, b in zip(cu_host, cu_host[1:]))
    if initial_state is not None:
        if tuple(initial_state.shape) != (N, HV, K, V):
            raise RuntimeError("npu_chunk_gated_delta_rule_fwd_h: initial_state shape does not match state_v_first.")
        initial_state = initial_state.float().contiguous()
    h = torch.empty((B, HV, NT, K, V), dtype=k.dtype, device=k.device)
    v_new = torch.empty_like(u)
    ht = torch.empty((N, HV, K, V), dtype=torch.float32, device=k.device) if output_final_state else None
    _stage_call("chunk_gated_delta_rule_fwd_h", dict(k=k, w=w, u=u, g=g, initial_state=initial_state, out0=h, out1=v_new, out2=ht),
                [k, w, u, g, initial_state, h, v_new, ht], u, cu_seqlens, chunk_size)
    return h, v_new, ht


def chunk_fwd_o(q, k, v, h, scale, *, g=None, g_gamma=None, cu_seqlens=None, chunk_indices=None, chunk_size=None,
                transpose_state_layout=False):
    """`o = scale (e^{g_i} q h_c + tril(q k^T e^{g_i - g_j}) v)` per chunk; v is the `v_new` of the state pass."""
    del chunk_indices
    if g_gamma is not None:   # reserved in the reference too (chunk_gdn_fwd/chunk_fwd_o/README.md:177: not used, pass None)
        raise RuntimeError("chunk_fwd_o: g_gamma is a reserved input and must be None")
    if transpose_state_layout:
        raise NotImplementedError("chunk_fwd_o: transpose_state_layout is not supported")
    if g is None:
        raise NotImplementedError("chunk_fwd_o: g is required")
    chunk_size = CHUNK if chunk_size is None else int(chunk_size)
    o = torch.empty_like(v)
    _stage_call("chunk_fwd_o", dict(q=q, k=k, v=v, h=h, g=g, out0=o), [q, k, v, h, g, o], v, cu_seqlens, chunk_size, scale=scale)
    return o


def chunk_bwd_dv_local(q, k, d_o, g, scale, chunk_size, *, g_gamma=None, A=None, cu_seqlens=None, chunk_indices=None):
    """Intra-chunk part of dv: `dv_j = sum_{i >= j} scale (k_j.q_i) e^{g_i - g_j} d_o_i`.  q, k `[B,HK,T,K]`, d_o `[B,HV,T,V]`,
    g `[B,HV,T]` (chunk-local cumulative gate)."""
    del chunk_indices
    if g_gamma is not None or A is not None:   # reserved in the reference too (chunk_gdn_bwd/chunk_bwd_dv_local/README.md:84-85)
        raise RuntimeError("chunk_bwd_dv_local: g_gamma and A are reserved inputs and must be None")
    dv = torch.empty_like(d_o)
    _stage_call("chunk_bwd_dv_local", dict(q=q, k=k, v=d_o, g=g, out0=dv), [q, k, d_o, g, dv], d_o, cu_seqlens, chunk_size, scale=scale)
    return dv


def chunk_gated_delta_rule_bwd_dhu(q, k, w, d_o, dv, scale, chunk_size, *, g=None, gK=None, h0=None, dht=None, cu_seqlens=None,
                                   chunk_indices=None, use_exp2=False, transpose_state_layout=False):
    """Reverse state pass of the backward: `dh_c = dS`, `dv2 = dv + e^{g_last - g} (k dS)`,
    `dS <- e^{g_last} dS + q^T (scale e^g d_o) - w^T dv2`.  Returns (dh `[B,HV,NT,K,V]`, dh0, dv2).
    dh0 is returned when `h0` is given, as fp32 `[N,HV,K,V]` (the reference allocates `[B,HV,NT,K,V]` and fills chunk 0);
    `dht` `[N,HV,K,V]` seeds dS (the reference accepts the argument and ignores it)."""
    del chunk_indices
    if gK is not None or g is None:
        raise NotImplementedError("chunk_gated_delta_rule_bwd_dhu: scalar gates (g) only; gK belongs to the fused KDA operator")
    if use_exp2 or transpose_state_layout:
        raise NotImplementedError("chunk_gated_delta_rule_bwd_dhu: use_exp2 / transpose_state_layout are not supported")
    if any(t.dtype != q.dtype for t in (k, w, d_o, dv)):
        raise ValueError("q, k, w, d_o and dv must have the same dtype.")
    B, HV, T, V = dv.shape
    K = q.shape[3]
    N = _num_sequences(B, cu_seqlens)
    if cu_seqlens is None:
        NT = (T + CHUNK - 1) // CHUNK
    else:
        cu_host = [int(x) for x in (cu_seqlens.tolist() if isinstance(cu_seqlens, torch.Tensor) else cu_seqlens)]
        NT = sum((b - a + CHUNK - 1) // CHUNK for a, b in zip(cu_host, cu_host[1:]))
    if dht is not None:
        if tuple(dht.shape) != (N, HV, K, V):
            raise RuntimeError(f"chunk_gated_delta_rule_bwd_dhu: dht must be {(N, HV, K, V)}, got {tuple(dht.shape)}")
        dht = dht.float().contiguous()
    dh = torch.empty((B, HV, NT, K, V), dtype=q.dtype, device=q.device)
    dv2 = torch.empty_like(dv)
    dh0 = torch.empty((N, HV, K, V), dtype=torch.float32, device=q.device) if h0 is not None else None
    _stage_call("chunk_gated_delta_rule_bwd_dhu", dict(q=q, k=k, w=w, u=d_o, v=dv, g=g, initial_state=dht, out0=dh, out1=dv2, out2=dh0),
                [q, k, w, d_o, dv, g, dht, dh, dv2, dh0], dv, cu_seqlens, chunk_size, scale=scale)
    return dh, dh0, dv2


def chunk_bwd_dqkwg(q, k, v, g, h, dox, dh, dv, chunk_size, *, cu_seqlens=None, chunk_indices=None, w=None, g_gamma=None, scale=None,
                    use_exp2=None, transpose_state_layout=None):
    """dq, dk (summed over the value heads of a group), dw and the pre-cumsum dg of one backward step from the per-chunk
    states.  q, k `[B,HK,T,K]`; v (= v_new), dox (= dO), dv (= dv2) `[B,HV,T,V]`; h, dh `[B,HV,NT,K,V]`; g `[B,HV,T]`.
    Returns (dq, dk, dw, dg); dw is produced when `w` is given (as in the reference, whose kernel only needs its presence)."""
    del chunk_indices
    if g is None or g_gamma is not None or use_exp2 or transpose_state_layout:
        raise NotImplementedError("chunk_bwd_dqkwg: scalar gates g only; g_gamma / use_exp2 / transpose_state_layout are not supported")
    scale = 1.0 if scale is None else float(scale)
    B, HV, T, V = v.shape
    dq, dk = torch.empty_like(q), torch.empty_like(k)
    dw = torch.empty((B, HV, T, q.shape[3]), dtype=q.dtype, device=q.device) if w is not None else None
    dg = torch.empty_like(g)
    _stage_call("chunk_bwd_dqkwg", dict(q=q, k=k, v=v, g=g, h=h, u=dox, A=dh, w=dv, out0=dq, out1=dk, out2=dw, out3=dg),
                [q, k, v, g, h, dox, dh, dv, dq, dk, dw, dg], v, cu_seqlens, chunk_size, scale=scale)
    return dq, dk, dw, dg


def _wy_outputs(k, v, beta, g):
    return torch.empty_like(k), torch.empty_like(v), torch.empty_like(beta), torch.empty_like(g)


def prepare_wy_repr_bwd(k, v, beta, A, dw, du, g, chunk_size, *, cu_seqlens=None, chunk_indices=None):
    """Backward of `w = A (k beta e^g)`, `u = A (v beta)` (A = the chunk inverses) from dw, du in one launch.
    k `[B,HK,T,K]`; v, du `[B,HV,T,V]`; dw `[B,HV,T,K]`; A `[B,HV,T,C]`; beta, g `[B,HV,T]`.
    Returns (dk `[B,HK,T,K]` summed over each group's value heads, dv, dbeta, dg)."""
    del chunk_indices
    dk, dv, dbeta, dg = _wy_outputs(k, v, beta, g)
    _stage_call("prepare_wy_repr_bwd", dict(k=k, v=v, beta=beta, A=A, w=dw, u=du, g=g, out0=dk, out1=dv, out2=dbeta, out3=dg),
                [k, v, beta, A, dw, du, g, dk, dv, dbeta, dg], v, cu_seqlens, chunk_size)
    return dk, dv, dbeta, dg


def prepare_wy_repr_bwd_da(k, v, beta, A, dw, du, g, *, chunk_size, cu_seqlens=None, chunk_indices=None):
    """Gradient of the chunk's strictly-lower score block, stored transposed within each chunk like the reference:
    `dA^T = strict_lower(-(A^T strict_lower(dw (k beta e^g)^T + du (v beta)^T) A^T) * e^{g_i - g_j})`.  `[B,HV,T,C]`, A's dtype."""
    del chunk_indices
    dA = torch.empty_like(A)
    _stage_call("prepare_wy_repr_bwd_da", dict(k=k, v=v, beta=beta, A=A, w=dw, u=du, g=g, out0=dA), [k, v, beta, A, dw, du, g, dA], v,
                cu_seqlens, chunk_size)
    return dA


def prepare_wy_repr_bwd_full(k, v, beta, A, dA, dw, du, g, chunk_size, *, cu_seqlens=None, chunk_indices=None):
    """dk, dv, dbeta, dg of the WY representation from dw, du and the dA of `prepare_wy_repr_bwd_da`."""
    del chunk_indices
    dk, dv, dbeta, dg = _wy_outputs(k, v, beta, g)
    _stage_call("prepare_wy_repr_bwd_full", dict(k=k, v=v, beta=beta, A=A, q=dA, w=dw, u=du, g=g, out0=dk, out1=dv, out2=dbeta, out3=dg),
                [k, v, beta, A, dA, dw, du, g, dk, dv, dbeta, dg], v, cu_seqlens, chunk_size)
    return dk, dv, dbeta, dg


def chunk_kda_bwd_intra(q, k, gk, beta, dAqk, dAkk, dq, dk, db, dg, *, cu_seqlens=None, chunk_indices=None, chunk_size=64,
                        safe_gate=True, layout="BSND"):
    """Intra-chunk part of the KDA backward, accumulated IN PLACE onto dq, dk, db, dg (which are also returned).
    Layouts as in the reference: "BSND" `[B,T,H,D]`, "BNSD" `[B,H,T,D]`, "TND" `[T,H,D]` (with `cu_seqlens`).
    q, k bf16; gk (base-2 cumulative gate), dAqk, dAkk `[..., 64]`, dq, dk, dg fp32; beta bf16 or fp32; db fp32."""
    del chunk_indices
    op = "npu_chunk_kda_bwd_intra"
    layout = str(layout)
    if layout not in {"BSND", "BNSD", "TND"}:
        raise RuntimeError(f"{op}: supports dense BSND/BNSD or varlen TND.")
    if not bool(safe_gate):
        raise RuntimeError(f"{op}: safe_gate=False is reserved but not supported in v1.")
    if int(chunk_size) != CHUNK:
        raise RuntimeError(f"{op}: chunk_size must be 64.")
    tensors = dict(q=q, k=k, gk=gk, beta=beta, dAqk=dAqk, dAkk=dAkk, dq=dq, dk=dk, db=db, dg=dg)
    want = dict(q=torch.bfloat16, k=torch.bfloat16, gk=torch.float32, dAqk=torch.float32, dAkk=torch.float32, dq=torch.float32,
                dk=torch.float32, db=torch.float32, dg=torch.float32)
    for name, t in tensors.items():
        if name == "beta":
            if t.dtype not in (torch.bfloat16, torch.float32):
                raise RuntimeError(f"{op}: beta must be torch.bfloat16 or torch.float32.")
        elif t.dtype != want[name]:
            raise RuntimeError(f"{op}: {name} must be {want[name]}.")
        if not t.is_contiguous():
            raise RuntimeError(f"{op}: {name} must be contiguous; implicit copies are disabled.")
    if cu_seqlens is not None and layout == "BNSD":
        raise RuntimeError(f"{op}: varlen supports TND or BSND, not BNSD.")
    if cu_seqlens is None and layout == "TND":
        raise RuntimeError(f"{op}: TND requires cu_seqlens.")
    rt.reject_requires_grad(op, dq=dq, dk=dk, db=db, dg=dg)

    def view(t):     # -> [B, T, H, .] (3-D gate tensors: [B, T, H])
        if layout == "TND":
            return t.unsqueeze(0)
        return t.transpose(1, 2) if layout == "BNSD" else t

    v = {n: view(t) for n, t in tensors.items()}
    B, T, H, K = v["q"].shape
    if K != 128:
        raise NotImplementedError(f"{op}: this build supports K = 128, got {K}")
    dev = q.device
    cu = co = None
    max_len, total_chunks = T, B * ((T + CHUNK - 1) // CHUNK)
    if cu_seqlens is not None:
        if B != 1:
            raise RuntimeError(f"{op}: varlen BSND compatibility requires B=1.")
        cu, co, max_len, total_chunks, _n, total = _varlen_meta(cu_seqlens, dev)
        if total != T:
            raise RuntimeError(f"{op}: cu_seqlens must start at 0 and end at T.")
    a = ChunkKdaBwdIntraArgs()
    a.q, a.k, a.gk, a.beta = rt.desc(v["q"]), rt.desc(v["k"]), rt.desc(v["gk"]), rt.desc(v["beta"])
    a.d_aqk, a.d_akk = rt.desc(v["dAqk"]), rt.desc(v["dAkk"])
    a.dq, a.dk, a.db, a.dg = rt.desc(v["dq"]), rt.desc(v["dk"]), rt.desc(v["db"]), rt.desc(v["dg"])
    a.cu_seqlens, a.chunk_offsets = rt.desc(cu), rt.desc(co)
    a.chunk_size, a.max_seqlen, a.total_chunks = CHUNK, int(max_len), int(total_chunks)
    rt.call("chunk_kda_bwd_intra", a, list(tensors.values()) + [cu, co])
    rt.mark_mutated(dq, dk, db, dg)
    return dq, dk, db, dg


npu_chunk_kda_bwd_intra = chunk_kda_bwd_intra
npu_prepare_wy_repr_bwd = prepare_wy_repr_bwd
npu_prepare_wy_repr_bwd_da = prepare_wy_repr_bwd_da
npu_prepare_wy_repr_bwd_full = prepare_wy_repr_bwd_full
npu_chunk_bwd_dqkwg = chunk_bwd_dqkwg
npu_kda_gate_cumsum = kda_gate_cumsum
npu_chunk_bwd_dv_local = chunk_bwd_dv_local
npu_chunk_gated_delta_rule_bwd_dhu = chunk_gated_delta_rule_bwd_dhu
npu_chunk_local_cumsum = chunk_local_cumsum
npu_chunk_scaled_dot_kkt = chunk_scaled_dot_kkt
npu_solve_tri = solve_tri
npu_recompute_w_u_fwd = recompute_w_u_fwd
npu_chunk_gated_delta_rule_fwd_h = chunk_gated_delta_rule_fwd_h
npu_chunk_fwd_o = chunk_fwd_o

"""Oracle for the stand-alone forward stages (test infrastructure only; never imported by the shipped package).

CPU restatements of the reference's per-operator goldens, on head-first `[B,H,T,D]` tensors, computed in fp64:
  chunk_local_cumsum    torch_custom/fla_npu/test/test_npu_chunk_local_cumsum.py:44-72
  chunk_scaled_dot_kkt  torch_custom/fla_npu/test/test_npu_chunk_scaled_dot_kkt.py:60-103
  solve_tri             torch_custom/fla_npu/test/test_npu_solve_tri_ascend910b.py:48-89
  recompute_w_u_fwd     torch_custom/fla_npu/test/test_npu_recompute_w_u_fwd.py:38-145
  fwd_h                 tests/atk/chunk_gated_delta_rule_fwd_h/executor_chunk_gated_delta_rule_fwd_h.py:75-126
                        ("fp64" mode), extended with an initial state and the final state the reference omits
  fwd_o                 fla/ops/ascendc/gdn/chunk_gdn_fwd/chunk_fwd_o/tests/pta/test_fwd_o.py:42-117
  dv_local              fla/ops/ascendc/gdn/chunk_gdn_bwd/chunk_bwd_dv_local/tests/ATK/executor_chunk_bwd_dv_local.py:57-130
  bwd_dhu               torch_custom/fla_npu/test/test_bwd_dhu.py:61-290 ("fp64" mode), extended with the cotangent of the
                        final state (the reference deletes `dht`) and a `[N,HV,K,V]` dh0
  dqkwg                 tests/atk/chunk_bwd_dqkwg/scripts/chunk_bwd_dqkwg_cpu.py:66-409 (benchmark = fp64 mode)
  wy bwd (dA)           torch_custom/fla_npu/test/test_npu_prepare_wy_repr_bwd_da.py:165-291
  wy bwd (dk,dv,dg,db)  torch_custom/fla_npu/test/test_npu_prepare_wy_repr_bwd_full.py:95-486 (the *_high_precision goldens)
Pinned by tests/golden/stages_golden.npz, which tests/golden/make_golden.py produces by running those reference
functions themselves.
"""
from __future__ import annotations

import torch


def chunk_ranges(T, chunk_size, cu_seqlens=None):
    """(start, end) of every chunk; chunks restart at each sequence boundary of `cu_seqlens`."""
    bounds = [0, T] if cu_seqlens is None else [int(x) for x in cu_seqlens]
    out = []
    for bos, eos in zip(bounds[:-1], bounds[1:]):
        for s in range(bos, eos, chunk_size):
            out.append((s, min(s + chunk_size, eos)))
    return out


def sequence_chunk_ranges(T, chunk_size, cu_seqlens=None):
    """Per sequence: the list of its chunks' (start, end)."""
    bounds = [0, T] if cu_seqlens is None else [int(x) for x in cu_seqlens]
    return [[(s, min(s + chunk_size, eos)) for s in range(bos, eos, chunk_size)] for bos, eos in zip(bounds[:-1], bounds[1:])]


def chunk_local_cumsum_ref(g, chunk_size, reverse=False, scale=1.0, cu_seqlens=None):
    """g [B,H,T] or [B,H,T,D] -> chunk-local (reverse) cumulative sum times scale, fp64."""
    g = g.double()
    out = torch.zeros_like(g)
    for s, e in chunk_ranges(g.shape[2], chunk_size, cu_seqlens):
        seg = g[:, :, s:e]
        out[:, :, s:e] = (seg.flip(2).cumsum(2).flip(2) if reverse else seg.cumsum(2)) * scale
    return out


def chunk_scaled_dot_kkt_ref(k, g, beta, chunk_size, cu_seqlens=None):
    """k [B,HK,T,K], g (chunk-local cumulative gate), beta [B,HV,T] -> A [B,HV,T,C]: strictly lower part of
    beta_i exp(clamp(g_i - g_j, -50, 50)) k_i.k_j per chunk."""
    B, HK, T, _ = k.shape
    HV = g.shape[1]
    kk = k.double().repeat_interleave(HV // HK, dim=1)
    g, beta = g.double(), beta.double()
    out = torch.zeros(B, HV, T, chunk_size, dtype=torch.float64)
    for s, e in chunk_ranges(T, chunk_size, cu_seqlens):
        n = e - s
        score = kk[:, :, s:e] @ kk[:, :, s:e].transpose(-1, -2)
        gate = torch.exp(torch.clamp(g[:, :, s:e, None] - g[:, :, None, s:e], -50.0, 50.0))
        val = score * gate * beta[:, :, s:e, None]
        out[:, :, s:e, :n] = torch.tril(val, diagonal=-1)
    return out


def solve_tri_ref(A, chunk_size, cu_seqlens=None):
    """A [B,H,T,C] -> per chunk inverse of I + strict_lower(A[:n, :n]); columns past a short chunk stay zero."""
    A = A.double()
    out = torch.zeros_like(A)
    for s, e in chunk_ranges(A.shape[2], chunk_size, cu_seqlens):
        n = e - s
        M = torch.eye(n, dtype=torch.float64) + torch.tril(A[:, :, s:e, :n], diagonal=-1)
        out[:, :, s:e, :n] = torch.linalg.inv(M)
    return out


def recompute_w_u_ref(k, v, beta, A, g, chunk_size, cu_seqlens=None):
    """w = A (k beta e^g), u = A (v beta) per chunk.  k [B,HK,T,K]; v [B,HV,T,V]; A [B,HV,T,C]; beta, g [B,HV,T]."""
    B, HV, T, V = v.shape
    HK = k.shape[1]
    kk = k.double().repeat_interleave(HV // HK, dim=1)
    v, beta, A, g = v.double(), beta.double(), A.double(), g.double()
    w = torch.zeros(B, HV, T, k.shape[3], dtype=torch.float64)
    u = torch.zeros(B, HV, T, V, dtype=torch.float64)
    for s, e in chunk_ranges(T, chunk_size, cu_seqlens):
        n = e - s
        Ac = A[:, :, s:e, :n]
        w[:, :, s:e] = Ac @ (kk[:, :, s:e] * (beta[:, :, s:e] * torch.exp(g[:, :, s:e]))[..., None])
        u[:, :, s:e] = Ac @ (v[:, :, s:e] * beta[:, :, s:e, None])
    return w, u


def chunk_fwd_h_ref(k, w, u, g, chunk_size, initial_state=None, cu_seqlens=None):
    """Sequential state pass in fp64.  Returns (h [B,HV,NT,K,V] = state at the start of every chunk,
    v_new [B,HV,T,V], final_state [N,HV,K,V])."""
    B, HV, T, V = u.shape
    HK, K = k.shape[1], k.shape[3]
    kk = k.double().repeat_interleave(HV // HK, dim=1)
    w, u, g = w.double(), u.double(), g.double()
    seqs = sequence_chunk_ranges(T, chunk_size, cu_seqlens)
    nt_total = sum(len(s) for s in seqs)
    packed = cu_seqlens is not None
    N = len(seqs) if packed else B
    h = torch.zeros(B, HV, nt_total, K, V, dtype=torch.float64)
    v_new = torch.zeros(B, HV, T, V, dtype=torch.float64)
    final = torch.zeros(N, HV, K, V, dtype=torch.float64)
    ci = 0
    for si, chunks in enumerate(seqs):
        rows = [0] if packed else list(range(B))
        state = torch.zeros(len(rows), HV, K, V, dtype=torch.float64)
        if initial_state is not None:
            state = initial_state.double()[[si] if packed else rows].clone()
        for (s, e) in chunks:
            h[rows, :, ci] = state
            cur = u[rows, :, s:e] - w[rows, :, s:e] @ state
            v_new[rows, :, s:e] = cur
            gl = g[rows, :, e - 1]
            decay = torch.exp(gl[..., None] - g[rows, :, s:e])[..., None]
            state = state * torch.exp(gl)[..., None, None] + kk[rows, :, s:e].transpose(-1, -2) @ (cur * decay)
            ci += 1
        if packed:
            final[si] = state[0]
        else:
            final[:] = state
    return h, v_new, final


def chunk_fwd_o_ref(q, k, v, h, g, scale, chunk_size, cu_seqlens=None):
    """o = scale (e^{g_i} q h_c + tril(q k^T e^{g_i - g_j}) v) per chunk, fp64.  h [B,HV,NT,K,V] indexed by the running
    chunk number."""
    B, HV, T, V = v.shape
    HK = k.shape[1]
    qq = q.double().repeat_interleave(HV // HK, dim=1)
    kk = k.double().repeat_interleave(HV // HK, dim=1)
    v, h, g = v.double(), h.double(), g.double()
    o = torch.zeros(B, HV, T, V, dtype=torch.float64)
    for ci, (s, e) in enumerate(chunk_ranges(T, chunk_size, cu_seqlens)):
        attn = qq[:, :, s:e] @ kk[:, :, s:e].transpose(-1, -2)
        attn = torch.tril(attn * torch.exp(g[:, :, s:e, None] - g[:, :, None, s:e]))
        inter = (qq[:, :, s:e] * torch.exp(g[:, :, s:e])[..., None]) @ h[:, :, ci]
        o[:, :, s:e] = (inter + attn @ v[:, :, s:e]) * scale
    return o


def chunk_bwd_dv_local_ref(q, k, d_o, g, scale, chunk_size, cu_seqlens=None):
    """dv_j = sum_{i >= j in chunk} scale (k_j.q_i) e^{g_i - g_j} d_o_i, fp64."""
    B, HV, T, V = d_o.shape
    HK = k.shape[1]
    qq = q.double().repeat_interleave(HV // HK, dim=1)
    kk = k.double().repeat_interleave(HV // HK, dim=1)
    d_o, g = d_o.double(), g.double()
    dv = torch.zeros(B, HV, T, V, dtype=torch.float64)
    for s, e in chunk_ranges(T, chunk_size, cu_seqlens):
        A = kk[:, :, s:e] @ qq[:, :, s:e].transpose(-1, -2) * scale            # [j, i]
        A = torch.triu(A * torch.exp(g[:, :, None, s:e] - g[:, :, s:e, None]))  # i >= j
        dv[:, :, s:e] = A @ d_o[:, :, s:e]
    return dv


def chunk_bwd_dhu_ref(q, k, w, d_o, dv, g, scale, chunk_size, dht=None, cu_seqlens=None):
    """Reverse state pass in fp64.  Returns (dh [B,HV,NT,K,V] = dS at the end of every chunk, dh0 [N,HV,K,V], dv2)."""
    B, HV, T, V = dv.shape
    HK, K = k.shape[1], k.shape[3]
    qq = q.double().repeat_interleave(HV // HK, dim=1)
    kk = k.double().repeat_interleave(HV // HK, dim=1)
    w, d_o, dv, g = w.double(), d_o.double(), dv.double(), g.double()
    seqs = sequence_chunk_ranges(T, chunk_size, cu_seqlens)
    nt_total = sum(len(s) for s in seqs)
    packed = cu_seqlens is not None
    N = len(seqs) if packed else B
    dh = torch.zeros(B, HV, nt_total, K, V, dtype=torch.float64)
    dv2 = torch.zeros(B, HV, T, V, dtype=torch.float64)
    dh0 = torch.zeros(N, HV, K, V, dtype=torch.float64)
    base = 0
    for si, chunks in enumerate(seqs):
        rows = [0] if packed else list(range(B))
        dS = torch.zeros(len(rows), HV, K, V, dtype=torch.float64)
        if dht is not None:
            dS = dht.double()[[si] if packed else rows].clone()
        for ci in range(len(chunks) - 1, -1, -1):
            s, e = chunks[ci]
            dh[rows, :, base + ci] = dS
            gl = g[rows, :, e - 1]
            cur = dv[rows, :, s:e] + torch.exp(gl[..., None] - g[rows, :, s:e])[..., None] * (kk[rows, :, s:e] @ dS)
            dv2[rows, :, s:e] = cur
            qg = qq[rows, :, s:e] * torch.exp(g[rows, :, s:e])[..., None]
            dS = dS * torch.exp(gl)[..., None, None] + scale * qg.transpose(-1, -2) @ d_o[rows, :, s:e] \
                - w[rows, :, s:e].transpose(-1, -2) @ cur
        if packed:
            dh0[si] = dS[0]
        else:
            dh0[:] = dS
        base += len(chunks)
    return dh, dh0, dv2


def chunk_bwd_dqkwg_ref(q, k, v, g, h, d_o, dh, dv, scale, chunk_size, cu_seqlens=None):
    """dq, dk [B,HK,T,K] (summed over each group's value heads), dw [B,HV,T,K], dg [B,HV,T] (before the reverse cumulative
    sum; the last row of a chunk carries e^{g_last} <h, dh> + sum_i k_i.dk_state_i), fp64."""
    B, HV, T, V = v.shape
    HK, K = k.shape[1], k.shape[3]
    G = HV // HK
    qq = q.double().repeat_interleave(G, dim=1)
    kk = k.double().repeat_interleave(G, dim=1)
    v, g, h, d_o, dh, dv = (t.double() for t in (v, g, h, d_o, dh, dv))
    dq = torch.zeros(B, HV, T, K, dtype=torch.float64)
    dk = torch.zeros_like(dq)
    dw = torch.zeros_like(dq)
    dg = torch.zeros(B, HV, T, dtype=torch.float64)
    for ci, (s, e) in enumerate(chunk_ranges(T, chunk_size, cu_seqlens)):
        gc, gl = g[:, :, s:e], g[:, :, e - 1]
        hc, dhc = h[:, :, ci], dh[:, :, ci]
        dq_state = (d_o[:, :, s:e] @ hc.transpose(-1, -2)) * torch.exp(gc)[..., None] * scale
        dk_state = (v[:, :, s:e] @ dhc.transpose(-1, -2)) * torch.exp(gl[..., None] - gc)[..., None]
        dw[:, :, s:e] = -(dv[:, :, s:e] @ hc.transpose(-1, -2))
        ds = torch.tril(d_o[:, :, s:e] @ v[:, :, s:e].transpose(-1, -2) * torch.exp(gc[..., :, None] - gc[..., None, :])) * scale
        ds2 = ds * (qq[:, :, s:e] @ kk[:, :, s:e].transpose(-1, -2))
        dgc = (dq_state * qq[:, :, s:e]).sum(-1) - (kk[:, :, s:e] * dk_state).sum(-1) + ds2.sum(-1) - ds2.sum(-2)
        dgc[:, :, -1] += (hc * dhc).sum((-1, -2)) * torch.exp(gl) + (dk_state * kk[:, :, s:e]).sum((-1, -2))
        dg[:, :, s:e] = dgc
        dq[:, :, s:e] = dq_state + ds @ kk[:, :, s:e]
        dk[:, :, s:e] = dk_state + ds.transpose(-1, -2) @ qq[:, :, s:e]
    return dq.view(B, HK, G, T, K).sum(2), dk.view(B, HK, G, T, K).sum(2), dw, dg


def prepare_wy_repr_bwd_ref(k, v, beta, A, dw, du, g, chunk_size, cu_seqlens=None, dA=None):
    """Backward of w = A (k beta e^g), u = A (v beta) in fp64.  Returns (dA stored transposed per chunk [B,HV,T,C],
    dk [B,HK,T,K] summed over groups, dv, dbeta, dg).  With `dA` given (transposed storage) it is used instead of the computed one."""
    B, HV, T, V = v.shape
    HK, K = k.shape[1], k.shape[3]
    G = HV // HK
    kk = k.double().repeat_interleave(G, dim=1)
    v, beta, A, dw, du, g = (t.double() for t in (v, beta, A, dw, du, g))
    dA_out = torch.zeros(B, HV, T, chunk_size, dtype=torch.float64)
    dk = torch.zeros(B, HV, T, K, dtype=torch.float64)
    dv = torch.zeros(B, HV, T, V, dtype=torch.float64)
    dbeta = torch.zeros(B, HV, T, dtype=torch.float64)
    dg = torch.zeros(B, HV, T, dtype=torch.float64)
    for s, e in chunk_ranges(T, chunk_size, cu_seqlens):
        n = e - s
        X = A[:, :, s:e, :n]
        kc, vc, bc, gc = kk[:, :, s:e], v[:, :, s:e], beta[:, :, s:e], g[:, :, s:e]
        eg = torch.exp(gc)
        kbg = kc * (bc * eg)[..., None]
        vb = vc * bc[..., None]
        if dA is None:
            P = torch.tril(dw[:, :, s:e] @ kbg.transpose(-1, -2) + du[:, :, s:e] @ vb.transpose(-1, -2), diagonal=-1)
            P6 = X.transpose(-1, -2) @ (P @ X.transpose(-1, -2))
            M = torch.tril(-P6 * torch.exp(gc[..., :, None] - gc[..., None, :]), diagonal=-1)
        else:
            M = torch.tril(dA.double()[:, :, s:e, :n].transpose(-1, -2), diagonal=-1)
        dA_out[:, :, s:e, :n] = M.transpose(-1, -2)
        dkbg = X.transpose(-1, -2) @ dw[:, :, s:e]
        dvb = X.transpose(-1, -2) @ du[:, :, s:e]
        dv[:, :, s:e] = dvb * bc[..., None]
        T1 = M @ kc
        dk[:, :, s:e] = M.transpose(-1, -2) @ (kc * bc[..., None]) + T1 * bc[..., None] + dkbg * (bc * eg)[..., None]
        kd = (dkbg * kc).sum(-1)
        dbeta[:, :, s:e] = (T1 * kc).sum(-1) + eg * kd + (dvb * vc).sum(-1)
        W = M * (kc @ kc.transpose(-1, -2)) * bc[..., None]
        dg[:, :, s:e] = bc * eg * kd + W.sum(-1) - W.sum(-2)
    return dA_out, dk.view(B, HK, G, T, K).sum(2), dv, dbeta, dg

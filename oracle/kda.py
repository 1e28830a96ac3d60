"""KDA oracle (test infrastructure only).

`naive_recurrent_kda` follows the reference's per-token loop
(tests/atk/recurrent_kda/executor_recurrent_kda.py:63-83), vectorised over batch and heads and
with the state kept K-first ([B,HV,K,V]) like the chunk operators' initial/final state:
    S <- diag(exp(g_t)) S;  d = beta_t (v_t - S^T k_t);  S <- S + k_t d^T;  o_t = S^T (scale q_t)
The reference has no KDA backward of its own (it defers to a third-party Triton package that is
not part of its tree), so gradients are pinned by autograd through this recurrence.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def naive_recurrent_kda(q, k, v, g, beta, *, scale, initial_state=None, dtype=torch.float32):
    """q,k [B,T,H,K]; v [B,T,H,V]; g [B,T,H,K] (log decay per channel); beta [B,T,H]; H = HV."""
    q, k, v, g, beta = [x.to(dtype) for x in (q, k, v, g, beta)]
    B, T, H, K = q.shape
    V = v.shape[-1]
    state = q.new_zeros(B, H, K, V) if initial_state is None else initial_state.to(dtype)
    outs = []
    for t in range(T):
        state = state * g[:, t].exp()[..., None]
        k_t = k[:, t]
        delta = beta[:, t][..., None] * (v[:, t] - torch.einsum("bhkv,bhk->bhv", state, k_t))
        state = state + k_t[..., None] * delta[..., None, :]
        outs.append(torch.einsum("bhkv,bhk->bhv", state, q[:, t] * scale))
    return torch.stack(outs, dim=1), state


def kda_reference_fwd_bwd(q, k, v, g, beta, *, scale=None, initial_state=None, do=None, dht=None,
                          use_qk_l2norm=False, dtype=torch.float32):
    """Forward (+ autograd backward) through the naive KDA recurrence; GVA by repeat_interleave."""
    HK, HV = q.shape[2], v.shape[2]
    rep = HV // HK
    K = q.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    need_grad = do is not None
    leaves = {}
    for name, t in (("q", q), ("k", k), ("v", v), ("g", g), ("beta", beta), ("h0", initial_state)):
        leaves[name] = None if t is None else t.detach().to(dtype).clone().requires_grad_(need_grad)
    q_i, k_i = leaves["q"], leaves["k"]
    if use_qk_l2norm:
        q_i, k_i = F.normalize(q_i, p=2, dim=-1), F.normalize(k_i, p=2, dim=-1)
    if rep != 1:
        q_i, k_i = q_i.repeat_interleave(rep, dim=2), k_i.repeat_interleave(rep, dim=2)
    o, ht = naive_recurrent_kda(q_i, k_i, leaves["v"], leaves["g"], leaves["beta"], scale=scale,
                                initial_state=leaves["h0"], dtype=dtype)
    res = {"o": o.detach(), "ht": ht.detach()}
    if need_grad:
        loss = (o * do.to(dtype)).sum()
        if dht is not None:
            loss = loss + (ht * dht.to(dtype)).sum()
        loss.backward()
        res.update(dq=leaves["q"].grad, dk=leaves["k"].grad, dv=leaves["v"].grad, dg=leaves["g"].grad,
                   dbeta=leaves["beta"].grad, dh0=None if leaves["h0"] is None else leaves["h0"].grad)
    return res


def kda_chunk_score_blocks_ref(q, k, g, beta, scale, cu_seqlens=None, chunk_size=64):
    """Per-chunk score blocks of the chunked KDA forward in fp64, `[B,T,H,.]` inputs (g = log decay per channel):
        gk  = chunk-local cumsum(g) / ln 2                                  [B,HV,T,K]
        Aqk = scale * tril(q k^T 2^{gk_i-gk_j})                              [B,HV,T,chunk]
        Akk = (I + beta_i strict_tril(k k^T 2^{gk_i-gk_j}))^-1               [B,HV,T,chunk]
    Restates the score / inverse part of the reference's chunked golden
    (tests/atk/chunk_kda_fwd/executor_chunk_kda_fwd.py:361-399 `_stable_causal_scores`, :455-468) without its 16-row
    anchoring, which only matters in float32."""
    import math
    C = chunk_size
    B, T, HK, K = q.shape
    HV = beta.shape[2]
    G = HV // HK
    qq = q.double().repeat_interleave(G, dim=2).permute(0, 2, 1, 3)
    kk = k.double().repeat_interleave(G, dim=2).permute(0, 2, 1, 3)
    gg = g.double().permute(0, 2, 1, 3)
    bb = beta.double().permute(0, 2, 1)
    aqk = torch.zeros(B, HV, T, C, dtype=torch.float64)
    akk = torch.zeros_like(aqk)
    gk = torch.zeros_like(gg)
    bounds = [0, T] if cu_seqlens is None else [int(x) for x in cu_seqlens]
    for bos, eos in zip(bounds[:-1], bounds[1:]):
        for s in range(bos, eos, C):
            e = min(s + C, eos)
            n = e - s
            gc = gg[:, :, s:e].cumsum(2) / math.log(2.0)
            gk[:, :, s:e] = gc
            D = torch.exp2(gc[:, :, :, None, :] - gc[:, :, None, :, :]) * torch.tril(torch.ones(n, n, dtype=torch.float64))[..., None]
            qk = torch.einsum("bhik,bhijk,bhjk->bhij", qq[:, :, s:e], D, kk[:, :, s:e]) * scale
            kkm = torch.einsum("bhik,bhijk,bhjk->bhij", kk[:, :, s:e], D, kk[:, :, s:e])
            lhs = torch.tril(kkm * bb[:, :, s:e, None], diagonal=-1) + torch.eye(n, dtype=torch.float64)
            aqk[:, :, s:e, :n] = qk
            akk[:, :, s:e, :n] = torch.linalg.inv(lhs)
    return aqk, akk, gk


def kda_chunk_intermediates_ref(q, k, v, g, beta, scale, initial_state=None, cu_seqlens=None, chunk_size=64):
    """The chunked KDA forward with every intermediate in fp64, `[B,T,H,.]` inputs (g = log decay per channel), head-first results:
        gk (base 2), qg = q 2^{gk}, kg = k 2^{gk_last - gk}, w = Akk (beta k 2^{gk}), u = Akk (beta v)       [B,HV,T,.]
        v_new = u - w S, S <- 2^{gk_last} S + kg^T v_new, o = scale qg S + Aqk v_new;  h = S at the start of every chunk  [chunks,HV,K,V]
    Restates the chunk loop of the reference's chunked golden (tests/atk/chunk_kda_fwd/executor_chunk_kda_fwd.py:447-492)
    on top of `kda_chunk_score_blocks_ref` (its score blocks), for any chunk size."""
    C = chunk_size
    B, T, HK, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    G = HV // HK
    aqk, akk, gk = kda_chunk_score_blocks_ref(q, k, g, beta, scale, cu_seqlens, C)
    qq = q.double().repeat_interleave(G, dim=2).permute(0, 2, 1, 3)
    kk = k.double().repeat_interleave(G, dim=2).permute(0, 2, 1, 3)
    vv = v.double().permute(0, 2, 1, 3)
    bb = beta.double().permute(0, 2, 1)
    out = {n: torch.zeros(B, HV, T, d, dtype=torch.float64) for n, d in (("w", K), ("u", V), ("qg", K), ("kg", K), ("v_new", V), ("o", V))}
    bounds = [0, T] if cu_seqlens is None else [int(x) for x in cu_seqlens]
    nseq = len(bounds) - 1
    N = B if cu_seqlens is None else nseq
    state = torch.zeros(N, HV, K, V, dtype=torch.float64) if initial_state is None else initial_state.double().clone()
    hs = []
    for b in range(B):
        for si, (bos, eos) in enumerate(zip(bounds[:-1], bounds[1:])):
            n_idx = b if cu_seqlens is None else si
            for s in range(bos, eos, C):
                e = min(s + C, eos)
                n = e - s
                gc = gk[b, :, s:e]                                               # [HV, n, K], base 2
                eg = torch.exp2(gc)
                qg = qq[b, :, s:e] * eg
                kg = kk[b, :, s:e] * torch.exp2(gc[:, -1:, :] - gc)
                A = akk[b, :, s:e, :n]
                w = A @ (kk[b, :, s:e] * bb[b, :, s:e, None] * eg)
                u = A @ (vv[b, :, s:e] * bb[b, :, s:e, None])
                S = state[n_idx]
                hs.append(S.clone())
                vn = u - w @ S
                out["o"][b, :, s:e] = scale * (qg @ S) + aqk[b, :, s:e, :n] @ vn
                state[n_idx] = torch.exp2(gc[:, -1, :]).unsqueeze(-1) * S + kg.transpose(1, 2) @ vn
                for name, val in (("w", w), ("u", u), ("qg", qg), ("kg", kg), ("v_new", vn)):
                    out[name][b, :, s:e] = val
    out.update(gk=gk, aqk=aqk, akk=akk, h=torch.stack(hs), final_state=state)
    return out


def chunk_kda_bwd_intra_ref(q, k, gk, beta, d_aqk, d_akk, dq, dk, db, dg, chunk_size=64, cu_seqlens=None):
    """Intra-chunk KDA backward accumulated onto dq, dk, db, dg (returns new tensors), fp64, `[B,T,H,.]` layout.
    Restates torch_custom/fla_npu/test/test_npu_chunk_kda_bwd_intra.py:7-91 without its 16-row anchoring (exact in fp64):
      dq_i += sum_{j<=i} dAqk[i][j] k_j 2^{g_i-g_j};  lower_i = sum_{j<=i} dAkk[i][j] k_j 2^{g_i-g_j};
      upper_j = sum_{i>=j} (dAqk[i][j] q_i + dAkk[i][j] beta_i k_i) 2^{g_i-g_j};
      dk_i += beta_i lower_i + upper_i;  db_i += lower_i.k_i;  dg_i += q_i dq_delta_i + k_i (beta_i lower_i - upper_i)."""
    q, k, gk, beta, d_aqk, d_akk = (t.double() for t in (q, k, gk, beta, d_aqk, d_akk))
    dq, dk, db, dg = (t.double().clone() for t in (dq, dk, db, dg))
    T = q.shape[1]
    bounds = [0, T] if cu_seqlens is None else [int(x) for x in cu_seqlens]
    for bos, eos in zip(bounds[:-1], bounds[1:]):
        for s in range(bos, eos, chunk_size):
            e = min(s + chunk_size, eos)
            n = e - s
            qc, kc, gc, bc = q[:, s:e], k[:, s:e], gk[:, s:e], beta[:, s:e]          # [B, n, H, K], [B, n, H]
            aqk = torch.tril(d_aqk[:, s:e, :, :n].permute(0, 2, 1, 3))               # [B, H, i, j]
            akk = torch.tril(d_akk[:, s:e, :, :n].permute(0, 2, 1, 3))
            gh = gc.permute(0, 2, 1, 3)                                              # [B, H, n, K]
            D = torch.exp2(gh[:, :, :, None, :] - gh[:, :, None, :, :]) * torch.tril(torch.ones(n, n, dtype=torch.float64))[..., None]
            kh, qh, bh = kc.permute(0, 2, 1, 3), qc.permute(0, 2, 1, 3), bc.permute(0, 2, 1)
            dq_delta = torch.einsum("bhij,bhijk,bhjk->bhik", aqk, D, kh)
            lower = torch.einsum("bhij,bhijk,bhjk->bhik", akk, D, kh)
            upper = torch.einsum("bhij,bhijk,bhik->bhjk", aqk, D, qh) + torch.einsum("bhij,bhijk,bhik->bhjk", akk, D, kh * bh[..., None])
            bl = bh[..., None] * lower
            dq[:, s:e] += dq_delta.permute(0, 2, 1, 3)
            dk[:, s:e] += (bl + upper).permute(0, 2, 1, 3)
            db[:, s:e] += (lower * kh).sum(-1).permute(0, 2, 1)
            dg[:, s:e] += (qh * dq_delta + kh * (bl - upper)).permute(0, 2, 1, 3)
    return dq, dk, db, dg

"""GDN oracle (test infrastructure only; never imported by the shipped package).

`naive_recurrent_gated_delta_rule` follows the reference's naive fp32 recurrence
(examples/flash_gated_delta_rule.py:1545-1571) and extends it with the two things the benchmark
configurations need and the reference version lacks: an `initial_state` and the final state as a
second return value.  `gdn_reference_fwd_bwd` follows the reference's autograd harness
(examples/flash_gated_delta_rule.py:1574-1631): GVA by repeat_interleave, optional q/k L2
normalisation, loss = sum(o * dO) (+ sum(ht * dht) for the final-state cotangent).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def naive_recurrent_gated_delta_rule(q, k, v, beta, g, *, scale, initial_state=None, dtype=torch.float32):
    """q,k [B,T,H,K]; v [B,T,H,V]; beta,g [B,T,H] (heads already expanded to H = HV).

    Returns (o [B,T,H,V], final_state [B,H,K,V]) in `dtype`.
    Per token: S <- exp(g) S;  d = beta (v - S^T k);  S <- S + k d^T;  o = S^T (scale q).
    """
    q, k, v, beta, g = [x.transpose(1, 2).contiguous().to(dtype) for x in (q, k, v, beta, g)]
    B, H, T, K = q.shape
    V = v.shape[-1]
    if initial_state is None:
        state = q.new_zeros(B, H, K, V)
    else:
        state = initial_state.to(dtype)
    outs = []
    q = q * scale
    for idx in range(T):
        q_i, k_i, v_i = q[:, :, idx], k[:, :, idx], v[:, :, idx]
        beta_i = beta[:, :, idx]
        decay = g[:, :, idx].exp()
        state = state * decay[..., None, None]
        delta_v = v_i - (state * k_i[..., None]).sum(-2)
        delta_v = delta_v * beta_i[..., None]
        state = state + k_i.unsqueeze(-1) * delta_v.unsqueeze(-2)
        outs.append(torch.einsum("bhd,bhdm->bhm", q_i, state))
    o = torch.stack(outs, dim=2)
    return o.transpose(1, 2).contiguous(), state


def gdn_reference_fwd_bwd(q, k, v, g, beta, *, scale=None, initial_state=None, do=None, dht=None,
                          use_qk_l2norm=False, dtype=torch.float32, cu_seqlens=None):
    """Forward (+ autograd backward when `do` is given) through the naive recurrence.

    Layouts follow the operator surface: q,k [B,T,HK,K]; v [B,T,HV,V]; g,beta [B,T,HV];
    initial_state [N,HV,K,V].  Inputs are used at their stored precision (bf16 inputs are upcast,
    so input rounding is not counted as error).  Returns a dict with o, ht and the gradients.
    """
    HK, HV = q.shape[2], v.shape[2]
    rep = HV // HK
    K = q.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    need_grad = do is not None
    leaves = {}
    for name, t in (("q", q), ("k", k), ("v", v), ("g", g), ("beta", beta), ("h0", initial_state)):
        if t is None:
            leaves[name] = None
        else:
            leaves[name] = t.detach().to(dtype).clone().requires_grad_(need_grad)

    def run(sl, h0):
        q_i, k_i = leaves["q"][:, sl], leaves["k"][:, sl]
        if use_qk_l2norm:
            q_i = F.normalize(q_i, p=2, dim=-1)
            k_i = F.normalize(k_i, p=2, dim=-1)
        if rep != 1:
            q_i = q_i.repeat_interleave(rep, dim=2)
            k_i = k_i.repeat_interleave(rep, dim=2)
        return naive_recurrent_gated_delta_rule(q_i, k_i, leaves["v"][:, sl], leaves["beta"][:, sl],
                                                leaves["g"][:, sl], scale=scale, initial_state=h0, dtype=dtype)

    if cu_seqlens is None:
        o, ht = run(slice(None), leaves["h0"])
    else:
        outs, hts = [], []
        for i in range(len(cu_seqlens) - 1):
            h0 = None if leaves["h0"] is None else leaves["h0"][i:i + 1]
            o_i, ht_i = run(slice(int(cu_seqlens[i]), int(cu_seqlens[i + 1])), h0)
            outs.append(o_i)
            hts.append(ht_i)
        o, ht = torch.cat(outs, dim=1), torch.cat(hts, dim=0)
    res = {"o": o.detach(), "ht": ht.detach()}
    if need_grad:
        loss = (o * do.to(dtype)).sum()
        if dht is not None:
            loss = loss + (ht * dht.to(dtype)).sum()
        loss.backward()
        res.update(dq=leaves["q"].grad, dk=leaves["k"].grad, dv=leaves["v"].grad, dg=leaves["g"].grad,
                   dbeta=leaves["beta"].grad,
                   dh0=None if leaves["h0"] is None else leaves["h0"].grad)
    return res


def chunk_gated_delta_rule_restated(q, k, v, g, beta, *, scale=None, initial_state=None, chunk_size=64,
                                    dtype=torch.float64):
    """Chunked restatement of the forward, stage by stage, in the form the CUDA kernels use.

    Follows the reference's stage math (chunk_scaled_dot_kkt README:13-27, solve_tri README:9-13,
    chunk_gated_delta_rule_fwd_h README:20-27, chunk_fwd_o README:11-16) with the WY factors folded:
        gam   = chunk-local cumsum(g)
        A     = strict_tril(beta_i exp(gam_i - gam_j) k_i.k_j);  X = (I + A)^-1
        v_new = X (beta * (V - exp(gam) * (K S)))          [ = u - w S of the reference ]
        o     = scale (exp(gam) * (Q S) + tril(Q K^T * exp(gam_i - gam_j)) v_new)
        S'    = exp(gam_L) S + K^T (exp(gam_L - gam) * v_new)
    Single sequence per batch entry, T a multiple of chunk_size is NOT required (tail chunk is short).
    Returns o, final state, and per-chunk intermediates (gam, X, S_c, v_new) for kernel bisection.
    """
    B, T, HK, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    rep = HV // HK
    scale = K ** -0.5 if scale is None else scale
    C = chunk_size
    qf, kf, vf, gf, bf = [x.to(dtype) for x in (q, k, v, g, beta)]
    o = torch.zeros(B, T, HV, V, dtype=dtype)
    NT = (T + C - 1) // C
    S = torch.zeros(B, HV, K, V, dtype=dtype) if initial_state is None else initial_state.to(dtype).clone()
    gam_all = torch.zeros(B, T, HV, dtype=dtype)
    X_all = torch.zeros(B, T, HV, C, dtype=dtype)
    S_all = torch.zeros(B, NT, HV, K, V, dtype=dtype)
    vn_all = torch.zeros(B, T, HV, V, dtype=dtype)
    for c in range(NT):
        sl = slice(c * C, min((c + 1) * C, T))
        L = sl.stop - sl.start
        S_all[:, c] = S
        for hv in range(HV):
            hk = hv // rep
            qc, kc = qf[:, sl, hk], kf[:, sl, hk]            # [B,L,K]
            vc, bc = vf[:, sl, hv], bf[:, sl, hv]            # [B,L,V], [B,L]
            gam = gf[:, sl, hv].cumsum(1)                    # [B,L]
            dec = torch.exp(gam[:, :, None] - gam[:, None, :])
            A = torch.tril(bc[:, :, None] * dec * (kc @ kc.transpose(1, 2)), -1)
            X = torch.linalg.inv(torch.eye(L, dtype=dtype) + A)
            Sh = S[:, hv]
            Z = bc[:, :, None] * (vc - gam.exp()[:, :, None] * (kc @ Sh))
            vn = X @ Z
            P = torch.tril(qc @ kc.transpose(1, 2) * dec)
            o[:, sl, hv] = scale * (gam.exp()[:, :, None] * (qc @ Sh) + P @ vn)
            gl = gam[:, -1]
            S[:, hv] = gl.exp()[:, None, None] * Sh + kc.transpose(1, 2) @ (torch.exp(gl[:, None] - gam)[:, :, None] * vn)
            gam_all[:, sl, hv] = gam
            X_all[:, sl, hv, :L] = X
            vn_all[:, sl, hv] = vn
    return {"o": o, "ht": S, "gam": gam_all, "X": X_all, "S": S_all, "v_new": vn_all}

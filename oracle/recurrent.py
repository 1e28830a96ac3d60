"""Decode-step oracle (test infrastructure only).

Follows the reference's CPU golden for recurrent_gated_delta_rule
(fla/ops/ascendc/gdn/recurrent_gdn/recurrent_gated_delta_rule/tests/pta/golden.py:14-105):
state pool [blocks, NV, dv, dk] (V-first), `actual_seq_lengths[0]` is a skipped prefix and entries
1.. are per-sequence token counts, the start state of a sequence is
state[ssm_state_indices[seq0 (+ accepted - 1)]], and the state after token t is written to
state[ssm_state_indices[t]].  Unlike the golden, the arithmetic dtype and the output dtype are
parameters so fp32 state pools can be checked at the 1e-5 bar.
"""
from __future__ import annotations

from typing import Optional

import torch


def recurrent_gated_delta_rule_golden(query, key, value, state, beta, scale, actual_seq_lengths,
                                      ssm_state_indices, num_accepted_tokens: Optional[torch.Tensor] = None,
                                      g: Optional[torch.Tensor] = None, gk: Optional[torch.Tensor] = None,
                                      dtype=torch.float32, out_dtype=torch.bfloat16, state_out_dtype=None):
    T, NK, dk = query.shape
    _, NV, dv = value.shape
    nseq = actual_seq_lengths.shape[0]
    q_f = query.to(dtype) * scale
    k_f, v_f, beta_f = key.to(dtype), value.to(dtype), beta.to(dtype)
    alpha = torch.exp(g.to(dtype)) if g is not None else None
    alpha_k = torch.exp(gk.to(dtype)) if gk is not None else None
    attn_out = torch.zeros(T, NV, dv, dtype=dtype)
    final_state = state.to(dtype).clone()
    rep = NV // NK
    seq_ptr = int(actual_seq_lengths[0])
    for b in range(1, nseq):
        seq0, seq1 = seq_ptr, seq_ptr + int(actual_seq_lengths[b])
        seq_ptr = seq1
        tok = seq0
        if num_accepted_tokens is not None:
            tok = seq0 + int(num_accepted_tokens[b - 1]) - 1
        S = final_state[int(ssm_state_indices[tok])].clone()          # [NV, dv, dk]
        for t in range(seq0, seq1):
            k_h = k_f[t].repeat_interleave(rep, dim=0)                 # [NV, dk]
            q_h = q_f[t].repeat_interleave(rep, dim=0)
            if alpha is not None:
                S = S * alpha[t][:, None, None]
            if alpha_k is not None:
                S = S * alpha_k[t][:, None, :]
            delta = (v_f[t] - torch.einsum("hvk,hk->hv", S, k_h)) * beta_f[t][:, None]
            S = S + delta[:, :, None] * k_h[:, None, :]
            attn_out[t] = torch.einsum("hvk,hk->hv", S, q_h)
            final_state[int(ssm_state_indices[t])] = S
    return attn_out.to(out_dtype), final_state.to(state_out_dtype or state.dtype)

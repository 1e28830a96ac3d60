"""A Gated-DeltaNet token-mixing block on the B200 operators.

The block of the reference's example (DemoGatedDeltaNet, examples/flash_gated_delta_rule.py:1249-1365): input
projections -> depthwise causal conv (SiLU) over [q | k | v] -> chunked gated delta rule with q/k l2-normalised
in the kernel -> gated RMSNorm -> output projection.  The projections and the norm are plain PyTorch (cuBLAS and
element-wise work outside the hot path); the conv and the delta rule are this package's kernels, used through
their differentiable operators.  q, k, v are strided views of the conv output: no repeat of q/k for grouped value
heads and no `.contiguous()` copies, unlike the reference block.

`step` adds what the reference leaves to its serving stack: one decode token per sequence through
`causal_conv1d_update` and the fused-recurrent kernel over caches that `forward(..., return_caches=True)` filled.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops


class RMSNormGated(nn.Module):
    """RMSNorm over the value head dim times SiLU(gate) (QwenStyleRMSNormGated of the reference example, :1231-1246)."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()
        return (y * F.silu(gate.float())).to(x.dtype)


class GatedDeltaNetBlock(nn.Module):
    def __init__(self, hidden_size: int, *, num_value_heads: int, num_key_heads: int, head_dim: int = 128,
                 conv_kernel_dim: int = 4, rms_norm_eps: float = 1e-6):
        super().__init__()
        if num_value_heads % num_key_heads:
            raise ValueError("num_value_heads must be a multiple of num_key_heads")
        self.hidden_size, self.HV, self.HK, self.D = hidden_size, num_value_heads, num_key_heads, head_dim
        self.key_dim, self.value_dim = head_dim * num_key_heads, head_dim * num_value_heads
        self.W = conv_kernel_dim
        conv_dim = 2 * self.key_dim + self.value_dim
        self.conv_weight = nn.Parameter(torch.randn(conv_dim, conv_kernel_dim) * 0.5)     # [D, W]
        self.dt_bias = nn.Parameter(torch.ones(num_value_heads))
        self.A_log = nn.Parameter(torch.log(torch.rand(num_value_heads) * 15.99 + 0.01))
        self.in_proj_qkv = nn.Linear(hidden_size, conv_dim, bias=False)
        self.in_proj_z = nn.Linear(hidden_size, self.value_dim, bias=False)
        self.in_proj_b = nn.Linear(hidden_size, num_value_heads, bias=False)
        self.in_proj_a = nn.Linear(hidden_size, num_value_heads, bias=False)
        self.norm = RMSNormGated(head_dim, eps=rms_norm_eps)
        self.out_proj = nn.Linear(self.value_dim, hidden_size, bias=False)

    def _split(self, mixed: torch.Tensor):
        B, T = mixed.shape[:2]
        q = mixed[..., : self.key_dim].unflatten(-1, (self.HK, self.D))
        k = mixed[..., self.key_dim: 2 * self.key_dim].unflatten(-1, (self.HK, self.D))
        v = mixed[..., 2 * self.key_dim:].unflatten(-1, (self.HV, self.D))
        return q, k, v

    def _gates(self, x: torch.Tensor):
        beta = self.in_proj_b(x).sigmoid()
        g = -self.A_log.float().exp() * F.softplus(self.in_proj_a(x).float() + self.dt_bias.float())
        return g, beta

    def forward(self, hidden_states: torch.Tensor, cu_seqlens: Optional[torch.Tensor] = None, return_caches: bool = False):
        """hidden_states `[B,T,hidden]` bf16 (B = 1 with `cu_seqlens`).  Returns the block output, plus
        ``(conv_state [N,D,W-1], recurrent_state [N,HV,K,V] fp32)`` with ``return_caches``."""
        B, T, _ = hidden_states.shape
        mixed, conv_state = ops.causal_conv1d(self.in_proj_qkv(hidden_states), self.conv_weight.to(hidden_states.dtype),
                                              activation="silu", cu_seqlens=cu_seqlens, output_final_state=return_caches)
        q, k, v = self._split(mixed)
        g, beta = self._gates(hidden_states)
        o, state = ops.chunk_gated_delta_rule(q, k, v, g, beta.to(hidden_states.dtype), use_qk_l2norm_in_kernel=True,
                                              cu_seqlens=cu_seqlens, output_final_state=return_caches)
        z = self.in_proj_z(hidden_states).unflatten(-1, (self.HV, self.D))
        y = self.out_proj(self.norm(o, z).flatten(-2))
        return (y, (conv_state, state)) if return_caches else y

    @torch.no_grad()
    def step(self, hidden_states: torch.Tensor, caches: Tuple[torch.Tensor, torch.Tensor]) -> torch.Tensor:
        """One decode token per sequence: hidden_states `[N,hidden]`; the caches are updated in place."""
        conv_state, state = caches
        mixed = ops.causal_conv1d_update(self.in_proj_qkv(hidden_states), conv_state,
                                         weight=self.conv_weight.to(hidden_states.dtype), activation="silu")
        q, k, v = self._split(mixed.unsqueeze(1))
        g, beta = self._gates(hidden_states)
        o, _ = ops.fused_recurrent_gated_delta_rule(q, k, v, g=g.unsqueeze(1), beta=beta.to(hidden_states.dtype).unsqueeze(1),
                                                    initial_state=state, use_qk_l2norm_in_kernel=True,
                                                    inplace_final_state=True)
        z = self.in_proj_z(hidden_states).unflatten(-1, (self.HV, self.D))
        return self.out_proj(self.norm(o.squeeze(1), z).flatten(-2))

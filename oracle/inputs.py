"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations
(test infrastructure only).  Everything is generated on the CPU in fp32 and then rounded to the
storage dtype, so the oracle and the kernels consume the same rounded values.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def make_gdn_inputs(B, T, HK, HV, K=128, V=128, *, seed=1001, dtype=torch.bfloat16, h0_scale=0.1, with_grad=True):
    g_ = _gen(seed)
    q = F.normalize(torch.randn(B, T, HK, K, generator=g_), dim=-1).to(dtype)
    k = F.normalize(torch.randn(B, T, HK, K, generator=g_), dim=-1).to(dtype)
    v = torch.randn(B, T, HV, V, generator=g_).to(dtype)
    g = F.logsigmoid(torch.randn(B, T, HV, generator=g_)).to(dtype)
    beta = torch.sigmoid(torch.randn(B, T, HV, generator=g_)).to(dtype)
    h0 = (h0_scale * torch.randn(B, HV, K, V, generator=g_)).float() if h0_scale else None
    out = dict(q=q, k=k, v=v, g=g, beta=beta, h0=h0)
    if with_grad:
        out["do"] = torch.randn(B, T, HV, V, generator=g_).to(dtype)
        out["dht"] = (0.1 * torch.randn(B, HV, K, V, generator=g_)).float()
    return out


def make_kda_inputs(B, T, HK, HV, K=128, V=128, *, seed=1003, dtype=torch.bfloat16, with_grad=True):
    g_ = _gen(seed)
    q = F.normalize(torch.randn(B, T, HK, K, generator=g_), dim=-1).to(dtype)
    k = F.normalize(torch.randn(B, T, HK, K, generator=g_), dim=-1).to(dtype)
    v = torch.randn(B, T, HV, V, generator=g_).to(dtype)
    g = (F.logsigmoid(torch.randn(B, T, HV, K, generator=g_)) / 16).to(dtype)
    beta = torch.sigmoid(torch.randn(B, T, HV, generator=g_)).to(dtype)
    out = dict(q=q, k=k, v=v, g=g, beta=beta, h0=None)
    if with_grad:
        out["do"] = torch.randn(B, T, HV, V, generator=g_).to(dtype)
    return out


def make_decode_inputs(N, HK, HV, K=128, V=128, *, seed=1004, tokens_per_seq=1, dtype=torch.bfloat16):
    g_ = _gen(seed)
    T = N * tokens_per_seq
    q = F.normalize(torch.randn(T, HK, K, generator=g_), dim=-1).to(dtype)
    k = F.normalize(torch.randn(T, HK, K, generator=g_), dim=-1).to(dtype)
    v = torch.randn(T, HV, V, generator=g_).to(dtype)
    g = F.logsigmoid(torch.randn(T, HV, generator=g_)).to(dtype)
    beta = torch.sigmoid(torch.randn(T, HV, generator=g_)).to(dtype)
    state = (0.1 * torch.randn(N, HV, K, V, generator=g_)).float()
    return dict(q=q, k=k, v=v, g=g, beta=beta, state=state)


def make_conv_inputs(B, T, D, W=4, *, seed=1001, dtype=torch.bfloat16, with_state=False):
    g_ = _gen(seed + 77)
    x = torch.randn(B, T, D, generator=g_).to(dtype)
    weight = (0.5 * torch.randn(D, W, generator=g_)).to(dtype)     # N(0, 1/4): variance 1/4, sigma 0.5
    bias = (0.1 * torch.randn(D, generator=g_)).to(dtype)
    out = dict(x=x, weight=weight, bias=bias)
    if with_state:
        out["state"] = torch.randn(B, D, W - 1, generator=g_).to(dtype)
    return out

"""The names the reference exports from its second operator package (`fla_npu.ops.triton`,
torch_custom/fla_npu/fla_npu/ops/triton/__init__.py:9-40; name list scripts/check_packaged_wheel_api.py:34-44), served by
the CUDA kernels of this library with that package's own layouts (sequence-first `[B,T,H,...]` gates and score blocks,
head-first `[B,HK,T,K]` keys for `chunk_scaled_dot_kkt_fwd`) and keyword names, so that
`from fla_npu.ops.triton import chunk_local_cumsum` becomes `from fla_b200.ops.upstream import chunk_local_cumsum`.
Not served: that package's `causal_conv1d` / `causal_conv1d_triton` (weight `[W,D]`, a head count argument, output re-laid
as `[B,H,T,D/H]` and a final state of W rather than W-1 inputs: fla/ops/triton/triton_core/causal_conv1d.py:720-880) --
the convolution of this library follows the operator `npu_causal_conv1d` instead (`fla_b200.ops.causal_conv1d`)."""
from __future__ import annotations

import functools

import torch

from . import stages as _st
from .l2norm import l2norm_bwd, l2norm_fwd  # noqa: F401


def chunk_local_cumsum(g, chunk_size, reverse=False, scale=None, cu_seqlens=None, chunk_indices_out=None, head_first=False,
                       output_dtype=torch.float, **kwargs):
    """fla/ops/triton/triton_core/cumsum.py:105-137: g `[B,T,H]` (`[B,H,T]` when `head_first`), 3-D only."""
    del chunk_indices_out, kwargs
    if cu_seqlens is not None and g.shape[0] != 1:
        raise ValueError(f"Only batch size 1 is supported when cu_seqlens are provided, current size is{g.shape[0]}")
    if g.dim() != 3:
        raise ValueError(f"Unsupported input shape {g.shape}, which should be (B, T, H, D) if `head_first=False` "
                         f"or (B, H, T, D) otherwise")
    return _st.chunk_local_cumsum(g, chunk_size, cu_seqlens=cu_seqlens, reverse=reverse, scale=1.0 if scale is None else scale,
                                  head_first=head_first, output_dtype=output_dtype or g.dtype)


chunk_local_cumsum_scalar = chunk_local_cumsum


def chunk_scaled_dot_kkt_fwd(k, g=None, gk=None, beta=None, cu_seqlens=None, chunk_indices=None, chunk_size=64,
                             output_dtype=torch.float32):
    """fla/ops/triton/triton_core/chunk_scaled_dot_kkt.py:325-360, with that function's own layouts: k is head-first
    `[B,HK,T,K]` (it unpacks `B, H_K, T, K = k.shape`, :359), g (chunk-local cumulative gate) and beta are `[B,T,HV]`
    -> A `[B,T,HV,chunk_size]`, `beta_i exp(clip(g_i - g_j, -50, 50)) k_i.k_j` strictly below the diagonal of every chunk
    (the reference kernel clamps the exponent the same way)."""
    del chunk_indices
    if gk is not None:
        raise NotImplementedError("chunk_scaled_dot_kkt_fwd: the per-channel gate gk is not supported")
    if beta is None:
        raise NotImplementedError("chunk_scaled_dot_kkt_fwd: beta is required")
    if k.dim() != 4 or beta.dim() != 3 or k.shape[0] != beta.shape[0] or k.shape[2] != beta.shape[1]:
        raise ValueError(f"chunk_scaled_dot_kkt_fwd: expected k [B, Hk, T, K] and beta [B, T, Hv], got {tuple(k.shape)} and "
                         f"{tuple(beta.shape)}")
    if beta.shape[-1] % k.shape[1] != 0:
        raise ValueError(f"Expected beta/g head count Hv to be a multiple of Hk, got Hk={k.shape[1]}, Hv={beta.shape[-1]}.")
    if g is None:
        g = torch.zeros(beta.shape, dtype=torch.float32, device=k.device)
    A = _st.chunk_scaled_dot_kkt(k, g.transpose(1, 2), beta.transpose(1, 2), cu_seqlens=cu_seqlens, chunk_size=chunk_size)
    A = A.transpose(1, 2)
    return A if output_dtype in (None, torch.float32) else A.to(output_dtype)


def solve_tril(A, cu_seqlens=None, chunk_indices_out=None, output_dtype=torch.float):
    """fla/ops/triton/triton_core/solve_tril_fast.py:613-634: `(I + A)^-1` per chunk, A `[B,T,H,64]` strictly lower."""
    del chunk_indices_out
    return _st.solve_tri(A, cu_seqlens=cu_seqlens, layout="bsnd", output_dtype=output_dtype)


solve_tril_npu = solve_tril


class _L2NormFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, eps, output_dtype):
        y, rstd = l2norm_fwd(x, eps, output_dtype)
        ctx.save_for_backward(y, rstd)
        ctx.eps, ctx.in_dtype = eps, x.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        y, rstd = ctx.saved_tensors
        return l2norm_bwd(y, rstd, dy.to(y.dtype).contiguous(), ctx.eps).to(ctx.in_dtype), None, None


def l2norm(x, eps=1e-6, output_dtype=None):
    """fla/ops/triton/triton_core/l2norm.py:261-266: `x * rsqrt(sum(x^2, -1) + eps)`, differentiable."""
    return _L2NormFunction.apply(x, eps, output_dtype)


l2_norm = l2norm


class L2Norm(torch.nn.Module):
    """fla/ops/triton/triton_core/l2norm.py:272-284."""

    def __init__(self, eps=1e-6, output_dtype=None):
        super().__init__()
        self.eps, self.output_dtype = eps, output_dtype

    def forward(self, x):
        return l2norm(x, self.eps, self.output_dtype)


def input_guard(fn):
    """fla/ops/triton/triton_core/utils.py: makes tensor arguments contiguous and runs `fn` on their device."""
    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        args = tuple(a.contiguous() if isinstance(a, torch.Tensor) else a for a in args)
        kwargs = {k: (v.contiguous() if isinstance(v, torch.Tensor) else v) for k, v in kwargs.items()}
        dev = next((a.device for a in list(args) + list(kwargs.values()) if isinstance(a, torch.Tensor)), None)
        if dev is not None and dev.type == "cuda":
            with torch.cuda.device(dev):
                return fn(*args, **kwargs)
        return fn(*args, **kwargs)
    return wrapper


autocast_custom_fwd = functools.partial(torch.amp.custom_fwd, device_type="cuda")
autocast_custom_bwd = functools.partial(torch.amp.custom_bwd, device_type="cuda")

__all__ = ["L2Norm", "autocast_custom_bwd", "autocast_custom_fwd", "chunk_local_cumsum",
           "chunk_local_cumsum_scalar", "chunk_scaled_dot_kkt_fwd", "input_guard", "l2norm", "l2norm_bwd", "l2norm_fwd",
           "solve_tril", "solve_tril_npu"]

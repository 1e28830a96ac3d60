"""fp16 tensors at the boundary of operators whose kernels multiply bf16 operands.

The reference's chunk and decode operators take fp16 as well as bf16 tensors and reject only fp32
(examples/flash_gated_delta_rule.py:1161-1162).  Here an fp16 tensor enters through the library's conversion kernel
(`fla_b200_convert`: rounded to bf16, 11 -> 8 significant bits) and results leave through it as fp16; gradients take the
same way back.  Nothing is cast through PyTorch."""
from __future__ import annotations

import ctypes

import torch

from .. import _runtime as rt
from .. import load_library


def convert(t: torch.Tensor, dtype: torch.dtype, op: str = "convert") -> torch.Tensor:
    """A dense copy of ``t`` (1 to 4 dims, innermost dim contiguous, any outer strides) in ``dtype``
    (float32 / bfloat16 / float16), made by the library's conversion kernel on the current stream."""
    if t.dim() < 1 or t.dim() > 4:
        raise RuntimeError(f"{op}: conversion takes 1 to 4 dims, got {t.dim()}")
    out = torch.empty(t.shape, dtype=dtype, device=t.device)
    if t.numel() == 0:
        return out
    if t.shape[-1] != 1 and t.stride(-1) != 1:
        t = t.contiguous()
    lib = load_library()
    rt._check_arch(t.device, op)
    src, dst = rt.desc(t), rt.desc(out)
    with torch.cuda.device(t.device):
        status = lib.fla_b200_convert(ctypes.byref(src), ctypes.byref(dst),
                                      ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream))
    if status != 0:
        raise RuntimeError(f"{op}: conversion {t.dtype} -> {dtype} failed with status={status}: "
                           f"{rt._STATUS_NAMES.get(status, '?')}")
    return out


class _ConvertFunction(torch.autograd.Function):
    """``convert`` with the gradient converted back to the source dtype."""

    @staticmethod
    def forward(ctx, t, dtype, op):
        ctx.src_dtype, ctx.op = t.dtype, op
        return convert(t, dtype, op)

    @staticmethod
    def backward(ctx, grad):
        return convert(grad, ctx.src_dtype, ctx.op), None, None


def to_dtype(t, dtype: torch.dtype, op: str = "convert"):
    """``t`` in ``dtype`` (differentiable); ``t`` itself when it already has that dtype or is None."""
    if t is None or t.dtype == dtype:
        return t
    return _ConvertFunction.apply(t, dtype, op)

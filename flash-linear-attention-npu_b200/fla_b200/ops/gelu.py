"""FastGELU operators of the reference surface (torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:224-239 and the
autograd binding torch_custom/fla_npu/fla_npu/ops/ascendc/__init__.py:270-296)."""
from __future__ import annotations

import ctypes

import torch

from .. import _runtime as rt
from .. import load_library
from ._structs import FastGeluArgs


def _call(fn_name, args, tensors):
    lib = load_library()
    dev = rt.common_device(tensors, fn_name)
    rt._check_arch(dev, fn_name)
    with torch.cuda.device(dev):
        status = getattr(lib, f"fla_b200_{fn_name}")(ctypes.byref(args),
                                                     ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    if status != 0:
        raise RuntimeError(f"{fn_name} failed with status={status}: {rt._STATUS_NAMES.get(status, '?')}")


def _flat(t, op):
    if t.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        raise TypeError(f"{op}: dtype must be float32, bfloat16 or float16, got {t.dtype}")
    return t.contiguous().view(-1)


def npu_fast_gelu_custom(self):
    """``self / (1 + exp(-1.702 * self))`` computed in fp32, returned in the dtype and shape of ``self``."""
    op = "npu_fast_gelu_custom"
    out = torch.empty(self.shape, dtype=self.dtype, device=self.device)
    if self.numel() == 0:
        return out
    x = _flat(self, op)
    a = FastGeluArgs()
    a.x, a.y = rt.desc(x), rt.desc(out.view(-1))
    _call("fast_gelu", a, [x, out])
    return out


def npu_fast_gelu_custom_backward(grad, self):
    """``grad * (s + 1.702 * self * s * (1 - s))`` with ``s = sigmoid(1.702 * self)``: the derivative of the forward."""
    op = "npu_fast_gelu_custom_backward"
    if grad.shape != self.shape or grad.dtype != self.dtype:
        raise RuntimeError(f"{op}: grad and self must have the same shape and dtype, got {tuple(grad.shape)} {grad.dtype} "
                           f"and {tuple(self.shape)} {self.dtype}")
    out = torch.empty(self.shape, dtype=self.dtype, device=self.device)
    if self.numel() == 0:
        return out
    x, g = _flat(self, op), _flat(grad, op)
    a = FastGeluArgs()
    a.x, a.dy, a.dx = rt.desc(x), rt.desc(g), rt.desc(out.view(-1))
    _call("fast_gelu_bwd", a, [x, g, out])
    return out


class _FastGeluCustomFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        ctx.save_for_backward(x)
        return npu_fast_gelu_custom(x)

    @staticmethod
    def backward(ctx, grad):
        (x,) = ctx.saved_tensors
        return npu_fast_gelu_custom_backward(grad.contiguous(), x)


def fast_gelu_custom(input_tensor):
    """FastGELU bound to its backward operator when the input requires a gradient."""
    if input_tensor.requires_grad and torch.is_grad_enabled():
        return _FastGeluCustomFunction.apply(input_tensor)
    return npu_fast_gelu_custom(input_tensor)

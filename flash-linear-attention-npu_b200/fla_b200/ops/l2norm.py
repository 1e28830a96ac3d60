"""Row-wise L2 normalisation kernels (reference: fla/ops/triton/triton_core/l2norm.py:131-234)."""
from __future__ import annotations

import ctypes

import torch

from .. import _runtime as rt
from .. import load_library
from ._structs import L2NormArgs


def _call(fn_name, args, tensors):
    lib = load_library()
    dev = rt.common_device(tensors, fn_name)
    rt._check_arch(dev, fn_name)
    with torch.cuda.device(dev):
        status = getattr(lib, f"fla_b200_{fn_name}")(ctypes.byref(args),
                                                     ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    if status != 0:
        raise RuntimeError(f"{fn_name} failed with status={status}: {rt._STATUS_NAMES.get(status, '?')}")


def _rows(t):
    t2 = t.reshape(-1, t.shape[-1])
    return t2 if t2.stride(-1) == 1 else t2.contiguous()


def l2norm_fwd(x, eps: float = 1e-6, output_dtype=None):
    """Returns ``(y, rstd)`` with ``y = x * rsqrt(sum(x^2, -1) + eps)`` and rstd of shape ``x.shape[:-1]`` (fp32)."""
    x2 = _rows(x)
    y2 = torch.empty(x2.shape, dtype=output_dtype or x.dtype, device=x.device)
    rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
    a = L2NormArgs()
    a.x, a.y, a.rstd, a.eps = rt.desc(x2), rt.desc(y2), rt.desc(rstd), float(eps)
    _call("l2norm_fwd", a, [x2, y2, rstd])
    return y2.view(x.shape), rstd.view(x.shape[:-1])


def l2norm_bwd(y, rstd, dy, eps: float = 1e-6):
    """Returns ``dx = dy * rstd - sum(dy * y, -1) * y * rstd`` in the dtype of ``y``."""
    y2, dy2 = _rows(y), _rows(dy)
    dx2 = torch.empty_like(y2)
    r = rstd.reshape(-1).contiguous()
    a = L2NormArgs()
    a.y, a.rstd, a.dy, a.dx, a.eps = rt.desc(y2), rt.desc(r), rt.desc(dy2), rt.desc(dx2), float(eps)
    _call("l2norm_bwd", a, [y2, r, dy2, dx2])
    return dx2.view(y.shape)

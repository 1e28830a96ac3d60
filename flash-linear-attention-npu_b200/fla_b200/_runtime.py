"""ctypes call layer between the Python operators and libfla_b200.so.

Mirrors the reference's FFI runtime (torch_custom/fla_npu/fla_npu/ops/ascendc/_runtime.py):
tensor descriptors built from shape / strides / dtype / data pointer (:210-256), a device guard
around every call (:153-174), launch on torch's current stream of the outputs' device (:177-188),
all tensors of one call on one device (:302-307, :442-460), two-phase workspace query + launch with
the workspace allocated as a uint8 torch tensor (:388-429), and non-zero status -> RuntimeError.
"""
from __future__ import annotations

import ctypes
import os
from typing import Iterable, Optional, Sequence

import torch

from . import load_library

FLA_MAX_DIMS = 6

_DTYPE_CODES = {
    torch.float32: 0,
    torch.bfloat16: 1,
    torch.float16: 2,
    torch.int32: 3,
    torch.int64: 4,
}

_STATUS_NAMES = {
    1: "FLA_ERR_NULL (required tensor missing)",
    2: "FLA_ERR_SHAPE (unsupported or inconsistent shape)",
    3: "FLA_ERR_DTYPE (unsupported dtype)",
    4: "FLA_ERR_LAYOUT (stride / alignment requirement not met)",
    5: "FLA_ERR_WORKSPACE (workspace too small)",
    6: "FLA_ERR_CUDA (CUDA runtime error)",
    7: "FLA_ERR_VALUE (scalar argument out of range)",
    8: "FLA_ERR_TIMEOUT (device-side wait ran out)",
    9: "FLA_ERR_TOO_LARGE (problem exceeds the built-in scratch of an allocation-free entry point)",
}


class TensorDesc(ctypes.Structure):
    """Binary twin of ``fla_tensor_t`` in include/fla_b200.h."""

    _fields_ = [
        ("data", ctypes.c_void_p),
        ("dtype", ctypes.c_int32),
        ("ndim", ctypes.c_int32),
        ("shape", ctypes.c_int64 * FLA_MAX_DIMS),
        ("stride", ctypes.c_int64 * FLA_MAX_DIMS),
    ]


def desc(t: Optional[torch.Tensor], name: str = "tensor") -> TensorDesc:
    """Describe a tensor for the C ABI; ``None`` becomes the null descriptor (tensor absent)."""
    d = TensorDesc()
    if t is None:
        return d
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor or None, got {type(t)!r}")
    if t.dtype not in _DTYPE_CODES:
        raise TypeError(f"{name}: unsupported dtype {t.dtype}")
    if t.dim() > FLA_MAX_DIMS:
        raise RuntimeError(f"{name}: rank {t.dim()} exceeds {FLA_MAX_DIMS}")
    d.data = t.data_ptr() if t.numel() > 0 else None
    d.dtype = _DTYPE_CODES[t.dtype]
    d.ndim = t.dim()
    for i, (s, st) in enumerate(zip(t.shape, t.stride())):
        d.shape[i] = s
        d.stride[i] = st
    return d


def common_device(tensors: Iterable[Optional[torch.Tensor]], op: str) -> torch.device:
    """All tensors of one call must live on one CUDA device; there is no CPU path."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if t.device.type != "cuda":
            raise RuntimeError(f"{op}: tensors must be on a CUDA device, got {t.device} (no CPU fallback exists)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"{op}: all tensors must be on the same device, got {dev} and {t.device}")
    if dev is None:
        raise RuntimeError(f"{op}: no tensors given")
    return dev


_checked_devices = set()


def _check_arch(dev: torch.device, op: str) -> None:
    if dev.index in _checked_devices:
        return
    major, _minor = torch.cuda.get_device_capability(dev)
    if major != 10:
        raise RuntimeError(f"{op}: libfla_b200 is built for sm_100a only; device {dev} is sm_{major}x")
    _checked_devices.add(dev.index)


# Operators whose kernels wait on barriers: byte 0 of their workspace is an int32 status word that a wait which ran
# out sets to FLA_ERR_TIMEOUT (include/fla_b200.h, "Device-side failure reporting").
_STATUS_WORD_OPS = frozenset({
    "gdn_chunk_fwd", "gdn_chunk_bwd", "kda_chunk_fwd", "kda_chunk_bwd", "chunk_local_cumsum", "chunk_scaled_dot_kkt",
    "solve_tri", "recompute_w_u_fwd", "chunk_gated_delta_rule_fwd_h", "chunk_fwd_o", "chunk_bwd_dv_local",
    "chunk_gated_delta_rule_bwd_dhu", "chunk_bwd_dqkwg", "prepare_wy_repr_bwd", "prepare_wy_repr_bwd_da",
    "prepare_wy_repr_bwd_full",
})

_check_device_status = os.environ.get("FLA_B200_CHECK", "0") not in ("", "0")


def set_device_status_check(enabled: bool) -> bool:
    """Turn the per-call read-back of the device status word on or off (also: ``FLA_B200_CHECK=1`` in the environment);
    returns the previous setting.  When on, every chunk operator waits for its stream after the launch and raises
    ``RuntimeError`` if a kernel recorded a failure - the synchronous behaviour of the reference, whose launches return
    an aclnnStatus (torch_custom/fla_npu/fla_npu/ops/ascendc/_runtime.py:410-411,427-428).  Off by default: launches
    stay asynchronous and a caller can check a workspace itself with :func:`read_device_status`."""
    global _check_device_status
    prev, _check_device_status = _check_device_status, bool(enabled)
    return prev


def read_device_status(workspace: torch.Tensor, op: str = "operator") -> None:
    """Wait for the current stream of ``workspace``'s device, read the int32 status word at its head and raise
    ``RuntimeError`` if a kernel left a non-zero status there (FLA_ERR_TIMEOUT: a bounded device-side wait ran out and
    the outputs of that call are invalid)."""
    lib = load_library()
    with torch.cuda.device(workspace.device):
        word = ctypes.c_int32(0)
        stream = ctypes.c_void_p(torch.cuda.current_stream(workspace.device).cuda_stream)
        status = lib.fla_b200_read_status_word(ctypes.c_void_p(workspace.data_ptr()), stream, ctypes.byref(word))
    if status != 0:
        raise RuntimeError(f"{op}: reading the device status word failed with status={status}: {_STATUS_NAMES.get(status, '?')}")
    if word.value != 0:
        raise RuntimeError(f"{op} failed on the device with status={word.value}: {_STATUS_NAMES.get(word.value, '?')}")


def call(op: str, args: ctypes.Structure, tensors: Sequence[Optional[torch.Tensor]]) -> None:
    """Two-phase call: ``fla_b200_<op>_workspace_size`` then ``fla_b200_<op>`` on the current stream."""
    lib = load_library()
    dev = common_device(tensors, op)
    _check_arch(dev, op)
    ws_fn = getattr(lib, f"fla_b200_{op}_workspace_size")
    run_fn = getattr(lib, f"fla_b200_{op}")
    with torch.cuda.device(dev):
        nbytes = ctypes.c_uint64(0)
        status = ws_fn(ctypes.byref(args), ctypes.byref(nbytes))
        if status != 0:
            raise RuntimeError(f"{op} workspace query failed with status={status}: {_STATUS_NAMES.get(status, '?')}")
        ws = None
        ws_ptr = ctypes.c_void_p(None)
        if nbytes.value:
            ws = torch.empty(nbytes.value, dtype=torch.uint8, device=dev)
            ws_ptr = ctypes.c_void_p(ws.data_ptr())
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        status = run_fn(ctypes.byref(args), ws_ptr, ctypes.c_uint64(nbytes.value), stream)
        if status != 0:
            raise RuntimeError(f"{op} failed with status={status}: {_STATUS_NAMES.get(status, '?')}")
        if _check_device_status and ws is not None and op in _STATUS_WORD_OPS:
            read_device_status(ws, op)
        # `ws` is released to the caching allocator in stream order when it goes out of scope


def mark_mutated(*tensors: Optional[torch.Tensor]) -> None:
    """Tell autograd that the kernel wrote these tensors in place
    (reference: ops/ascendc/__init__.py:61-71,169-183)."""
    for t in tensors:
        if t is not None:
            torch.autograd.graph.increment_version(t)


def reject_requires_grad(op: str, **tensors: Optional[torch.Tensor]) -> None:
    for name, t in tensors.items():
        if t is not None and t.requires_grad:
            raise RuntimeError(f"{op}: {name} is updated in place and must not require grad")

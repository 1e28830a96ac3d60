"""B200-native (sm_100a) GDN / KDA linear-attention operators.

Importing the package locates and dlopens ``libfla_b200.so`` (the role of
``load_ascendc_opapi_libraries`` in the reference, torch_custom/fla_npu/fla_npu/__init__.py:129-150).
There is no CPU or PyTorch fallback: every operator in :mod:`fla_b200.ops` raises if the
library is missing or the tensors are not on a CUDA device.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

__version__ = "0.1.0"

_LIB = None
_LIB_PATH_ENV = "FLA_B200_LIB"


def library_path() -> Path:
    """Resolve the shared library: ``$FLA_B200_LIB`` overrides the in-tree build."""
    override = os.environ.get(_LIB_PATH_ENV)
    if override:
        return Path(override)
    return Path(__file__).resolve().parent / "lib" / "libfla_b200.so"


def load_library() -> ctypes.CDLL:
    """dlopen the kernel library once per process (RTLD_GLOBAL | RTLD_NOW) and cache the handle."""
    global _LIB
    if _LIB is None:
        path = library_path()
        if not path.exists():
            raise RuntimeError(
                f"fla_b200: kernel library not found at {path}. Build it with "
                f"`python {Path(__file__).resolve().parent.parent / 'build.py'}` "
                f"or point ${_LIB_PATH_ENV} at libfla_b200.so. There is no fallback path."
            )
        mode = ctypes.RTLD_GLOBAL | getattr(os, "RTLD_NOW", 2)
        _LIB = ctypes.CDLL(str(path), mode=mode)
    return _LIB

"""ctypes loader for the in-tree kernel library (``hippolm_b200/lib/libhippo_kernels.so``).

On a machine with a CUDA device the library must exist and load; a missing or broken build raises
instead of falling back to torch ops, so GPU tests never pass on a silent fallback.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

_LIB: Optional[ctypes.CDLL] = None
_HOST: Optional[ctypes.CDLL] = None
_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib")


def lib_path() -> str:
    """``HIPPO_DEBUG_BOUNDS=1`` selects the library built with checked data-dependent indices (see csrc/build.py)."""
    dbg = os.environ.get("HIPPO_DEBUG_BOUNDS", "0") not in ("", "0")
    return os.path.join(_DIR, "libhippo_kernels_dbg.so" if dbg else "libhippo_kernels.so")


def is_loaded() -> bool:
    return _LIB is not None


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        p = lib_path()
        if not os.path.exists(p):
            raise RuntimeError(f"{p} is missing: run `python -m hippolm_b200.csrc.build` "
                               "(CUDA tensors never fall back to torch ops)")
        _LIB = ctypes.CDLL(p)
    return _LIB


def host_lib() -> Optional[ctypes.CDLL]:
    global _HOST
    if _HOST is None:
        p = os.path.join(_DIR, "libhippo_host.so")
        if os.path.exists(p):
            _HOST = ctypes.CDLL(p)
    return _HOST


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_LAUNCHES = [0]


def launch_count() -> int:
    """Number of kernel-launcher calls into the library since the last reset."""
    return _LAUNCHES[0]


def reset_launch_count() -> None:
    _LAUNCHES[0] = 0


def check(rc: int, what: str) -> None:
    _LAUNCHES[0] += 1
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


def device_status():
    """(code, detail, block, count) of the first bounded wait that ran out, (0,0,0,0) when clean."""
    out = (ctypes.c_int * 4)()
    check(lib().hippo_get_status(out), "hippo_get_status")
    return tuple(out)


def clear_device_status() -> None:
    check(lib().hippo_clear_status(), "hippo_clear_status")

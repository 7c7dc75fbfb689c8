"""ctypes loader for the CUDA kernel library (``lib/libmlcb200_kernels.so``).

The library is built in-tree by :mod:`mlc_llm_b200.build`.  On a machine with a GPU a missing or
unloadable library is a hard error: the CUDA ops never fall back to PyTorch silently.
"""

from __future__ import annotations

import ctypes
import threading
from typing import Optional

import torch

_LIB: Optional[ctypes.CDLL] = None
_LOCK = threading.Lock()
_STATUS = {}


class KernelError(RuntimeError):
    """A kernel launch was rejected or a bounded device-side wait ran out."""


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        with _LOCK:
            if _LIB is None:
                from .. import build  # pylint: disable=import-outside-toplevel

                path = build.kernels_lib_path()
                if not path.exists():
                    build.build_kernels()
                _LIB = ctypes.CDLL(str(path))
    return _LIB


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 word that kernels set when a bounded wait expires or an index is bad."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    st = _STATUS.get(key)
    if st is None:
        st = torch.zeros(1, dtype=torch.int32, device=device)
        _STATUS[key] = st
    return st


def check_status(device: torch.device) -> None:
    """Synchronising check of the status word (call at step boundaries, not per kernel)."""
    st = status_word(device)
    code = int(st.item())
    if code != 0:
        st.zero_()
        names = {
            1: "wait for TMA data timed out",
            2: "wait for MMA completion timed out",
            3: "wait for epilogue timed out",
            4: "producer wait timed out",
            5: "wait for a peer GPU timed out",
            6: "index out of range",
            7: "wait for dequantised tile timed out",
            8: "a fixed-capacity exchange buffer overflowed",
        }
        raise KernelError(f"device status {code}: {names.get(code, 'unknown')}")


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")


DTYPE_CODE = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}

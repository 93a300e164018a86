"""ctypes binding of ``libdizo_b200.so`` (the sm_100a kernels).

The library is built ahead of time by :mod:`dizo_b200.ops.build` and lives beside this
file.  There is no silent fallback: asking for the library on a machine where it has
not been built raises, and every entry point's return code is checked.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libdizo_b200.so"
_lock = threading.Lock()
_lib = None
_err_words: dict[int, torch.Tensor] = {}

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float
c_u64 = ctypes.c_uint64
c_u32 = ctypes.c_uint32


class KernelError(RuntimeError):
    """An entry point returned a non-zero code, or a kernel reported a timed-out wait."""


_RC_NAMES = {1: "bad argument", 2: "misaligned pointer or stride", 3: "tensor-map encode failed",
             4: "size beyond the supported maximum"}


def available() -> bool:
    return _LIB_PATH.exists()


def lib() -> ctypes.CDLL:
    """Load (once) and return the kernel library; build it first if nvcc is present."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not _LIB_PATH.exists() or os.environ.get("DIZO_B200_REBUILD") == "1":
                from . import build as _build
                _build.build()
            _lib = ctypes.CDLL(str(_LIB_PATH))
    return _lib


launch_count = 0     # entry points called so far (each launches one kernel)


def check(rc: int, what: str) -> None:
    global launch_count
    if rc == 0:
        launch_count += 1
        return
    if rc >= 1000:
        raise KernelError(f"{what}: CUDA error {rc - 1000} "
                          f"({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no gpu'})")
    raise KernelError(f"{what}: {_RC_NAMES.get(rc, 'error')} (code {rc})")


def stream_ptr() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> c_void_p:
    if t is None:
        return c_void_p(0)
    return c_void_p(t.data_ptr())


def err_word(device: torch.device | int | None = None) -> torch.Tensor:
    """Per-device 32-bit word in which kernels record a wait that ran out of time."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    w = _err_words.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
        _err_words[idx] = w
    return w


_ERR_CODES = {1: "consumer waited for a TMA-filled stage", 2: "producer waited for a free stage",
              3: "epilogue waited for an accumulator", 4: "MMA issuer waited for a drained accumulator",
              5: "wait on a peer GPU's flag", 6: "wait", 7: "bad argument seen on the device"}


def check_device_errors(device: torch.device | int | None = None) -> None:
    """Synchronising read of the device error word; raises if a kernel gave up a wait."""
    w = err_word(device)
    v = int(w.item()) & 0xFFFFFFFF
    if v:
        w.zero_()
        code, cta = v & 0xFF, v >> 8
        raise KernelError(f"device wait timed out: {_ERR_CODES.get(code, code)} (CTA {cta})")

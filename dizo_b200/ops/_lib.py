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
# DIZO_DEBUG_BOUNDS=1: load the checked-store build (see the end of this file)
DEBUG_BOUNDS = os.environ.get("DIZO_DEBUG_BOUNDS") == "1"
_LIB_PATH = _HERE / ("libdizo_b200_dbg.so" if DEBUG_BOUNDS else "libdizo_b200.so")
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
                _build.build(debug_bounds=DEBUG_BOUNDS)
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
    if DEBUG_BOUNDS and t.is_cuda:
        note(t)
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
    if DEBUG_BOUNDS:
        debug_check()
    if v:
        w.zero_()
        code, cta = v & 0xFF, v >> 8
        raise KernelError(f"device wait timed out: {_ERR_CODES.get(code, code)} (CTA {cta})")


# ---------------------------------------------------------------------------------- checked stores
# The debug build (``python -m dizo_b200.ops.build --debug-bounds``, loaded with DIZO_DEBUG_BOUNDS=1)
# checks every global store of the instrumented kernels against a table of address ranges and skips the
# store when it falls outside all of them.  The table holds the storage of every tensor passed to an
# entry point (``ptr`` registers it; ``note`` does so for tensors handed over as raw addresses, and
# ``note_range`` for peer memory); each translation unit of the library keeps its own copy, refreshed
# when the table changes.  ``debug_check`` (called by ``check_device_errors``) raises if a kernel
# recorded a skipped store.  Stands in for compute-sanitizer where that tool is closed.
_DBG_MAX = 256
_DBG_TUS = ("zo", "norm", "lmhead", "bwd", "peft", "gemm1", "gemm2", "commgemm", "llama")


class _DbgState(ctypes.Structure):
    _fields_ = [("lo", ctypes.c_uint64 * _DBG_MAX), ("hi", ctypes.c_uint64 * _DBG_MAX), ("n", ctypes.c_int),
                ("violations", ctypes.c_uint), ("first_addr", ctypes.c_uint64), ("first_line", ctypes.c_int),
                ("pad", ctypes.c_int)]


_dbg_ranges: dict[int, int] = {}      # base address -> end address, insertion-ordered (oldest first)


def note_range(lo: int, nbytes: int) -> None:
    """Allow stores into [lo, lo + nbytes) (debug build only)."""
    if not DEBUG_BOUNDS or nbytes <= 0:
        return
    hi = lo + nbytes
    if _dbg_ranges.get(lo) == hi:
        _dbg_ranges[lo] = _dbg_ranges.pop(lo)     # most recently used last: eviction takes the oldest
        return
    _dbg_ranges.pop(lo, None)
    _dbg_ranges[lo] = hi
    while len(_dbg_ranges) > _DBG_MAX:
        _dbg_ranges.pop(next(iter(_dbg_ranges)))
    _dbg_push()


def note(t: torch.Tensor) -> torch.Tensor:
    """Register the storage of ``t`` as writable for the kernels (no-op in the normal build)."""
    if DEBUG_BOUNDS and t is not None and t.is_cuda:
        st = t.untyped_storage()
        note_range(st.data_ptr(), st.nbytes())
    return t


def forget(t: torch.Tensor) -> None:
    """Drop ``t``'s storage from the table (tests: the next store into it must be reported)."""
    if DEBUG_BOUNDS:
        st = t.untyped_storage()
        lo, hi = st.data_ptr(), st.data_ptr() + st.nbytes()
        # ranges of freed tensors linger (the allocator reuses their memory): drop every overlap
        for k in [k for k, v in _dbg_ranges.items() if k < hi and v > lo]:
            _dbg_ranges.pop(k)
        _dbg_push()


def _dbg_push() -> None:
    st = _DbgState()
    for i, (lo, hi) in enumerate(_dbg_ranges.items()):
        st.lo[i], st.hi[i] = lo, hi
    st.n = len(_dbg_ranges)
    L = lib()
    for tu in _DBG_TUS:
        prev = _DbgState()
        getattr(L, f"dz_debug_get_{tu}")(ctypes.byref(prev))     # keep what the kernels recorded so far
        st.violations, st.first_addr, st.first_line = prev.violations, prev.first_addr, prev.first_line
        rc = getattr(L, f"dz_debug_set_{tu}")(ctypes.byref(st))
        if rc:
            raise KernelError(f"dz_debug_set_{tu}: CUDA error {rc}")


def debug_violations(reset: bool = True) -> list[tuple[str, int, int, int]]:
    """[(translation unit, skipped stores, first address, source line)] recorded since the last reset."""
    if not DEBUG_BOUNDS:
        return []
    torch.cuda.synchronize()
    out = []
    L = lib()
    for tu in _DBG_TUS:
        st = _DbgState()
        getattr(L, f"dz_debug_get_{tu}")(ctypes.byref(st))
        if st.violations:
            out.append((tu, int(st.violations), int(st.first_addr), int(st.first_line)))
            if reset:
                st.violations, st.first_addr, st.first_line = 0, 0, 0
                getattr(L, f"dz_debug_set_{tu}")(ctypes.byref(st))
    return out


def debug_check() -> None:
    bad = debug_violations()
    if bad:
        tu, n, addr, line = bad[0]
        raise KernelError(f"{n} store(s) outside every registered range were skipped in {tu} "
                          f"(first at 0x{addr:x}, source line {line}); all: {bad}")

"""Ahead-of-time build of the sm_100a kernels into one in-tree shared library.

Every ``csrc/*.cu`` file is compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` and linked into
``dizo_b200/ops/libdizo_b200.so``.  The library exports plain ``extern "C"`` entry
points taking raw device pointers and a ``cudaStream_t``; Python binds them with
``ctypes`` (see ``dizo_b200/ops/_lib.py``).  There is no JIT cache: the built ``.so``
sits beside the sources, and a stale library (older than any source) is rebuilt.

``--debug-bounds`` builds a second library, ``libdizo_b200_dbg.so``, with ``-DDZ_DEBUG_BOUNDS``: every
global store of the instrumented kernels is checked against the address ranges the host registered and
skipped (and recorded) when it falls outside them; ``DIZO_DEBUG_BOUNDS=1`` makes the package load it.

Run ``python -m dizo_b200.ops.build [--force] [--verbose] [--debug-bounds]``.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD = HERE / "_build"
LIB = HERE / "libdizo_b200.so"
BUILD_DBG = HERE / "_build_dbg"
LIB_DBG = HERE / "libdizo_b200_dbg.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=default",
    "--use_fast_math",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest(src: Path, flags) -> str:
    h = hashlib.sha256()
    h.update(" ".join(flags).encode())
    h.update(src.read_bytes())
    for hdr in sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(hdr.read_bytes())
    return h.hexdigest()[:16]


def _compile_one(src: Path, verbose: bool, build_dir: Path, flags) -> Path:
    obj = build_dir / f"{src.stem}.{_digest(src, flags)}.o"
    if obj.exists():
        return obj
    for old in build_dir.glob(f"{src.stem}.*.o"):
        old.unlink()
    cmd = [_nvcc(), *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return obj


def _variant(debug_bounds: bool):
    if debug_bounds:
        return BUILD_DBG, LIB_DBG, NVCC_FLAGS + ["-DDZ_DEBUG_BOUNDS"]
    return BUILD, LIB, NVCC_FLAGS


def stale(debug_bounds: bool = False) -> bool:
    build_dir, lib, flags = _variant(debug_bounds)
    if not lib.exists():
        return True
    stamp = build_dir / "link.stamp"
    want = "\n".join(f"{s.stem}.{_digest(s, flags)}" for s in _sources())
    return not stamp.exists() or stamp.read_text() != want


def build(force: bool = False, verbose: bool = False, debug_bounds: bool = False) -> Path:
    """Compile every kernel for sm_100a and link the shared library. Returns its path."""
    build_dir, lib, flags = _variant(debug_bounds)
    build_dir.mkdir(exist_ok=True)
    if force:
        for old in build_dir.glob("*.o"):
            old.unlink()
    elif not stale(debug_bounds):
        return lib
    srcs = _sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs) or 1)) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, verbose, build_dir, flags), srcs))
    cmd = [_nvcc(), "-shared", "-o", str(lib), *map(str, objs)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    (build_dir / "link.stamp").write_text("\n".join(f"{s.stem}.{_digest(s, flags)}" for s in srcs))
    return lib


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register/smem usage")
    ap.add_argument("--debug-bounds", action="store_true", help="build the checked-store library instead")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose, debug_bounds=a.debug_bounds))

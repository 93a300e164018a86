"""Ahead-of-time build of the sm_100a kernels into one in-tree shared library.

Every ``csrc/*.cu`` file is compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` and linked into
``dizo_b200/ops/libdizo_b200.so``.  The library exports plain ``extern "C"`` entry
points taking raw device pointers and a ``cudaStream_t``; Python binds them with
``ctypes`` (see ``dizo_b200/ops/_lib.py``).  There is no JIT cache: the built ``.so``
sits beside the sources, and a stale library (older than any source) is rebuilt.

Run ``python -m dizo_b200.ops.build [--force] [--verbose]``.
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


def _digest(src: Path) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(src.read_bytes())
    for hdr in sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(hdr.read_bytes())
    return h.hexdigest()[:16]


def _compile_one(src: Path, verbose: bool) -> Path:
    obj = BUILD / f"{src.stem}.{_digest(src)}.o"
    if obj.exists():
        return obj
    for old in BUILD.glob(f"{src.stem}.*.o"):
        old.unlink()
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return obj


def stale() -> bool:
    if not LIB.exists():
        return True
    stamp = BUILD / "link.stamp"
    want = "\n".join(f"{s.stem}.{_digest(s)}" for s in _sources())
    return not stamp.exists() or stamp.read_text() != want


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every kernel for sm_100a and link the shared library. Returns its path."""
    BUILD.mkdir(exist_ok=True)
    if force:
        for old in BUILD.glob("*.o"):
            old.unlink()
    elif not stale():
        return LIB
    srcs = _sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs) or 1)) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, verbose), srcs))
    cmd = [_nvcc(), "-shared", "-o", str(LIB), *map(str, objs)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    (BUILD / "link.stamp").write_text("\n".join(f"{s.stem}.{_digest(s)}" for s in srcs))
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register/smem usage")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))

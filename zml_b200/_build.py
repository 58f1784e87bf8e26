"""In-tree build of the native libraries.

Two shared objects are produced next to the sources, never installed elsewhere:

* ``zml_b200/_C/libzb_cuda.so``  - every ``csrc/*.cu`` compiled by ``nvcc`` for
  ``sm_100a`` only (``-gencode arch=compute_100a,code=sm_100a``).  nvcc
  cross-compiles, so this builds on a machine without a GPU.
* ``zml_b200/_C/libzb_host.so``  - ``csrc/host/*.cpp`` compiled by ``g++``: the
  threaded file reader behind the weight loader (``file_stream.cpp``) and the span
  recorder (``tracer.cpp``).  CPU only.

The reference gets its native parts from Bazel rules and from binaries downloaded at build time
(platforms/cuda/cuda.bzl, third_party/*/repo.bzl); here everything native is compiled from the sources in this
tree by the two functions below.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OUT = ROOT / "_C"
OBJ = ROOT.parent / "build" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-diag-suppress", "177",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread"]


def _nvcc() -> str | None:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    return None


def _newer(target: Path, deps: list[Path]) -> bool:
    """True when `target` exists and is newer than every dependency."""
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(d.stat().st_mtime <= t for d in deps)


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))


def build_cuda(force: bool = False, verbose: bool = False, extra_flags: list[str] | None = None,
               variant: str = "") -> Path:
    """Builds `_C/libzb_cuda.so`.  With `variant` (and usually `extra_flags`) the same sources are built into
    `_C/libzb_cuda_<variant>.so` with objects of their own - e.g. `variant="bc", extra_flags=["-DZB_BOUNDS_CHECK"]`,
    the checking build that `ZB_CUDA_LIB` then selects."""
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build libzb_cuda.so")
    srcs = sorted(CSRC.glob("*.cu"))
    hdrs = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    target = OUT / (f"libzb_cuda_{variant}.so" if variant else "libzb_cuda.so")
    if not force and _newer(target, srcs + hdrs):
        return target
    obj_dir = OBJ.parent / (f"obj_{variant}" if variant else "obj")
    OUT.mkdir(parents=True, exist_ok=True)
    obj_dir.mkdir(parents=True, exist_ok=True)
    flags = NVCC_FLAGS + (extra_flags or []) + (["-Xptxas", "-v"] if verbose else [])

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        if force or not _newer(obj, [src] + hdrs):
            _run([nvcc, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)])
        return obj

    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs) or 1)) as ex:
        objs = list(ex.map(compile_one, srcs))
    # link beside the target and rename: a reader never sees a half-written library
    tmp = target.with_suffix(".so.tmp")
    _run([nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-lpthread", "-ldl"])
    # every symbol must resolve at load time (works without a GPU or a driver)
    import ctypes
    ctypes.CDLL(str(tmp), mode=getattr(os, "RTLD_NOW", 2))
    os.replace(tmp, target)
    return target


def build_host(force: bool = False) -> Path:
    srcs = sorted((CSRC / "host").glob("*.cpp"))
    hdrs = sorted((CSRC / "host").glob("*.h"))
    target = OUT / "libzb_host.so"
    if not srcs:
        return target
    if not force and _newer(target, srcs + hdrs):
        return target
    OUT.mkdir(parents=True, exist_ok=True)
    cxx = os.environ.get("CXX", "g++")
    _run([cxx, *CXX_FLAGS, "-shared", "-o", str(target), *map(str, srcs), "-ldl"])
    return target


def build_all(force: bool = False, verbose: bool = False) -> dict[str, Path]:
    return {"host": build_host(force), "cuda": build_cuda(force, verbose)}


if __name__ == "__main__":
    out = build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    for k, v in out.items():
        print(k, v)

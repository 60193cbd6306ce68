"""Builds the native library (``libtplr_b200.so``) in-tree with nvcc for sm_100a.

``python -m templar_b200.ops.build`` (or :func:`build`) compiles every ``csrc/*.cu``
translation unit with ``-gencode arch=compute_100a,code=sm_100a -lineinfo`` and links
them into ``templar_b200/ops/_lib/libtplr_b200.so``.  nvcc cross-compiles without a GPU.
Objects are rebuilt only when a source or header is newer than the object.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIBDIR = HERE / "_lib"
LIBNAME = "libtplr_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]
# Approximate intrinsics and flush-to-zero only where the arithmetic is a softmax in base 2 (the flash
# attention kernels).  The loss, the norms, the optimizer, the quantiser and the compression kernels are
# compiled with IEEE division / square root and keep denormals; where they want a fast exponential they
# call __expf explicitly.
FAST_MATH_SOURCES = {"attention.cu"}


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")
    return cand


def lib_path() -> Path:
    return LIBDIR / LIBNAME


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale(obj: Path, src: Path, headers: list[Path]) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    return any(p.stat().st_mtime > t for p in [src, *headers])


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile and link the library; returns its path."""
    nvcc = _nvcc()
    LIBDIR.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    objs, jobs = [], []
    for src in sources():
        obj = LIBDIR / (src.stem + ".o")
        objs.append(obj)
        if force or _stale(obj, src, headers):
            extra = ["--use_fast_math"] if src.name in FAST_MATH_SOURCES else []
            cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
        return r.stderr

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for out in ex.map(run, jobs):
                if verbose and out:
                    print(out, file=sys.stderr)
    lib = lib_path()
    if jobs or not lib.exists():
        tmp = lib.with_suffix(".so.tmp")          # link beside the target, then rename: readers never see a partial file
        run([nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-lcudart"])
        os.replace(tmp, lib)
    return lib


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))

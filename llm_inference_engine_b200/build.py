"""Builds libmuse_proj.so (the sm_100a kernels + C ABI) in-tree with nvcc.

    python -m llm_inference_engine_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU. The library links the CUDA runtime statically and fetches the one
driver entry point it needs at run time, so it loads on a machine without a driver.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
# MUSE_TRACE=1 in the environment builds (and _capi loads) a separate diagnostic library whose kernels
# stamp their phases; the ordinary library carries none of that code.
TRACE = bool(os.environ.get("MUSE_TRACE"))
LIB_PATH = PKG_DIR / ("libmuse_proj_trace.so" if TRACE else "libmuse_proj.so")
SOURCES = ["gemv1.cu", "fewtok_mma.cu", "fewtok_zip.cu", "ffn_boundary.cu", "skinny_tc.cu", "gemm_tc.cu", "capi.cu"]
NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "--shared",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found: set NVCC or put /usr/local/cuda/bin on PATH")
    return cand


def _stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = [CSRC / s for s in SOURCES] + [CSRC / "common.cuh", PKG_DIR.parent / "include" / "muse_proj.h"]
    return any(d.stat().st_mtime > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if it is missing or older than its sources; return its path."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = _nvcc()
    compile_flags = ([f for f in NVCC_FLAGS if f != "--shared"] + (["-Xptxas", "-v"] if verbose else [])
                     + (["-DMUSE_TRACE"] if TRACE else []))
    objs = [CSRC / (Path(s).stem + (".trace.o" if TRACE else ".o")) for s in SOURCES]

    def compile_one(src_obj):
        src, obj = src_obj
        return subprocess.run([nvcc, *compile_flags, "-c", str(CSRC / src), "-o", str(obj)], capture_output=True, text=True)

    from concurrent.futures import ThreadPoolExecutor

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:   # one nvcc per translation unit, side by side
        results = list(pool.map(compile_one, zip(SOURCES, objs)))
    for src, proc in zip(SOURCES, results):
        if verbose or proc.returncode != 0:
            sys.stderr.write(proc.stdout + proc.stderr)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed ({proc.returncode}) on {src}")
    link = subprocess.run([nvcc, "--shared", "-Xcompiler", "-fPIC", "-gencode", "arch=compute_100a,code=sm_100a",
                           *[str(o) for o in objs], "-o", str(LIB_PATH)], capture_output=True, text=True)
    if link.returncode != 0:
        sys.stderr.write(link.stdout + link.stderr)
        raise RuntimeError(f"link failed ({link.returncode})")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))

"""Builds libdfdx_b200.so (sm_100a only) in-tree with nvcc.

    python -m dfdx_b200.build            # incremental
    python -m dfdx_b200.build --force

Each .cu is compiled to an object in `dfdx_b200/lib/obj/` (in parallel), then linked into
`dfdx_b200/lib/libdfdx_b200.so` with a statically linked CUDA runtime.  The driver API is not linked:
the one driver entry point the library needs (tensor-map encoding) is resolved at run time, so the
library loads on a machine without a GPU driver.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
OBJDIR = LIBDIR / "obj"
LIB = LIBDIR / "libdfdx_b200.so"
SOURCES = ["api.cu", "gemm_simt.cu", "gemm_tc.cu", "gemm_tc_pair.cu", "conv2d.cu", "attention.cu", "attention_bwd.cu", "rowwise.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _deps_mtime() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [PKG.parent / "include" / "dfdx_b200.h"]
    return max(p.stat().st_mtime for p in hdrs if p.exists())


def _compile(src: str, force: bool) -> Path:
    obj = OBJDIR / (src.replace(".cu", ".o"))
    srcp = CSRC / src
    if not force and obj.exists() and obj.stat().st_mtime >= max(srcp.stat().st_mtime, _deps_mtime()):
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(srcp), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    (OBJDIR / (src + ".log")).write_text(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJDIR.mkdir(parents=True, exist_ok=True)
    with ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        objs = list(ex.map(lambda s: _compile(s, force), SOURCES))
    if force or not LIB.exists() or any(o.stat().st_mtime > LIB.stat().st_mtime for o in objs):
        cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-cudart", "static",
               "-o", str(LIB), *map(str, objs)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    if verbose:
        print(f"built {LIB}")
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)

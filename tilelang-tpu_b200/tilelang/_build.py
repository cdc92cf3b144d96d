"""Ahead-of-time build of libtl_b200.so (the sm_100a kernel library).

Takes the place of the reference's per-program `LibraryGenerator`
(tilelang/jit/adapter/libgen.py:19-415), which shells out to the SOPHGO toolchain on every
`compile()`.  Here every kernel is hand-written CUDA, compiled once with nvcc for sm_100a and
kept in-tree next to the package.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_ROOT = Path(__file__).resolve().parent.parent          # .../tilelang-tpu_b200
REPO_ROOT = PKG_ROOT.parent
CSRC = PKG_ROOT / "csrc"
LIB_DIR = PKG_ROOT / "lib"
OBJ_DIR = PKG_ROOT / "build"
LIB_PATH = LIB_DIR / "libtl_b200.so"
INCLUDE = REPO_ROOT / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-I", str(INCLUDE), "-I", str(CSRC),
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: libtl_b200.so cannot be built")
    return exe


def _newest_header_mtime() -> float:
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    return max((h.stat().st_mtime for h in headers), default=0.0)


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile every csrc/*.cu to an object and link lib/libtl_b200.so.  Incremental by mtime."""
    nvcc = _nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    hdr_m = _newest_header_mtime()
    jobs = []
    objs = []
    for src in sources():
        obj = OBJ_DIR / (src.stem + ".o")
        objs.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m)
        if stale:
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            if ptxas_info:
                cmd += ["-Xptxas", "-v"]
            jobs.append(cmd)

    def run(cmd):
        if verbose:
            print(" ".join(cmd), file=sys.stderr)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed:\n{' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
        if ptxas_info or verbose:
            sys.stderr.write(res.stderr)
        return res

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            list(pool.map(run, jobs))
    need_link = force or bool(jobs) or not LIB_PATH.exists() or any(
        o.stat().st_mtime > LIB_PATH.stat().st_mtime for o in objs)
    if need_link:
        run([nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs), "-lcuda",
             "-gencode", "arch=compute_100a,code=sm_100a"])
    return LIB_PATH


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv)
    print(p)

"""Builds libmach_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

Every source is compiled to an object under `build/` (in parallel, only when it or a header
is newer than the object) and the objects are linked into the shared library.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG.parent / "csrc"
OBJ = PKG.parent / "build"
LIB = PKG / "libmach_b200.so"
HEADER = PKG.parent.parent / "include" / "mach_b200.h"
SOURCES = ["host_util.cu", "quant_kernels.cu", "gemm_mx.cu", "gemm_mx_tm.cu", "gemm_mx_2cta.cu", "gemm_mx_mid.cu",
           "gemm_blockfp8.cu", "gemm_blockfp8_tm.cu", "ar_norm.cu", "moe.cu", "moe_small.cu", "gemm_mx_grouped.cu"]
FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
         "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _headers_mtime() -> float:
    return max(p.stat().st_mtime for p in list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [HEADER])


def needs_build() -> bool:
    if not LIB.exists():
        return True
    newest = max(max(p.stat().st_mtime for p in CSRC.glob("*.cu")), _headers_mtime())
    return newest > LIB.stat().st_mtime


def _compile(src: str, force: bool, verbose: bool, defines: list[str]) -> tuple[Path, str]:
    obj = OBJ / (src + ".o")
    source = CSRC / src
    if (not force and obj.exists()
            and obj.stat().st_mtime > max(source.stat().st_mtime, _headers_mtime())):
        return obj, ""
    cmd = [_nvcc(), *FLAGS, *defines, "-c", str(source), "-o", str(obj)]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n" + proc.stdout + proc.stderr)
    return obj, proc.stderr


def build(force: bool = False, verbose: bool = False, defines: list[str] | None = None) -> Path:
    """`defines`: extra -D flags (e.g. ["-DMACH_EXPERIMENTS"] for the tile-sweep build)."""
    if not force and not defines and not needs_build():
        return LIB
    OBJ.mkdir(exist_ok=True)
    defines = list(defines or [])
    force = force or bool(defines)
    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 4)) as pool:
        results = list(pool.map(lambda s: _compile(s, force, verbose, defines), SOURCES))
    proc = subprocess.run([_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
                           *[str(o) for o, _ in results], "-o", str(LIB)],
                          capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("link failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv,
                defines=[a for a in sys.argv[1:] if a.startswith("-D")]))

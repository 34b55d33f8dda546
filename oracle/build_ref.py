"""TEST INFRASTRUCTURE: builds oracle/_ref/libar_ref.so from the reference's own sources.

The fused all-reduce tail of the reference (FusedOp::operator(), rms_norm, the MXFP8 branch,
vec_add, allreduce_sum, blockReduceSumV2) is device code inside
native/ar_norm/trtllm_allreduce_fusion_mxfp8.cuh. The header as a whole needs FlashInfer and
CUDA 13; these definitions alone are plain C++ once vec_t and a handful of intrinsics exist.
This recipe cuts them out of the header WHERE IT LIES in the reference checkout (nothing is
copied into the repository: the cut goes to the git-ignored oracle/_ref/), and compiles them
with oracle/ar_ref_harness.cpp by g++ into a shared library that tests/test_oracle_cpu.py uses
to pin oracle.mx_oracle.allreduce_rmsnorm and the MXFP8 activation rule.

    python oracle/build_ref.py [reference root]
                  (default: $MACH_REFERENCE_ROOT, else the `reference` checkout that lies
                   beside this repository's folder)

Returns silently without building when the reference checkout is absent (the GPU box): the
prebuilt library travels with the repository snapshot.
"""
from __future__ import annotations

import re
import subprocess
import sys
from pathlib import Path

import os

HERE = Path(__file__).resolve().parent
DEFAULT_REFERENCE = os.environ.get("MACH_REFERENCE_ROOT") or str(HERE.parent.parent / "reference")
OUT = HERE / "_ref"
LIB = OUT / "libar_ref.so"
HEADER = "native/ar_norm/trtllm_allreduce_fusion_mxfp8.cuh"

# (first line pattern, pattern of the first line AFTER the region)
REGIONS = [
    # warpReduceSumV2, warpReduceSumPartialV2, blockReduceSumV2
    (r"^template <typename T, int NUM>\n__inline__ __device__ T warpReduceSumV2\(",
     r"^template <typename T, int NUM>\n__inline__ __device__ T warpReduceMaxV2\("),
    # vec_add, pattern and quantisation enums, pattern traits
    (r"^template <typename T, uint32_t VEC_SIZE>\n__device__ __forceinline__ vec_t<T, VEC_SIZE> vec_add\(",
     r"^template <typename T>\nstruct AllReduceFusionParams \{"),
    # class FusedOp
    (r"^template <AllReduceFusionPattern Pattern, typename T>\nclass FusedOp \{",
     r"^template <typename T>\nstruct neg_zero \{"),
    # allreduce_sum
    (r"^template <typename T, uint32_t VEC_SIZE, int NRanks, bool Fp32Acc>\n__device__ __forceinline__ vec_t<T, VEC_SIZE> allreduce_sum\(",
     r"^template <typename T>\n(?:__device__|__global__|class|struct|inline)"),
]


def extract(text: str) -> str:
    parts = []
    for i, (first, after) in enumerate(REGIONS):
        a = re.search(first, text, re.M)
        if a is None:
            raise RuntimeError(f"region {i}: start not found in {HEADER}")
        b = re.compile(after, re.M).search(text, a.end())
        if b is None:
            raise RuntimeError(f"region {i}: end not found in {HEADER}")
        body = text[a.start():b.start()]
        # the harness maps __shared__ to `static` (one object per block)
        body = body.replace("static __shared__", "__shared__").replace("extern __shared__", "extern")
        if i == 0:
            body = "namespace utils {\nstatic constexpr int kWarpSize = 32;\n" \
                   "static constexpr unsigned int kFullWarpMask = 0xffffffffU;\n" + body + "}\n"
        parts.append(f"// ---- cut {i} of {HEADER}\n{body}")
    return "\n".join(parts)


def build(reference_root: str = DEFAULT_REFERENCE, force: bool = False) -> Path | None:
    header = Path(reference_root) / HEADER
    if not header.exists():
        return LIB if LIB.exists() else None
    OUT.mkdir(exist_ok=True)
    inc = OUT / "ar_extract.inc"
    harness = HERE / "ar_ref_harness.cpp"
    newest = max(header.stat().st_mtime, harness.stat().st_mtime, Path(__file__).stat().st_mtime)
    if not force and LIB.exists() and LIB.stat().st_mtime > newest:
        return LIB
    inc.write_text(extract(header.read_text()))
    cmd = ["g++", "-std=c++20", "-O1", "-shared", "-fPIC", "-pthread", "-w",
           "-I/usr/local/cuda/include", f"-I{HERE}", str(harness), "-o", str(LIB)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("g++ failed on the reference cut:\n" + proc.stderr[-4000:])
    return LIB


if __name__ == "__main__":
    print(build(*(sys.argv[1:2]), force=True))

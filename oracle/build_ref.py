"""Compiles the reference's own arch-agnostic kernels (in place, from the reference checkout) plus
oracle/ref_harness.cu into oracle/_ref/libeps_ref.so for sm_100a.

TEST INFRASTRUCTURE ONLY.  Needs the reference checkout ($EPS_REFERENCE, or the default location in the code);
where it is absent the prebuilt library, if any, is used as is.  Nothing from the reference is copied.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT_DIR, "libeps_ref.so")

REF_SOURCES = [
    "src/scheduler/comm_expander.cu",
    "src/scheduler/comm_expander_ver2.cu",
    "src/scheduler/gemm_expander.cu",
    "src/scheduler/gemm_expander_ver2.cu",
    "src/scheduler/local_reducer.cu",
    "src/scheduler/local_reducer_ver2.cu",
    "src/scheduler/global_reducer.cu",
    "src/scheduler/global_reducer_ver2.cu",
    "src/scheduler/zero_reducer.cu",
    "src/executor/activations.cu",
    "src/quant/fp8.cu",
    "src/common/debug.cu",
    "src/utils/topk_sigmoid.cu",
    "src/utils/rms_norm.cu",
    "src/fast_ep/all_to_all/fast_ep_kernels.cu",
]


def build(force: bool = False) -> str | None:
    ref = os.environ.get("EPS_REFERENCE", "/root/reference")
    if not os.path.isdir(os.path.join(ref, "src")):
        return LIB if os.path.exists(LIB) else None
    if os.path.exists(LIB) and not force:
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    srcs = [os.path.join(ref, s) for s in REF_SOURCES] + [os.path.join(HERE, "ref_harness.cu")]
    cmd = [nvcc, "-std=c++17", "-O3", "-shared", "-Xcompiler", "-fPIC", "-DENABLE_BF16", "-DENABLE_FP8", "-DNDEBUG",
           "--expt-relaxed-constexpr", "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static",
           "-I", ref, "-I", os.path.join(HERE, "ref_stubs"), "-o", LIB, *srcs]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout[-4000:] + r.stderr[-8000:])
        raise RuntimeError("building the reference kernels failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))

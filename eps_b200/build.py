"""Builds libeps_b200.so (sm_100a) from eps_b200/csrc with nvcc, in-tree.

Usage: python -m eps_b200.build [--force]
nvcc cross-compiles without a GPU, so this also serves as the build check on a CPU-only machine.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libeps_b200.so")
OBJ_DIR = os.path.join(HERE, "csrc", "_obj")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps():
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hdrs.append(os.path.join(HERE, "..", "include", "eps_b200.h"))
    return hdrs


def _stale(target, inputs):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(i) > t for i in inputs)


def build(force: bool = False, verbose: bool = False) -> str:
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    os.makedirs(OBJ_DIR, exist_ok=True)
    srcs, deps = _sources(), _deps()
    jobs = []
    for src in srcs:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        if force or _stale(obj, [src] + deps):
            jobs.append((src, obj))

    def compile_one(job):
        src, obj = job
        cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".ptxas.log")
        with open(log, "w") as f:
            f.write(r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(compile_one, jobs))
    objs = [os.path.join(OBJ_DIR, os.path.basename(s)[:-3] + ".o") for s in srcs]
    if force or jobs or _stale(LIB, objs):
        cmd = [nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
               "-cudart", "static", "-Xcompiler", "-fPIC"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


TORCH_SRC = os.path.join(HERE, "csrc_torch", "executor_ops.cpp")
TORCH_LIB = os.path.join(HERE, "libexecutor_.so")


def build_torch_ops(force: bool = False) -> str:
    """Builds libexecutor_.so: the TORCH_LIBRARY registration of the executor ops (namespace `executor`, the
    reference's library name) over libeps_b200.so.  Host-only C++ (g++), linked against the installed torch."""
    import sysconfig

    import torch
    from torch.utils import cpp_extension as ce

    build()
    if not force and not _stale(TORCH_LIB, [TORCH_SRC, LIB, os.path.join(HERE, "..", "include", "eps_b200.h")]):
        return TORCH_LIB
    inc = ce.include_paths() + [sysconfig.get_paths()["include"], "/usr/local/cuda/include"]
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", TORCH_SRC, "-o", TORCH_LIB,
           *[f"-I{i}" for i in inc], f"-L{libdir}", "-ltorch", "-ltorch_cpu", "-lc10", "-lc10_cuda", f"-L{HERE}",
           "-l:libeps_b200.so", f"-Wl,-rpath,{libdir}", "-Wl,-rpath,$ORIGIN"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"building libexecutor_.so failed:\n{r.stderr[-4000:]}")
    return TORCH_LIB


def load_torch_ops():
    """torch.ops.load_library(libexecutor_.so) -> torch.ops.executor (reference python/eps/executor/ops.py:9-17)."""
    import torch

    if not os.path.exists(TORCH_LIB):
        raise RuntimeError(f"{TORCH_LIB} is missing: run eps_b200.build.build_torch_ops()")
    torch.ops.load_library(TORCH_LIB)
    return torch.ops.executor


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--torch-ops" in sys.argv:
        print(build_torch_ops(force="--force" in sys.argv))

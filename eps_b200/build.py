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


TORCH_DIR = os.path.join(HERE, "csrc_torch")
COMPAT = os.path.join(HERE, "eps")   # the drop-in `eps` package: eps/<pkg>/lib<name>.so next to its ops.py
# library -> (source, package directory, needs NCCL): the six names python/eps/<pkg>/ops.py loads in the reference
TORCH_LIBS = {
    "libscheduler_.so": ("scheduler_ops.cpp", "scheduler", True),
    "libexecutor_.so": ("executor_ops.cpp", "executor", False),
    "libfast_ep.so": ("fast_ep_ops.cpp", "fast_ep", True),
    "libfast_oep.so": ("fast_oep_ops.cpp", "fast_oep", True),
    "libcommunication_.so": ("communication_ops.cpp", "communication", True),
    "libutils_.so": ("utils_ops.cpp", "utils", False),
}


def torch_lib_path(name: str) -> str:
    return os.path.join(COMPAT, TORCH_LIBS[name][1], name)


def build_torch_ops(force: bool = False) -> list:
    """Builds the six torch-op libraries (TORCH_LIBRARY registrations with the reference's namespaces and op names)
    over libeps_b200.so into eps_b200/eps/<pkg>/, where the drop-in `eps` package loads them from.  Host-only C++
    (g++), linked against the installed torch, its NCCL and its CUDA runtime."""
    import sysconfig

    import torch
    from torch.utils import cpp_extension as ce

    build()
    site = os.path.dirname(os.path.dirname(torch.__file__))
    inc = ce.include_paths() + [sysconfig.get_paths()["include"], "/usr/local/cuda/include",
                                os.path.join(site, "nvidia", "nccl", "include")]
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    nccl_dir = os.path.join(site, "nvidia", "nccl", "lib")
    rt_dir = os.path.join(site, "nvidia", "cuda_runtime", "lib")
    if not os.path.exists(os.path.join(rt_dir, "libcudart.so.12")):
        rt_dir = "/usr/local/cuda/lib64"
    hdrs = [os.path.join(TORCH_DIR, f) for f in os.listdir(TORCH_DIR) if f.endswith(".hpp")]
    hdrs += [LIB, os.path.join(HERE, "..", "include", "eps_b200.h")]
    out = []

    def one(item):
        name, (src, pkg, nccl) = item
        src = os.path.join(TORCH_DIR, src)
        if not os.path.exists(src):
            return None
        dst = torch_lib_path(name)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        if not force and not _stale(dst, [src] + hdrs):
            return dst
        cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-Wno-deprecated-declarations",
               f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", src, "-o", dst,
               *[f"-I{i}" for i in inc], f"-L{libdir}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
               f"-L{HERE}", "-l:libeps_b200.so", f"-L{rt_dir}", "-l:libcudart.so.12",
               f"-Wl,-rpath,{libdir}", f"-Wl,-rpath,{rt_dir}", "-Wl,-rpath,$ORIGIN/../.."]
        if nccl:
            cmd += [f"-L{nccl_dir}", "-l:libnccl.so.2", f"-Wl,-rpath,{nccl_dir}"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"building {name} failed:\n{r.stderr[-6000:]}")
        return dst

    with ThreadPoolExecutor(max_workers=6) as ex:
        out = [p for p in ex.map(one, TORCH_LIBS.items()) if p]
    return out


def load_torch_ops(name: str = "libexecutor_.so"):
    """torch.ops.load_library(<name>) -> its torch.ops namespace (reference python/eps/<pkg>/ops.py:9-17)."""
    import torch

    path = torch_lib_path(name)
    if not os.path.exists(path):
        raise RuntimeError(f"{path} is missing: run eps_b200.build.build_torch_ops()")
    torch.ops.load_library(path)
    return getattr(torch.ops, TORCH_LIBS[name][1])


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--torch-ops" in sys.argv:
        print(build_torch_ops(force="--force" in sys.argv))

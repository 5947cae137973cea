"""Builds the native libraries in-tree (no JIT cache, nothing installed elsewhere):

    mops_b200/lib/libmops.so        the sm_100a kernels + C++ API + C ABI (no torch dependency)
    mops_b200/lib/libmops_torch.so  TORCH_LIBRARY(mops) autograd ops on top of it

    python -m mops_b200.build [--force] [--no-torch]

Objects are rebuilt only when a source or header is newer. nvcc cross-compiles for
sm_100a without a GPU.
"""
import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "lib")
OBJ = os.path.join(HERE, "build")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
HOST_CXX = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH + ["-lineinfo", "-O3", "-std=c++17", "-ccbin", HOST_CXX, "-Xcompiler",
                     "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr"]

KERNEL_SOURCES = ["runtime.cu", "hpe.cu", "sap.cu", "opsa.cu", "sasaw.cu", "sort.cu", "capi.cu",
                  "host_stubs.cpp"]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".hpp", ".cuh", ".h"))]
    hs.append(os.path.join(INCLUDE, "mops.h"))
    return hs


def _run(cmd):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + r.stdout)
    return r.stdout


def build_core(force=False, verbose=False):
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    headers = _headers()
    jobs, objs = [], []
    for src in KERNEL_SOURCES:
        path = os.path.join(CSRC, src)
        obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
        objs.append(obj)
        if force or _newer(obj, [path] + headers):
            cmd = [NVCC] + NVCC_FLAGS + ["-x", "cu", "-c", path, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            for out in ex.map(_run, jobs):
                if verbose and out:
                    print(out)
    lib = os.path.join(LIB, "libmops.so")
    if force or jobs or _newer(lib, objs):
        _run([NVCC] + ARCH + ["-shared", "-ccbin", HOST_CXX, "-o", lib] + objs +
             ["-cudart", "shared"])
    return lib


def build_torch(force=False):
    import torch
    from torch.utils import cpp_extension

    core = build_core()
    src = os.path.join(CSRC, "torch_ops.cpp")
    if not os.path.exists(src):
        return None
    lib = os.path.join(LIB, "libmops_torch.so")
    if not (force or _newer(lib, [src, core] + _headers())):
        return lib
    inc = []
    for p in cpp_extension.include_paths(device_type="cuda"):
        inc += ["-isystem", p]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = [HOST_CXX, "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
           "-I", CSRC, "-I", INCLUDE] + inc + [src, "-o", lib, "-L", LIB, "-lmops",
           "-L", torch_lib, "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
           "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    _run(cmd)
    return lib


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--no-torch", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register/spill report")
    a = ap.parse_args()
    print(build_core(a.force, a.verbose))
    if not a.no_torch:
        print(build_torch(a.force))


if __name__ == "__main__":
    sys.exit(main())

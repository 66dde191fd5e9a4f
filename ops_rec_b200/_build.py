"""In-tree build of the native libraries (no JIT cache: the .so files sit next to this file).

  libhstu_b200.so   the C-ABI library: CUDA kernels for sm_100a + entry points (include/hstu_b200.h); nvcc only
  _torch_shim.so    registers the operators with torch under the reference's schema strings - ops_rec::hstu_jagged
                    (.equal / .delta), hstu_jagged_backward (.equal / .delta), hstu_dense, hstu_paged, ln_mul,
                    distance_in_linear_silu - with their Meta implementations, and forwards to the C ABI

Run `python ops_rec_b200/_build.py` (or call build_all()) after changing anything under csrc/.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
ROOT = os.path.dirname(PKG)
LIB = os.path.join(PKG, "libhstu_b200.so")
SHIM = os.path.join(PKG, "_torch_shim.so")

CUDA_SOURCES = ["hstu_api.cu", "hstu_sched.cu", "hstu_generic.cu", "hstu_tc.cu", "hstu_static.cu", "hstu_paged.cu", "hstu_bwd_generic.cu", "hstu_bwd_tc.cu", "ln_mul.cu", "in_linear_silu.cu", "in_linear_silu_bwd.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc():
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    exe = os.path.join(cuda_home, "bin", "nvcc")
    return exe if os.path.exists(exe) else (shutil.which("nvcc") or "nvcc")


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _deps():
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(ROOT, "include", "hstu_b200.h"))
    deps.append(os.path.join(ROOT, "include", "hstu_b200_testing.h"))
    return deps


def build_lib(force=False, verbose=False):
    srcs = [os.path.join(CSRC, s) for s in CUDA_SOURCES]
    if not force and not _stale(LIB, _deps()):
        return LIB
    cmd = [_nvcc(), "-O3", "-std=c++17", "-lineinfo", "--threads", "0", *ARCH, "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared",
           "-cudart", "shared", "-I", os.path.join(ROOT, "include"), "-o", LIB, *srcs]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    _run(cmd)
    return LIB


def build_shim(force=False):
    src = os.path.join(CSRC, "torch_shim.cpp")
    if not force and not _stale(SHIM, [src, os.path.join(ROOT, "include", "hstu_b200.h")]):
        return SHIM
    import torch
    from torch.utils import cpp_extension as ce

    inc = [f"-I{p}" for p in ce.include_paths(device_type="cuda")] + [f"-I{os.path.join(ROOT, 'include')}"]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_lib = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "lib64")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
           "-DTORCH_API_INCLUDE_EXTENSION_H", *inc, src, "-o", SHIM,
           f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
           f"-L{cuda_lib}", "-lcudart", f"-L{PKG}", "-l:libhstu_b200.so",
           f"-Wl,-rpath,{torch_lib}", "-Wl,-rpath,$ORIGIN"]
    _run(cmd)
    return SHIM


def _run(cmd):
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build failed:\n" + " ".join(cmd) + "\n" + proc.stdout)
    if proc.stdout.strip():
        sys.stderr.write(proc.stdout)


def build_all(force=False, verbose=False):
    build_lib(force=force, verbose=verbose)
    build_shim(force=force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built", LIB, SHIM)

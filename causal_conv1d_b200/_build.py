"""In-tree build of the two native libraries of this package.

``libcc1d.so``       CUDA kernels + the C ABI of ``include/cc1d.h``; nvcc, sm_100a only,
                     no torch dependency.
``_cc1d_torch.so``   the PyTorch extension (``csrc/causal_conv1d.cpp``) that fills the C-ABI
                     parameter blocks; g++, links ``libcc1d.so`` through ``$ORIGIN``.

Both land next to this file so that they travel with the source tree.  ``build()`` is
incremental: a library is rebuilt when any of its sources is newer than it.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(ROOT, "include")
OBJ = os.environ.get("CC1D_BUILD_DIR", os.path.join(ROOT, "build", "cc1d"))

LIB_CC1D = os.path.join(PKG, "libcc1d.so")
LIB_TORCH = os.path.join(PKG, "_cc1d_torch.so")

CU_SOURCES = ["cc1d_api.cu", "cc1d_fwd.cu", "cc1d_bwd.cu", "cc1d_update.cu", "cc1d_varlen.cu",
              "cc1d_prefill.cu", "cc1d_peer.cu"]
CU_HEADERS = ["cc1d_common.cuh", "cc1d_kernels.h", "cc1d_tma.cuh", os.path.join(INCLUDE, "cc1d.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "--use_fast_math",   # flush-to-zero special-function paths; state copies never go through arithmetic
    "-Xptxas", "-v",
]


# extra nvcc flags (e.g. -DCC1D_CF_KVECS=8) for tuning experiments
NVCC_FLAGS += os.environ.get("CC1D_EXTRA_NVCC_FLAGS", "").split()


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if os.path.exists(cand):
        return cand
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found: the CUDA kernels of causal_conv1d_b200 cannot be built")
    return found


def _newer(srcs, target) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in srcs)


def _run(cmd, log_name):
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    os.makedirs(OBJ, exist_ok=True)
    with open(os.path.join(OBJ, log_name), "w") as f:
        f.write(" ".join(cmd) + "\n" + res.stdout)
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError(f"build step failed: {' '.join(cmd[:3])} ... (log: build/cc1d/{log_name})")
    return res.stdout


def build_kernels(force: bool = False, verbose: bool = False) -> str:
    """nvcc: csrc/*.cu -> libcc1d.so (sm_100a)."""
    hdrs = [h if os.path.isabs(h) else os.path.join(CSRC, h) for h in CU_HEADERS]
    srcs = [os.path.join(CSRC, s) for s in CU_SOURCES]
    if not (force or _newer(srcs + hdrs + [__file__], LIB_CC1D)):
        return LIB_CC1D
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()

    def compile_one(src):
        obj = os.path.join(OBJ, os.path.basename(src) + ".o")
        if force or _newer([src] + hdrs + [__file__], obj):
            out = _run([nvcc, *NVCC_FLAGS, "-I", INCLUDE, "-I", CSRC, "-c", src, "-o", obj],
                       os.path.basename(src) + ".log")
            if verbose:
                print(out)
        return obj

    with ThreadPoolExecutor(max_workers=len(srcs)) as ex:
        objs = list(ex.map(compile_one, srcs))
    _run([nvcc, "-shared", "-o", LIB_CC1D, *objs, "-gencode", "arch=compute_100a,code=sm_100a"], "link_cc1d.log")
    return LIB_CC1D


def build_torch_ext(force: bool = False) -> str:
    """g++: csrc/causal_conv1d.cpp -> _cc1d_torch.so (pybind11 module linking libcc1d.so)."""
    src = os.path.join(CSRC, "causal_conv1d.cpp")
    if not (force or _newer([src, os.path.join(INCLUDE, "cc1d.h"), LIB_CC1D, __file__], LIB_TORCH)):
        return LIB_TORCH
    import sysconfig

    import torch
    from torch.utils import cpp_extension as ce

    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc = ce.include_paths() + [sysconfig.get_paths()["include"], os.path.join(cuda_home, "include"), INCLUDE]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           "-DTORCH_EXTENSION_NAME=_cc1d_torch", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for i in inc:
        cmd += ["-isystem", i]
    cmd += [src, "-o", LIB_TORCH,
            "-L", PKG, "-l:libcc1d.so", "-Wl,-rpath,$ORIGIN",
            "-L", torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            f"-Wl,-rpath,{torch_lib}"]
    _run(cmd, "torch_ext.log")
    return LIB_TORCH


def build(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force=force, verbose=verbose)
    build_torch_ext(force=force)


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB_CC1D)
    print(LIB_TORCH)

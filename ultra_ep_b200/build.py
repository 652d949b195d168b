"""In-tree build of the native library (nvcc, sm_100a) and of the PyTorch extension shim.

    python -m ultra_ep_b200.build            # build both if stale
    python -m ultra_ep_b200.build --force

Products (kept out of version control, carried to GPU machines as files):
    ultra_ep_b200/lib/libuep_b200.so     C-ABI library: kernels + host runtime (no torch)
    ultra_ep_b200/_C*.so                 pybind/torch shim exposing the reference's `_C` surface
"""

from __future__ import annotations

import argparse
import concurrent.futures
import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "_build")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libuep_b200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

CUDA_SOURCES = ["host_common.cu", "plan.cu", "reroute.cu", "weight_sync.cu", "grad_reduce.cu", "manager.cu"]
HEADERS = ["common.cuh", "solver.cuh", "internal.h", os.path.join(INCLUDE, "uep_b200.h")]

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "--expt-extended-lambda", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
]


def _nvcc() -> str:
    path = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(path):
        raise RuntimeError("nvcc not found: the native library cannot be built on this machine")
    return path


def _newest(paths) -> float:
    return max(os.path.getmtime(p) for p in paths)


def _header_paths():
    return [h if os.path.isabs(h) else os.path.join(CSRC, h) for h in HEADERS]


def native_is_stale() -> bool:
    srcs = [os.path.join(CSRC, s) for s in CUDA_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    if not os.path.exists(LIB_PATH):
        return True
    return os.path.getmtime(LIB_PATH) < _newest(srcs + _header_paths())


def build_native(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu for sm_100a and link libuep_b200.so. Returns its path."""
    if not force and not native_is_stale():
        return LIB_PATH
    os.makedirs(OBJ_DIR, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)
    nvcc = _nvcc()
    srcs = [s for s in CUDA_SOURCES if os.path.exists(os.path.join(CSRC, s))]
    hdr_time = _newest(_header_paths())

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        src_path = os.path.join(CSRC, src)
        if not force and os.path.exists(obj) and os.path.getmtime(obj) > max(os.path.getmtime(src_path), hdr_time):
            return obj
        cmd = [nvcc, *NVCC_FLAGS, "-I", INCLUDE, "-c", src_path, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            sys.stderr.write(res.stderr)
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(6, len(srcs))) as pool:
        objs = list(pool.map(compile_one, srcs))
    link = [nvcc, "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


def ext_path() -> str:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return os.path.join(HERE, "_C" + suffix)


def ext_is_stale() -> bool:
    p = ext_path()
    src = os.path.join(CSRC, "torch_ext.cpp")
    if not os.path.exists(src):
        return False
    if not os.path.exists(p):
        return True
    return os.path.getmtime(p) < _newest([src, os.path.join(INCLUDE, "uep_b200.h")])


def build_ext(force: bool = False) -> str | None:
    """Compile the torch/pybind shim against libuep_b200.so (g++, torch headers)."""
    src = os.path.join(CSRC, "torch_ext.cpp")
    if not os.path.exists(src):
        return None
    if not force and not ext_is_stale():
        return ext_path()
    import torch
    from torch.utils import cpp_extension

    includes = cpp_extension.include_paths()
    try:
        includes = cpp_extension.include_paths("cuda")
    except TypeError:
        pass
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-Wall", "-Wno-unused-variable",
           "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           "-I", INCLUDE, "-I", sysconfig.get_paths()["include"]]
    for inc in includes:
        cmd += ["-isystem", inc]
    cuda_inc = "/usr/local/cuda/include"
    if os.path.isdir(cuda_inc):
        cmd += ["-isystem", cuda_inc]
    cmd += [src, "-o", ext_path(), f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10",
            "-ltorch_cuda", "-lc10_cuda", f"-L{LIB_DIR}", "-luep_b200",
            f"-Wl,-rpath,{torch_lib}", "-Wl,-rpath,$ORIGIN/lib"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"torch extension build failed:\n{res.stdout}\n{res.stderr}")
    return ext_path()


def build_all(force: bool = False, verbose: bool = False):
    lib = build_native(force=force, verbose=verbose)
    ext = build_ext(force=force)
    return lib, ext


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas resource usage")
    ap.add_argument("--native-only", action="store_true")
    a = ap.parse_args()
    print(build_native(force=a.force, verbose=a.verbose))
    if not a.native_only:
        print(build_ext(force=a.force))

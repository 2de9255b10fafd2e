"""In-tree build of the CUDA library (``librmn_b200.so``) for sm_100a.

nvcc cross-compiles without a GPU; the shared object lands beside the
sources' package (``riemannengine_b200/lib/``) so that it travels with the
source tree. Nothing is cached outside the tree.
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
LIB_DIR = os.path.join(PKG, "lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")
LIB_PATH = os.path.join(LIB_DIR, "librmn_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-I" + INCLUDE, "-I" + CSRC,
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps_mtime() -> float:
    files = sources() + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    files += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE)]
    return max(os.path.getmtime(f) for f in files)


def build_library(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    """Compile every ``csrc/*.cu`` and link ``librmn_b200.so``; returns its path."""
    if not force and os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= _deps_mtime():
        return LIB_PATH
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    newest_hdr = max([os.path.getmtime(os.path.join(CSRC, f)) for f in os.listdir(CSRC) if f.endswith(".cuh")]
                     + [os.path.getmtime(os.path.join(INCLUDE, f)) for f in os.listdir(INCLUDE)])

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), newest_hdr):
            return obj
        cmd = [nvcc] + NVCC_FLAGS + extra + ["-c", src, "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode != 0 or ptxas_info:
            sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources()))) as ex:
        objs = list(ex.map(compile_one, sources()))
    tmp = LIB_PATH + f".tmp{os.getpid()}"
    cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", tmp] + objs
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("link failed")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv))


# ------------------------------------------------------------------------------------------
# C++20 / LibTorch host layer (riemann_cpp) + its pybind11 module
# ------------------------------------------------------------------------------------------
HOST_DIR = os.path.join(PKG, "riemann_cpp")
HOST_LIB = os.path.join(LIB_DIR, "_C.so")


def build_host_extension(force: bool = False, verbose: bool = False) -> str:
    """Compile ``riemann_cpp/*.cpp`` with g++ against LibTorch and link them to librmn_b200.so."""
    import sysconfig

    import torch

    build_library()
    srcs = sorted(os.path.join(HOST_DIR, f) for f in os.listdir(HOST_DIR) if f.endswith(".cpp"))
    deps = srcs + [os.path.join(HOST_DIR, f) for f in os.listdir(HOST_DIR) if f.endswith(".hpp")]
    deps.append(os.path.join(INCLUDE, "rmn_b200.h"))
    if not force and os.path.exists(HOST_LIB) and os.path.getmtime(HOST_LIB) >= max(os.path.getmtime(f) for f in deps):
        return HOST_LIB
    tdir = os.path.dirname(torch.__file__)
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(_nvcc())), "include")
    flags = ["-std=c++20", "-O2", "-fPIC", "-w", "-DTORCH_EXTENSION_NAME=_C",
             f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
             "-I" + INCLUDE, "-I" + HOST_DIR, "-isystem", os.path.join(tdir, "include"),
             "-isystem", os.path.join(tdir, "include", "torch", "csrc", "api", "include"),
             "-isystem", sysconfig.get_paths()["include"], "-isystem", cuda_inc]
    os.makedirs(OBJ_DIR, exist_ok=True)

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ_DIR, "host_" + os.path.basename(src)[:-4] + ".o")
        newest = max(os.path.getmtime(f) for f in deps if not f.endswith(".cpp"))
        if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), newest):
            return obj
        cmd = [cxx] + flags + ["-c", src, "-o", obj]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"g++ failed on {src}")
        return obj

    with ThreadPoolExecutor(max_workers=len(srcs)) as ex:
        objs = list(ex.map(compile_one, srcs))
    tmp = HOST_LIB + f".tmp{os.getpid()}"
    cmd = [cxx, "-shared", "-o", tmp] + objs + [
        "-L" + os.path.join(tdir, "lib"), "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
        "-ltorch_python", "-L" + LIB_DIR, "-lrmn_b200", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + os.path.join(tdir, "lib")]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
        raise RuntimeError("host extension link failed")
    os.replace(tmp, HOST_LIB)
    return HOST_LIB

"""Builds ``lib/libkan_b200.so`` (the C-ABI library) with nvcc for sm_100a.

    python torchsplinekan_b200/build.py [--force] [--verbose]

The library has no dependency on PyTorch or on libcuda at link time; it is
loaded with ctypes.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libkan_b200.so")
SOURCES = ["kan_capi.cu", "kan_simt.cu", "kan_reg.cu", "kan_dense64.cu", "kan_tc.cu", "kan_tc_edge.cu", "kan_refit.cu", "kan_collective.cu"]
# test-only library (operand-layout self-test); never loaded by the package
SELFTEST_SOURCE = "kan_selftest.cu"
SELFTEST_PATH = os.path.join(LIB_DIR, "libkan_b200_selftest.so")
# PyTorch operator layer (TORCH_LIBRARY + pybind + autograd node), host C++ only
EXT_SOURCE = "kan_torch_ext.cpp"
HEADERS = ["kan_device.cuh", "kan_dmma.cuh", "kan_internal.h", "kan_table.cuh", "kan_tc_ptx.cuh", "kan_tc_common.cuh", os.path.join("..", "..", "include", "kan_b200.h")]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the KAN B200 library cannot be built")
    return cand


def _older_than(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _stale() -> bool:
    return _older_than(LIB_PATH, [os.path.join(CSRC, s) for s in SOURCES + HEADERS])


def ext_path() -> str:
    import sysconfig
    return os.path.join(PKG, "_C" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_selftest(force: bool = False) -> str:
    """The operand-layout self-test kernel as a library of its own (loaded by the tests only)."""
    src = os.path.join(CSRC, SELFTEST_SOURCE)
    if not force and not _older_than(SELFTEST_PATH, [src, os.path.join(CSRC, "kan_tc_ptx.cuh"), os.path.join(CSRC, "kan_dmma.cuh")]):
        return SELFTEST_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [_nvcc(), *ARCH_FLAGS, *NVCC_FLAGS, "-shared", src, "-o", SELFTEST_PATH + ".tmp"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {SELFTEST_SOURCE}:\n{r.stdout}\n{r.stderr}")
    os.replace(SELFTEST_PATH + ".tmp", SELFTEST_PATH)
    return SELFTEST_PATH


def build_extension(force: bool = False) -> str:
    """Compiles the PyTorch operator layer (csrc/kan_torch_ext.cpp) into ``_C.<abi>.so`` beside the
    package's Python files; it links libkan_b200.so (found at run time through ``$ORIGIN/lib``)."""
    import sysconfig
    target = ext_path()
    src = os.path.join(CSRC, EXT_SOURCE)
    if not force and not _older_than(target, [src, os.path.join(PKG, "..", "include", "kan_b200.h"), LIB_PATH]):
        return target
    import torch
    from torch.utils import cpp_extension as ce
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cudart_dir = os.path.join(os.path.dirname(torch.__file__), "..", "nvidia", "cuda_runtime", "lib")
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cudart = ["-L" + cudart_dir, "-l:libcudart.so.12", "-Wl,-rpath," + os.path.abspath(cudart_dir)] \
        if os.path.exists(os.path.join(cudart_dir, "libcudart.so.12")) else ["-L" + os.path.join(cuda_home, "lib64"), "-lcudart"]
    # The system compiler, whatever $CXX says: the extension must use the same libstdc++ as the
    # interpreter's other extension modules (a toolchain that links its own copy statically breaks
    # stream formatting inside the module).
    cxx = shutil.which("g++", path="/usr/bin:/usr/local/bin:/bin") or shutil.which("g++") or "g++"
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *["-I" + p for p in ce.include_paths()], "-I" + sysconfig.get_paths()["include"],
           "-I" + os.path.join(cuda_home, "include"), src, "-o", target + ".tmp",
           "-L" + torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
           "-L" + LIB_DIR, "-lkan_b200", "-Wl,-rpath,$ORIGIN/lib", "-Wl,-rpath," + torch_lib, *cudart]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"g++ failed for {EXT_SOURCE}:\n{r.stdout}\n{r.stderr[-6000:]}")
    os.replace(target + ".tmp", target)
    return target


def build_all(force: bool = False, verbose: bool = False) -> str:
    """Library, self-test library and operator extension, each only when out of date."""
    build_library(force, verbose)
    build_selftest(force)
    build_extension(force)
    return LIB_PATH


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compiles the CUDA sources if the library is missing or older than them."""
    if not force and not _stale():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    obj_dir = os.path.join(PKG, "build")
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = _nvcc()

    def compile_one(src: str) -> str:
        obj = os.path.join(obj_dir, src.replace(".cu", ".o"))
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=len(SOURCES)) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    tmp = LIB_PATH + ".tmp"
    cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", tmp, *objs]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose="--verbose" in sys.argv))

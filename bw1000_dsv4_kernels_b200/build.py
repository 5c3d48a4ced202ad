"""In-tree build of the native code: explicit nvcc / g++ command lines, no JIT cache.

  libdsv4_w8a8.so            the CUDA kernels behind the C-ABI of include/dsv4_w8a8.h
  dsv4_native_ext.<abi>.so   the pybind11 / torch operator module on top of it

Both land next to this file so that they travel with the source tree.  `python -m
bw1000_dsv4_kernels_b200.build` builds what is out of date; `--force` rebuilds.
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(ROOT, "include")

LIB_NAME = "libdsv4_w8a8.so"
LIB_PATH = os.path.join(HERE, LIB_NAME)
EXT_PATH = os.path.join(HERE, "dsv4_native_ext" + sysconfig.get_config_var("EXT_SUFFIX"))

CUDA_SOURCES = ["rowwise_quant.cu", "gemm_i8_sm100.cu", "moe_segments.cu", "c_abi.cu"]
CUDA_HEADERS = ["w8a8_arith.cuh", "sm100_ptx.cuh", "launch_common.h", "gemm_i8_common.cuh", "gemm_i8_tile_kernel.cuh",
                "gemm_i8_pair_kernel.cuh", "gemm_i8_wt_kernel.cuh", "gemm_i8_stream_kernels.cuh"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _cuda_home() -> str:
    return os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)


def build_cuda_lib(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    srcs = [os.path.join(CSRC, s) for s in CUDA_SOURCES]
    deps = srcs + [os.path.join(CSRC, h) for h in CUDA_HEADERS] + [os.path.join(INCLUDE, "dsv4_w8a8.h"), __file__]
    if not force and _newer(LIB_PATH, deps):
        return LIB_PATH
    nvcc = os.path.join(_cuda_home(), "bin", "nvcc")
    # -fmad=false: a multiply and an add that the sources write as two rounded steps must stay two
    # instructions (fused forms are written explicitly where they are meant)
    cmd = [nvcc, *ARCH_FLAGS, "-lineinfo", "-O3", "-fmad=false", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
           "-Xcompiler", "-fvisibility=hidden", "--threads", "4", "-o", LIB_PATH, *srcs]
    if ptxas_info:
        cmd[1:1] = ["-Xptxas", "-v"]
    _run(cmd, verbose)
    return LIB_PATH


def build_torch_ext(force: bool = False, verbose: bool = False) -> str:
    src = os.path.join(CSRC, "torch_ext.cpp")
    deps = [src, os.path.join(INCLUDE, "dsv4_w8a8.h"), LIB_PATH, __file__]
    if not force and _newer(EXT_PATH, deps):
        return EXT_PATH
    import torch
    from torch.utils import cpp_extension as ce
    import pybind11

    inc = ce.include_paths() + [pybind11.get_include(), sysconfig.get_paths()["include"],
                                os.path.join(_cuda_home(), "include")]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
           "-DTORCH_EXTENSION_NAME=dsv4_native_ext", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    cmd += [f"-I{p}" for p in inc]
    cmd += [src, "-o", EXT_PATH, f"-L{HERE}", "-ldsv4_w8a8", f"-L{torch_lib}", "-lc10", "-lc10_cuda",
            "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    _run(cmd, verbose)
    return EXT_PATH


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cuda_lib(force, verbose)
    build_torch_ext(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
    print(LIB_PATH)
    print(EXT_PATH)

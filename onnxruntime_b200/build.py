"""In-tree native build: writes a ninja file and runs it.

Two shared objects are produced inside the package directory:

* ``lib/libortb200_kernels.so`` -- every ``csrc/cuda/*.cu`` compiled for
  sm_100a only (``-gencode arch=compute_100a,code=sm_100a``).  Pure CUDA, no
  PyTorch headers, C ABI (``csrc/cuda/ortb200_kernels.h``).
* ``_core*.so`` -- the C++ runtime (ONNX protobuf reader/writer, graph IR,
  optimizer, planner, executor, CPU kernels over ATen, GPU op wrappers) as a
  PyTorch C++ extension that links the kernel library.

Run ``python -m onnxruntime_b200.build`` (add ``--kernels-only`` to skip the
C++ runtime).  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import argparse
import glob
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "build")
LIBDIR = os.path.join(HERE, "lib")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
    "--expt-relaxed-constexpr",
]


def _cuda_home() -> str:
    for cand in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if cand and os.path.exists(os.path.join(cand, "bin", "nvcc")):
            return cand
    raise RuntimeError("nvcc not found")


def core_ext_name() -> str:
    return "_core" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so")


def write_ninja(kernels_only: bool = False) -> str:
    os.makedirs(BUILD, exist_ok=True)
    os.makedirs(LIBDIR, exist_ok=True)
    cuda = _cuda_home()
    cu_srcs = sorted(glob.glob(os.path.join(CSRC, "cuda", "*.cu")))
    cu_hdrs = sorted(glob.glob(os.path.join(CSRC, "cuda", "*.h")) + glob.glob(os.path.join(CSRC, "cuda", "*.cuh")))
    lines = [
        "ninja_required_version = 1.5",
        f"nvcc = {cuda}/bin/nvcc",
        "cxx = g++",
        "nvflags = " + " ".join(NVCC_FLAGS) + f" -I{CSRC}/cuda",
        "rule nvcc",
        "  command = $nvcc $nvflags -c $in -o $out",
        "  description = NVCC $in",
        "rule nvlink",
        f"  command = $nvcc -shared -o $out $in -L{cuda}/lib64 -lcudart",
        "  description = LINK $out",
    ]
    objs = []
    for src in cu_srcs:
        obj = os.path.join(BUILD, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        lines.append(f"build {obj}: nvcc {src} | " + " ".join(cu_hdrs))
    kern_so = os.path.join(LIBDIR, "libortb200_kernels.so")
    lines.append(f"build {kern_so}: nvlink " + " ".join(objs))
    defaults = [kern_so]

    cpp_srcs = sorted(glob.glob(os.path.join(CSRC, "core", "*.cc")))
    if cpp_srcs and not kernels_only:
        from torch.utils import cpp_extension as ce
        import pybind11

        incs = ce.include_paths() + [pybind11.get_include(), sysconfig.get_paths()["include"], f"{cuda}/include",
                                     os.path.join(CSRC, "cuda"), os.path.join(CSRC, "core")]
        torch_lib = ce.library_paths()[0]
        cxxflags = ("-O2 -g0 -std=c++17 -fPIC -fvisibility=hidden -Wall -Wno-unused-function -Wno-sign-compare "
                    "-Wno-unknown-pragmas -D_GLIBCXX_USE_CXX11_ABI=1 -DTORCH_EXTENSION_NAME=_core "
                    "-DTORCH_API_INCLUDE_EXTENSION_H " + " ".join(f"-isystem {i}" for i in incs))
        lines += [
            f"cxxflags = {cxxflags}",
            "rule cxx",
            "  command = $cxx -MMD -MF $out.d $cxxflags -c $in -o $out",
            "  depfile = $out.d",
            "  deps = gcc",
            "  description = CXX $in",
            "rule cxxlink",
            f"  command = $cxx -shared -o $out $in -L{torch_lib} -L{LIBDIR} -L{cuda}/lib64 "
            "-lc10 -ltorch_cpu -ltorch -ltorch_python -lc10_cuda -ltorch_cuda -lcudart -lortb200_kernels "
            f"-Wl,-rpath,{torch_lib} -Wl,-rpath,'$$ORIGIN/lib' -Wl,-rpath,{cuda}/lib64",
            "  description = LINK $out",
        ]
        cobjs = []
        for src in cpp_srcs:
            obj = os.path.join(BUILD, "core_" + os.path.basename(src)[:-3] + ".o")
            cobjs.append(obj)
            lines.append(f"build {obj}: cxx {src}")
        core_so = os.path.join(HERE, core_ext_name())
        lines.append(f"build {core_so}: cxxlink " + " ".join(cobjs) + f" | {kern_so}")
        defaults.append(core_so)
        # the same runtime without the Python bindings, behind the C API (ortb200_c_api.h)
        lines += [
            "rule cxxlink_c",
            f"  command = $cxx -shared -o $out $in -L{torch_lib} -L{LIBDIR} -L{cuda}/lib64 "
            "-lc10 -ltorch_cpu -ltorch -lc10_cuda -ltorch_cuda -lcudart -lortb200_kernels "
            f"-Wl,-rpath,{torch_lib} -Wl,-rpath,'$$ORIGIN' -Wl,-rpath,{cuda}/lib64",
            "  description = LINK $out",
        ]
        python_only = ("core_bindings.o", "core_python_ops.o")
        c_objs = [o for o in cobjs if os.path.basename(o) not in python_only]
        c_so = os.path.join(LIBDIR, "libortb200.so")
        lines.append(f"build {c_so}: cxxlink_c " + " ".join(c_objs) + f" | {kern_so}")
        defaults.append(c_so)
    lines.append("default " + " ".join(defaults))
    path = os.path.join(BUILD, "build.ninja")
    with open(path, "w") as f:
        f.write("\n".join(lines) + "\n")
    return path


def build(kernels_only: bool = False, verbose: bool = False) -> None:
    path = write_ninja(kernels_only)
    cmd = ["ninja", "-f", path] + (["-v"] if verbose else [])
    jobs = os.environ.get("ORTB200_BUILD_JOBS")
    if jobs:
        cmd += ["-j", jobs]
    res = subprocess.run(cmd, cwd=BUILD)
    if res.returncode != 0:
        raise RuntimeError("native build failed")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernels-only", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    build(a.kernels_only, a.verbose)
    print("build ok")

"""In-tree build of the mcop_b200 native code for sm_100a.

    python -m mcoplib_b200.build            # build what is out of date
    python -m mcoplib_b200.build --force

Two artefacts land next to this file:
  libmcop_b200.so  - the CUDA kernels behind the C ABI of include/mcop_b200.h (no torch dependency);
  op.<abi>.so      - the pybind11 / torch-library shims (csrc/torch_ext.cpp), linked against the first.
nvcc cross-compiles without a GPU, so the build also runs on a CPU-only machine.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(ROOT, "include")
BUILD = os.path.join(HERE, "build")

CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")

CU_SOURCES = ["api_common.cu", "norm_quant.cu", "norm_pad_quant.cu", "rope_kv.cu", "moe_route.cu", "moe_scatter.cu", "moe_gather.cu", "moe_act_quant.cu"]
# -fmad=false: products and sums are rounded separately, as the CPU evaluation of the same formulas does.
# Never --use_fast_math: division, sqrt and expf stay IEEE / full precision.
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-fmad=false", "-lineinfo",
              "-Xcompiler", "-fPIC", "-I" + INCLUDE, "-I" + CSRC]

LIB_NAME = "libmcop_b200.so"
EXT_SUFFIX = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
OP_NAME = "op" + EXT_SUFFIX


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed:\n" + " ".join(cmd) + "\n" + r.stdout)
    if verbose and r.stdout.strip():
        print(r.stdout)


def build_kernels(force=False, verbose=False, extra_nvcc=()) -> str:
    os.makedirs(BUILD, exist_ok=True)
    headers = [os.path.join(CSRC, h) for h in ("common.cuh", "tma_pipe.cuh", "rope_pipe.inl")] + [os.path.join(INCLUDE, "mcop_b200.h")]
    objs, jobs = [], []
    for src in CU_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(BUILD, src + ".o")
        objs.append(o)
        if force or not _newer(o, [s] + headers):
            jobs.append([NVCC] + NVCC_FLAGS + list(extra_nvcc) + ["-c", s, "-o", o])
    with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 1) or 1) as ex:
        list(ex.map(lambda c: _run(c, verbose), jobs))
    lib = os.path.join(HERE, LIB_NAME)
    if force or jobs or not _newer(lib, objs):
        _run([NVCC, "-shared", "-o", lib] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"], verbose)
    return lib


def moe_namespace(namespace: str) -> str:
    """torch.ops namespace of the MoE routing operators: `_moe_C` beside `_C`, `mcop_moe_C` beside `mcop_C`."""
    return namespace[:-1] + "moe_C" if namespace.endswith("_C") else namespace + "_moe"


def build_torch_ext(force=False, verbose=False, namespace="mcop_C") -> str:
    import torch
    from torch.utils import cpp_extension as ce

    src = os.path.join(CSRC, "torch_ext.cpp")
    out = os.path.join(HERE, OP_NAME)
    lib = os.path.join(HERE, LIB_NAME)
    if not force and _newer(out, [src, lib, os.path.join(INCLUDE, "mcop_b200.h"), os.path.join(CSRC, "debug_trace.hpp")]):
        return out
    inc = ["-I" + p for p in ce.include_paths()] + ["-I" + sysconfig.get_paths()["include"], "-I" + INCLUDE,
                                                    "-I" + os.path.join(CUDA_HOME, "include")]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-DTORCH_EXTENSION_NAME=op", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={abi}", f"-DMCOP_TORCH_NS={namespace}", f"-DMCOP_TORCH_NS_MOE={moe_namespace(namespace)}",
           "-Wno-attributes"] + inc + [src, "-o", out,
           "-L" + HERE, "-lmcop_b200", "-L" + torch_lib, "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
           "-ltorch_python", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + torch_lib]
    _run(cmd, verbose)
    return out


def build_all(force=False, verbose=False, namespace="mcop_C"):
    lib = build_kernels(force, verbose)
    ext = build_torch_ext(force, verbose, namespace)
    return lib, ext


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", "-v", action="store_true")
    ap.add_argument("--namespace", default="mcop_C", help="torch.ops namespace (use _C for a drop-in deployment)")
    a = ap.parse_args()
    print(build_all(a.force, a.verbose, a.namespace))

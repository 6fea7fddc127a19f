"""Build ``libmxmoe_b200.so`` in-tree with nvcc for sm_100a.

``python -m mxmoe_b200.build`` (or :func:`build`) compiles the CUDA sources under
``mxmoe_b200/csrc`` into ``mxmoe_b200/libmxmoe_b200.so``.  nvcc cross-compiles
without a GPU; the CUDA runtime is linked statically so the library loads on a
machine without a driver (the first call that needs a device then fails with
``MXMOE_ERR_NO_DEVICE``).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libmxmoe_b200.so")
SOURCES = ["capi.cu", "gg_kernel.cu", "gg_pair_kernel.cu", "gg_swap_kernel.cu", "act_kernels.cu", "had_kernels.cu", "route_kernels.cu", "ep_kernels.cu"]
HEADERS = ["ptx.cuh", "gg_common.cuh", "gg_types.h", "act_kernels.h", "had_kernels.h", "route_kernels.h", "ep_kernels.h", os.path.join("..", "..", "include", "mxmoe_b200.h")]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC=/path/to/nvcc")


def is_stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS]
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile the library if it is missing or older than its sources; return its path."""
    if not force and not is_stale():
        return LIB
    cmd = [
        _nvcc(), "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
        "-shared", "-Xcompiler", "-fPIC",
        "-Xptxas", "-v" if verbose else "-warn-spills",
        "-o", LIB + ".tmp",
    ] + os.environ.get("MXMOE_NVCC_FLAGS", "").split() + [os.path.join(CSRC, s) for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libmxmoe_b200.so (see stderr)")
    os.replace(LIB + ".tmp", LIB)   # a reader never sees a half-written library
    return LIB


OPS_LIB = os.path.join(HERE, "mxmoe_ops.so")


def build_torch_ext(force: bool = False) -> str:
    """Compile ``mxmoe_b200/mxmoe_ops.so``, the torch C++ extension with the reference's operator names
    (csrc/torch_ops.cpp), against the torch this interpreter imports and link it to ``libmxmoe_b200.so``."""
    src = os.path.join(CSRC, "torch_ops.cpp")
    if not force and os.path.exists(OPS_LIB) and os.path.getmtime(OPS_LIB) > max(os.path.getmtime(src), os.path.getmtime(LIB)):
        return OPS_LIB
    import sysconfig
    import torch
    from torch.utils import cpp_extension as ce
    inc = [f"-I{d}" for d in ce.include_paths()] + [f"-I{sysconfig.get_paths()['include']}"]
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(_nvcc())), "include")
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = (["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-DTORCH_EXTENSION_NAME=mxmoe_ops",
            f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-DTORCH_API_INCLUDE_EXTENSION_H"]
           + inc + [f"-I{cuda_inc}", src, "-o", OPS_LIB + ".tmp", f"-L{HERE}", "-l:libmxmoe_b200.so",
                    f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-lc10", "-lc10_cuda", "-ltorch_cuda",
                    "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"])
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr[-6000:])
        raise RuntimeError("building mxmoe_ops.so failed (see stderr)")
    os.replace(OPS_LIB + ".tmp", OPS_LIB)
    return OPS_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--ops" in sys.argv:
        print(build_torch_ext(force="--force" in sys.argv))

"""Builds libsessd.so (the CUDA library behind include/sessd.h) in-tree for sm_100a."""
from __future__ import annotations

import os
import shutil
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_HERE)
_CSRC = os.path.join(_HERE, "csrc")
LIB_PATH = os.path.join(_HERE, "libsessd.so")

SOURCES = ["capi.cu", "voxelize.cu", "rulebook.cu", "conv_simt.cu", "conv_umma.cu", "sparse2dense.cu", "voxelize_static.cu",
           "postprocess.cu", "nms.cu", "plugins.cu", "formats.cu", "trt_shim.cpp"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return nvcc


def tensorrt_include_dir():
    """Directory that holds TensorRT's NvInferPlugin.h, or None. csrc/trt_shim.cpp (the IPluginV2DynamicExt classes
    over the plugin mirrors) compiles to an empty object without it; with it the library also links nvinfer."""
    roots = [os.environ.get("TENSORRT_ROOT", ""), "/usr", "/usr/local", "/usr/local/cuda", "/usr/local/tensorrt",
             "/opt/tensorrt"]
    dirs = [os.path.join(r, sub) for r in roots if r for sub in ("include", "include/x86_64-linux-gnu", "targets/x86_64-linux/include")]
    dirs += [d for d in os.environ.get("CPATH", "").split(":") if d]
    for d in dirs:
        if os.path.exists(os.path.join(d, "NvInferPlugin.h")):
            return d
    return None


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(_CSRC, f) for f in os.listdir(_CSRC)] + [os.path.join(_ROOT, "include", "sessd.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles every .cu of the package into libsessd.so; returns its path."""
    if not force and not _stale():
        return LIB_PATH
    srcs = [os.path.join(_CSRC, s) for s in SOURCES if os.path.exists(os.path.join(_CSRC, s))]
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", os.path.join(_ROOT, "include"), "-I", _CSRC, "-o", LIB_PATH, *srcs]
    trt = tensorrt_include_dir()
    if trt:
        cmd += ["-I", trt, "-lnvinfer"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
        print(" ".join(cmd))
    subprocess.check_call(cmd)
    return LIB_PATH


if __name__ == "__main__":
    import sys

    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))

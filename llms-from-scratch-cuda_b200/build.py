"""In-tree build of libb200_linear.so (nvcc, sm_100a only).

    python llms-from-scratch-cuda_b200/build.py [--force] [--verbose]

The shared library lands next to this file so that it travels with the source tree; nothing
is installed into site-packages and no JIT cache is used.
"""
import argparse
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libb200_linear.so")
SHIM_LIB = os.path.join(HERE, "libb200_cublas_shim.so")
NVCC_FLAGS = ["-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "-shared"]


def _sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh"))) + [
        os.path.join(HERE, "..", "include", "b200_linear.h"), os.path.join(HERE, "..", "include", "b200_layers.h")]


def _fresh(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build(force=False, verbose=False):
    """Compile every CUDA translation unit of the package. Returns the library path."""
    if not force and _fresh(LIB, _sources()) and _fresh(SHIM_LIB, _sources()):
        return LIB
    if shutil.which("nvcc") is None:
        if os.path.exists(LIB):
            return LIB
        raise RuntimeError("nvcc not found and libb200_linear.so is not prebuilt")
    extra = ["-Xptxas", "-v"] if verbose else []
    units = [os.path.join(CSRC, f) for f in ("api.cu", "kernels_cuh_abi.cu", "layers_api.cu") if os.path.exists(os.path.join(CSRC, f))]
    subprocess.run(["nvcc"] + NVCC_FLAGS + extra + units + ["-o", LIB], check=True)
    shim = os.path.join(CSRC, "cublas_shim.cu")
    if os.path.exists(shim):
        subprocess.run(["nvcc"] + NVCC_FLAGS + [shim, "-o", SHIM_LIB], check=True)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))

"""Build recipe for the test oracle (TEST INFRASTRUCTURE — not part of the product).

  oracle/liboracle.so          gcc build of oracle/oracle_gemm.c (fp64 oracle, fp32 CPU baseline)
  oracle/_ref/libref_matmul.so the reference's unmodified cuda/matmul.cu (cuBLAS) plus the
                               extern "C" doorway oracle/ref_shim.cu, compiled from the
                               reference checkout where it lies.  Only built where that checkout
                               exists; the built file travels with the repository snapshot.

Run:  python oracle/build.py [--reference /path/to/llms-from-scratch-cuda]
"""
import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_REFERENCE = os.environ.get("LFS_CUDA_REFERENCE", "/root/reference")


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force=False):
    src = os.path.join(HERE, "oracle_gemm.c")
    out = os.path.join(HERE, "liboracle.so")
    if not force and _newer(out, [src]):
        return out
    if shutil.which("gcc") is None:
        if os.path.exists(out):
            return out
        raise RuntimeError("gcc not found and oracle/liboracle.so is not prebuilt")
    # x86-64-v3 (AVX2+FMA): the file is built on one machine and run on another.
    cmd = ["gcc", "-O3", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-shared", src, "-o", out, "-lm"]
    subprocess.run(cmd, check=True)
    return out


def build_reference(reference=DEFAULT_REFERENCE, force=False):
    """Returns the path of libref_matmul.so, or None when the reference checkout is absent
    and nothing was prebuilt."""
    out_dir = os.path.join(HERE, "_ref")
    out = os.path.join(out_dir, "libref_matmul.so")
    ref_src = os.path.join(reference, "cuda", "matmul.cu")
    shim = os.path.join(HERE, "ref_shim.cu")
    if not os.path.exists(ref_src) or shutil.which("nvcc") is None:
        return out if os.path.exists(out) else None
    if not force and _newer(out, [ref_src, shim]):
        return out
    os.makedirs(out_dir, exist_ok=True)
    cmd = ["nvcc", "-std=c++17", "-O3", "--use_fast_math", "-gencode", "arch=compute_100a,code=sm_100a",
           "-I", os.path.join(reference, "cuda"), "-shared", "-Xcompiler", "-fPIC",
           ref_src, shim, "-o", out, "-lcublas",
           "-Xlinker", "-rpath=/usr/local/cuda/lib64"]
    subprocess.run(cmd, check=True)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build_oracle(a.force))
    print(build_reference(a.reference, a.force))

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
# Where the reference checkout lies: --reference, else $LFS_CUDA_REFERENCE, else a directory named
# "reference" beside this repository.  Where none exists, only prebuilt files under oracle/_ref are used.
DEFAULT_REFERENCE = os.environ.get("LFS_CUDA_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


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
    ref_ce = os.path.join(reference, "cuda", "crossentropy.cu")
    # the layers that call the GEMMs, and what they call in turn
    ref_layers = [os.path.join(reference, "cuda", f) for f in ("attention.cu", "swiglu.cu", "rope.cu", "softmax.cu", "residual.cu",
                                                                  "adamw.cu")]
    shim = os.path.join(HERE, "ref_shim.cu")
    if not os.path.exists(ref_src) or shutil.which("nvcc") is None:
        return out if os.path.exists(out) else None
    if not force and _newer(out, [ref_src, ref_ce, shim] + ref_layers):
        return out
    os.makedirs(out_dir, exist_ok=True)
    cmd = ["nvcc", "-std=c++17", "-O3", "--use_fast_math", "-gencode", "arch=compute_100a,code=sm_100a",
           "-I", os.path.join(reference, "cuda"), "-shared", "-Xcompiler", "-fPIC",
           ref_src, ref_ce, shim] + ref_layers + ["-o", out, "-lcublas",
           "-Xlinker", "-rpath=/usr/local/cuda/lib64"]
    subprocess.run(cmd, check=True)
    return out


KERNEL_SOURCES = ["embedding.cu", "rmsnorm.cu", "rope.cu", "flash_attention.cu", "attention.cu", "swiglu.cu",
                  "softmax.cu", "crossentropy.cu", "residual.cu", "adamw.cu"]
# the callers of the GEMM path that the library also replaces (csrc/layers_api.cu exports their signatures)
LAYER_SOURCES = ["flash_attention.cu", "attention.cu", "swiglu.cu", "crossentropy.cu", "rmsnorm.cu", "residual.cu", "adamw.cu"]


def build_train(reference=DEFAULT_REFERENCE, model="llama2-mistral", force=False):
    """The reference's `train` program three times, from its sources where they lie:
         oracle/_ref/train_ref_<model>          as the reference builds it (cuda/matmul.cu -> cuBLAS)
         oracle/_ref/train_b200_<model>         the same host and kernel objects, with cuda/matmul.cu left out
                                                and libb200_linear.so (+ the cuBLAS stand-in) linked instead
         oracle/_ref/train_b200_layers_<model>  with cuda/attention.cu, flash_attention.cu, swiglu.cu,
                                                crossentropy.cu and rmsnorm.cu left out as well (the library's layer drop-ins)
       Returns (ref_path, b200_path) or (None, None) when the checkout or nvcc is absent."""
    out_dir = os.path.join(HERE, "_ref")
    tag = model.replace("-", "_")
    ref_bin = os.path.join(out_dir, "train_ref_" + tag)
    our_bin = os.path.join(out_dir, "train_b200_" + tag)
    layers_bin = os.path.join(out_dir, "train_b200_layers_" + tag)
    cuda_dir = os.path.join(reference, "cuda")
    src_dir = os.path.join(reference, model, "src")
    if not os.path.isdir(src_dir) or shutil.which("nvcc") is None:
        return (ref_bin if os.path.exists(ref_bin) else None, our_bin if os.path.exists(our_bin) else None)
    pkg = os.path.join(os.path.dirname(HERE), "llms-from-scratch-cuda_b200")
    ours = [os.path.join(pkg, "libb200_linear.so"), os.path.join(pkg, "libb200_cublas_shim.so")]
    srcs = [os.path.join(cuda_dir, f) for f in KERNEL_SOURCES] + \
           [os.path.join(src_dir, f) for f in ("main.cpp", "model.cpp", "dataloader.cpp")]
    if not force and _newer(ref_bin, srcs) and _newer(our_bin, srcs + ours) and _newer(layers_bin, srcs + ours):
        return ref_bin, our_bin
    os.makedirs(out_dir, exist_ok=True)
    obj_dir = os.path.join(out_dir, "obj_" + tag)
    os.makedirs(obj_dir, exist_ok=True)
    common = ["nvcc", "-std=c++17", "-O3", "--use_fast_math", "-gencode", "arch=compute_100a,code=sm_100a",
              "-I", cuda_dir, "-I", src_dir]
    objs = []
    for src in srcs + [os.path.join(cuda_dir, "matmul.cu")]:
        obj = os.path.join(obj_dir, os.path.basename(src) + ".o")
        subprocess.run(common + ["-x", "cu", "-c", src, "-o", obj], check=True)
        objs.append(obj)
    matmul_obj = objs.pop()
    subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-o", ref_bin] + objs + [matmul_obj, "-lcublas",
                                                    "-Xlinker", "-rpath=/usr/local/cuda/lib64"], check=True)
    subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-o", our_bin] + objs + ["-L", pkg, "-lb200_linear", "-lb200_cublas_shim",
                   "-Xlinker", "-rpath=$ORIGIN/../../llms-from-scratch-cuda_b200"], check=True)
    slim = [o for o in objs if os.path.basename(o)[:-2] not in LAYER_SOURCES]
    subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-o", layers_bin] + slim + ["-L", pkg, "-lb200_linear", "-lb200_cublas_shim",
                   "-Xlinker", "-rpath=$ORIGIN/../../llms-from-scratch-cuda_b200"], check=True)
    return ref_bin, our_bin


def build_train_dp(reference=DEFAULT_REFERENCE, model="llama2-mistral", force=False):
    """The package's multi-GPU driver (llms-from-scratch-cuda_b200/csrc/train_dp.cpp) linked with the reference's
    unmodified model.cpp, dataloader.cpp and kernel objects (the ones build_train compiles, without main.cpp), twice:
         oracle/_ref/train_dp_b200_<model>       linear layers, attention, SwiGLU and cross-entropy from
                                                 libb200_linear.so (the reference's attention.cu, flash_attention.cu,
                                                 swiglu.cu, crossentropy.cu, rmsnorm.cu and matmul.cu left out), no libcublas
         oracle/_ref/train_dp_b200_gemm_<model>  only the linear layers from libb200_linear.so
         oracle/_ref/train_dp_ref_<model>        linear layers from the reference's own cuda/matmul.cu (cuBLAS); the
                                                 same driver, so that all three print the loss with the same digits
       Returns (b200_path, ref_path); None for what cannot be built (checkout, nvcc or nccl.h absent) and is not prebuilt."""
    out_dir = os.path.join(HERE, "_ref")
    tag = model.replace("-", "_")
    out = os.path.join(out_dir, "train_dp_b200_" + tag)
    out_gemm = os.path.join(out_dir, "train_dp_b200_gemm_" + tag)
    out_ref = os.path.join(out_dir, "train_dp_ref_" + tag)
    cuda_dir = os.path.join(reference, "cuda")
    src_dir = os.path.join(reference, model, "src")
    pkg = os.path.join(os.path.dirname(HERE), "llms-from-scratch-cuda_b200")
    driver = os.path.join(pkg, "csrc", "train_dp.cpp")
    prebuilt = (out if os.path.exists(out) else None, out_ref if os.path.exists(out_ref) else None)
    if not os.path.isdir(src_dir) or shutil.which("nvcc") is None or not os.path.exists("/usr/include/nccl.h"):
        return prebuilt
    ref_bin, our_bin = build_train(reference, model, force)
    if our_bin is None:
        return prebuilt
    obj_dir = os.path.join(out_dir, "obj_" + tag)
    objs = [os.path.join(obj_dir, f + ".o") for f in KERNEL_SOURCES + ["model.cpp", "dataloader.cpp"]]
    ours = [os.path.join(pkg, "libb200_linear.so"), os.path.join(pkg, "libb200_cublas_shim.so")]
    deps = objs + ours + [driver, os.path.join(pkg, "csrc", "rank_rendezvous.h"), os.path.join(pkg, "..", "include", "b200_linear.h")]
    if not force and _newer(out, deps) and _newer(out_ref, deps) and _newer(out_gemm, deps):
        return out, out_ref
    drv_obj = os.path.join(obj_dir, "train_dp.cpp.o")
    subprocess.run(["nvcc", "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-I", cuda_dir, "-I", src_dir,
                    "-x", "cu", "-c", driver, "-o", drv_obj], check=True)
    rpath = "-rpath=$ORIGIN/../../llms-from-scratch-cuda_b200"
    slim = [o for o in objs if os.path.basename(o)[:-2] not in LAYER_SOURCES]
    subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-o", out, drv_obj] + slim + ["-L", pkg, "-lb200_linear", "-lb200_cublas_shim", "-lnccl",
                   "-Xlinker", rpath], check=True)
    subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-o", out_gemm, drv_obj] + objs + ["-L", pkg, "-lb200_linear", "-lb200_cublas_shim", "-lnccl",
                   "-Xlinker", rpath], check=True)
    # the reference's own matmul.o comes first: its matmul_forward / matmul_backward win over the library's
    subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-o", out_ref, drv_obj] + objs + [os.path.join(obj_dir, "matmul.cu.o"), "-L", pkg, "-lb200_linear",
                   "-lcublas", "-lnccl", "-Xlinker", rpath, "-Xlinker", "-rpath=/usr/local/cuda/lib64"], check=True)
    return out, out_ref


MODELS = ("llama2-mistral", "llama3")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build_oracle(a.force))
    print(build_reference(a.reference, a.force))
    for model in MODELS:
        print(build_train(a.reference, model, a.force))
        print(build_train_dp(a.reference, model, a.force))

"""Generates tests/golden/reference_cublas.npz on a GPU box: outputs of the reference's own,
unmodified cuda/matmul.cu (cuBLAS; built by oracle/build.py into oracle/_ref/) on seeded inputs
that the oracle's generator reproduces from (seed, shape) alone.

    python tests/golden/make_reference_golden.py [out.npz]

The file stores only outputs and the (seed, shape) of each input.
"""
import ctypes
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import oracle  # noqa: E402

# (M, N, K); inputs: A seed 101+i*10 N(0,1), B seed 102+i*10 N(0,0.02), dC seed 103+i*10 N(0,1),
# dB_old seed 104+i*10 N(0,1).  bf16 cases round the inputs to bf16 first.
CASES = [(128, 96, 64), (64, 64, 160), (192, 128, 72)]


def main():
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "reference_cublas.npz")
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_matmul.so"))
    vp, ci = ctypes.c_void_p, ctypes.c_int
    lib.ref_create.argtypes = [ctypes.POINTER(vp)]
    lib.ref_create_fp32.argtypes = [ctypes.POINTER(vp)]
    for n in ("ref_matmul_forward_bf16", "ref_matmul_forward_f32"):
        getattr(lib, n).argtypes = [vp, vp, vp, vp, ci, ci, ci]
        getattr(lib, n).restype = None
    for n in ("ref_matmul_backward_bf16", "ref_matmul_backward_f32"):
        getattr(lib, n).argtypes = [vp, vp, vp, vp, vp, vp, ci, ci, ci]
        getattr(lib, n).restype = None
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    res = {"cases": np.array(CASES, dtype=np.int32)}
    for dt, sfx, create in ((torch.bfloat16, "bf16", lib.ref_create), (torch.float32, "f32", lib.ref_create_fp32)):
        h = vp()
        assert create(ctypes.byref(h)) == 0
        for i, (M, N, K) in enumerate(CASES):
            bf = dt == torch.bfloat16
            A = oracle.normal((M, K), 101 + 10 * i, bf16=bf)
            B = oracle.normal((K, N), 102 + 10 * i, std=0.02, bf16=bf)
            dC = oracle.normal((M, N), 103 + 10 * i, bf16=bf)
            old = oracle.normal((K, N), 104 + 10 * i, bf16=bf)
            a, b, dc, db = (torch.from_numpy(v).to(dev, dt) for v in (A, B, dC, old))
            c = torch.empty(M, N, device=dev, dtype=dt)
            da = torch.empty(M, K, device=dev, dtype=dt)
            getattr(lib, "ref_matmul_forward_" + sfx)(h, c.data_ptr(), a.data_ptr(), b.data_ptr(), M, N, K)
            getattr(lib, "ref_matmul_backward_" + sfx)(h, da.data_ptr(), db.data_ptr(), dc.data_ptr(), a.data_ptr(),
                                                       b.data_ptr(), M, N, K)
            torch.cuda.synchronize()
            res[f"{sfx}_{i}_fwd"] = c.float().cpu().numpy()
            res[f"{sfx}_{i}_dgrad"] = da.float().cpu().numpy()
            res[f"{sfx}_{i}_wgrad"] = db.float().cpu().numpy()
    if any(k.startswith("bf16") for k in res):
        for k in list(res):
            if k.startswith("bf16"):
                # bf16 values: keep the upper 16 bits only (halves the file)
                res[k] = (res[k].view(np.uint32) >> 16).astype(np.uint16)
    np.savez_compressed(out_path, **res)
    print("wrote", out_path)


if __name__ == "__main__":
    main()

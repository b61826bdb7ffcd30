"""Runs the reference's own `train` program in its two builds (TEST INFRASTRUCTURE — not part of the
product): oracle/_ref/train_ref_* (the reference as it is: cuda/matmul.cu -> cuBLAS) and
oracle/_ref/train_b200_* (the same host and kernel objects linked against libb200_linear.so instead),
both produced by oracle/build.py from the reference checkout.

    python oracle/train_dropin.py overfit      # the reference README's overfit-one-batch recipe, 200 steps
    python oracle/train_dropin.py throughput   # B=16, T=512, accum=16 (131072 tokens/step), wall clock

The token files are synthetic (uniform ids in [0, 32000), fixed seed): the corpus slice the reference's
README uses is not redistributable and throughput does not depend on token values.
"""
import json
import os
import re
import subprocess
import sys
import tempfile
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
STEP_RE = re.compile(r"step\s+(\d+) \| loss ([0-9.]+|nan|inf|-nan)")


def binaries(model="llama2_mistral"):
    ref = os.path.join(REF, "train_ref_" + model)
    ours = os.path.join(REF, "train_b200_" + model)
    return (ref if os.path.exists(ref) else None, ours if os.path.exists(ours) else None)


def write_tokens(path, n, seed=42, vocab=32000):
    np.random.default_rng(seed).integers(0, vocab, n, dtype=np.int32).tofile(path)


def run(binary, data, args, cwd):
    t0 = time.time()
    out = subprocess.run([binary, data] + args, cwd=cwd, capture_output=True, text=True, timeout=3000)
    wall = time.time() - t0
    losses = {int(m.group(1)): float(m.group(2)) for m in STEP_RE.finditer(out.stdout)}
    return {"rc": out.returncode, "wall_s": wall, "losses": losses, "tail": out.stdout[-400:] + out.stderr[-400:]}


def overfit(steps=200, repeats_ref=2):
    """README recipe (README.md:76-80 of the reference): B=1, T=512, one batch, lr 3e-4, warmup 20."""
    ref, ours = binaries()
    if not ref or not ours:
        raise FileNotFoundError("oracle/_ref/train_* not built (run oracle/build.py where the reference checkout is)")
    args = ["--bf16", "--batch", "1", "--steps", str(steps), "--accum", "1", "--lr", "3e-4", "--warmup", "20",
            "--save", "1000000"]
    with tempfile.TemporaryDirectory() as d:
        data = os.path.join(d, "overfit.bin")
        write_tokens(data, 513)
        res = {"reference": [run(ref, data, args, d) for _ in range(repeats_ref)], "b200": run(ours, data, args, d)}
    return res


def throughput(steps=2):
    ref, ours = binaries()
    if not ref or not ours:
        raise FileNotFoundError("oracle/_ref/train_* not built")
    args = ["--bf16", "--batch", "16", "--steps", str(steps), "--accum", "16", "--save", "1000000"]
    with tempfile.TemporaryDirectory() as d:
        data = os.path.join(d, "data.bin")
        write_tokens(data, 131072 * 2 + 1)
        res = {}
        for name, b in (("reference", ref), ("b200", ours)):
            r = run(b, data, args, d)
            r["tokens_per_s_wall"] = steps * 131072 / r["wall_s"]  # includes model build and data load
            res[name] = r
    return res


TOKS_RE = re.compile(r"step\s+(\d+) \| loss [0-9.naif-]+ \|.*\| (\d+) tok/s")


def dp_binary(model="llama2_mistral"):
    p = os.path.join(REF, "train_dp_b200_" + model)
    return p if os.path.exists(p) else None


def data_parallel(ranks_list=(1, 2), steps=3, batch=16, accum=4, lr="3e-4", warmup="20"):
    """The package's data-parallel driver (csrc/train_dp.cpp around the reference's ModelBF16) on the same token
    stream at every rank count: losses per step and the wall-clock tokens/s it prints for steps 2..S."""
    b = dp_binary()
    if not b:
        raise FileNotFoundError("oracle/_ref/train_dp_b200_* not built")
    res = {}
    with tempfile.TemporaryDirectory() as d:
        data = os.path.join(d, "data.bin")
        write_tokens(data, batch * 512 * accum * steps + 1)
        for r in ranks_list:
            out = run(b, data, ["--ranks", str(r), "--steps", str(steps), "--batch", str(batch), "--accum", str(accum),
                                "--lr", lr, "--warmup", warmup], d)
            toks = [int(m.group(2)) for m in TOKS_RE.finditer(out["tail"])]
            out["tokens_per_s"] = toks[-1] if toks else None
            res[r] = out
    return res


if __name__ == "__main__":
    mode = sys.argv[1] if len(sys.argv) > 1 else "overfit"
    if mode == "dp":
        print(json.dumps(data_parallel(tuple(int(x) for x in sys.argv[2].split(",")) if len(sys.argv) > 2 else (1, 2),
                                       *(int(x) for x in sys.argv[3:6]))))
    else:
        print(json.dumps(overfit() if mode == "overfit" else throughput(int(sys.argv[2]) if len(sys.argv) > 2 else 2)))

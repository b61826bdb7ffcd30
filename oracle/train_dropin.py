"""Runs the reference's training program and the package's multi-GPU driver in their different links
(TEST INFRASTRUCTURE — not part of the product).  All binaries are produced by oracle/build.py from the
reference checkout, for the models "llama2_mistral" and "llama3":

    oracle/_ref/train_ref_<model>      the reference as it is: cuda/matmul.cu -> cuBLAS
    oracle/_ref/train_b200_<model>     the same host and kernel objects linked against libb200_linear.so
    oracle/_ref/train_dp_b200_<model>  csrc/train_dp.cpp around the reference's ModelBF16, libb200_linear.so
    oracle/_ref/train_dp_ref_<model>   the same driver with the reference's own matmul.cu (cuBLAS)

    python oracle/train_dropin.py overfit             # the reference README's overfit-one-batch recipe, 200 steps
    python oracle/train_dropin.py overfit_digits      # the same recipe through the driver: loss printed with 8 digits
    python oracle/train_dropin.py throughput [steps]  # B=16, T=512, accum=16 (131072 tokens/step), wall clock
    python oracle/train_dropin.py dp 1,2 [steps batch accum]
    python oracle/train_dropin.py vp <model> 1,2 [steps batch seq accum]   # vocabulary-parallel LM head vs the plain path
    python oracle/train_dropin.py checkpoint          # checkpoint written by one program, resumed by the other

The token files are synthetic (uniform ids, fixed seed): the corpus slice the reference's README uses is not
redistributable and throughput does not depend on token values.
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
TOKS_RE = re.compile(r"step\s+(\d+) \| loss [0-9.naif-]+ \|.*\| (\d+) tok/s")
PHASES_RE = re.compile(r"phases, seconds per step.*?: (.*)")
VOCAB = {"llama2_mistral": 32000, "llama3": 128256}


def _existing(name):
    p = os.path.join(REF, name)
    return p if os.path.exists(p) else None


def binaries(model="llama2_mistral"):
    """(reference build, drop-in build) of the reference's own `train` program."""
    return _existing("train_ref_" + model), _existing("train_b200_" + model)


def dp_binaries(model="llama2_mistral"):
    """(this library: linear layers and the layers around them, reference cuBLAS) links of the package's driver."""
    return _existing("train_dp_b200_" + model), _existing("train_dp_ref_" + model)


def dp_gemm_binary(model="llama2_mistral"):
    """The driver with only the linear layers from this library (the reference's own attention, SwiGLU, RMSNorm and
    cross-entropy kernels around them)."""
    return _existing("train_dp_b200_gemm_" + model)


def dp_binary(model="llama2_mistral"):
    return dp_binaries(model)[0]


def write_tokens(path, n, seed=42, vocab=32000):
    np.random.default_rng(seed).integers(0, vocab, n, dtype=np.int32).tofile(path)


def run(binary, data, args, cwd, timeout=3000):
    t0 = time.time()
    out = subprocess.run([binary, data] + [str(a) for a in args], cwd=cwd, capture_output=True, text=True, timeout=timeout)
    wall = time.time() - t0
    losses = {int(m.group(1)): float(m.group(2)) for m in STEP_RE.finditer(out.stdout)}
    toks = [int(m.group(2)) for m in TOKS_RE.finditer(out.stdout)]
    ph = PHASES_RE.search(out.stdout)
    phases = None
    if ph:
        phases = {k.strip(): float(v) for k, v in (item.rsplit(" ", 1) for item in ph.group(1).split(" | "))}
    return {"rc": out.returncode, "wall_s": wall, "losses": losses, "tokens_per_s": toks[-1] if toks else None,
            "phases": phases, "stdout": out.stdout[-3000:], "tail": out.stdout[-600:] + out.stderr[-600:]}


OVERFIT_ARGS = ["--batch", "1", "--accum", "1", "--lr", "3e-4", "--warmup", "20"]


def overfit(steps=200, repeats_ref=2):
    """README recipe (README.md:76-80 of the reference): B=1, T=512, one batch, lr 3e-4, warmup 20; the reference's
    own program in both links (it prints the loss with four decimals)."""
    ref, ours = binaries()
    if not ref or not ours:
        raise FileNotFoundError("oracle/_ref/train_* not built (run oracle/build.py where the reference checkout is)")
    args = ["--bf16", "--steps", steps, "--save", "1000000"] + OVERFIT_ARGS
    with tempfile.TemporaryDirectory() as d:
        data = os.path.join(d, "overfit.bin")
        write_tokens(data, 513)
        res = {"reference": [run(ref, data, args, d) for _ in range(repeats_ref)], "b200": run(ours, data, args, d)}
    return res


def overfit_digits(steps=200, repeats_ref=3, repeats_ours=2):
    """The same recipe through the package's driver at one rank, linked once against the reference's own
    matmul.cu (cuBLAS) and once against this library: same host code, same kernels around the GEMMs, loss
    printed with eight decimals, so that the end of the curve (1e-4 and below) can be compared."""
    layers, ref = dp_binaries()
    gemm = dp_gemm_binary()
    if not ref or not layers or not gemm:
        raise FileNotFoundError("oracle/_ref/train_dp_* not built (run oracle/build.py where the reference checkout is)")
    args = ["--ranks", "1", "--steps", steps] + OVERFIT_ARGS
    with tempfile.TemporaryDirectory() as d:
        data = os.path.join(d, "overfit.bin")
        write_tokens(data, 513)
        res = {"reference": [run(ref, data, args, d) for _ in range(repeats_ref)],
               "b200": [run(gemm, data, args, d) for _ in range(repeats_ours)],          # linear layers only
               "b200_layers": [run(layers, data, args, d) for _ in range(repeats_ours)]}  # + attention, SwiGLU, RMSNorm, CE
    return res


def throughput(steps=2):
    ref, ours = binaries()
    if not ref or not ours:
        raise FileNotFoundError("oracle/_ref/train_* not built")
    args = ["--bf16", "--batch", "16", "--steps", steps, "--accum", "16", "--save", "1000000"]
    with tempfile.TemporaryDirectory() as d:
        data = os.path.join(d, "data.bin")
        write_tokens(data, 131072 * 2 + 1)
        res = {}
        for name, b in (("reference", ref), ("b200", ours)):
            r = run(b, data, args, d)
            r["tokens_per_s_wall"] = steps * 131072 / r["wall_s"]  # includes model build and data load
            res[name] = r
    return res


def data_parallel(ranks_list=(1, 2), steps=3, batch=16, accum=4, lr="3e-4", warmup="20", model="llama2_mistral", seq=512,
                  timers=False):
    """The package's driver on the same token stream at every rank count: losses per step and the wall-clock
    tokens/s it prints for steps 2..S."""
    b = dp_binary(model)
    if not b:
        raise FileNotFoundError("oracle/_ref/train_dp_b200_* not built")
    res = {}
    with tempfile.TemporaryDirectory() as d:
        data = os.path.join(d, "data.bin")
        write_tokens(data, batch * seq * accum * steps + 1, vocab=VOCAB[model])
        for r in ranks_list:
            res[r] = run(b, data, ["--ranks", r, "--steps", steps, "--batch", batch, "--seq", seq, "--accum", accum,
                                   "--lr", lr, "--warmup", warmup] + (["--timers"] if timers else []), d)
    return res


def vocab_parallel(model="llama3", ranks_list=(1, 2), steps=3, batch=2, seq=512, accum=2, lr="3e-4", warmup="20",
                   timers=False):
    """The driver with the LM head and the cross-entropy sharded by vocabulary at every rank count in
    `ranks_list`, next to the plain path (the reference's own full-vocabulary GEMM + crossentropy.cu) on one
    GPU, key 0: same tokens, same micro-batches per step."""
    b = dp_binary(model)
    if not b:
        raise FileNotFoundError("oracle/_ref/train_dp_b200_%s not built" % model)
    res = {}
    common = ["--steps", steps, "--batch", batch, "--seq", seq, "--accum", accum, "--lr", lr, "--warmup", warmup]
    if timers:
        common.append("--timers")
    with tempfile.TemporaryDirectory() as d:
        data = os.path.join(d, "data.bin")
        write_tokens(data, batch * seq * accum * steps + 1, vocab=VOCAB[model])
        res[0] = run(b, data, ["--ranks", 1] + common, d)
        for r in ranks_list:
            res[r] = run(b, data, ["--ranks", r, "--vocab-parallel"] + common, d)
    return res


def checkpoint_roundtrip(model="llama2_mistral"):
    """On-disk compatibility (llama2-mistral/src/main.cpp:212-254 writes, :93-112 and model.cpp:564-580 read):
    two steps in one program, checkpoint, third step in the other program, both ways round, against each
    program continuing from its own file."""
    ref, _ = binaries(model)
    ours, _ = dp_binaries(model)
    if not ref or not ours:
        raise FileNotFoundError("oracle/_ref/train_ref_* / train_dp_b200_* not built")
    small = ["--batch", "1", "--accum", "1", "--lr", "3e-4", "--warmup", "20"]
    res = {}
    with tempfile.TemporaryDirectory() as d:
        data = os.path.join(d, "tokens.bin")
        write_tokens(data, 3 * 512 + 1, vocab=VOCAB[model])
        res["token_file_bytes"] = os.path.getsize(data)
        for writer, wbin, wargs in (("driver", ours, ["--ranks", "1", "--steps", "2", "--save-every", "2"] + small),
                                    ("reference", ref, ["--bf16", "--steps", "2", "--save", "2"] + small)):
            wd = os.path.join(d, writer)
            os.makedirs(os.path.join(wd, "checkpoints"))
            w = run(wbin, data, wargs, wd)
            ck = os.path.join(wd, "checkpoints", "step_2.bin")
            entry = {"write": w, "bytes": os.path.getsize(ck) if os.path.exists(ck) else 0}
            if entry["bytes"]:
                # the reference's program restarts its data loader at the head of the file on resume, the driver too
                entry["resume_reference"] = run(ref, data, ["--bf16", "--checkpoint", ck, "--steps", "1", "--save", "1000000"] + small, wd)
                entry["resume_driver"] = run(ours, data, ["--ranks", "1", "--checkpoint", ck, "--steps", "1"] + small, wd)
                os.remove(ck)
            res[writer] = entry
    return res


if __name__ == "__main__":
    mode = sys.argv[1] if len(sys.argv) > 1 else "overfit"
    ints = lambda xs: [int(x) for x in xs]
    if mode == "dp":
        out = data_parallel(tuple(ints(sys.argv[2].split(","))) if len(sys.argv) > 2 else (1, 2), *ints(sys.argv[3:6]), timers=True)
    elif mode == "vp":
        out = vocab_parallel(sys.argv[2] if len(sys.argv) > 2 else "llama3",
                             tuple(ints(sys.argv[3].split(","))) if len(sys.argv) > 3 else (1, 2), *ints(sys.argv[4:8]), timers=True)
    elif mode == "overfit_digits":
        out = overfit_digits()
    elif mode == "checkpoint":
        out = checkpoint_roundtrip()
    elif mode == "throughput":
        out = throughput(int(sys.argv[2]) if len(sys.argv) > 2 else 2)
    else:
        out = overfit()
    print(json.dumps(out))

#!/usr/bin/env python
"""Benchmark of the linear-layer GEMM path (contract: one JSON line on stdout from rank 0).

Workload ("step"): every GEMM of one LLaMA-2/Mistral-125M decoder layer plus the LM head,
forward + backward, for one micro-batch of B=16 x T=512 = 8192 tokens in bf16 — the second
configuration of BASELINE.json.  As the reference launches them (cuda/attention.cu:597-599,616;
cuda/swiglu.cu:161-162,169; llama2-mistral/src/model.cpp:612,635): projections
Q 768->768, K 768->256, V 768->256, O 768->768, gate 768->2048, up 768->2048, down 2048->768,
LM head 768->32000; each runs matmul_forward once and matmul_backward once (dgrad, and wgrad
accumulating into dW with beta=1), 24 GEMMs and 1.517e12 FLOP per step.  Inputs are seeded
synthetic tensors (weights N(0,0.02), activations and upstream gradients N(0,1)).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

TOKENS = 8192  # B=16 x T=512
# name, N (out features), K (in features)
PROJECTIONS = [("q", 768, 768), ("k", 256, 768), ("v", 256, 768), ("o", 768, 768),
               ("gate", 2048, 768), ("up", 2048, 768), ("down", 768, 2048), ("lm_head", 32000, 768)]
STEP_FLOP = sum(3 * 2 * TOKENS * n * k for _, n, k in PROJECTIONS)
ACCUM = 16  # micro-batches per optimizer step in the reference's training config


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"bf16_tflops": d.get("bf16_tflops"), "bf16_tflops_sustained": d.get("bf16_tflops_sustained"),
                "hbm_gbs": d.get("hbm_gbs"), "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in self.rows:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9 or not (t0 - 0.05 <= ts <= t1 + 0.15):
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "samples": len(sm),
                "reasons": sorted(reasons)}


def make_buffers(torch, dev, oracle_mod, host=False):
    """Per-projection operand set. Device tensors; with host=True also pinned host copies of the
    per-micro-batch operands (A and dC)."""
    bufs = []
    g = torch.Generator(device=dev).manual_seed(1234)
    for i, (name, n, k) in enumerate(PROJECTIONS):
        b = {"name": name, "N": n, "K": k}
        b["A"] = torch.randn(TOKENS, k, device=dev, generator=g).to(torch.bfloat16)
        b["B"] = (0.02 * torch.randn(k, n, device=dev, generator=g)).to(torch.bfloat16)
        b["dC"] = torch.randn(TOKENS, n, device=dev, generator=g).to(torch.bfloat16)
        b["C"] = torch.empty(TOKENS, n, device=dev, dtype=torch.bfloat16)
        b["dA"] = torch.empty(TOKENS, k, device=dev, dtype=torch.bfloat16)
        b["dB"] = torch.zeros(k, n, device=dev, dtype=torch.bfloat16)
        if host:
            b["A_host"] = b["A"].cpu().pin_memory()
            b["dC_host"] = b["dC"].cpu().pin_memory()
            b["dA_host"] = torch.empty(TOKENS, k, dtype=torch.bfloat16).pin_memory()
        bufs.append(b)
    return bufs


PREHEAT_S = 1.0
BLOCKS = 10  # the K-step block is timed this many times back to back; value = median block

WORKLOAD = ("configs[1]: decoder-layer projections (Q,K,V,O,gate,up,down) + LM head 768->32000, "
            "M=8192 tokens (B16xT512), fwd + dgrad + wgrad(beta=1), 24 GEMMs/step")


def common_config(world):
    """The same keys in both arms, so that the two lines describe one configuration."""
    return {"workload": WORKLOAD,
            "l2": "no flush: the step's working set (~1.7 GB, every GEMM its own buffers) exceeds the 126 MB L2",
            "preheat": "%.1f s of untimed steps right before the timed region, in both arms (thermal / power-cap steady state)" % PREHEAT_S,
            "timing": "%d blocks of --steps steps back to back, CUDA events around each block; value and ms_per_step "
                      "are the median block (maximum over ranks per block), ms_per_step_min/max the spread" % BLOCKS,
            "parallelism": "dp%d by tokens, dW all-reduce (NCCL) every %d micro-batches" % (world, ACCUM),
            "flop_per_step": STEP_FLOP}


def time_blocks(torch, step_fn, steps, after_step=None):
    """BLOCKS blocks of `steps` steps, one CUDA event between blocks (no host synchronisation inside the region).
    Returns the list of block durations in milliseconds."""
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(BLOCKS + 1)]
    ev[0].record()
    n = 0
    for b in range(BLOCKS):
        for _ in range(steps):
            step_fn()
            n += 1
            if after_step is not None:
                after_step(n)
        ev[b + 1].record()
    torch.cuda.synchronize()
    return [ev[b].elapsed_time(ev[b + 1]) for b in range(BLOCKS)]


def median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2] if len(xs) % 2 else 0.5 * (xs[len(xs) // 2 - 1] + xs[len(xs) // 2])


def preheat(torch, step_fn, seconds=PREHEAT_S):
    """Untimed steps until the board is at its power-capped steady state.  A replayed graph of this step takes
    1.23 ms on a GPU that has idled for a second and 1.35 ms half a second of load later (either library), so
    a 0.27 s timed region would otherwise measure how long the process idled before it -- and which arm ran
    first.  Both arms call this right before their timed region."""
    t_end = time.time() + seconds
    n = 0
    while time.time() < t_end:
        for _ in range(20):
            step_fn()
        torch.cuda.synchronize()
        n += 20
    return n


def time_e2e(torch, bufs, step_device, steps, barrier):
    """The step with host buffers on both sides: every projection's A and dC copied from pinned host
    memory, the 24 GEMMs, every dA read back to pinned host memory; all inside the timed region.
    Both arms (this library, the reference's cuBLAS build) are timed by this one function.
    Returns (milliseconds, steps timed, host-to-device bytes per step, device-to-host bytes per step)."""
    h2d = sum(b["A_host"].numel() + b["dC_host"].numel() for b in bufs) * 2
    d2h = sum(b["dA_host"].numel() for b in bufs) * 2

    def step_e2e():
        for b in bufs:
            b["A"].copy_(b["A_host"], non_blocking=True)
            b["dC"].copy_(b["dC_host"], non_blocking=True)
        step_device()
        for b in bufs:
            b["dA_host"].copy_(b["dA"], non_blocking=True)

    e2e_steps = max(1, min(steps, 5))
    step_e2e()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(e2e_steps):
        step_e2e()
    e1.record()
    barrier()
    return e0.elapsed_time(e1), e2e_steps, h2d, d2h


def run_ours(args):
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    pkg = load_package()  # raises if the CUDA library is missing: there is no fallback

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    h = pkg.Handle()
    bufs = make_buffers(torch, dev, None, host=True)

    def step_device():
        for b in bufs:
            pkg.matmul_forward(h, b["C"], b["A"], b["B"], TOKENS, b["N"], b["K"])
        for b in reversed(bufs):
            pkg.matmul_backward(h, b["dA"], b["dB"], b["dC"], b["A"], b["B"], TOKENS, b["N"], b["K"])

    grad_flat = None
    if world > 1:
        # data parallel by tokens: every rank holds the same weights and its own 8192-token
        # micro-batch; the dW buckets are summed across ranks once per optimizer step.
        grad_flat = torch.zeros(sum(b["dB"].numel() for b in bufs), device=dev, dtype=torch.bfloat16)
        off = 0
        for b in bufs:
            n = b["dB"].numel()
            b["dB"] = grad_flat[off:off + n].view_as(b["dB"])
            off += n

    def exchange():
        if world > 1:
            dist.all_reduce(grad_flat)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step_device()
    exchange()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    preheat(torch, step_device)
    barrier()
    launches0 = h.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()

    def after_step(n):  # the dW exchange, once per ACCUM micro-batches (at least once per block)
        if n % ACCUM == 0 or (args.steps < ACCUM and n % args.steps == 0):
            exchange()

    block_ms = time_blocks(torch, step_device, args.steps, after_step)
    barrier()
    t1 = time.time()
    h.sync()
    launches = (h.launches - launches0) // BLOCKS
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    if world > 1:
        t = torch.tensor(block_ms, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        block_ms = t.tolist()
    ms = median(block_ms)
    value = world * args.steps * STEP_FLOP / (ms * 1e-3) / 1e12

    # ---- end to end: host buffers in, host buffers out, through the same calls
    ms_e2e, e2e_steps, h2d, d2h = time_e2e(torch, bufs, step_device, args.steps, barrier)
    if world > 1:
        t = torch.tensor([ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = t.item()
    e2e_value = world * e2e_steps * STEP_FLOP / (ms_e2e * 1e-3) / 1e12

    # ---- the vocabulary-sharded LM head + cross-entropy of configs[3] on these ranks (a sub-record)
    vocab_parallel = run_vocab_parallel(torch, dist, pkg, h, dev, world, rank) if args.vocab_parallel else None
    # ---- a whole training step of the 125M model through the multi-GPU driver (a sub-record)
    train_step = run_train_step(dist, world, rank, args) if args.train_step else None

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        if vocab_parallel is not None and not vocab_parallel.get("parity_ok", True):
            sys.exit(3)
        return

    # ---- per-GEMM timing (rank 0): CUDA events on the launching stream, each GEMM alone
    per = []
    dominant = None
    side = torch.cuda.Stream()
    h.set_stream(side)  # per-GEMM timing: 10 launches captured in a CUDA graph, replayed, timed with events on that stream
    for b in bufs:
        for kind, call, flop in (
                ("fwd_nn", lambda: pkg.gemm(h, pkg.FWD_NN, 0, b["C"], b["A"], b["B"], TOKENS, b["N"], b["K"]), 1),
                ("dgrad_nt", lambda: pkg.gemm(h, pkg.DGRAD_NT, 0, b["dA"], b["dC"], b["B"], TOKENS, b["N"], b["K"]), 1),
                ("wgrad_tn", lambda: pkg.gemm(h, pkg.WGRAD_TN, 1, b["dB"], b["A"], b["dC"], TOKENS, b["N"], b["K"]), 1)):
            reps = 10
            l0 = h.launches
            with torch.cuda.stream(side):
                for _ in range(3):
                    call()
                side.synchronize()
                l0 = h.launches
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for _ in range(reps):
                        call()
                launches_in_graph = h.launches - l0
                graph.replay()
                side.synchronize()
                e0.record(side)
                graph.replay()
                e1.record(side)
                side.synchronize()
            l0 = h.launches - launches_in_graph
            us = e0.elapsed_time(e1) / reps * 1e3
            fl = 2.0 * TOKENS * b["N"] * b["K"]
            # algorithmic bytes: both operands and the output once (the beta = 1 output twice), 2 bytes each
            nbytes = 2.0 * (TOKENS * b["K"] + b["K"] * b["N"] + TOKENS * b["N"]) + (2.0 * b["K"] * b["N"] if kind == "wgrad_tn" else 0.0)
            rec = {"proj": b["name"], "gemm": kind, "us": round(us, 2), "tflops": round(fl / us / 1e6, 1),
                   "hbm_gbs": round(nbytes / us / 1e3, 1), "launches_per_call": (h.launches - l0) // reps}
            per.append(rec)
            if dominant is None or us > dominant["us"]:
                dominant = dict(rec, flop=fl, N=b["N"], K=b["K"])
    # ---- the same projections as their callers issue them: one grouped launch per direction for Q, K, V and for
    # gate, up (attention.cu:597-599, 671-688; swiglu.cu:161-162, 197-208), beside the sum of the single products above
    def time_graph(call, reps=10):
        with torch.cuda.stream(side):
            for _ in range(3):
                call()
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(reps):
                    call()
            graph.replay()
            side.synchronize()
            e0.record(side)
            graph.replay()
            e1.record(side)
            side.synchronize()
        return e0.elapsed_time(e1) / reps * 1e3

    by_name = {b["name"]: b for b in bufs}
    grouped = []
    for names in (("q", "k", "v"), ("gate", "up")):
        if not all(n in by_name for n in names):
            continue
        g = [by_name[n] for n in names]
        Ns, K = [b["N"] for b in g], g[0]["K"]
        x = g[0]["A"]
        fl = sum(2.0 * TOKENS * n * K for n in Ns)
        single = {kind: sum(r["us"] for r in per if r["proj"] in names and r["gemm"] == kind) for kind in ("fwd_nn", "dgrad_nt", "wgrad_tn")}
        for kind, call in (
                ("fwd_nn", lambda: pkg.gemm_grouped(h, pkg.FWD_NN, 0, [b["C"] for b in g], x, [b["B"] for b in g], TOKENS, Ns, K)),
                ("dgrad_nt", lambda: pkg.gemm_grouped(h, pkg.DGRAD_NT, 0, g[0]["dA"], [b["dC"] for b in g], [b["B"] for b in g], TOKENS, Ns, K)),
                ("wgrad_tn", lambda: pkg.gemm_grouped(h, pkg.WGRAD_TN, 1, [b["dB"] for b in g], x, [b["dC"] for b in g], TOKENS, Ns, K))):
            us = time_graph(call)
            grouped.append({"group": "+".join(names), "gemm": kind, "us": round(us, 2), "tflops": round(fl / us / 1e6, 1),
                            "single_products_us": round(single[kind], 2)})
    h.sync()
    h.set_stream(torch.cuda.current_stream())
    # ---- the same 24 products as this library's layer functions issue them: Q, K, V and gate, up of one input as one
    # grouped launch per direction (16 launches in all).  Not the headline: `value` keeps one call per product, which is
    # what the other arm's interface offers.
    step_grouped = None
    if all(n in by_name for n in ("q", "k", "v", "gate", "up")):
        groups = [[by_name[n] for n in ("q", "k", "v")], [by_name[n] for n in ("gate", "up")]]
        rest = [b for b in bufs if b["name"] not in ("q", "k", "v", "gate", "up")]

        def step_device_grouped():
            for g in groups:
                pkg.gemm_grouped(h, pkg.FWD_NN, 0, [b["C"] for b in g], g[0]["A"], [b["B"] for b in g], TOKENS, [b["N"] for b in g], g[0]["K"])
            for b in rest:
                pkg.matmul_forward(h, b["C"], b["A"], b["B"], TOKENS, b["N"], b["K"])
            for b in reversed(rest):
                pkg.matmul_backward(h, b["dA"], b["dB"], b["dC"], b["A"], b["B"], TOKENS, b["N"], b["K"])
            for g in reversed(groups):
                pkg.matmul_backward_grouped(h, g[0]["dA"], [b["dB"] for b in g], [b["dC"] for b in g], g[0]["A"],
                                            [b["B"] for b in g], TOKENS, [b["N"] for b in g], g[0]["K"])

        for _ in range(max(3, args.warmup)):
            step_device_grouped()
        torch.cuda.synchronize()
        preheat(torch, step_device_grouped)
        gms = median(time_blocks(torch, step_device_grouped, args.steps))
        h.sync()
        step_grouped = {"ms_per_step": round(gms / args.steps, 4), "tflops": round(args.steps * STEP_FLOP / (gms * 1e-3) / 1e12, 2),
                        "launches_per_step": 16,
                        "what": "the same 24 products with Q, K, V and gate, up of one input issued as grouped launches "
                                "(b200_linear_gemm_bf16_grouped / _backward_bf16_grouped), rank 0, no gradient exchange"}
    in_step = None
    if args.breakdown:
        calls = [(b["name"] + ":fwd", (lambda b=b: pkg.matmul_forward(h, b["C"], b["A"], b["B"], TOKENS, b["N"], b["K"]))) for b in bufs]
        calls += [(b["name"] + ":bwd", (lambda b=b: pkg.matmul_backward(h, b["dA"], b["dB"], b["dC"], b["A"], b["B"], TOKENS, b["N"], b["K"]))) for b in reversed(bufs)]
        in_step = step_breakdown(torch, calls)
    peaks = measured_peaks()
    total_us = sum(r["us"] for r in per)
    roofline = {"bound": "tensor", "kernel": "gemm_bf16_sm100 (%s %s, M=8192)" % (dominant["proj"], dominant["gemm"]),
                "achieved": round(dominant["flop"] / dominant["us"] / 1e6, 1), "peak": peaks["bf16_tflops"],
                "unit": "TFLOP/s", "frac": round(dominant["flop"] / dominant["us"] / 1e6 / peaks["bf16_tflops"], 4),
                "peak_source": peaks["source"] + " (burst: kernel timed alone)",
                "share_of_step": round(dominant["us"] / total_us, 3), "traffic": None,
                "traffic_note": "DRAM bytes per launch come from an ncu capture, not from this run: see the kernel's summary "
                                "under profiles/ (a capture at full size is too large to take under the profiler)",
                "algorithmic_bytes": int(2.0 * (TOKENS * dominant["K"] + dominant["K"] * dominant["N"] + TOKENS * dominant["N"]) +
                                         (2.0 * dominant["K"] * dominant["N"] if dominant["gemm"] == "wgrad_tn" else 0.0)),
                "hbm_peak_gbs": peaks["hbm_gbs"],  # secondary bound: compare per_gemm[].hbm_gbs for the thin k/v shapes
                "step_frac_of_sustained": round(value / world / peaks["bf16_tflops_sustained"], 4)}

    cpu = cpu_baseline_port()
    line = {"metric": "bf16 GEMM TFLOP/s, all linear-layer GEMMs of one 125M decoder layer + LM head, fwd+bwd",
            "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms / args.steps, 4), "ms_per_step_min": round(min(block_ms) / args.steps, 4),
            "ms_per_step_max": round(max(block_ms) / args.steps, 4), "blocks": BLOCKS,
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": common_config(world),
            "clocks": clocks, "gpu_launches": launches,
            "e2e": {"value": round(e2e_value, 2), "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "what": "A and dC of every projection copied from pinned host memory, 24 GEMMs through the C ABI, every dA read back"},
            "roofline": roofline, "cpu_baseline": cpu, "per_gemm": per, "grouped_gemm": grouped, "step_grouped": step_grouped}
    if in_step:
        line["in_step_us"] = in_step
    if vocab_parallel is not None:
        line["vocab_parallel"] = vocab_parallel
    if train_step is not None:
        line["train_step"] = train_step
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    if vocab_parallel is not None and not vocab_parallel.get("parity_ok", True):
        sys.exit(3)


def run_vocab_parallel(torch, dist, pkg, h, dev, world, rank):
    """The LM head of BASELINE.json configs[3] (LLaMA-3 272M: 16384 tokens = B2 x T8192, vocabulary 128256, K = 768)
    sharded by vocabulary over the ranks of this run, forward + cross-entropy + backward, as the multi-GPU driver
    runs it (csrc/train_dp.cpp; replaces llama2-mistral/src/model.cpp:612-614,634-635 in that mode): every rank
    multiplies by its own 256-column tiles of w_out where they lie (pitched operands), the row maxima and the sums
    of exponentials cross the ranks in two small all-reduces, dlogits is formed in place, the weight gradient lands
    in the rank's own columns of dw_out and the input gradient is summed over the ranks.  Total work is fixed
    (strong scaling); every rank also runs the whole vocabulary alone once (n1_ms) for the efficiency figure.
    A small case is checked against float64 first: parity_ok False makes the run exit non-zero."""
    import importlib
    dmod = importlib.import_module(pkg.__name__ + ".dist")
    rows, V, K = 16384, 128256, 768
    shards = dmod.vocab_shards(V, world)

    def lm_head(x, w, dw, targets, logits, dx, col0, cols, exchange, fused_stats=True):
        n_rows = x.shape[0]
        if fused_stats:   # row maximum / sum of exponentials / target logit from the forward GEMM's epilogue
            stats = pkg.forward_ce_stats(h, logits, x, w[:, col0:col0 + cols], n_rows, cols, x.shape[1], targets, col0)
        else:             # the same from a pass over the stored logits
            pkg.gemm_ld(h, pkg.FWD_NN, 0, logits, x, w[:, col0:col0 + cols], n_rows, cols, x.shape[1])
            stats = None
        loss, d = dmod.vocab_parallel_cross_entropy(logits, targets, col0, in_place=True, exchange=exchange, stats=stats)
        pkg.gemm_ld(h, pkg.DGRAD_NT, 0, dx, d, w[:, col0:col0 + cols], n_rows, cols, x.shape[1])
        pkg.gemm_ld(h, pkg.WGRAD_TN, 1, dw[:, col0:col0 + cols], x, d, n_rows, cols, x.shape[1])
        if exchange:
            dmod.reduce_input_gradient(dx)
        return loss

    # ---- parity on a small case (every rank computes it; the float64 result on the host)
    g = torch.Generator(device="cpu").manual_seed(99)
    r_s, v_s, k_s = 512, 2048 + 256 * world, 256
    xs = torch.randn(r_s, k_s, generator=g).to(torch.bfloat16)
    ws = (0.05 * torch.randn(k_s, v_s, generator=g)).to(torch.bfloat16)
    ts = torch.randint(0, v_s, (r_s,), generator=g, dtype=torch.int32)
    s_col0, s_cols = dmod.vocab_shards(v_s, world)[rank]
    x_d, w_d, t_d = xs.to(dev), ws.to(dev), ts.to(dev)
    dw_d = torch.zeros(k_s, v_s, device=dev, dtype=torch.bfloat16)
    lg_d = torch.empty(r_s, s_cols, device=dev, dtype=torch.bfloat16)
    dx_d = torch.empty(r_s, k_s, device=dev, dtype=torch.bfloat16)
    loss_s = lm_head(x_d, w_d, dw_d, t_d, lg_d, dx_d, s_col0, s_cols, True)
    h.sync()
    if world > 1:
        dist.all_reduce(dw_d)  # every rank wrote its own columns only
    l64 = (xs.double() @ ws.double()).to(torch.bfloat16).double()  # the logits as the GEMM stores them
    loss64 = torch.logsumexp(l64, 1) - l64.gather(1, ts.long()[:, None]).squeeze(1)
    d64 = torch.softmax(l64, 1)
    d64[torch.arange(r_s), ts.long()] -= 1.0
    d64 /= r_s
    dx64, dw64 = d64 @ ws.double().T, xs.double().T @ d64
    e_loss = (loss_s.double().cpu() - loss64).abs().max().item()
    e_dx = ((dx_d.double().cpu() - dx64).abs().max() / dx64.abs().max()).item()
    e_dw = ((dw_d.double().cpu() - dw64).abs().max() / dw64.abs().max()).item()
    ok = torch.tensor([1 if (e_loss <= 5e-3 and e_dx <= 2e-2 and e_dw <= 2e-2) else 0], device=dev)
    if world > 1:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    parity = {"parity_ok": bool(ok.item()), "loss_abs_err": round(e_loss, 6), "dx_rel_err": round(e_dx, 5),
              "dw_rel_err": round(e_dw, 5), "case": "rows %d, vocabulary %d, K %d vs float64" % (r_s, v_s, k_s),
              "tolerance": "loss 5e-3 abs, dX and dW 2e-2 of their maximum (bf16 dlogits)"}
    del x_d, w_d, dw_d, lg_d, dx_d

    # ---- timing at configs[3] size
    g = torch.Generator(device=dev).manual_seed(4321)
    x = torch.randn(rows, K, device=dev, generator=g).to(torch.bfloat16)
    w = (0.02 * torch.randn(K, V, device=dev, generator=g)).to(torch.bfloat16)
    dw = torch.zeros(K, V, device=dev, dtype=torch.bfloat16)
    targets = torch.randint(0, V, (rows,), device=dev, generator=g, dtype=torch.int32)
    dx = torch.empty(rows, K, device=dev, dtype=torch.bfloat16)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(col0, cols, exchange, reps=5, fused_stats=True):
        logits = torch.empty(rows, cols, device=dev, dtype=torch.bfloat16)
        for _ in range(2):
            lm_head(x, w, dw, targets, logits, dx, col0, cols, exchange, fused_stats)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            lm_head(x, w, dw, targets, logits, dx, col0, cols, exchange, fused_stats)
        e1.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        del logits
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        return ms

    col0, cols = shards[rank]
    ms = timed(col0, cols, True)
    n1_ms = ms if world == 1 else timed(0, V, False, reps=3)
    ms_separate = timed(col0, cols, True, fused_stats=False)   # statistics by a pass of their own over the logits
    h.sync()
    flop = 3 * 2.0 * rows * V * K
    rec = {"workload": "configs[3] LM head: 16384 tokens x 128256 vocabulary x 768, forward + cross-entropy + dgrad + wgrad(beta=1), "
                       "vocabulary sharded in whole 256-column tiles over %d rank(s)" % world,
           "ranks": world, "ms": round(ms, 3), "tflops": round(flop / ms / 1e9, 1), "n1_ms": round(n1_ms, 3),
           "efficiency_vs_n1": round(n1_ms / (world * ms), 3), "scaling": "strong",
           "columns_per_rank": [n for _, n in shards],
           "exchange_bytes_per_rank": {"all_reduce_max_fp32": rows * 4, "all_reduce_sum_fp32": 2 * rows * 4,
                                       "all_reduce_dx_bf16": rows * K * 2},
           "logits_bytes_per_rank": rows * cols * 2,
           "ms_with_separate_statistics_pass": round(ms_separate, 3),
           "what": "row maximum, sum of exponentials and target logit come out of the forward GEMM's epilogue "
                   "(b200_linear_forward_ce_stats_bf16); ms_with_separate_statistics_pass is the same step with "
                   "b200_ce_shard_stats_bf16 reading the stored logits instead"}
    rec.update(parity)
    return rec


def run_train_step(dist, world, rank, args, link="b200"):
    """The metric's second half: tokens/s of a whole LLaMA-2/Mistral-125M training step (B=16, T=512, 16 micro-batches
    = 131072 tokens per optimizer step, bf16, AdamW) on the ranks of this run, through the package's multi-GPU
    driver csrc/train_dp.cpp (the reference's own model objects with this library's linear layers, one process per
    GPU, NCCL gradient sum).  Rank 0 starts the driver, which forks its own ranks; the ranks of this benchmark hold
    no kernels meanwhile (they wait on the host).  Present only where the binary was built."""
    import tempfile
    binary = os.path.join(ROOT, "oracle", "_ref", "train_dp_%s_llama2_mistral" % link)
    store = None
    if world > 1:
        from torch.distributed.distributed_c10d import _get_default_store
        store = _get_default_store()
    rec = None
    if rank == 0:
        if not os.path.exists(binary):
            rec = {"unavailable": "driver binary not built (needs the reference checkout at build time)"}
        else:
            import re
            import numpy as np
            steps, batch, seq, accum = 2, 16, 512, 16
            with tempfile.TemporaryDirectory() as d:
                data = os.path.join(d, "tokens.bin")
                np.random.default_rng(42).integers(0, 32000, batch * seq * accum * steps + 1, dtype=np.int32).tofile(data)
                t0 = time.time()
                try:
                    out = subprocess.run([binary, data, "--ranks", str(world), "--steps", str(steps), "--batch", str(batch),
                                          "--seq", str(seq), "--accum", str(accum), "--timers"], cwd=d, capture_output=True,
                                         text=True, timeout=args.train_step_timeout)
                    text, rc = out.stdout, out.returncode
                except subprocess.TimeoutExpired:
                    text, rc = "", -1
                wall = time.time() - t0
            toks = re.findall(r"\| (\d+) tok/s", text)
            losses = [float(x) for x in re.findall(r"loss ([0-9.]+)", text)]
            phases = re.search(r"phases, seconds per step.*?: (.*)", text)
            if rc != 0 or not toks:
                rec = {"unavailable": "driver run failed (rc %d)" % rc, "tail": text[-300:]}
            else:
                rec = {"metric": "LLaMA-125M train tok/s", "tokens_per_s": int(toks[-1]), "ranks": world,
                       "tokens_per_step": batch * seq * accum, "steps": steps, "timed": "wall clock of step 2 (step 1 carries set-up)",
                       "losses": losses, "phases_s_per_step": phases.group(1) if phases else None, "wall_s": round(wall, 1),
                       "what": ("csrc/train_dp.cpp around the reference's ModelBF16; linear layers, attention, SwiGLU, RMSNorm and "
                                "cross-entropy from this library; micro-batches dealt to the ranks, one NCCL gradient sum per step")
                               if link == "b200" else
                               "the same driver at one rank with the reference's own, unmodified kernels and cuda/matmul.cu (cuBLAS)"}
        if store is not None:
            store.set("b200_train_step_done", "1")
    elif store is not None:
        import datetime
        store.wait(["b200_train_step_done"], datetime.timedelta(seconds=args.train_step_timeout + 60))
    return rec


def step_breakdown(torch, calls, steps=20):
    """Device time of every call of the step, measured inside the running step (events between calls)."""
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(calls) + 1)] for _ in range(steps)]
    for _, fn in calls:
        fn()
    torch.cuda.synchronize()
    for s_ in range(steps):
        ev[s_][0].record()
        for i, (_, fn) in enumerate(calls):
            fn()
            ev[s_][i + 1].record()
    torch.cuda.synchronize()
    out = {}
    for i, (name, _) in enumerate(calls):
        out[name] = round(sum(ev[s_][i].elapsed_time(ev[s_][i + 1]) for s_ in range(steps)) / steps * 1e3, 2)
    out["total"] = round(sum(out.values()), 2)
    return out


def cpu_baseline_port(seconds_hint=15.0):
    """The oracle's fp32 host GEMM (a CPU restatement of cuda/matmul.cu: the reference has no CPU
    code) on a bounded sample: the seven decoder-layer projections at M=8192, fwd+dgrad+wgrad."""
    import numpy as np
    from oracle import oracle
    flops, secs = 0.0, 0.0
    rng = np.random.default_rng(0)
    passes = 0
    while secs < 10.0 and passes < 8:
      passes += 1
      for name, n, k in PROJECTIONS[:-1]:
        A = rng.standard_normal((TOKENS, k), dtype=np.float32)
        B = (0.02 * rng.standard_normal((k, n), dtype=np.float32))
        dC = rng.standard_normal((TOKENS, n), dtype=np.float32)
        C = np.empty((TOKENS, n), np.float32)
        dA = np.empty((TOKENS, k), np.float32)
        dB = np.zeros((k, n), np.float32)
        t = time.time()
        oracle.gemm_f32(0, 0, C, A, B, TOKENS, n, k)
        oracle.gemm_f32(1, 0, dA, dC, B, TOKENS, n, k)
        oracle.gemm_f32(2, 1, dB, A, dC, TOKENS, n, k)
        secs += time.time() - t
        flops += 3 * 2.0 * TOKENS * n * k
    return {"value": round(flops / secs / 1e12, 4), "unit": "TFLOP/s", "cores": oracle.num_threads(), "kind": "port",
            "seconds": round(secs, 2),
            "sample": "fp32 OpenMP host GEMM (oracle/oracle_gemm.c), the 7 decoder-layer projections at M=8192, "
                      "fwd+dgrad+wgrad, %d pass(es) (no LM head)" % passes}


def run_reference(args):
    """The reference's own, unmodified cuda/matmul.cu (cuBLAS) from oracle/_ref on the same workload
    and GPU; where that build is absent, the oracle's CPU port on a bounded sample."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import ctypes
    path = os.path.join(ROOT, "oracle", "_ref", "libref_matmul.so")
    base = {"impl": "reference", "metric": "bf16 GEMM TFLOP/s, all linear-layer GEMMs of one 125M decoder layer + LM head, fwd+bwd",
            "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "data": "synthetic"}
    import torch
    if not os.path.exists(path) or not torch.cuda.is_available():
        cpu = cpu_baseline_port()
        base.update({"value": cpu["value"], "dtype": "f32", "ms_per_step": None, "cpu_baseline": cpu,
                     "config": {"workload": cpu["sample"]},
                     "e2e": {"value": cpu["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        print(json.dumps(base))
        return
    lib = ctypes.CDLL(path)
    vp, ci = ctypes.c_void_p, ctypes.c_int
    lib.ref_create.argtypes = [ctypes.POINTER(vp)]
    lib.ref_matmul_forward_bf16.argtypes = [vp, vp, vp, vp, ci, ci, ci]
    lib.ref_matmul_forward_bf16.restype = None
    lib.ref_matmul_backward_bf16.argtypes = [vp, vp, vp, vp, vp, vp, ci, ci, ci]
    lib.ref_matmul_backward_bf16.restype = None
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    hd = vp()
    assert lib.ref_create(ctypes.byref(hd)) == 0
    bufs = make_buffers(torch, dev, None, host=True)

    def step():
        for b in bufs:
            lib.ref_matmul_forward_bf16(hd, b["C"].data_ptr(), b["A"].data_ptr(), b["B"].data_ptr(), TOKENS, b["N"], b["K"])
        for b in reversed(bufs):
            lib.ref_matmul_backward_bf16(hd, b["dA"].data_ptr(), b["dB"].data_ptr(), b["dC"].data_ptr(),
                                         b["A"].data_ptr(), b["B"].data_ptr(), TOKENS, b["N"], b["K"])

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    time.sleep(0.3)
    preheat(torch, step)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.time()
    block_ms = time_blocks(torch, step, args.steps)
    t1 = time.time()
    ms = median(block_ms)
    value = args.steps * STEP_FLOP / (ms * 1e-3) / 1e12
    ms_e2e, e2e_steps, h2d, d2h = time_e2e(torch, bufs, step, args.steps, torch.cuda.synchronize)
    e2e_value = e2e_steps * STEP_FLOP / (ms_e2e * 1e-3) / 1e12
    per = []
    for b in bufs:
        for kind, call in (("fwd_nn", lambda: lib.ref_matmul_forward_bf16(hd, b["C"].data_ptr(), b["A"].data_ptr(), b["B"].data_ptr(), TOKENS, b["N"], b["K"])),
                           ("dgrad+wgrad", lambda: lib.ref_matmul_backward_bf16(hd, b["dA"].data_ptr(), b["dB"].data_ptr(), b["dC"].data_ptr(), b["A"].data_ptr(), b["B"].data_ptr(), TOKENS, b["N"], b["K"]))):
            for _ in range(3):
                call()
            e0.record()
            for _ in range(10):
                call()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / 10 * 1e3
            fl = 2.0 * TOKENS * b["N"] * b["K"] * (1 if kind == "fwd_nn" else 2)
            per.append({"proj": b["name"], "gemm": kind, "us": round(us, 2), "tflops": round(fl / us / 1e6, 1)})
    if args.train_step:
        base["train_step"] = run_train_step(None, 1, 0, args, link="ref")
    if args.breakdown:
        calls = [(b["name"] + ":fwd", (lambda b=b: lib.ref_matmul_forward_bf16(hd, b["C"].data_ptr(), b["A"].data_ptr(), b["B"].data_ptr(), TOKENS, b["N"], b["K"]))) for b in bufs]
        calls += [(b["name"] + ":bwd", (lambda b=b: lib.ref_matmul_backward_bf16(hd, b["dA"].data_ptr(), b["dB"].data_ptr(), b["dC"].data_ptr(), b["A"].data_ptr(), b["B"].data_ptr(), TOKENS, b["N"], b["K"]))) for b in reversed(bufs)]
        base["in_step_us"] = step_breakdown(torch, calls)
    base.update({"value": round(value, 2), "dtype": "bf16", "ms_per_step": round(ms / args.steps, 4),
                 "ms_per_step_min": round(min(block_ms) / args.steps, 4), "ms_per_step_max": round(max(block_ms) / args.steps, 4),
                 "blocks": BLOCKS,
                 "implementation": "reference cuda/matmul.cu unmodified (cuBLAS) on the same GPU; the reference has no CPU implementation of this path",
                 "config": common_config(1),
                 "clocks": sampler.stop(t0, t1),
                 "cpu_baseline": {"value": round(value, 2), "unit": "TFLOP/s", "cores": 0, "kind": "reference",
                                  "sample": "whole workload on the GPU (cuBLAS); not a CPU run"},
                 "e2e": {"value": round(e2e_value, 2), "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                         "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                         "what": "the same host copies as the other arm (A and dC in from pinned memory, dA out) around the "
                                 "reference's own calls, so that the two end-to-end numbers compare like with like"},
                 "per_gemm": per})
    print(json.dumps(base))


def run_only(args):
    """One GEMM of the workload, a few launches, at a reduced token count: the small case that
    profiler captures use (still larger than L2 for the LM head)."""
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    h = pkg.Handle()
    proj, kind = args.only.split(":")
    n, k = {name: (n, k) for name, n, k in PROJECTIONS}[proj]
    M = args.tokens
    g = torch.Generator(device=dev).manual_seed(7)
    A = torch.randn(M, k, device=dev, generator=g).to(torch.bfloat16)
    B = (0.02 * torch.randn(k, n, device=dev, generator=g)).to(torch.bfloat16)
    dC = torch.randn(M, n, device=dev, generator=g).to(torch.bfloat16)
    which = {"fwd_nn": pkg.FWD_NN, "dgrad_nt": pkg.DGRAD_NT, "wgrad_tn": pkg.WGRAD_TN}[kind]
    out = torch.zeros({0: (M, n), 1: (M, k), 2: (k, n)}[which], device=dev, dtype=torch.bfloat16)
    x, y = {0: (A, B), 1: (dC, B), 2: (A, dC)}[which]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pkg.gemm(h, which, which == 2, out, x, y, M, n, k)
    e0.record()
    for _ in range(args.reps):
        pkg.gemm(h, which, which == 2, out, x, y, M, n, k)
    e1.record()
    torch.cuda.synchronize()
    h.sync()
    us = e0.elapsed_time(e1) / args.reps * 1e3
    print(json.dumps({"only": args.only, "tokens": M, "N": n, "K": k, "us": round(us, 2),
                      "tflops": round(2.0 * M * n * k / us / 1e6, 1), "launches": h.launches}))


SWEEP_M = [512, 2048, 8192, 16384, 65536]
SWEEP_NK = [768, 1280, 2048, 4096, 8192, 32000, 128256]


def run_sweep(args):
    """Shape / layout / dtype / beta sweep (BASELINE.json configs[4]), this library and the reference's
    cuBLAS build in the same process, every case timed as 5 launches captured in a CUDA graph.  The grid is
    thinned to fit a time budget: cases are ordered by FLOPs and skipped (and listed) once the budget is
    spent or when a case would need more than --sweep-gb of device memory."""
    import ctypes
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    h = pkg.Handle()
    side = torch.cuda.Stream()
    h.set_stream(side)
    ref = None
    path = os.path.join(ROOT, "oracle", "_ref", "libref_matmul.so")
    if os.path.exists(path):
        ref = ctypes.CDLL(path)
        vp, ci = ctypes.c_void_p, ctypes.c_int
        ref.ref_create.argtypes = [ctypes.POINTER(vp)]
        ref.ref_create_fp32.argtypes = [ctypes.POINTER(vp)]
        ref.ref_set_stream.argtypes = [vp, vp]
        for n in ("ref_matmul_forward_bf16", "ref_matmul_forward_f32"):
            getattr(ref, n).argtypes = [vp, vp, vp, vp, ci, ci, ci]
            getattr(ref, n).restype = None
        for n in ("ref_matmul_backward_bf16", "ref_matmul_backward_f32"):
            getattr(ref, n).argtypes = [vp, vp, vp, vp, vp, vp, ci, ci, ci]
            getattr(ref, n).restype = None
        hb, hf = vp(), vp()
        ref.ref_create(ctypes.byref(hb))
        ref.ref_create_fp32(ctypes.byref(hf))
        ref.ref_set_stream(hb, vp(side.cuda_stream))
        ref.ref_set_stream(hf, vp(side.cuda_stream))
    peaks = measured_peaks()

    def tgraph(fn, reps=5):
        with torch.cuda.stream(side):
            fn()
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for _ in range(reps):
                    fn()
            g.replay()
            side.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            g.replay()
            e1.record(side)
            side.synchronize()
        return e0.elapsed_time(e1) / reps * 1e3

    cases = []
    for M in SWEEP_M:
        for N in SWEEP_NK:
            for K in SWEEP_NK:
                cases.append((2.0 * M * N * K, M, N, K))
    cases.sort()
    t_start = time.time()
    skipped = []
    for flop, M, N, K in cases:
        for dt, sfx in ((torch.bfloat16, "bf16"), (torch.float32, "f32")):
            es = 2 if sfx == "bf16" else 4
            gb = es * (M * K + K * N + M * N) * 2 / 1e9  # operands + outputs + gradients, roughly
            if gb > args.sweep_gb or (sfx == "f32" and flop > args.sweep_f32_flop) or time.time() - t_start > args.sweep_seconds:
                skipped.append([sfx, M, N, K])
                continue
            g = torch.Generator(device=dev).manual_seed(M + N + K)
            A = torch.randn(M, K, device=dev, generator=g).to(dt)
            B = torch.randn(K, N, device=dev, generator=g).to(dt)
            dC = torch.randn(M, N, device=dev, generator=g).to(dt)
            for which, name, x, y, shape in ((0, "NN", A, B, (M, N)), (1, "NT", dC, B, (M, K)), (2, "TN", A, dC, (K, N))):
                for beta in (0, 1):
                    out = torch.randn(shape, device=dev, generator=g).to(dt)
                    us = tgraph(lambda: pkg.gemm(h, which, beta, out, x, y, M, N, K))
                    rec = {"dtype": sfx, "layout": name, "beta": beta, "M": M, "N": N, "K": K, "us": round(us, 1),
                           "tflops": round(flop / us / 1e6, 1)}
                    if sfx == "bf16":
                        rec["frac_of_measured_peak"] = round(flop / us / 1e6 / peaks["bf16_tflops"], 3)
                    # the reference's API has no beta argument: forward = NN beta0, backward = NT beta0 + TN beta1
                    if ref is not None and ((which == 0 and beta == 0) or (which == 1 and beta == 0)):
                        hh = hb if sfx == "bf16" else hf
                        if which == 0:
                            fn = getattr(ref, "ref_matmul_forward_" + sfx)
                            rus = tgraph(lambda: fn(hh, out.data_ptr(), A.data_ptr(), B.data_ptr(), M, N, K))
                            rec["reference_us"] = round(rus, 1)
                        else:
                            fn = getattr(ref, "ref_matmul_backward_" + sfx)
                            dB = torch.zeros(K, N, device=dev, dtype=dt)
                            rus = tgraph(lambda: fn(hh, out.data_ptr(), dB.data_ptr(), dC.data_ptr(), A.data_ptr(), B.data_ptr(), M, N, K))
                            rec["reference_backward_us (NT+TN)"] = round(rus, 1)
                    print(json.dumps(rec), flush=True)
            del A, B, dC
    h.sync()
    print(json.dumps({"skipped": skipped, "seconds": round(time.time() - t_start, 1)}))


def run_ce_shard(args):
    """The vocabulary-sharded cross-entropy kernels on one rank's shard of config 4 (16384 tokens, llama3
    vocabulary 128256 over 8 ranks = 16032 columns): HBM-bound, timed alone with CUDA events against the
    measured copy bandwidth.  The reference's own cross-entropy kernels (one thread per row) are timed on the
    same shard when oracle/_ref has them (rows a multiple of 256: their forward has no bounds check)."""
    import ctypes
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    rows, cols = args.ce_rows, 16032
    g = torch.Generator(device=dev).manual_seed(5)
    logits = (3.0 * torch.randn(rows, cols, device=dev, generator=g)).to(torch.bfloat16)  # 525 MB > L2
    targets = torch.randint(0, cols, (rows,), device=dev, generator=g, dtype=torch.int32)
    out = torch.empty_like(logits)
    peaks = measured_peaks()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps * 1e3

    lm, sm, tg = pkg.ce_shard_stats(logits, targets, 0)
    us_stats = timed(lambda: pkg.ce_shard_stats(logits, targets, 0))
    us_bwd = timed(lambda: pkg.ce_shard_backward(logits, targets, 0, lm, sm, 1.0 / rows, out=out))
    nbytes = logits.numel() * 2
    line = {"metric": "vocabulary-sharded cross-entropy kernels, one rank's shard of config 4", "unit": "GB/s",
            "config": {"workload": "logits [%d, 16032] bf16 (%d MB, larger than L2), int32 targets" % (rows, rows * cols * 2 // 1000000)},
            "stats": {"us": round(us_stats, 1), "gbs": round(nbytes / us_stats / 1e3, 1),
                      "frac_of_measured_hbm": round(nbytes / us_stats / 1e3 / peaks["hbm_gbs"], 3),
                      "algorithmic_bytes": nbytes},
            "backward": {"us": round(us_bwd, 1), "gbs": round(2 * nbytes / us_bwd / 1e3, 1),
                         "frac_of_measured_hbm": round(2 * nbytes / us_bwd / 1e3 / peaks["hbm_gbs"], 3),
                         "algorithmic_bytes": 2 * nbytes},
            "peak": peaks["hbm_gbs"], "peak_source": peaks["source"]}
    path = os.path.join(ROOT, "oracle", "_ref", "libref_matmul.so")
    if os.path.exists(path):
        lib = ctypes.CDLL(path)
        if hasattr(lib, "ref_crossentropy_forward_bf16"):
            vp, ci = ctypes.c_void_p, ctypes.c_int
            lib.ref_crossentropy_forward_bf16.argtypes = [vp, vp, vp, ci, ci, ci]
            lib.ref_crossentropy_forward_bf16.restype = None
            lib.ref_crossentropy_backward_bf16.argtypes = [vp, vp, vp, ci, ci, ci, ctypes.c_float]
            lib.ref_crossentropy_backward_bf16.restype = None
            probs = logits.clone()
            loss = torch.empty(rows, device=dev, dtype=torch.float32)
            us_rf = timed(lambda: lib.ref_crossentropy_forward_bf16(loss.data_ptr(), probs.data_ptr(), targets.data_ptr(), 2, rows // 2, cols), reps=3)
            us_rb = timed(lambda: lib.ref_crossentropy_backward_bf16(out.data_ptr(), probs.data_ptr(), targets.data_ptr(), 2, rows // 2, cols, 1.0), reps=3)
            line["reference"] = {"forward_us": round(us_rf, 1), "backward_us": round(us_rb, 1),
                                 "what": "cuda/crossentropy.cu bf16 overloads, unmodified, whole-row version on the same matrix"}
    print(json.dumps(line))


def run_attention(args):
    """The fused causal grouped-query attention core (csrc/attention_sm100.cuh: what fills the reference's empty
    flash_attention_forward / flash_attention_backward, cuda/flash_attention.cu:12-17,51-57) timed alone on the two
    model shapes: LLaMA-2/Mistral 125M (B=16, T=512) and LLaMA-3 272M (B=2, T=8192); 12 query heads, 4 KV heads,
    head dimension 64, bf16.  FLOP counted for the causal half only: forward 4*B*nh*T^2*64/2, backward 2.5 x that."""
    import importlib
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    layers = importlib.import_module(pkg.__name__ + ".layers")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    peaks = measured_peaks()
    out = {"metric": "fused causal GQA attention core, bf16, head_dim 64, 12 query / 4 KV heads", "unit": "TFLOP/s",
           "peak": peaks["bf16_tflops"], "peak_source": peaks["source"], "cases": []}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    shapes = [(16, 512), (2, 8192)] if args.attn_shape is None else [tuple(int(x) for x in args.attn_shape.split("x"))]
    for B, T in shapes:
        nh, nkv, hd = 12, 4, 64
        g = torch.Generator(device=dev).manual_seed(B * T)
        q = torch.randn(B * T, nh * hd, device=dev, generator=g).to(torch.bfloat16)
        k = torch.randn(B * T, nkv * hd, device=dev, generator=g).to(torch.bfloat16)
        v = torch.randn(B * T, nkv * hd, device=dev, generator=g).to(torch.bfloat16)
        do = torch.randn(B * T, nh * hd, device=dev, generator=g).to(torch.bfloat16)
        ctx, lse = torch.empty_like(q), torch.empty(B, nh, T, device=dev, dtype=torch.float32)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        fwd = lambda: layers.flash_attention_forward(ctx, lse, q, k, v, B, T, nh, nkv, hd)
        bwd = lambda: layers.flash_attention_backward(dq, dk, dv, do, q, k, v, lse, B, T, nh, nkv, hd, context=ctx)
        rec = {"B": B, "T": T}
        for name, fn, mult in (("forward", fwd, 1.0), ("backward", bwd, 2.5)):
            for _ in range(args.reps):
                fn()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(args.reps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / args.reps * 1e3
            flop = mult * 4.0 * B * nh * T * T * hd / 2
            rec[name] = {"us": round(us, 1), "tflops": round(flop / us / 1e6, 1),
                         "frac_of_measured_peak": round(flop / us / 1e6 / peaks["bf16_tflops"], 3)}
        out["cases"].append(rec)
    print(json.dumps(out))


def main():
    # stdout carries the one JSON line: whatever NCCL prints at its debug level (a version banner, warnings) goes to stderr
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":   # that level's banner is a bare printf to stdout
        os.environ["NCCL_DEBUG"] = "WARN"
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None, help="profile mode: <projection>:<fwd_nn|dgrad_nt|wgrad_tn>")
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--breakdown", action="store_true", help="also time every call inside the running step")
    ap.add_argument("--sweep", action="store_true", help="shape/layout/dtype/beta sweep against the reference's cuBLAS")
    ap.add_argument("--sweep-seconds", type=float, default=240.0)
    ap.add_argument("--sweep-gb", type=float, default=40.0)
    ap.add_argument("--sweep-f32-flop", type=float, default=3e12)
    ap.add_argument("--ce-shard", action="store_true", help="time the vocabulary-sharded cross-entropy kernels")
    ap.add_argument("--ce-rows", type=int, default=16384, help="rows of the shard for --ce-shard (a multiple of 512)")
    ap.add_argument("--no-vocab-parallel", dest="vocab_parallel", action="store_false",
                    help="skip the vocabulary-sharded LM head + cross-entropy sub-record")
    ap.add_argument("--train-step-timeout", type=float, default=600.0)
    ap.add_argument("--attention", action="store_true", help="time the fused attention core on the two model shapes")
    ap.add_argument("--attn-shape", default=None, help="BxT for --attention (default: 16x512 and 2x8192)")
    ap.add_argument("--no-train-step", dest="train_step", action="store_false",
                    help="skip the whole-training-step sub-record (the multi-GPU driver, 2 optimizer steps)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.attention:
        run_attention(args)
    elif args.ce_shard:
        run_ce_shard(args)
    elif args.sweep:
        run_sweep(args)
    elif args.only:
        run_only(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

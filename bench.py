#!/usr/bin/env python
"""Headline benchmark: greedy decode tokens/s of a Llama-3-8B-architecture Q4_K model (synthetic
seeded weights, 512-token random-id prompt, paged fp16 KV with 16-token pages, context 4096) and
the achieved HBM bandwidth of the quantised matrix-vector kernel against the measured peak.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--batch B] [--format Q4_K|Q8_0|Q4_0] [--arch 8b|1b|tiny] [--prompt P]

One process per GPU (torchrun sets RANK/LOCAL_RANK/WORLD_SIZE). Rank 0 prints ONE JSON line.

value  : tokens/s with token feedback resident on the device (jl_generate: no host round trip).
e2e    : tokens/s through the reference-facing call (BatchExecutor.decodeStep -> jl_decode) with
         host token/position arrays going in and sampled ids coming back every step.
roofline: the dominant kernel (RMSNorm + gate/up + SwiGLU matrix-vector launch) timed alone with
         CUDA events over all layers' weights (2.1 GB for the 8B shape, so every launch reads HBM),
         algorithmic bytes / time against MEASURED_PEAKS.json.
cpu_baseline / --impl reference: the C restatement of jitLLM's CPU path (oracle/) on the host
         cores, a bounded number of decode steps of the same model.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

ARCHS = {
    # dim, hidden, layers, heads, kv_heads, vocab, ctx, tied
    "8b": (4096, 14336, 32, 32, 8, 128256, 4096, False),
    "1b": (2048, 8192, 16, 32, 8, 128256, 2048, True),
    "tiny": (512, 1024, 4, 8, 2, 4096, 1024, False),
    # Llama-3-70B architecture: the tensor-parallel configuration (B=16, 1024-token prompts)
    "70b": (8192, 28672, 80, 64, 8, 128256, 4096, False),
    # four layers of the 8B layer shapes with a small vocabulary: the profiling-sized case
    "8b4": (4096, 14336, 4, 32, 8, 16384, 4096, False),
}
BYTES_PER_EL = {"Q4_K": 144 / 256, "Q4_0": 18 / 32, "Q8_0": 34 / 32}
EXTRA_BYTES_PER_EL = {"Q4_1": 20 / 32, "Q5_K": 176 / 256, "Q6_K": 210 / 256}  # stand-alone operators only
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the gate/up kernel for the 8B layer
# shape, from one ncu capture of that launch (the summary is kept with the other profile summaries)
NCU_TRAFFIC_BYTES = {("Q4_K", 4096, 14336): 66.89e6}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--format", default="Q4_K", choices=list(BYTES_PER_EL))
    ap.add_argument("--arch", default="8b", choices=list(ARCHS))
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--seed", type=int, default=20261125)
    ap.add_argument("--cpu-seconds", type=float, default=15.0, help="budget of the CPU baseline leg")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile-matmul", default="",
                    help="ROWSxCOLSxN: launch the standalone product on three copies of one matrix --steps times and "
                         "exit: the small case ncu captures of the tensor-core kernel are taken on")
    ap.add_argument("--also-batch", type=int, default=32,
                    help="after the B=1 measurement on one GPU, also time this many sequences decoded together "
                         "(the metric names B=1 and B=32) and report it under \"batched\"; 0 skips it")
    ap.add_argument("--sweep", action="store_true",
                    help="standalone quantised mat-vec / mat-mat sweep (formats x shapes x N): one JSON line per case")
    ap.add_argument("--parallel", default="tp", choices=["tp", "replicas"],
                    help="with more than one GPU: tensor parallelism over one model (strong scaling, the default) "
                         "or one whole model per GPU (weak scaling)")
    ap.add_argument("--profile-op", type=int, default=-1,
                    help="launch one matrix-vector operator (0 qkv, 1 out, 2 gate/up, 3 down, 4 vocab) "
                         "--steps times and exit: the small case ncu captures are taken on")
    ap.add_argument("--sweep-formats", default="Q8_0,Q4_0,Q4_K,Q4_1,Q5_K,Q6_K",
                    help="comma-separated formats of --sweep")
    ap.add_argument("--sweep-shapes", default="4096x4096,14336x4096,4096x14336,128256x4096",
                    help="comma-separated rows x cols of --sweep")
    ap.add_argument("--mixed", action="store_true",
                    help="Q6_K value / down projections (every other layer) and output matrix, as in a mixed-precision file")
    ap.add_argument("--prefill-sweep", action="store_true",
                    help="prompt ingestion rate for prompts of 512, 2048 and 8192 tokens, 1 and 4 sequences (the batched "
                         "prefill configuration; use --format Q8_0): one JSON line per case")
    ap.add_argument("--timeline", action="store_true",
                    help="print the launch timeline of one decode step (--batch sequences) from the trace build of the "
                         "library: run as JITLLM_B200_TRACE=1 python bench.py --timeline ... after "
                         "python jitllm_b200/build.py --trace")
    return ap.parse_args()


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs (read-only)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        inside = [r for ts, r in self.rows if t0 - 0.05 <= ts <= t1 + 0.15 and len(r) >= 8] or \
                 [r for _, r in self.rows if len(r) >= 8]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(float(r[1]) for r in inside)
        reasons = []
        for name, col in (("hw_slowdown", 4), ("hw_thermal_slowdown", 5), ("sw_thermal_slowdown", 6),
                          ("sw_power_cap", 7)):
            if any(r[col].lower().startswith("active") for r in inside):
                reasons.append(name)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(inside[0][2]), "reasons": reasons,
                "samples": len(inside), "power_w_max": max(float(r[3]) for r in inside)}


def model_bytes(cfg, fmt):
    """Algorithmic bytes one decode step must read: every weight matrix once."""
    bpe = BYTES_PER_EL[fmt]
    dim, hid, L, kv = cfg.dim, cfg.hiddenDim, cfg.numberOfLayers, cfg.kvDim
    per_layer = dim * dim * 2 + kv * dim * 2 + hid * dim * 3
    return (per_layer * L + cfg.vocabularySize * dim) * bpe


def op_bytes(cfg, fmt, op, shards=1):
    """Algorithmic bytes of one launch on one GPU: the weight slice once, the input vector, the output."""
    bpe = BYTES_PER_EL[fmt]
    dim, hid, kv, V = cfg.dim, cfg.hiddenDim // shards, cfg.kvDim // shards, cfg.vocabularySize // shards
    qd = dim // shards
    rows, cols = {0: (qd + 2 * kv, dim), 1: (dim, qd), 2: (2 * hid, dim), 3: (dim, hid), 4: (V, dim)}[op]
    out_rows = hid if op == 2 else rows
    return rows * cols * bpe + 4 * cols + 4 * out_rows


def run_sweep(jl, args):
    """Formats {Q8_0, Q4_0, Q4_K, Q4_1, Q5_K, Q6_K} x shapes x N through jl_gemv_dev with device-resident operands.
    Each case cycles over enough copies of the matrix to exceed L2 (126 MB), so every launch reads HBM."""
    import numpy as np
    dev = jl.Device(0)
    peak, peak_kind = measured_peak()
    shapes = tuple(tuple(int(v) for v in sh.split("x")) for sh in args.sweep_shapes.split(",") if sh)
    for fmt_name in [f for f in args.sweep_formats.split(",") if f]:
        t = jl.GGMLType[fmt_name]
        extra = fmt_name in EXTRA_BYTES_PER_EL  # no encoder here: random blocks with sane scales
        for rows, cols in shapes:
            w = (jl.random_blocks(t, rows * cols, seed=args.seed + rows + cols) if extra
                 else jl.synth_tensor(t, rows * cols, seed=args.seed + rows + cols))
            wbytes = rows * cols * (EXTRA_BYTES_PER_EL if extra else BYTES_PER_EL)[fmt_name]
            copies = int(min(32, max(1, -(-300e6 // wbytes))))
            mats = [dev.upload_matrix(t, w, rows, cols) for _ in range(copies)]
            for n in (1, 8, 32, 512, 2048):
                x = np.random.default_rng(args.seed + n).standard_normal((n, cols)).astype(np.float32)
                xd, yd = dev.alloc(x.nbytes), dev.alloc(n * rows * 4)
                dev.h2d(xd, x)
                for m in mats:
                    m.matmul_dev(xd, n, yd)
                reps = max(1, min(8, 64 // copies)) if n <= 32 else 1
                dev.synchronize()
                dev.timer_start()
                for _ in range(reps):
                    for m in mats:
                        m.matmul_dev(xd, n, yd)
                us = dev.timer_stop() * 1000.0 / (reps * copies)
                by = wbytes + 4 * cols * n + 4 * rows * n
                print(json.dumps({"sweep": fmt_name, "rows": rows, "cols": cols, "n": n, "us": round(us, 2),
                                  "bytes": by, "gbs": round(by / us / 1e3, 1), "hbm_frac": round(by / us / 1e3 / peak, 4),
                                  "tflops": round(2.0 * rows * cols * n / us / 1e6, 2), "peak_kind": peak_kind,
                                  "kernel": "gemv" if n < 8 else "gemm_tc"}), flush=True)
                dev.free(xd)
                dev.free(yd)
            for m in mats:
                m.close()
    return 0


def batched_leg(jl, dev, kv, cfg, tensors, cr, ci, args):
    """The same model with `--also-batch` sequences decoded together (tensor-core path): prompts of the
    same length, token feedback on the device, CUDA events around the timed steps."""
    import numpy as np
    Bn, P, K = getattr(args, "also_batch_now", args.also_batch), args.prompt, max(8, min(args.steps, 64))
    kv.close()
    model = jl.load_model(dev, cfg, tensors, cr, ci, maxBatch=Bn)  # replaces the B=1 model on this context
    bps = cfg.contextLength // 16
    need = (P + K + 3 + 64 + 15) // 16
    store = model.createKvStorage(jl.KvStorageRequest(Bn * need, bps, Bn, 16, cfg.numberOfLayers, cfg.kvDim))
    table = np.full(Bn * bps, jl.UNMAPPED, dtype=np.int32)
    for b in range(Bn):
        table[b * bps:b * bps + need] = np.arange(b * need, (b + 1) * need)
    store.publishBlockTable(table)
    ex = jl.B200BatchExecutor(model)
    prompts = np.random.default_rng(args.seed + 1).integers(0, cfg.vocabularySize, size=(Bn, P))
    for b in range(Bn):
        jl.B200InvocationBoundary(model, kvSlot=b, copyLogits=False).prefill(prompts[b, :P - 1], 0)
    slots, active = list(range(Bn)), [True] * Bn
    hist = ex.generate(jl.BatchSlots(active, [int(t) for t in prompts[:, P - 1]], [P - 1] * Bn, slots), 3)
    dev.synchronize()
    dev.timer_start()
    ex.generate(jl.BatchSlots(active, [int(t) for t in hist[-1]], [P + 2] * Bn, slots), K)
    ms = dev.timer_stop()
    weights_b = model_bytes(cfg, args.format)
    kv_b = Bn * (P + 2 + K // 2) * cfg.numberOfLayers * cfg.kvDim * 2 * 2
    peak, _ = measured_peak()
    store.close()
    return {"batch": Bn, "value": Bn * K / (ms / 1000.0), "unit": "tok/s", "steps": K, "ms_per_step": ms / K,
            "frac_of_measured_hbm_peak": (weights_b + kv_b) / (ms / K) / 1e6 / peak, "kernel": "gemm_tc_kernel (tcgen05)"}


def cpu_decode_rate(cfg, tensors, budget_s, max_steps, seed, depth=0):
    """tokens/s of the oracle's forwardJava on this host: decode steps from position `depth`. The
    K/V cache below `depth` is filled with seeded random binary16 rows instead of an hour of CPU
    prefill, so that attention does the same work per step as on the GPU arm at that depth."""
    from oracle import binding as oracle
    om = oracle.Model(cfg, tensors)
    rng = np.random.default_rng(seed)
    if depth > 0:
        om.fill_cache(depth, rng)
    toks = rng.integers(0, cfg.vocabularySize, size=max_steps + 1)
    om.forward(int(toks[0]), depth)  # untimed warm-up, as JitllmBench does
    t0 = time.perf_counter()
    done = 0
    while done < max_steps:
        om.forward(int(toks[done + 1]), depth + done + 1)
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    cores = oracle.lib().orc_get_threads()
    om.close()
    return done / dt, cores, done, dt


def cpu_sample_text(done, depth, dt):
    return (f"{done} single-sequence decode steps from position {depth + 1} (K/V cache below it pre-filled with "
            f"seeded random rows, no CPU prefill), all layers, scalar summation mode, {dt:.1f} s")


def run_prefill_sweep(jl, args):
    """Prompt tokens per second through jl_prefill (chunks of up to 512 rows: tcgen05 projections, tiled
    tensor-core attention), CUDA-event time of the whole ingestion, for the batched-prefill configuration."""
    dims = list(ARCHS[args.arch])
    dims[6] = max(dims[6], 8192 + 256)
    cfg = jl.Configuration(dim=dims[0], hiddenDim=dims[1], numberOfLayers=dims[2], numberOfHeads=dims[3],
                           numberOfKeyValueHeads=dims[4], vocabularySize=dims[5], contextLength=dims[6],
                           tiedEmbeddings=dims[7])
    tensors = jl.synth_model_tensors(cfg, jl.GGMLType[args.format], args.seed, threads=os.cpu_count())
    cr, ci = jl.precomputeFreqsCis(cfg.contextLength, cfg.headSize, cfg.ropeTheta)
    dev = jl.Device(0)
    model = jl.load_model(dev, cfg, tensors, cr, ci, maxBatch=4)
    bps = cfg.contextLength // 16
    kv = model.createKvStorage(jl.KvStorageRequest(4 * bps, bps, 4, 16, cfg.numberOfLayers, cfg.kvDim))
    kv.publishBlockTable(np.arange(4 * bps, dtype=np.int32))
    flops_per_token = 2.0 * (model_bytes(cfg, args.format) / BYTES_PER_EL[args.format] - cfg.vocabularySize * cfg.dim)
    warm = np.random.default_rng(1).integers(0, cfg.vocabularySize, size=600)
    jl.B200InvocationBoundary(model, kvSlot=0, copyLogits=False).prefill(warm, 0)
    for P in (512, 2048, 8192):
        for batch in (1, 4):
            prompts = np.random.default_rng(P + batch).integers(0, cfg.vocabularySize, size=(batch, P))
            bounds = [jl.B200InvocationBoundary(model, kvSlot=b, copyLogits=False) for b in range(batch)]
            dev.synchronize()
            dev.timer_start()
            for b in range(batch):
                bounds[b].prefill(prompts[b], 0)
            ms = dev.timer_stop()
            rate = batch * P / (ms / 1e3)
            print(json.dumps({"prefill": {"arch": args.arch, "format": args.format, "prompt": P, "sequences": batch},
                              "ms": round(ms, 2), "prompt_tok_s": round(rate, 1),
                              "projection_tflops": round(rate * flops_per_token / 1e12, 1)}), flush=True)
    return 0


def run_mixed(jl, args):
    """Decode rate of a model with the tensor mix of a mixed-precision file next to the same model in one format:
    the value and down projections of every other layer and the output matrix in Q6_K (random payloads of
    weight-like magnitude: there is no Q6_K encoder here). One JSON line."""
    import numpy as np
    dims = ARCHS[args.arch]
    cfg = jl.Configuration(dim=dims[0], hiddenDim=dims[1], numberOfLayers=dims[2], numberOfHeads=dims[3],
                           numberOfKeyValueHeads=dims[4], vocabularySize=dims[5], contextLength=dims[6],
                           tiedEmbeddings=dims[7])
    B, P, K = args.batch, args.prompt, max(args.steps, 4)
    base = jl.synth_model_tensors(cfg, jl.GGMLType[args.format], args.seed, threads=os.cpu_count())
    R, Q6 = jl.TensorRole, jl.GGMLType.Q6_K
    mixed = dict(base)
    q6_bytes = 0
    for (role, layer) in list(mixed):
        if (role in (R.ATTENTION_VALUE, R.FFN_DOWN) and layer % 2 == 0) or role == R.OUTPUT:
            rows, cols = cfg.matrix_shape(role)
            mixed[(role, layer)] = (Q6, jl.random_blocks(Q6, rows * cols, args.seed + 31 * layer + int(role), 3e-5))
            q6_bytes += mixed[(role, layer)][1].size
    cr, ci = jl.precomputeFreqsCis(cfg.contextLength, cfg.headSize, cfg.ropeTheta)
    out = {}
    for name, tensors in (("one_format", base), ("mixed", mixed)):
        dev = jl.Device(0)
        model = jl.load_model(dev, cfg, tensors, cr, ci, maxBatch=B)
        bps = cfg.contextLength // 16
        need = (P + 2 * K + 24 + 15) // 16
        kv = model.createKvStorage(jl.KvStorageRequest(B * need, bps, B, 16, cfg.numberOfLayers, cfg.kvDim))
        table = np.full(B * bps, jl.UNMAPPED, dtype=np.int32)
        for b in range(B):
            table[b * bps:b * bps + need] = np.arange(b * need, (b + 1) * need)
        kv.publishBlockTable(table)
        ex = jl.B200BatchExecutor(model)
        prompts = np.random.default_rng(args.seed).integers(0, cfg.vocabularySize, size=(B, P))
        for b in range(B):
            jl.B200InvocationBoundary(model, kvSlot=b, copyLogits=False).prefill(prompts[b, :P - 1], 0)
        slots, active = list(range(B)), [True] * B
        hist = ex.generate(jl.BatchSlots(active, [int(t) for t in prompts[:, P - 1]], [P - 1] * B, slots), 4)
        dev.synchronize()
        dev.timer_start()
        ex.generate(jl.BatchSlots(active, [int(t) for t in hist[-1]], [P + 3] * B, slots), K)
        ms = dev.timer_stop() / K
        out[name] = {"ms_per_step": round(ms, 4), "tok_s": round(B * 1000.0 / ms, 1)}
        kv.close()
        dev.close()
    print(json.dumps({"mixed_formats": {"arch": args.arch, "format": args.format, "batch": B, "prompt": P, "steps": K,
                                        "q6_k_bytes": q6_bytes, **out}}), flush=True)
    return 0


def run_timeline(jl, args):
    """One decode step of --batch sequences as a table of launches, from the stamps the trace build of the
    library leaves (first CTA of every launch: entry, dependency resolved, operands staged, loop done, exit)."""
    if os.environ.get("JITLLM_B200_TRACE") != "1":
        print("--timeline needs the trace build: JITLLM_B200_TRACE=1 python bench.py --timeline ...", file=sys.stderr)
        return 2
    dims = ARCHS[args.arch]
    cfg = jl.Configuration(dim=dims[0], hiddenDim=dims[1], numberOfLayers=dims[2], numberOfHeads=dims[3],
                           numberOfKeyValueHeads=dims[4], vocabularySize=dims[5], contextLength=dims[6],
                           tiedEmbeddings=dims[7])
    B, P = args.batch, args.prompt
    tensors = jl.synth_model_tensors(cfg, jl.GGMLType[args.format], args.seed, threads=os.cpu_count())
    cr, ci = jl.precomputeFreqsCis(cfg.contextLength, cfg.headSize, cfg.ropeTheta)
    dev = jl.Device(0)
    model = jl.load_model(dev, cfg, tensors, cr, ci, maxBatch=B)
    bps = cfg.contextLength // 16
    need = (P + 64 + 15) // 16
    kv = model.createKvStorage(jl.KvStorageRequest(B * need, bps, B, 16, cfg.numberOfLayers, cfg.kvDim))
    table = np.full(B * bps, jl.UNMAPPED, dtype=np.int32)
    for b in range(B):
        table[b * bps:b * bps + need] = np.arange(b * need, (b + 1) * need)
    kv.publishBlockTable(table)
    ex = jl.B200BatchExecutor(model)
    prompts = np.random.default_rng(args.seed).integers(0, cfg.vocabularySize, size=(B, P))
    for b in range(B):
        jl.B200InvocationBoundary(model, kvSlot=b, copyLogits=False).prefill(prompts[b, :P - 1], 0)
    slots, active = list(range(B)), [True] * B
    hist = ex.generate(jl.BatchSlots(active, [int(t) for t in prompts[:, P - 1]], [P - 1] * B, slots), 4)
    dev.synchronize()
    dev.timer_start()
    hist = ex.generate(jl.BatchSlots(active, [int(t) for t in hist[-1]], [P + 3] * B, slots), 16)
    ms = dev.timer_stop() / 16
    cap = dev._lib.jl_debug_trace(dev.handle, None, 0)  # arm
    ex.generate(jl.BatchSlots(active, [int(t) for t in hist[-1]], [P + 19] * B, slots), 3)
    buf = np.zeros(cap * 8, dtype=np.uint64)
    n = dev._lib.jl_debug_trace(dev.handle, buf.ctypes.data, cap)
    rec = buf.reshape(cap, 8)[:n].astype(np.int64)
    rec = rec[np.argsort(rec[:, 1])]
    step = rec[n // 3: 2 * n // 3]  # the middle one of the three traced steps
    names = {1: "mat-vec", 2: "attention", 3: "embedding", 4: "advance", 5: "mat-mat", 6: "row kernel", 7: "exchange"}
    print(f"# one decode step, {args.arch} {args.format}, B={B}, {P + 20} keys; {ms:.3f} ms/step in the trace build; "
          f"{len(step)} launches; times in us, first CTA of each launch")
    print("# mat-vec: A = wait for the kernel ahead, B = stage the activations, C = weight loop, D = epilogue to exit")
    print("# mat-mat: A = set-up (barriers, tensor memory), B = wait for the first weights, C = main loop (it fills the "
          "operand ring, then waits for the kernel ahead before the first results), D = tail; other kernels stamp entry "
          "(and exit) only")
    print("| launch | kernel | entry | A | B | C | D |")
    print("| ---: | --- | ---: | ---: | ---: | ---: | ---: |")
    per_layer = max(1, (len(step) - 3) // cfg.numberOfLayers)
    shown = list(range(min(len(step), 1 + 2 * per_layer))) + list(range(max(0, len(step) - 3), len(step)))
    for i in sorted(set(shown)):
        r = step[i]
        ent, a, b_, c, d = (int(v) for v in r[1:6])
        def us(x, y):
            return "%.2f" % ((x - y) / 1e3) if x and y else "-"
        print(f"| {i} | {names.get(int(r[0]), str(int(r[0])))} | {(ent - int(step[0, 1])) / 1e3:.2f} | {us(a, ent)} | {us(b_, a)} | "
              f"{us(c, b_)} | {us(d, c) if c else us(d, a)} |")
    print(f"step span {(int(step[-1, 5] or step[-1, 1]) - int(step[0, 1])) / 1e3:.1f} us; one layer = {per_layer} launches")
    return 0


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    n_gpus = args.gpus

    import jitllm_b200 as jl

    if args.sweep:
        return run_sweep(jl, args) if rank == 0 else 0
    if args.timeline:
        return run_timeline(jl, args) if rank == 0 else 0
    if args.prefill_sweep:
        return run_prefill_sweep(jl, args) if rank == 0 else 0
    if args.mixed:
        return run_mixed(jl, args) if rank == 0 else 0
    if args.profile_matmul:
        if rank != 0:
            return 0
        rows, cols, n = (int(v) for v in args.profile_matmul.lower().split("x"))
        t = jl.GGMLType[args.format]
        dev = jl.Device(0)
        w = jl.synth_tensor(t, rows * cols, seed=args.seed)
        mats = [dev.upload_matrix(t, w, rows, cols) for _ in range(3)]
        x = np.random.default_rng(args.seed).standard_normal((n, cols)).astype(np.float32)
        xd, yd = dev.alloc(x.nbytes), dev.alloc(n * rows * 4)
        dev.h2d(xd, x)
        for _ in range(max(args.warmup, 1)):
            for m in mats:
                m.matmul_dev(xd, n, yd)
        dev.synchronize()
        dev.timer_start()
        for _ in range(args.steps):
            for m in mats:
                m.matmul_dev(xd, n, yd)
        us = dev.timer_stop() * 1000.0 / (3 * args.steps)
        by = rows * cols * BYTES_PER_EL[args.format] + 4 * cols * n + 4 * rows * n
        print(json.dumps({"profile_matmul": args.profile_matmul, "format": args.format, "launches": 3 * args.steps,
                          "us_per_launch": us, "bytes_per_launch": by, "flops_per_launch": 2.0 * rows * cols * n}), flush=True)
        return 0

    dims = ARCHS[args.arch]
    cfg = jl.Configuration(dim=dims[0], hiddenDim=dims[1], numberOfLayers=dims[2], numberOfHeads=dims[3],
                           numberOfKeyValueHeads=dims[4], vocabularySize=dims[5], contextLength=dims[6],
                           tiedEmbeddings=dims[7])
    fmt = jl.GGMLType[args.format]
    B, K, W, P = args.batch, args.steps, args.warmup, args.prompt
    workload = f"llama3-{args.arch}-arch {args.format} greedy decode, B={B}, {P}-token prompt, ctx {cfg.contextLength}, 16-token fp16 KV pages"
    config = {"workload": workload, "batch": B, "prompt_len": P, "format": args.format,
              "cache": "weights of one step (%.2f GB) exceed L2; no flush needed" % (model_bytes(cfg, args.format) / 1e9)}

    if args.impl == "reference":
        if rank != 0:
            return 0
        t0 = time.time()
        tensors = jl.synth_model_tensors(cfg, fmt, args.seed)
        budget = min(240.0, max(10.0, 3.0 * K))
        depth = P + max(W, 3)  # where the other arm's timed region starts
        rate, cores, done, dt = cpu_decode_rate(cfg, tensors, budget, max(1, K), args.seed, depth=depth)
        line = {"impl": "reference", "metric": "decode tok/s", "value": rate, "unit": "tok/s", "n_gpus": n_gpus,
                "steps": K, "steps_measured": done, "warmup": max(W, 3), "ms_per_step": 1000.0 / rate,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": config,
                "cpu_baseline": {"value": rate, "unit": "tok/s", "cores": cores, "kind": "port",
                                 "sample": cpu_sample_text(done, depth, dt) +
                                           f"; one untimed step first; model built in {time.time() - t0 - dt:.0f} s"},
                "e2e": {"value": rate, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line), flush=True)
        return 0

    import torch
    import torch.distributed as dist

    distributed = world > 1
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    def barrier():
        if distributed:
            dist.barrier()

    use_tp = distributed and args.parallel == "tp"
    tp = jl.TensorParallel(rank, world) if use_tp else jl.TensorParallel()
    shards = tp.size  # the matrices of one step are spread over this many GPUs
    t_build = time.time()
    threads = max(1, (os.cpu_count() or 1) // max(1, world))
    tensors = jl.synth_model_tensors(cfg, fmt, args.seed, threads=threads, tp=tp if use_tp else None)
    cr, ci = jl.precomputeFreqsCis(cfg.contextLength, cfg.headSize, cfg.ropeTheta)
    dev = jl.Device(local_rank)
    model = jl.load_model(dev, cfg, tensors, cr, ci, maxBatch=B, tp=tp, broadcast=jl.torch_broadcast,
                          presharded=use_tp)
    t_build = time.time() - t_build

    if args.profile_op >= 0:
        model.benchOp(args.profile_op, 0, max(W, 1))
        dev.synchronize()
        dev.timer_start()
        model.benchOp(args.profile_op, 0, K)
        t_ms = dev.timer_stop()
        print(json.dumps({"profile_op": args.profile_op, "launches": K, "us_per_launch": t_ms * 1000.0 / K,
                          "bytes_per_launch": op_bytes(cfg, args.format, args.profile_op, shards)}), flush=True)
        return 0

    # KV pool: only the pages this run touches are mapped; the rest stay UNMAPPED (scratch block).
    bps = cfg.contextLength // 16
    total_tokens = P + W + 3 * K + 64
    if total_tokens > cfg.contextLength:
        raise SystemExit(f"prompt + steps ({total_tokens}) exceed the context ({cfg.contextLength})")
    need = (total_tokens + 15) // 16
    kv = model.createKvStorage(jl.KvStorageRequest(B * need, bps, B, 16, cfg.numberOfLayers, model.localKvDim))
    table = np.full(B * bps, jl.UNMAPPED, dtype=np.int32)
    for b in range(B):
        table[b * bps:b * bps + need] = np.arange(b * need, (b + 1) * need)
    kv.publishBlockTable(table)
    ex = jl.B200BatchExecutor(model)

    rng = np.random.default_rng(args.seed + (0 if use_tp else rank))  # one prompt for the whole group under TP
    prompts = rng.integers(0, cfg.vocabularySize, size=(B, P))
    t_prefill = time.perf_counter()
    for b in range(B):
        jl.B200InvocationBoundary(model, kvSlot=b, copyLogits=False).prefill(prompts[b, :P - 1], 0)
    dev.synchronize()
    t_prefill = time.perf_counter() - t_prefill

    active = [True] * B
    slots = list(range(B))
    pos = P - 1
    last = [int(t) for t in prompts[:, P - 1]]

    logits_tp = None
    if use_tp:
        # one step with the logits gathered, for the parity record below (re-decoding position P-1 in the
        # warm-up writes the same K/V rows again)
        _, logits_tp = ex.decodeStep(jl.BatchSlots(active, last, [pos] * B, slots), wantLogits=True)
    # warm-up (also captures the step graph)
    hist = ex.generate(jl.BatchSlots(active, last, [pos] * B, slots), max(W, 3))
    warm_hist = hist
    pos += max(W, 3)
    last = [int(t) for t in hist[-1]]

    # ---- timed region 1: device-resident token feedback
    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)
    c0 = dev.counters()
    barrier()
    dev.synchronize()
    wall0 = time.time()
    dev.timer_start()
    hist = ex.generate(jl.BatchSlots(active, last, [pos] * B, slots), K)
    ms = dev.timer_stop()
    wall1 = time.time()
    barrier()
    c1 = dev.counters()
    clocks = sampler.stop(wall0, wall1)
    mid_pos = pos + K // 2
    pos += K
    last = [int(t) for t in hist[-1]]
    if distributed:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())

    # ---- timed region 2: end to end through decodeStep with host arrays every step
    tok = list(last)
    for _ in range(3):
        out = ex.decodeStep(jl.BatchSlots(active, tok, [pos] * B, slots))
        tok = [int(t) for t in out]
        pos += 1
    barrier()
    dev.synchronize()
    e0 = time.perf_counter()
    for _ in range(K):
        out = ex.decodeStep(jl.BatchSlots(active, tok, [pos] * B, slots))
        tok = [int(t) for t in out]
        pos += 1
    dev.synchronize()
    e_ms = (time.perf_counter() - e0) * 1000.0
    if distributed:
        t = torch.tensor([e_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e_ms = float(t.item())

    # ---- device-side temperature / top-p sampling of the same steps (single GPU): what jl_sample adds to a step,
    # and the step rate with it, against copying the rows of logits out for a host-side sampler
    sampling = None
    if rank == 0 and not use_tp:
        smp = jl.Sampler.selectSampler(cfg.vocabularySize, 0.8, 0.9, rngSeed=args.seed)
        n_s = max(4, min(K, 32))
        s_tok, s_pos, sample_ms = list(tok), pos, 0.0
        dev.synchronize()
        s0 = time.perf_counter()
        for _ in range(n_s):
            out = ex.decodeStep(jl.BatchSlots(active, s_tok, [s_pos] * B, slots), sampler=smp)
            sample_ms += dev.counters()["last_step_ms"]
            s_tok = [int(t) for t in out]
            s_pos += 1
        dev.synchronize()
        s_wall = (time.perf_counter() - s0) * 1000.0
        dev.synchronize()
        h0 = time.perf_counter()
        for _ in range(n_s):
            ex.decodeStep(jl.BatchSlots(active, s_tok, [s_pos] * B, slots), wantLogits=True)
            s_pos += 1
        dev.synchronize()
        h_wall = (time.perf_counter() - h0) * 1000.0
        sampling = {"temperature": 0.8, "topp": 0.9, "steps": n_s,
                    "sample_kernel_us": round(1000.0 * sample_ms / n_s, 1),
                    "tok_s_with_device_sampling": round(B * n_s / (s_wall / 1000.0), 1),
                    "tok_s_with_logits_copied_out": round(B * n_s / (h_wall / 1000.0), 1),
                    "d2h_bytes_per_step": 4 * B, "d2h_bytes_per_step_host_sampler": 4 * B * cfg.vocabularySize}

    # ---- per-kernel roofline: each matrix-vector launch shape alone, over all layers' weights
    peak, peak_kind = measured_peak()
    names = {0: "rmsnorm+qkv", 1: "attn-out+residual", 2: "rmsnorm+gate/up+swiglu", 3: "down+residual",
             4: "rmsnorm+vocab+argmax"}
    ops = []
    for op in (2, 0, 1, 3, 4):
        reps = cfg.numberOfLayers * (2 if op != 4 else 1) if op != 4 else 8
        model.benchOp(op, 0, cfg.numberOfLayers if op != 4 else 3)  # warm-up
        dev.synchronize()
        if op == 4:
            dev.flush_l2()  # one matrix only: start it cold
        dev.timer_start()
        model.benchOp(op, 0, reps)
        t_ms = dev.timer_stop()
        by = op_bytes(cfg, args.format, op, shards)
        us = t_ms * 1000.0 / reps
        ops.append({"kernel": names[op], "bytes_per_launch": by, "us_per_launch": round(us, 3),
                    "gbs": round(by / us / 1e3, 1), "frac": round(by / us / 1e3 / peak, 4), "launches": reps})
    dom = ops[0]
    if True:
        # attention of one layer at the depth the run has reached (row 0's position on the device)
        attn_pos = pos
        kv_row = 2 * model.localKvDim * 2  # K and V, binary16
        model.benchOp(5, 0, cfg.numberOfLayers)
        dev.synchronize()
        dev.timer_start()
        reps = 2 * cfg.numberOfLayers
        model.benchOp(5, 0, reps)
        us = dev.timer_stop() * 1000.0 / reps
        by = kv_row * (attn_pos + 1) + 4 * (cfg.dim // shards) * 2
        ops.append({"kernel": "rope+kv-append+attention", "bytes_per_launch": by, "us_per_launch": round(us, 3),
                    "gbs": round(by / us / 1e3, 1), "frac": round(by / us / 1e3 / peak, 4), "launches": reps,
                    "keys": attn_pos + 1, "note": "latency-bound at this depth: one launch per layer"})

    weights_b = model_bytes(cfg, args.format) / shards  # per GPU
    kv_b = B * (mid_pos + 1) * cfg.numberOfLayers * model.localKvDim * 2 * 2
    step_ms = ms / K
    tokens = B * K
    replicas = world if distributed and not use_tp else 1
    parallelism = "tp%d (Megatron split, one all-reduce per sublayer: %s)" % (world, model.exchangeMode) if use_tp else \
        ("replicas x%d" % replicas if replicas > 1 else "single GPU")
    value = tokens * replicas / (ms / 1000.0)
    line = {
        "metric": "decode tok/s", "value": value, "unit": "tok/s", "n_gpus": n_gpus, "steps": K, "warmup": max(W, 3),
        "ms_per_step": step_ms, "higher_is_better": True,
        "scaling": "weak" if replicas > 1 else "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": config, "parallelism": parallelism,
        "clocks": clocks,
        "e2e": {"value": tokens * replicas / (e_ms / 1000.0), "unit": "tok/s", "h2d_bytes_per_step": 13 * B,
                "d2h_bytes_per_step": 4 * B + 4, "ms_per_step": e_ms / K},
        "gpu_launches": int(c1["kernel_launches"] - c0["kernel_launches"]),
        "roofline": {"bound": "hbm", "kernel": "gemv_kernel<%s> %s" % (args.format, dom["kernel"]),
                     "achieved": dom["gbs"], "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                     "frac": dom["frac"], "traffic": NCU_TRAFFIC_BYTES.get((args.format, cfg.dim, cfg.hiddenDim)) if shards == 1 else None, "bytes_per_launch": dom["bytes_per_launch"],
                     "us_per_launch": dom["us_per_launch"]},
        "step_roofline": {"weight_bytes": weights_b, "kv_bytes": kv_b, "achieved_gbs": (weights_b + kv_b) / step_ms / 1e6,
                          "frac_of_measured_peak": (weights_b + kv_b) / step_ms / 1e6 / peak,
                          "frac_of_8tbs": (weights_b + kv_b) / step_ms / 1e6 / 8000.0},
        "kernels": ops,
        "sampling": sampling,
        "setup": {"synth_and_upload_s": round(t_build, 1), "prefill_tok_s": round(B * (P - 1) / t_prefill, 1)},
    }
    if rank == 0 and n_gpus == 1 and B == 1 and args.also_batch > 1 and args.arch in ("8b", "8b4", "tiny", "1b"):
        # the metric names B=1 and B=32; B=8 and B=64 are the other batch sizes of that configuration
        legs = []
        for bn in sorted({8, args.also_batch, 64}):
            args.also_batch_now = bn
            legs.append(batched_leg(jl, dev, kv, cfg, tensors, cr, ci, args))
        line["batched"] = next(l for l in legs if l["batch"] == args.also_batch)
        line["batched_all"] = legs
    if rank == 0 and n_gpus == 1 and not args.no_cpu_baseline:
        depth = P + max(W, 3)
        rate, cores, done, dt = cpu_decode_rate(cfg, tensors, args.cpu_seconds, 64, args.seed, depth=depth)
        line["cpu_baseline"] = {"value": rate, "unit": "tok/s", "cores": cores, "kind": "port",
                                "sample": cpu_sample_text(done, depth, dt)}
        # the host-side sampler chain the device sampler replaces (temperature, softmax, top-p), one row, one core
        from oracle import binding as oracle
        row = np.random.default_rng(args.seed).standard_normal(cfg.vocabularySize).astype(np.float32)
        oracle.sample(row, 0.8, 0.9, 0.5)
        t0 = time.perf_counter()
        for k in range(5):
            oracle.sample(row, 0.8, 0.9, 0.1 + 0.2 * k)
        line["cpu_baseline"]["sampler_ms_per_row"] = round((time.perf_counter() - t0) * 1000.0 / 5, 3)
    else:
        line["cpu_baseline"] = None
    if rank == 0 and use_tp and args.arch != "70b":
        # Tensor-parallel correctness inside the record: the same prompts on a single-GPU copy of the
        # whole model on this GPU -- logits of the first decode step side by side, then the same
        # greedy steps. Sums are taken in a different order on N GPUs, so tokens may part ways at a
        # near-tie; the count of identical leading tokens and the logit distance say how close it is.
        t_par = time.time()
        # the whole model the ranks hold between them: every rank's slices, put back together
        from jitllm_b200.tensor_parallel import assemble_tensor
        per_rank = [tensors if r == rank else
                    jl.synth_model_tensors(cfg, fmt, args.seed, threads=os.cpu_count() or 1, tp=jl.TensorParallel(r, world))
                    for r in range(world)]
        full = {key: (per_rank[0][key][0], assemble_tensor(cfg, key[0], [pr[key][1] for pr in per_rank]))
                for key in per_rank[0]}
        dev1 = jl.Device(local_rank)
        m1 = jl.load_model(dev1, cfg, full, cr, ci, maxBatch=B)
        kv1 = m1.createKvStorage(jl.KvStorageRequest(B * need, bps, B, 16, cfg.numberOfLayers, cfg.kvDim))
        kv1.publishBlockTable(table)
        ex1 = jl.B200BatchExecutor(m1)
        for b in range(B):
            jl.B200InvocationBoundary(m1, kvSlot=b, copyLogits=False).prefill(prompts[b, :P - 1], 0)
        first = [int(t) for t in prompts[:, P - 1]]
        _, logits_1 = ex1.decodeStep(jl.BatchSlots(active, first, [P - 1] * B, slots), wantLogits=True)
        ref_hist = ex1.generate(jl.BatchSlots(active, first, [P - 1] * B, slots), max(W, 3) + K)
        tp_hist = np.concatenate([np.asarray(warm_hist), np.asarray(hist)], axis=0)
        same = 0
        for a_row, b_row in zip(tp_hist, ref_hist):
            if not np.array_equal(a_row, b_row):
                break
            same += 1
        line["tp_parity"] = {"tokens_equal": "%d/%d" % (same, len(tp_hist)), "tokens_equal_frac": same / len(tp_hist),
                             "max_abs_logit_diff": float(np.max(np.abs(np.asarray(logits_tp) - np.asarray(logits_1)))),
                             "against": "the same prompts decoded by the whole model on one GPU, greedy, %d steps" % len(tp_hist),
                             "seconds": round(time.time() - t_par, 1)}
        kv1.close()
    if rank == 0:
        print(json.dumps(line), flush=True)
    barrier()
    if distributed:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

"""In-tree build of the native libraries.

`python -m jitllm_b200.build` compiles

* ``jitllm_b200/lib/libjitllm_b200.so`` -- the sm_100a CUDA library behind the C ABI of
  ``include/jitllm_b200.h`` (nvcc cross-compiles without a GPU);
* ``jitllm_b200/lib/libjl_synth.so``    -- the host-side synthetic weight generator / encoders.

Nothing is installed outside the tree; the built files are what a GPU machine loads.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "lib"

CUDA_SOURCES = ["gemv.cu", "ops.cu", "engine.cu", "static_entry.cu", "gemm_tc.cu", "tp_exchange.cu", "gguf_loader.cu",
                "sampler.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]
HOST_CC = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
HOST_CFLAGS = ["-O2", "-march=x86-64-v3", "-fopenmp", "-fPIC", "-shared", "-std=c11", "-Wall"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def _stale(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(s.stat().st_mtime > t for s in sources)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print("+", " ".join(cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout)
        sys.stderr.write(proc.stderr)
        raise RuntimeError(f"build step failed: {' '.join(cmd)}")
    if verbose and proc.stderr:
        sys.stderr.write(proc.stderr)


def build_cuda(force: bool = False, verbose: bool = False, ptxas_info: bool = False, trace: bool = False,
               trace_events: bool = False) -> Path:
    """Compiles every .cu file to its own object (in parallel) and links the shared library.

    trace=True builds ``libjitllm_b200_trace.so`` with -DJL_TRACE: the same kernels plus nanosecond
    stamps that ``jl_debug_trace`` reads back; the default library carries none of that code.
    trace_events=True (with trace) adds -DJL_TRACE_EVENTS: the tensor-core kernel's per-stage event log of one
    CTA, which costs registers and therefore is no part of the timeline build; always rebuilt."""
    LIB.mkdir(exist_ok=True)
    objdir = PKG / "build" / ("trace" if trace else "release")
    objdir.mkdir(parents=True, exist_ok=True)
    target = LIB / ("libjitllm_b200_trace.so" if trace else "libjitllm_b200.so")
    headers = sorted(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "jitllm_b200.h", Path(__file__)]
    flags = list(NVCC_FLAGS) + (["-DJL_TRACE"] if trace else []) + (["-DJL_TRACE_EVENTS"] if trace and trace_events else [])
    force = force or (trace and trace_events)
    if ptxas_info:
        flags += ["-Xptxas", "-v"]
    jobs = []
    for src in CUDA_SOURCES:
        obj = objdir / (src[:-3] + ".o")
        if force or ptxas_info or _stale(obj, [CSRC / src, *headers]):
            jobs.append([_nvcc(), *flags, "-c", "-o", str(obj), str(CSRC / src)])
    if jobs:
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
            list(pool.map(lambda c: _run(c, verbose or ptxas_info), jobs))
    objs = [objdir / (s[:-3] + ".o") for s in CUDA_SOURCES]
    if jobs or _stale(target, objs):
        _run([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", str(target), *[str(o) for o in objs]], verbose)
    return target


def build_microbench(verbose: bool = False) -> Path:
    """The stand-alone bulk-copy bandwidth benchmark (not part of the library)."""
    LIB.mkdir(exist_ok=True)
    target = LIB / "bulk_copy_bench"
    src = CSRC / "microbench" / "bulk_copy_bench.cu"
    if _stale(target, [src]):
        _run([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-o", str(target), str(src)], verbose)
    return target


def build_synth(force: bool = False, verbose: bool = False) -> Path:
    LIB.mkdir(exist_ok=True)
    target = LIB / "libjl_synth.so"
    src = CSRC / "synth.c"
    if force or _stale(target, [src]):
        _run([HOST_CC, *HOST_CFLAGS, "-o", str(target), str(src), "-lm"], verbose)
    return target


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cuda(force, verbose)
    build_synth(force, verbose)


if __name__ == "__main__":
    if "--ptxas" in sys.argv:
        build_cuda(force=True, ptxas_info=True)
    elif "--microbench" in sys.argv:
        build_microbench(verbose=True)
    elif "--trace" in sys.argv:
        build_cuda(force="--force" in sys.argv, verbose=True, trace=True, trace_events="--trace-events" in sys.argv)
    else:
        build_all(force="--force" in sys.argv, verbose=True)

"""Host-side mirror of the jitLLM interfaces the CUDA library sits behind.

The reference's host is Java; no JDK exists in this build environment, so the classes below
restate -- with the reference's own names, argument meaning and error behaviour -- the Java
seams a Panama shim would implement on top of the same C ABI (include/jitllm_b200.h). Paths cite
src/main/java/org/beehive/jitllm/ of the reference.

    Configuration            model/Configuration.java, model/llama/LlamaConfiguration.java:5-16
    GGMLType                 format/GGMLType.java:7,13,18-20
    TensorRole               runtime/tensor/TensorRole.java:17-59
    KvStorageRequest/KvStorage   runtime/kv/KvStorageRequest.java:5-12, runtime/kv/KvStorage.java,
                             backend/tornado/kv/TornadoKvStore.java
    BatchSlots/BatchExecutor runtime/batch/BatchSlots.java:15, runtime/batch/BatchExecutor.java:20-41
    InvocationBoundary       backend/tornado/lowering/InvocationBoundary.java:33-49
    Logits.argmax            inference/Logits.java:49-60

Java exceptions map to Python ones: IllegalArgumentException -> ValueError,
IllegalStateException -> IllegalStateError, InsufficientDeviceMemoryException (GPUL-MEM-001)
-> InsufficientDeviceMemoryError.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass
from typing import Dict, Optional, Sequence, Tuple

import numpy as np

from . import _lib
from .tensor_parallel import TensorParallel, check_divisible, init_group, local_shape, shard_tensor


class IllegalStateError(RuntimeError):
    """java.lang.IllegalStateException."""


class InsufficientDeviceMemoryError(MemoryError):
    """InsufficientDeviceMemoryException, GPUL-MEM-001."""


class DeviceTimeoutError(RuntimeError):
    """A bounded device-side wait gave up; the context stays usable."""


class GGMLType(enum.IntEnum):
    F32 = 0
    F16 = 1
    Q4_0 = 2
    Q4_1 = 3   # Q4_1, Q5_K, Q6_K: dequantize() and matmul() only, not model tensors
    Q8_0 = 8
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14

    @property
    def block_size(self) -> int:
        return {0: 1, 1: 1, 2: 32, 3: 32, 8: 32, 12: 256, 13: 256, 14: 256}[int(self)]

    @property
    def type_size(self) -> int:
        return {0: 4, 1: 2, 2: 18, 3: 20, 8: 34, 12: 144, 13: 176, 14: 210}[int(self)]

    def byte_size_for(self, n_elements: int) -> int:
        assert n_elements % self.block_size == 0
        return n_elements // self.block_size * self.type_size


class TensorRole(enum.IntEnum):
    TOKEN_EMBEDDING = 0
    ATTENTION_NORM = 1
    ATTENTION_QUERY = 2
    ATTENTION_KEY = 3
    ATTENTION_VALUE = 4
    ATTENTION_OUTPUT = 5
    FFN_NORM = 6
    FFN_GATE = 7
    FFN_UP = 8
    FFN_DOWN = 9
    OUTPUT_NORM = 10
    OUTPUT = 11


GLOBAL_ROLES = (TensorRole.TOKEN_EMBEDDING, TensorRole.OUTPUT_NORM, TensorRole.OUTPUT)

UNMAPPED = -1  # runtime/kv/BlockPool.java:61


@dataclass(frozen=True)
class Configuration:
    dim: int
    hiddenDim: int
    numberOfLayers: int
    numberOfHeads: int
    numberOfKeyValueHeads: int
    vocabularySize: int
    contextLength: int
    rmsNormEps: float = 1e-5
    ropeTheta: float = 500000.0
    tiedEmbeddings: bool = False

    @property
    def headSize(self) -> int:
        return self.dim // self.numberOfHeads

    @property
    def kvDim(self) -> int:
        return self.dim * self.numberOfKeyValueHeads // self.numberOfHeads

    def matrix_shape(self, role: TensorRole) -> Tuple[int, int]:
        c = self
        return {
            TensorRole.TOKEN_EMBEDDING: (c.vocabularySize, c.dim),
            TensorRole.OUTPUT: (c.vocabularySize, c.dim),
            TensorRole.ATTENTION_QUERY: (c.dim, c.dim),
            TensorRole.ATTENTION_KEY: (c.kvDim, c.dim),
            TensorRole.ATTENTION_VALUE: (c.kvDim, c.dim),
            TensorRole.ATTENTION_OUTPUT: (c.dim, c.dim),
            TensorRole.FFN_GATE: (c.hiddenDim, c.dim),
            TensorRole.FFN_UP: (c.hiddenDim, c.dim),
            TensorRole.FFN_DOWN: (c.dim, c.hiddenDim),
            TensorRole.ATTENTION_NORM: (1, c.dim),
            TensorRole.FFN_NORM: (1, c.dim),
            TensorRole.OUTPUT_NORM: (1, c.dim),
        }[role]


def _ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class Device:
    """One GPU context (jl_ctx). Everything else in this module hangs off one of these."""

    def __init__(self, device_id: int = 0):
        self._lib = _lib.load()
        h = C.c_void_p()
        rc = self._lib.jl_init(device_id, C.byref(h))
        if rc != 0:
            msg = self._lib.jl_last_error(None).decode()
            raise _exception(rc, msg)
        self._h = h
        self.device_id = device_id

    # -- error plumbing
    def _check(self, rc: int) -> None:
        if rc != 0:
            raise _exception(rc, self._lib.jl_last_error(self._h).decode())

    @property
    def handle(self):
        if self._h is None:
            raise IllegalStateError("GPUL-LIFE-001: this device context is closed")
        return self._h

    def close(self) -> None:
        if self._h is not None:
            self._lib.jl_destroy(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- standalone operators
    def dequantize(self, ggml_type: GGMLType, blocks: np.ndarray, n_elements: int) -> np.ndarray:
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
        if n_elements >= 0 and GGMLType(ggml_type).block_size > 1 and n_elements % GGMLType(ggml_type).block_size == 0:
            need = GGMLType(ggml_type).byte_size_for(n_elements)
            if blocks.size != need:
                raise ValueError(f"GPUL-CFG-002: {n_elements} elements need {need} bytes, got {blocks.size}")
        out = np.empty(max(n_elements, 0), dtype=np.float32)
        self._check(self._lib.jl_dequant(self.handle, int(ggml_type), _ptr(blocks), n_elements, _ptr(out)))
        return out

    def matmul(self, ggml_type: GGMLType, weight: np.ndarray, rows: int, cols: int, x: np.ndarray) -> np.ndarray:
        """FloatTensor.matmul with host buffers: x is [cols] or [n, cols]; returns [rows] / [n, rows]."""
        weight = np.ascontiguousarray(weight, dtype=np.uint8)
        x2 = np.ascontiguousarray(x, dtype=np.float32)
        single = x2.ndim == 1
        x2 = x2.reshape(-1, cols)
        need = rows * (cols // GGMLType(ggml_type).block_size) * GGMLType(ggml_type).type_size
        if weight.size != need:
            raise ValueError(f"GPUL-CFG-002: {rows}x{cols} {GGMLType(ggml_type).name} needs {need} bytes, got {weight.size}")
        y = np.empty((x2.shape[0], rows), dtype=np.float32)
        self._check(self._lib.jl_gemv(self.handle, int(ggml_type), rows, cols, _ptr(weight), _ptr(x2), x2.shape[0], _ptr(y)))
        return y[0] if single else y

    # -- device-resident operators (benchmarks)
    def upload_matrix(self, ggml_type: GGMLType, weight: np.ndarray, rows: int, cols: int) -> "DeviceMatrix":
        weight = np.ascontiguousarray(weight, dtype=np.uint8)
        t = C.c_void_p()
        self._check(self._lib.jl_tensor_upload(self.handle, int(ggml_type), rows, cols, _ptr(weight), weight.size, C.byref(t)))
        return DeviceMatrix(self, t, GGMLType(ggml_type), rows, cols)

    def alloc(self, nbytes: int) -> int:
        p = self._lib.jl_device_alloc(self.handle, nbytes)
        if not p:
            raise _exception(2, self._lib.jl_last_error(self._h).decode())
        return p

    def free(self, p: int) -> None:
        self._check(self._lib.jl_device_free(self.handle, C.c_void_p(p)))

    def h2d(self, dst: int, src: np.ndarray) -> None:
        src = np.ascontiguousarray(src)
        self._check(self._lib.jl_memcpy_h2d(self.handle, C.c_void_p(dst), _ptr(src), src.nbytes))

    def d2h(self, dst: np.ndarray, src: int) -> None:
        self._check(self._lib.jl_memcpy_d2h(self.handle, _ptr(dst), C.c_void_p(src), dst.nbytes))

    def synchronize(self) -> None:
        self._check(self._lib.jl_synchronize(self.handle))

    def timer_start(self) -> None:
        self._check(self._lib.jl_timer_start(self.handle))

    def timer_stop(self) -> float:
        ms = C.c_float()
        self._check(self._lib.jl_timer_stop(self.handle, C.byref(ms)))
        return ms.value

    def peer_wait_self_test(self, timeout_ms: int = 50) -> None:
        """Runs a peer exchange whose partner never answers; raises DeviceTimeoutError when the bounded
        wait gives up (the expected outcome) and leaves the context usable."""
        self._check(self._lib.jl_debug_peer_wait_timeout(self.handle, int(timeout_ms)))

    def flush_l2(self) -> None:
        self._check(self._lib.jl_flush_l2(self.handle))

    def counters(self) -> dict:
        c = _lib.JlCounters()
        self._check(self._lib.jl_get_counters(self.handle, C.byref(c)))
        return {name: getattr(c, name) for name, _ in c._fields_}


class DeviceMatrix:
    def __init__(self, dev: Device, handle, ggml_type: GGMLType, rows: int, cols: int):
        self.dev, self._h, self.type, self.rows, self.cols = dev, handle, ggml_type, rows, cols

    def matmul_dev(self, x_dev: int, n: int, y_dev: int) -> None:
        self.dev._check(self.dev._lib.jl_gemv_dev(self.dev.handle, self._h, C.c_void_p(x_dev), n, C.c_void_p(y_dev)))

    def close(self) -> None:
        if self._h is not None and self.dev._h is not None:
            self.dev._lib.jl_tensor_free(self.dev.handle, self._h)
        self._h = None


def _exception(rc: int, msg: str) -> Exception:
    if rc == 2:
        return InsufficientDeviceMemoryError(msg)
    if rc == 4:
        return IllegalStateError(msg)
    if rc == 5:
        return DeviceTimeoutError(msg)
    if rc in (1, 6):
        return ValueError(msg)
    return RuntimeError(msg)


# --------------------------------------------------------------------------------------------- KV

@dataclass(frozen=True)
class KvStorageRequest:
    totalBlocks: int
    blocksPerSlot: int
    maxSlots: int
    blockSizeTokens: int
    numberOfLayers: int
    kvDim: int
    fp16KeyValue: bool = True

    def __post_init__(self):
        if min(self.totalBlocks, self.blocksPerSlot, self.maxSlots, self.blockSizeTokens,
               self.numberOfLayers, self.kvDim) <= 0:
            raise ValueError(
                "every key/value pool dimension must be positive, got "
                f"totalBlocks={self.totalBlocks} blocksPerSlot={self.blocksPerSlot} "
                f"maxSlots={self.maxSlots} blockSizeTokens={self.blockSizeTokens} "
                f"numberOfLayers={self.numberOfLayers} kvDim={self.kvDim}")


class KvStorage:
    """Device page pool behind the storage SPI; created by B200Model.createKvStorage."""

    def __init__(self, model: "B200Model", request: KvStorageRequest):
        self._model = model
        self._req = request
        self._closed = False
        dev = model.dev
        dev._check(dev._lib.jl_kv_create(dev.handle, request.totalBlocks, request.blocksPerSlot,
                                         request.maxSlots, request.blockSizeTokens,
                                         1 if request.fp16KeyValue else 0))

    def publishBlockTable(self, blockTable: Sequence[int]) -> None:
        if self._closed:
            raise IllegalStateError("this KV store is closed")
        t = np.ascontiguousarray(blockTable, dtype=np.int32)
        dev = self._model.dev
        dev._check(dev._lib.jl_kv_publish_block_table(dev.handle, _ptr(t), t.size))

    def blockSizeTokens(self) -> int:
        return self._req.blockSizeTokens

    def blocksPerSlot(self) -> int:
        return self._req.blocksPerSlot

    def bytesPerBlock(self) -> int:
        r = self._req
        return 2 * r.kvDim * r.blockSizeTokens * r.numberOfLayers * (2 if r.fp16KeyValue else 4)

    def fill(self, half_bits: int = 0x7E00) -> None:
        """Every K and V element becomes this binary16 pattern (default: NaN, the reference's poison)."""
        dev = self._model.dev
        dev._check(dev._lib.jl_kv_fill(dev.handle, half_bits))

    def readRow(self, which: str, slot: int, layer: int, pos: int) -> np.ndarray:
        """One position's K or V row as raw binary16 bits (test access)."""
        out = np.empty(self._req.kvDim, dtype=np.uint16)
        dev = self._model.dev
        dev._check(dev._lib.jl_kv_read_row(dev.handle, 0 if which == "k" else 1, slot, layer, pos, _ptr(out)))
        return out

    def close(self) -> None:
        self._closed = True


# ------------------------------------------------------------------------------------------ model

class B200Model:
    """Device-resident weights + per-step workspace of one Llama-architecture model."""

    def __init__(self, dev: Device, config: Configuration, maxBatch: int = 1,
                 tp: Optional[TensorParallel] = None):
        self.dev = dev
        self.config = config
        self.maxBatch = maxBatch
        self.tp = tp or TensorParallel()
        check_divisible(config, self.tp.size)
        d = _lib.JlModelDesc(
            dim=config.dim, hidden=config.hiddenDim, layers=config.numberOfLayers,
            heads=config.numberOfHeads, kv_heads=config.numberOfKeyValueHeads,
            head_dim=config.headSize, vocab=config.vocabularySize, ctx_len=config.contextLength,
            rms_eps=config.rmsNormEps, tied_embeddings=1 if config.tiedEmbeddings else 0,
            max_batch=maxBatch, tp_rank=self.tp.rank, tp_size=self.tp.size)
        dev._check(dev._lib.jl_model_create(dev.handle, C.byref(d)))

    @classmethod
    def adopt(cls, dev: Device, config: Configuration, maxBatch: int = 1,
              tp: Optional[TensorParallel] = None) -> "B200Model":
        """Wraps a model the library has already created on `dev` (the native GGUF reader does that)."""
        self = cls.__new__(cls)
        self.dev, self.config, self.maxBatch, self.tp = dev, config, maxBatch, tp or TensorParallel()
        return self

    def uploadTensor(self, role: TensorRole, layer: int, ggml_type: GGMLType, data: np.ndarray,
                     presharded: bool = False) -> None:
        """`data` is the whole GGUF tensor; under tensor parallelism this GPU's slice is cut here
        (or, with `presharded`, `data` already is that slice)."""
        role = TensorRole(role)
        rows, cols = local_shape(self.config, role, self.tp.size)
        data = np.ascontiguousarray(data)
        if not presharded:
            data = np.ascontiguousarray(shard_tensor(self.config, role, ggml_type, data, self.tp))
        self.dev._check(self.dev._lib.jl_upload_tensor(
            self.dev.handle, int(role), layer, int(ggml_type), rows, cols, _ptr(data), data.nbytes))

    def uploadRope(self, cos: np.ndarray, sin: np.ndarray) -> None:
        cos = np.ascontiguousarray(cos, dtype=np.float32)
        sin = np.ascontiguousarray(sin, dtype=np.float32)
        self.dev._check(self.dev._lib.jl_upload_rope(self.dev.handle, _ptr(cos), _ptr(sin), cos.size))

    def initTensorParallel(self, broadcast) -> None:
        """Joins the NCCL group (collective; every rank calls it between construction and finalize)."""
        init_group(self.dev, self.tp, broadcast)

    def finalize(self) -> None:
        self.dev._check(self.dev._lib.jl_model_finalize(self.dev.handle))

    @property
    def exchangeMode(self) -> str:
        """How the tensor-parallel ranks trade partial sums: 'single', 'nccl', 'peer-memory' (one small
        kernel per exchange) or 'peer-memory, fused' (the all-reduce of the row-parallel projections
        happens inside the mat-vec kernel's epilogue; the arg-max exchange stays its own kernel)."""
        mode = self.dev._lib.jl_tp_exchange_mode(self.dev.handle)
        note = (self.dev._lib.jl_tp_exchange_note(self.dev.handle) or b"").decode()
        return ["single", "nccl", "peer-memory", "peer-memory, fused"][mode] + (f" ({note})" if note else "")

    @property
    def localKvDim(self) -> int:
        return self.config.kvDim // self.tp.size

    def createKvStorage(self, request: KvStorageRequest) -> KvStorage:
        c = self.config
        if request.numberOfLayers != c.numberOfLayers or request.kvDim != self.localKvDim:
            raise ValueError("GPUL-CFG-002: KV request does not match the model's layers / kvDim")
        return KvStorage(self, request)

    def benchOp(self, op: int, firstLayer: int, iters: int) -> None:
        self.dev._check(self.dev._lib.jl_bench_op(self.dev.handle, op, firstLayer, iters))

    def debugRead(self, name: str, row: int = 0) -> np.ndarray:
        c = self.config
        t = self.tp.size
        n = {"x": c.dim, "q": c.dim // t, "xb": c.dim, "k": c.kvDim // t, "v": c.kvDim // t,
             "hb": c.hiddenDim // t, "logits": c.vocabularySize // t}[name]
        out = np.empty(n, dtype=np.float32)
        self.dev._check(self.dev._lib.jl_debug_read(self.dev.handle, name.encode(), row, _ptr(out), n))
        return out


@dataclass(frozen=True)
class BatchSlots:
    active: Sequence[bool]
    tokens: Sequence[int]
    positions: Sequence[int]
    kvSlots: Sequence[int]

    def __post_init__(self):
        n = len(self.active)
        if not (len(self.tokens) == n and len(self.positions) == n and len(self.kvSlots) == n):
            raise ValueError(
                f"a batch is fixed width: got {n} active, {len(self.tokens)} tokens, "
                f"{len(self.positions)} positions, {len(self.kvSlots)} kv slots")

    def width(self) -> int:
        return len(self.active)

    def activeCount(self) -> int:
        return sum(1 for a in self.active if a)


class Sampler:
    """What Sampler.selectSampler(vocabularySize, temperature, topp, rngSeed) returns
    (inference/sampler/Sampler.java:63-110), with the arithmetic moved to the device: temperature 0 is
    greedy (the arg-max every step already returns); otherwise temperature scaling, softmax and
    categorical or top-p sampling run in jl_sample on the rows of logits the step left on the GPU. The
    random generator stays on the host, as the reference's does: `rng` is anything with a `random()`
    method returning a float in [0, 1) (numpy Generator, random.Random); a Java host passes
    rng.nextFloat(1f). Values are rounded down to a multiple of 2^-24, the granularity of nextFloat."""

    def __init__(self, vocabularySize: int, temperature: float, topp: float, rng=None, rngSeed: int = 0):
        self.vocabularySize = int(vocabularySize)
        self.temperature = float(temperature)
        self.topp = float(topp)
        self.greedy = self.temperature == 0.0
        self._rng = rng if rng is not None else np.random.default_rng(rngSeed)

    @staticmethod
    def selectSampler(vocabularySize: int, temperature: float, topp: float, rngSeed: int) -> "Sampler":
        return Sampler(vocabularySize, temperature, topp, rngSeed=rngSeed)

    def nextFloat(self) -> np.float32:
        return np.float32(int(float(self._rng.random()) * (1 << 24)) / float(1 << 24))


class B200BatchExecutor:
    """BatchExecutor over the CUDA library: one jl_decode per engine step."""

    def __init__(self, model: B200Model, stopTokens: Sequence[int] = ()):
        self._model = model
        self._stop = frozenset(int(t) for t in stopTokens)

    def maxBatchSize(self) -> int:
        return self._model.maxBatch

    def decodeStep(self, batch: BatchSlots, wantLogits: bool = False, sampler: "Optional[Sampler]" = None):
        """One step for every active row. Without a sampler (or with a greedy one) the tokens are the
        device-side arg-max; with a temperature sampler the rows of logits stay on the device and
        jl_sample draws from them (inference/sampler/Sampler.java:63-110), one random number per row
        from the sampler's generator, drawn for every row in row order whether active or not."""
        w = batch.width()
        tokens = np.ascontiguousarray(batch.tokens, dtype=np.int32)
        positions = np.ascontiguousarray(batch.positions, dtype=np.int32)
        slots = np.ascontiguousarray(batch.kvSlots, dtype=np.int32)
        active = np.ascontiguousarray(batch.active, dtype=np.uint8)
        out = np.empty(w, dtype=np.int32)
        logits = np.empty((w, self._model.config.vocabularySize), dtype=np.float32) if wantLogits else None
        dev = self._model.dev
        dev._check(dev._lib.jl_decode(dev.handle, w, _ptr(tokens), _ptr(positions), _ptr(slots),
                                      _ptr(active), _ptr(out), _ptr(logits)))
        if sampler is not None and not sampler.greedy:
            u = np.ascontiguousarray([sampler.nextFloat() for _ in range(w)], dtype=np.float32)
            dev._check(dev._lib.jl_sample(dev.handle, w, C.c_float(sampler.temperature), C.c_float(sampler.topp),
                                          _ptr(u), _ptr(out)))
        return (out, logits) if wantLogits else out

    def generate(self, batch: BatchSlots, steps: int) -> np.ndarray:
        """`steps` greedy steps with on-device token feedback; returns [steps, width] token ids."""
        w = batch.width()
        tokens = np.ascontiguousarray(batch.tokens, dtype=np.int32)
        positions = np.ascontiguousarray(batch.positions, dtype=np.int32)
        slots = np.ascontiguousarray(batch.kvSlots, dtype=np.int32)
        active = np.ascontiguousarray(batch.active, dtype=np.uint8)
        out = np.empty((steps, w), dtype=np.int32)
        dev = self._model.dev
        dev._check(dev._lib.jl_generate(dev.handle, w, _ptr(tokens), _ptr(positions), _ptr(slots),
                                        _ptr(active), steps, _ptr(out)))
        return out

    def isStopToken(self, token: int) -> bool:
        return int(token) in self._stop


@dataclass
class InvocationResult:
    logits: Optional[np.ndarray]
    sampledToken: int


class B200InvocationBoundary:
    """InvocationBoundary.invoke(token, position) for a single sequence bound to one KV slot."""

    def __init__(self, model: B200Model, kvSlot: int = 0, copyLogits: bool = True):
        self._exec = B200BatchExecutor(model)
        self._slot = kvSlot
        self._copy = copyLogits

    def invoke(self, token: int, position: int) -> InvocationResult:
        batch = BatchSlots([True], [token], [position], [self._slot])
        if self._copy:
            out, logits = self._exec.decodeStep(batch, wantLogits=True)
            return InvocationResult(logits[0], int(out[0]))
        out = self._exec.decodeStep(batch)
        return InvocationResult(None, int(out[0]))

    def prefill(self, tokens: Sequence[int], startPosition: int = 0) -> None:
        """BatchPrefillDecodePlan.tornadoVMForwardBatchPrefill: KV written, no logits."""
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        dev = self._exec._model.dev
        dev._check(dev._lib.jl_prefill(dev.handle, self._slot, _ptr(t), startPosition, t.size))


def argmax(logits: np.ndarray) -> int:
    """Logits.argmax: first index of the maximum (strict >)."""
    return int(np.argmax(logits))


# --------------------------------------------------------------------------- synthetic weights

def synth_tensor(ggml_type: GGMLType, n_elements: int, seed: int, std: float = 0.02, threads: int = 0) -> np.ndarray:
    """Seeded N(0, std) values encoded as `ggml_type` blocks (or raw F32)."""
    lib = _lib.load_synth()
    nbytes = lib.jls_tensor_bytes(int(ggml_type), n_elements)
    if nbytes < 0:
        raise ValueError(f"GPUL-CFG-002: cannot encode {n_elements} elements as {GGMLType(ggml_type).name}")
    out = np.empty(nbytes, dtype=np.uint8)
    rc = lib.jls_synth_tensor(int(ggml_type), n_elements, seed & (2**64 - 1), std, _ptr(out), threads)
    if rc != 0:
        raise ValueError("GPUL-CFG-002: synthetic tensor generation failed")
    return out.view(np.float32) if ggml_type == GGMLType.F32 else out


def random_blocks(ggml_type: GGMLType, n_elements: int, seed: int, scale: float = 0.01) -> np.ndarray:
    """Blocks of any block format with random payload bytes and block scales of magnitude `scale` (a random fp16 bit
    pattern is often infinite): test and benchmark input for the formats that have no encoder here (Q4_1, Q5_K,
    Q6_K)."""
    t = GGMLType(ggml_type)
    if t.block_size == 1 or n_elements % t.block_size:
        raise ValueError(f"GPUL-CFG-002: {n_elements} elements are no whole number of {t.name} blocks")
    n = n_elements // t.block_size
    rng = np.random.default_rng(seed)
    raw = rng.integers(0, 256, size=(n, t.type_size), dtype=np.uint8)
    for off in {GGMLType.Q4_0: (0,), GGMLType.Q8_0: (0,), GGMLType.Q4_1: (0, 2), GGMLType.Q4_K: (0, 2),
                GGMLType.Q5_K: (0, 2), GGMLType.Q6_K: (208,)}[t]:
        vals = (rng.uniform(0.2, 1.0, n) * scale * rng.choice([-1.0, 1.0], n)).astype(np.float16)
        raw[:, off:off + 2] = vals.view(np.uint8).reshape(n, 2)
    return raw.reshape(-1)


def quantize(ggml_type: GGMLType, values: np.ndarray, threads: int = 0) -> np.ndarray:
    lib = _lib.load_synth()
    values = np.ascontiguousarray(values, dtype=np.float32).ravel()
    nbytes = lib.jls_tensor_bytes(int(ggml_type), values.size)
    if nbytes < 0:
        raise ValueError(f"GPUL-CFG-002: cannot encode {values.size} elements as {GGMLType(ggml_type).name}")
    out = np.empty(nbytes, dtype=np.uint8)
    if lib.jls_quantize(int(ggml_type), _ptr(values), values.size, _ptr(out), threads) != 0:
        raise ValueError("GPUL-CFG-002: quantisation failed")
    return out


def synth_model_tensors(config: Configuration, ggml_type: GGMLType, seed: int, std: float = 0.02,
                        threads: int = 0, tp: Optional[TensorParallel] = None
                        ) -> Dict[Tuple[TensorRole, int], Tuple[GGMLType, np.ndarray]]:
    """All tensors of a synthetic model: matrices N(0, std) in `ggml_type`, norm weights 1.0.
    With `tp`, only this GPU's slices are generated (pass them to load_model with presharded=True):
    each slice of a split matrix draws from its own seed, so the ranks together hold one consistent
    random model of the full shape, though not the one a single GPU would draw from `seed`."""
    out: Dict[Tuple[TensorRole, int], Tuple[GGMLType, np.ndarray]] = {}
    index = 0
    size = tp.size if tp else 1

    def matrix(role: TensorRole, layer: int):
        nonlocal index
        rows, cols = local_shape(config, role, size)
        split = (rows, cols) != config.matrix_shape(role)
        s = seed * 1000003 + index + (7919 * 1000003 * (tp.rank + 1) if split else 0)
        out[(role, layer)] = (ggml_type, synth_tensor(ggml_type, rows * cols, s, std, threads))
        index += 1

    matrix(TensorRole.TOKEN_EMBEDDING, -1)
    for l in range(config.numberOfLayers):
        out[(TensorRole.ATTENTION_NORM, l)] = (GGMLType.F32, np.ones(config.dim, dtype=np.float32))
        for role in (TensorRole.ATTENTION_QUERY, TensorRole.ATTENTION_KEY, TensorRole.ATTENTION_VALUE,
                     TensorRole.ATTENTION_OUTPUT):
            matrix(role, l)
        out[(TensorRole.FFN_NORM, l)] = (GGMLType.F32, np.ones(config.dim, dtype=np.float32))
        for role in (TensorRole.FFN_GATE, TensorRole.FFN_UP, TensorRole.FFN_DOWN):
            matrix(role, l)
    out[(TensorRole.OUTPUT_NORM, -1)] = (GGMLType.F32, np.ones(config.dim, dtype=np.float32))
    if not config.tiedEmbeddings:
        matrix(TensorRole.OUTPUT, -1)
    return out


def load_model(dev: Device, config: Configuration, tensors, rope_cos: np.ndarray, rope_sin: np.ndarray,
               maxBatch: int = 1, tp: Optional[TensorParallel] = None, broadcast=None,
               presharded: bool = False) -> B200Model:
    """`tensors` holds whole tensors; with `tp` each GPU keeps its slice and `broadcast` carries the
    NCCL id between the ranks (see tensor_parallel.init_group)."""
    model = B200Model(dev, config, maxBatch, tp)
    for (role, layer), (t, data) in tensors.items():
        model.uploadTensor(role, layer if role not in GLOBAL_ROLES else -1, t, data, presharded)
    model.uploadRope(rope_cos, rope_sin)
    if model.tp.size > 1:
        if broadcast is None:
            raise ValueError("GPUL-CFG-002: tensor parallelism needs a broadcast channel for the NCCL id")
        model.initTensorParallel(broadcast)
    model.finalize()
    return model


def precomputeFreqsCis(contextLength: int, headSize: int, theta: float) -> Tuple[np.ndarray, np.ndarray]:
    """RopeFrequencies.precomputeFreqsCis without scaling (model/loader/RopeFrequencies.java:14-54):
    freq = (float)(1 / theta^(i/headSize)), val = pos * freq in binary32, cos/sin in double then
    narrowed. Returns two [contextLength * headSize/2] float32 arrays."""
    i = np.arange(0, headSize, 2, dtype=np.float64)
    freq = (1.0 / np.power(np.float64(theta), i / np.float64(headSize))).astype(np.float32)
    pos = np.arange(contextLength, dtype=np.float32)
    val = (pos[:, None] * freq[None, :]).astype(np.float32)
    cr = np.cos(val.astype(np.float64)).astype(np.float32).ravel()
    ci = np.sin(val.astype(np.float64)).astype(np.float32).ravel()
    return cr, ci

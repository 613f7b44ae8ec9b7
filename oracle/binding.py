"""ctypes binding of the CPU oracle (oracle/jl_oracle.h) -- TEST INFRASTRUCTURE.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this module; the product
package never does.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "libjl_oracle.so"


class OrcConfig(C.Structure):
    _fields_ = [("dim", C.c_int), ("hidden", C.c_int), ("layers", C.c_int), ("heads", C.c_int),
                ("kv_heads", C.c_int), ("head_dim", C.c_int), ("vocab", C.c_int),
                ("ctx_len", C.c_int), ("eps", C.c_float), ("theta", C.c_float)]


def build(force: bool = False) -> Path:
    src = [HERE / "jl_oracle.c", HERE / "jl_oracle.h"]
    if force or not LIB.exists() or any(s.stat().st_mtime > LIB.stat().st_mtime for s in src):
        subprocess.run(["make", "-C", str(HERE), "-B"], check=True, capture_output=True)
    return LIB


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(LIB))
        P, I, I64, F = C.c_void_p, C.c_int, C.c_int64, C.c_float
        L.orc_f16_to_f32.restype = F
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f32_to_f16.argtypes = [F]
        L.orc_get_float.restype = F
        L.orc_get_float.argtypes = [I, P, I64]
        L.orc_dequant.argtypes = [I, P, I64, P]
        L.orc_dot.restype = F
        L.orc_dot.argtypes = [I, P, I64, P, I64]
        L.orc_matmul.argtypes = [I, P, P, P, I, I]
        L.orc_matmul_batch.argtypes = [I, P, P, P, I, I, I]
        L.orc_sample.restype = I
        L.orc_sample.argtypes = [P, I, F, F, F, P]
        L.orc_rmsnorm.argtypes = [P, P, P, I, F]
        L.orc_rope.argtypes = [P, P, P, P, I, I, I, I]
        L.orc_swiglu.argtypes = [P, P, I]
        L.orc_argmax.restype = I
        L.orc_argmax.argtypes = [P, I]
        L.orc_rope_tables.argtypes = [I, I, C.c_double, P, P]
        L.orc_attention.argtypes = [P, P, P, P, P, I, I, I, I, I, I]
        L.orc_kv_offset.restype = I64
        L.orc_kv_offset.argtypes = [P, I, I, I, I, I, I, I]
        L.orc_model_create.restype = P
        L.orc_model_create.argtypes = [C.POINTER(OrcConfig)]
        L.orc_model_free.argtypes = [P]
        L.orc_model_set_tensor.restype = I
        L.orc_model_set_tensor.argtypes = [P, I, I, I, P]
        L.orc_model_set_rope.argtypes = [P, P, P]
        L.orc_model_rope_cos.restype = C.POINTER(F)
        L.orc_model_rope_cos.argtypes = [P]
        L.orc_model_rope_sin.restype = C.POINTER(F)
        L.orc_model_rope_sin.argtypes = [P]
        L.orc_state_create.restype = P
        L.orc_state_create.argtypes = [P]
        L.orc_state_free.argtypes = [P]
        L.orc_forward.restype = C.POINTER(F)
        L.orc_forward.argtypes = [P, P, I, I]
        L.orc_forward_no_logits.argtypes = [P, P, I, I]
        L.orc_state_buffer.restype = C.POINTER(F)
        L.orc_state_buffer.argtypes = [P, C.c_char_p]
        L.orc_state_kcache.restype = C.POINTER(C.c_uint16)
        L.orc_state_kcache.argtypes = [P, I]
        L.orc_state_vcache.restype = C.POINTER(C.c_uint16)
        L.orc_state_vcache.argtypes = [P, I]
        L.orc_set_vector_bits.argtypes = [I]
        L.orc_get_vector_bits.restype = I
        L.orc_set_threads.argtypes = [I]
        L.orc_get_threads.restype = I
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def dequant(t: int, blocks: np.ndarray, n: int) -> np.ndarray:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    out = np.empty(n, dtype=np.float32)
    lib().orc_dequant(int(t), _p(blocks), n, _p(out))
    return out


def get_float(t: int, blocks: np.ndarray, index: int) -> float:
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    return float(lib().orc_get_float(int(t), _p(blocks), index))


def rmsnorm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """CpuOperations.rmsNorm (inference/op/CpuOperations.java:55-73) of one vector."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    weight = np.ascontiguousarray(weight, dtype=np.float32)
    out = np.empty_like(x)
    lib().orc_rmsnorm(_p(out), _p(x), _p(weight), int(x.size), C.c_float(eps))
    return out


def matmul(t: int, w: np.ndarray, x: np.ndarray, rows: int, cols: int) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.float32)
    if x.ndim == 1:
        out = np.empty(rows, dtype=np.float32)
        lib().orc_matmul(int(t), _p(w), _p(x), _p(out), rows, cols)
        return out
    out = np.empty((x.shape[0], rows), dtype=np.float32)
    lib().orc_matmul_batch(int(t), _p(w), _p(x), _p(out), rows, cols, x.shape[0])
    return out


def sample(logits: np.ndarray, temperature: float, topp: float, u: float):
    """The reference's sampler chain on one row (a copy is modified); returns (token, margin): margin is the
    distance of the scaled random number from the nearest boundary of the cumulative distribution."""
    row = np.ascontiguousarray(logits, dtype=np.float32).copy()
    margin = C.c_float()
    tok = lib().orc_sample(_p(row), int(row.size), C.c_float(temperature), C.c_float(topp), C.c_float(u), C.byref(margin))
    return int(tok), float(margin.value)


class Model:
    """The oracle's forwardJava over borrowed tensor bytes."""

    def __init__(self, config, tensors):
        """config: jitllm_b200.Configuration-like; tensors: {(role, layer): (type, ndarray)}."""
        L = lib()
        c = OrcConfig(config.dim, config.hiddenDim, config.numberOfLayers, config.numberOfHeads,
                      config.numberOfKeyValueHeads, config.headSize, config.vocabularySize,
                      config.contextLength, config.rmsNormEps, config.ropeTheta)
        self.config = config
        self._keep = []
        self._m = L.orc_model_create(C.byref(c))
        for (role, layer), (t, data) in tensors.items():
            data = np.ascontiguousarray(data)
            self._keep.append(data)
            rc = L.orc_model_set_tensor(self._m, int(role), int(layer), int(t), _p(data))
            assert rc == 0, (role, layer)
        self._s = L.orc_state_create(self._m)

    def set_rope_tables(self, cr: np.ndarray, ci: np.ndarray) -> None:
        cr = np.ascontiguousarray(cr, dtype=np.float32)
        ci = np.ascontiguousarray(ci, dtype=np.float32)
        lib().orc_model_set_rope(self._m, _p(cr), _p(ci))

    def rope_tables(self):
        n = self.config.contextLength * (self.config.headSize // 2)
        L = lib()
        cr = np.ctypeslib.as_array(L.orc_model_rope_cos(self._m), shape=(n,)).copy()
        ci = np.ctypeslib.as_array(L.orc_model_rope_sin(self._m), shape=(n,)).copy()
        return cr, ci

    def forward(self, token: int, position: int) -> np.ndarray:
        p = lib().orc_forward(self._m, self._s, token, position)
        return np.ctypeslib.as_array(p, shape=(self.config.vocabularySize,)).copy()

    def forward_no_logits(self, token: int, position: int) -> None:
        lib().orc_forward_no_logits(self._m, self._s, token, position)

    def buffer(self, name: str, n: int) -> np.ndarray:
        p = lib().orc_state_buffer(self._s, name.encode())
        return np.ctypeslib.as_array(p, shape=(n,)).copy()

    def kcache(self, layer: int, pos: int) -> np.ndarray:
        kv = self.config.kvDim
        p = lib().orc_state_kcache(self._s, layer)
        return np.ctypeslib.as_array(p, shape=((pos + 1) * kv,))[pos * kv:(pos + 1) * kv].copy()

    def vcache(self, layer: int, pos: int) -> np.ndarray:
        kv = self.config.kvDim
        p = lib().orc_state_vcache(self._s, layer)
        return np.ctypeslib.as_array(p, shape=((pos + 1) * kv,))[pos * kv:(pos + 1) * kv].copy()

    def fill_cache(self, depth: int, rng) -> None:
        """Writes seeded random binary16 rows (|v| < 1) into positions [0, depth) of every layer's K and V
        cache: a stand-in for a prefill when only the cost of attention at that depth matters."""
        kv = self.config.kvDim
        L = lib()
        for layer in range(self.config.numberOfLayers):
            for getter in (L.orc_state_kcache, L.orc_state_vcache):
                view = np.ctypeslib.as_array(getter(self._s, layer), shape=(depth * kv,))
                view[:] = (rng.random(depth * kv, dtype=np.float32) - 0.5).astype(np.float16).view(np.uint16)

    def close(self):
        L = lib()
        if self._s:
            L.orc_state_free(self._s)
            self._s = None
        if self._m:
            L.orc_model_free(self._m)
            self._m = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

"""ctypes binding of include/jitllm_b200.h. Fails loudly when the CUDA library is missing:
there is no CPU fallback anywhere in this package."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
import os

# JITLLM_B200_TRACE=1 selects the build with launch-timeline stamps (python -m jitllm_b200.build --trace).
LIB_PATH = PKG / "lib" / ("libjitllm_b200_trace.so" if os.environ.get("JITLLM_B200_TRACE") == "1" else "libjitllm_b200.so")
SYNTH_PATH = PKG / "lib" / "libjl_synth.so"


class JlModelDesc(C.Structure):
    _fields_ = [
        ("dim", C.c_int32), ("hidden", C.c_int32), ("layers", C.c_int32), ("heads", C.c_int32),
        ("kv_heads", C.c_int32), ("head_dim", C.c_int32), ("vocab", C.c_int32),
        ("ctx_len", C.c_int32), ("rms_eps", C.c_float), ("tied_embeddings", C.c_int32),
        ("max_batch", C.c_int32), ("tp_rank", C.c_int32), ("tp_size", C.c_int32),
    ]


class JlCounters(C.Structure):
    _fields_ = [
        ("decode_calls", C.c_uint64), ("prefill_calls", C.c_uint64),
        ("kernel_launches", C.c_uint64), ("h2d_bytes", C.c_uint64), ("d2h_bytes", C.c_uint64),
        ("weight_bytes", C.c_uint64), ("kv_bytes", C.c_uint64), ("workspace_bytes", C.c_uint64),
        ("last_step_ms", C.c_float),
    ]


_P = C.c_void_p
_I32 = C.c_int32
_I64 = C.c_int64

# name -> (restype, argtypes); mirrors the header declaration by declaration.
SIGNATURES = {
    "jl_init": (_I32, [_I32, C.POINTER(_P)]),
    "jl_destroy": (_I32, [_P]),
    "jl_last_error": (C.c_char_p, [_P]),
    "jl_model_create": (_I32, [_P, C.POINTER(JlModelDesc)]),
    "jl_upload_tensor": (_I32, [_P, _I32, _I32, _I32, _I64, _I64, _P, C.c_size_t]),
    "jl_upload_rope": (_I32, [_P, _P, _P, _I64]),
    "jl_model_finalize": (_I32, [_P]),
    "jl_kv_create": (_I32, [_P, _I32, _I32, _I32, _I32, _I32]),
    "jl_kv_publish_block_table": (_I32, [_P, _P, _I64]),
    "jl_kv_bytes_per_block": (_I64, [_P]),
    "jl_kv_fill": (_I32, [_P, C.c_uint16]),
    "jl_kv_read_row": (_I32, [_P, _I32, _I32, _I32, _I32, _P]),
    "jl_decode": (_I32, [_P, _I32, _P, _P, _P, _P, _P, _P]),
    "jl_generate": (_I32, [_P, _I32, _P, _P, _P, _P, _I32, _P]),
    "jl_sample": (_I32, [_P, _I32, C.c_float, C.c_float, _P, _P]),
    "jl_prefill": (_I32, [_P, _I32, _P, _I32, _I32]),
    "jl_debug_read": (_I32, [_P, C.c_char_p, _I32, _P, _I64]),
    "jl_dequant": (_I32, [_P, _I32, _P, _I64, _P]),
    "jl_gemv": (_I32, [_P, _I32, _I64, _I64, _P, _P, _I32, _P]),
    "jl_tensor_upload": (_I32, [_P, _I32, _I64, _I64, _P, C.c_size_t, C.POINTER(_P)]),
    "jl_tensor_free": (_I32, [_P, _P]),
    "jl_gemv_dev": (_I32, [_P, _P, _P, _I32, _P]),
    "jl_device_alloc": (_P, [_P, C.c_size_t]),
    "jl_device_free": (_I32, [_P, _P]),
    "jl_memcpy_h2d": (_I32, [_P, _P, _P, C.c_size_t]),
    "jl_memcpy_d2h": (_I32, [_P, _P, _P, C.c_size_t]),
    "jl_synchronize": (_I32, [_P]),
    "jl_stream": (_P, [_P]),
    "jl_timer_start": (_I32, [_P]),
    "jl_timer_stop": (_I32, [_P, C.POINTER(C.c_float)]),
    "jl_debug_trace": (_I32, [_P, _P, _I32]),
    "jl_bench_op": (_I32, [_P, _I32, _I32, _I32]),
    "jl_get_counters": (_I32, [_P, C.POINTER(JlCounters)]),
    "jl_flush_l2": (_I32, [_P]),
    "jl_tp_unique_id": (_I32, [_P, C.c_char_p, _P]),
    "jl_tp_init": (_I32, [_P, C.c_char_p, _P, _I32, _I32]),
    "jl_tp_exchange_mode": (_I32, [_P]),
    "jl_debug_peer_wait_timeout": (_I32, [_P, _I32]),
    "jl_tp_exchange_note": (C.c_char_p, [_P]),
    "jl_debug_tp_next_sequence": (C.c_uint32, [C.c_uint32]),
    "jl_gemv_argmax_static": (_I32, [_I32, _I64, _I64, _P, _P, _P, C.c_float, _P, _P, _P]),
    "jl_static_last_error": (C.c_char_p, []),
    "jl_static_status": (_I32, [_P]),
    "jl_gguf_open": (_I32, [C.c_char_p, C.POINTER(_P)]),
    "jl_gguf_describe": (_I32, [_P, C.POINTER(JlModelDesc), C.POINTER(C.c_float), C.POINTER(C.c_int64)]),
    "jl_gguf_upload": (_I32, [_P, _P, _I32, _I32, _I32, _P, _P, C.c_int64]),
    "jl_gguf_close": (None, [_P]),
    "jl_gguf_last_error": (C.c_char_p, []),
}

_lib = None
_synth = None


def load() -> C.CDLL:
    """The CUDA library. Raises if it has not been built: nothing here runs without it."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing; run `python -m jitllm_b200.build` "
                "(this package has no CPU fallback)"
            )
        lib = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError = header and library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def load_synth() -> C.CDLL:
    global _synth
    if _synth is None:
        if not SYNTH_PATH.exists():
            raise RuntimeError(f"{SYNTH_PATH} is missing; run `python -m jitllm_b200.build`")
        lib = C.CDLL(str(SYNTH_PATH))
        lib.jls_tensor_bytes.restype = _I64
        lib.jls_tensor_bytes.argtypes = [C.c_int, _I64]
        lib.jls_quantize.restype = C.c_int
        lib.jls_quantize.argtypes = [C.c_int, _P, _I64, _P, C.c_int]
        lib.jls_fill_normal.restype = C.c_int
        lib.jls_fill_normal.argtypes = [_P, _I64, _I64, C.c_uint64, C.c_float, C.c_int]
        lib.jls_synth_tensor.restype = C.c_int
        lib.jls_synth_tensor.argtypes = [C.c_int, _I64, C.c_uint64, C.c_float, _P, C.c_int]
        _synth = lib
    return _synth

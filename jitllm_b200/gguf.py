"""GGUF v3 writer for synthetic Llama-architecture models, and the Python face of the native reader.

The file layout is the one the reference parses (format/GGUF.java:60-110, 296-330): magic
0x46554747, version 3, tensor count, key/value count, the key/value pairs, the tensor infos (name,
n_dims, dims innermost first, ggml type, offset relative to the data section), padding to
`general.alignment` (32), then the tensor bytes, each padded to the alignment. Metadata keys are the
ones LlamaModelLoader reads (model/loader/LlamaModelLoader.java:49-67); tensor names follow the
llama.cpp convention the reference's TensorRole maps from (runtime/tensor/TensorRole.java:17-59).
"""
from __future__ import annotations

import struct
from typing import Dict, Tuple

import numpy as np

GGUF_MAGIC = 0x46554747
ALIGNMENT = 32
# gguf_metadata_value_type
_T_U32, _T_F32, _T_STRING = 4, 6, 8

LAYER_NAMES = {
    "ATTENTION_NORM": "blk.%d.attn_norm.weight",
    "ATTENTION_QUERY": "blk.%d.attn_q.weight",
    "ATTENTION_KEY": "blk.%d.attn_k.weight",
    "ATTENTION_VALUE": "blk.%d.attn_v.weight",
    "ATTENTION_OUTPUT": "blk.%d.attn_output.weight",
    "FFN_NORM": "blk.%d.ffn_norm.weight",
    "FFN_GATE": "blk.%d.ffn_gate.weight",
    "FFN_UP": "blk.%d.ffn_up.weight",
    "FFN_DOWN": "blk.%d.ffn_down.weight",
}
GLOBAL_NAMES = {
    "TOKEN_EMBEDDING": "token_embd.weight",
    "OUTPUT_NORM": "output_norm.weight",
    "OUTPUT": "output.weight",
}


def tensor_name(role, layer: int) -> str:
    if role.name in GLOBAL_NAMES:
        return GLOBAL_NAMES[role.name]
    return LAYER_NAMES[role.name] % layer


def _string(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _kv(key: str, vtype: int, value) -> bytes:
    head = _string(key) + struct.pack("<I", vtype)
    if vtype == _T_U32:
        return head + struct.pack("<I", int(value))
    if vtype == _T_F32:
        return head + struct.pack("<f", float(value))
    return head + _string(str(value))


def _pad(n: int) -> int:
    return (-n) % ALIGNMENT


def write_gguf(path, config, tensors: Dict[Tuple[object, int], Tuple[object, np.ndarray]]) -> int:
    """Writes `tensors` ({(role, layer): (ggml_type, bytes-or-float32 array)}, the dictionary
    synth_model_tensors returns) as one GGUF file; returns the number of bytes written."""
    c = config
    kvs = [
        _kv("general.architecture", _T_STRING, "llama"),
        _kv("general.alignment", _T_U32, ALIGNMENT),
        _kv("llama.vocab_size", _T_U32, c.vocabularySize),
        _kv("llama.embedding_length", _T_U32, c.dim),
        _kv("llama.feed_forward_length", _T_U32, c.hiddenDim),
        _kv("llama.block_count", _T_U32, c.numberOfLayers),
        _kv("llama.attention.head_count", _T_U32, c.numberOfHeads),
        _kv("llama.attention.head_count_kv", _T_U32, c.numberOfKeyValueHeads),
        _kv("llama.context_length", _T_U32, c.contextLength),
        _kv("llama.attention.layer_norm_rms_epsilon", _T_F32, c.rmsNormEps),
        _kv("llama.rope.freq_base", _T_F32, c.ropeTheta),
    ]
    infos, blobs, offset = [], [], 0
    for (role, layer), (gtype, data) in tensors.items():
        rows, cols = c.matrix_shape(role)
        raw = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        dims = (cols,) if rows == 1 else (cols, rows)  # innermost dimension first
        info = _string(tensor_name(role, layer)) + struct.pack("<I", len(dims))
        info += b"".join(struct.pack("<Q", d) for d in dims)
        info += struct.pack("<I", int(gtype)) + struct.pack("<Q", offset)
        infos.append(info)
        blobs.append(raw)
        offset += raw.size + _pad(raw.size)
    header = struct.pack("<IIQQ", GGUF_MAGIC, 3, len(infos), len(kvs)) + b"".join(kvs) + b"".join(infos)
    with open(path, "wb") as f:
        f.write(header)
        f.write(b"\0" * _pad(len(header)))
        for raw in blobs:
            f.write(raw.tobytes())
            f.write(b"\0" * _pad(raw.size))
        return f.tell()


class GgufFile:
    """A GGUF file opened by the native reader (header, metadata and tensor infos parsed; tensor bytes
    stay in the mapping until they are uploaded). Needs the built library, not a GPU."""

    def __init__(self, path):
        import ctypes as C
        from . import _lib
        self._lib = _lib.load()
        self._h = C.c_void_p()
        rc = self._lib.jl_gguf_open(str(path).encode(), C.byref(self._h))
        if rc != 0:
            raise ValueError(self._lib.jl_gguf_last_error().decode())

    def describe(self):
        """(Configuration, number of tensors) from the llama.* metadata keys."""
        import ctypes as C
        from . import _lib
        from .api import Configuration
        d = _lib.JlModelDesc()
        theta, n = C.c_float(), C.c_int64()
        rc = self._lib.jl_gguf_describe(self._h, C.byref(d), C.byref(theta), C.byref(n))
        if rc != 0:
            raise ValueError(self._lib.jl_gguf_last_error().decode())
        cfg = Configuration(dim=d.dim, hiddenDim=d.hidden, numberOfLayers=d.layers, numberOfHeads=d.heads,
                            numberOfKeyValueHeads=d.kv_heads, vocabularySize=d.vocab, contextLength=d.ctx_len,
                            rmsNormEps=d.rms_eps, ropeTheta=theta.value, tiedEmbeddings=bool(d.tied_embeddings))
        return cfg, int(n.value)

    def close(self) -> None:
        if self._h:
            self._lib.jl_gguf_close(self._h)
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


def load_model_gguf(dev, path, maxBatch: int = 1, tp=None, broadcast=None, rope_cos=None, rope_sin=None):
    """Model straight from a GGUF file: the native reader uploads every tensor (this rank's slices
    under tensor parallelism) from the file mapping. RoPE tables: pass the host's own to share them
    bit for bit with a CPU path, or leave None to have them computed natively."""
    from .api import B200Model, _exception, _ptr
    from .tensor_parallel import TensorParallel, check_divisible, init_group
    tp = tp or TensorParallel()
    with GgufFile(path) as g:
        cfg, _ = g.describe()
        check_divisible(cfg, tp.size)
        cos = None if rope_cos is None else np.ascontiguousarray(rope_cos, dtype=np.float32)
        sin = None if rope_sin is None else np.ascontiguousarray(rope_sin, dtype=np.float32)
        rc = dev._lib.jl_gguf_upload(dev.handle, g._h, int(maxBatch), tp.rank, tp.size, _ptr(cos), _ptr(sin),
                                     0 if cos is None else cos.size)
        if rc != 0:
            raise _exception(rc, dev._lib.jl_gguf_last_error().decode())
    model = B200Model.adopt(dev, cfg, maxBatch, tp)
    if tp.size > 1:
        if broadcast is None:
            raise ValueError("GPUL-CFG-002: tensor parallelism needs a broadcast channel for the NCCL id")
        init_group(dev, tp, broadcast)
    model.finalize()
    return model

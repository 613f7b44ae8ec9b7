"""Host side of tensor parallelism: which slice of each GGUF tensor a GPU holds, and the set-up of
the NCCL group the library reduces over.

The reference runs on one device; its plan is a chain of per-layer task graphs
(backend/tornado/layers/LlamaQ8_0FFNLayers.java:150-213). The split here is the Megatron one, cut so
that every quantised block stays whole:

* rows of wq / wk / wv (whole heads), w1 (gate), w3 (up) and the vocabulary matrix are divided into
  `size` contiguous ranges -- a row of a GGUF matrix is one run of blocks, so this is a byte slice;
* columns of wo and w2 (down) are divided into `size` contiguous ranges of whole 256-element
  groups -- a per-row slice of blocks;
* norm weights, RoPE tables and the token embedding are replicated.

Each GPU then produces a partial [dim] vector from wo and from w2; the library sums them over the
group (one all-reduce per sublayer) before the residual add.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import numpy as np

ROW_SPLIT = ("ATTENTION_QUERY", "ATTENTION_KEY", "ATTENTION_VALUE", "FFN_GATE", "FFN_UP", "OUTPUT")
COL_SPLIT = ("ATTENTION_OUTPUT", "FFN_DOWN")
COLUMN_GROUP = 256  # the kernels' unit along a row: a whole number of blocks in every format


@dataclass(frozen=True)
class TensorParallel:
    rank: int = 0
    size: int = 1

    def __post_init__(self):
        if self.size < 1 or not (0 <= self.rank < self.size):
            raise ValueError(f"GPUL-CFG-002: rank {self.rank} of {self.size} is not a valid placement")


def check_divisible(config, size: int) -> None:
    """The conditions jl_model_create checks, stated on the host so a bad split fails before any upload."""
    c = config
    problems = []
    if c.numberOfHeads % size:
        problems.append(f"heads {c.numberOfHeads}")
    if c.numberOfKeyValueHeads % size:
        problems.append(f"kv heads {c.numberOfKeyValueHeads}")
    if c.vocabularySize % size:
        problems.append(f"vocabulary {c.vocabularySize}")
    if c.dim % size or (c.dim // size) % COLUMN_GROUP:
        problems.append(f"dim {c.dim} (needs {COLUMN_GROUP}-column groups per GPU)")
    if c.hiddenDim % size or (c.hiddenDim // size) % COLUMN_GROUP:
        problems.append(f"hidden {c.hiddenDim} (needs {COLUMN_GROUP}-column groups per GPU)")
    if problems:
        raise ValueError("GPUL-CFG-002: cannot split over %d GPUs: %s" % (size, ", ".join(problems)))


def local_shape(config, role, size: int) -> Tuple[int, int]:
    rows, cols = config.matrix_shape(role)
    if role.name in ROW_SPLIT:
        return rows // size, cols
    if role.name in COL_SPLIT:
        return rows, cols // size
    return rows, cols


def assemble_tensor(config, role, shards) -> np.ndarray:
    """The whole tensor whose slices, in rank order, are `shards`: the inverse of shard_tensor."""
    size = len(shards)
    if size == 1 or (role.name not in ROW_SPLIT and role.name not in COL_SPLIT):
        return shards[0]
    rows, _ = config.matrix_shape(role)
    if role.name in ROW_SPLIT:
        return np.concatenate([np.ascontiguousarray(s).reshape(-1) for s in shards])
    return np.ascontiguousarray(np.concatenate([np.ascontiguousarray(s).reshape(rows, -1) for s in shards], axis=1)).reshape(-1)


def shard_tensor(config, role, ggml_type, data: np.ndarray, tp: TensorParallel) -> np.ndarray:
    """This GPU's slice of one tensor, as bytes (quantised / F16) or float32 (F32), contiguous."""
    if tp.size == 1:
        return data
    rows, cols = config.matrix_shape(role)
    if role.name in ROW_SPLIT:
        flat = np.ascontiguousarray(data).reshape(rows, -1)
        n = rows // tp.size
        return np.ascontiguousarray(flat[tp.rank * n:(tp.rank + 1) * n]).reshape(-1)
    if role.name in COL_SPLIT:
        per = cols // tp.size
        if per % COLUMN_GROUP:
            raise ValueError(f"GPUL-CFG-002: {role.name}: {per} columns per GPU is not a multiple of {COLUMN_GROUP}")
        flat = np.ascontiguousarray(data).reshape(rows, -1)  # one row = cols / block_size blocks
        unit = flat.shape[1] * per // cols  # array elements per GPU per row
        return np.ascontiguousarray(flat[:, tp.rank * unit:(tp.rank + 1) * unit]).reshape(-1)
    return data


def nccl_library_path() -> Optional[str]:
    """The NCCL build PyTorch ships (its own collectives use the same one), else the loader's default."""
    override = os.environ.get("JITLLM_B200_NCCL")
    if override:
        return override
    try:
        import nvidia.nccl as pkg  # type: ignore
        for base in list(pkg.__path__):
            cand = os.path.join(base, "lib", "libnccl.so.2")
            if os.path.exists(cand):
                return cand
    except ImportError:
        pass
    return None


def init_group(dev, tp: TensorParallel, broadcast: Callable[[Optional[bytes]], bytes]) -> None:
    """Collective over the group. `broadcast(payload)` is the host's channel: rank 0 passes the 128-byte
    id, the others pass None, all get rank 0's bytes back (torch.distributed, MPI, a socket ...)."""
    if tp.size == 1:
        return
    path = nccl_library_path()
    cpath = path.encode() if path else None
    ident = (C.c_ubyte * 128)()
    if tp.rank == 0:
        dev._check(dev._lib.jl_tp_unique_id(dev.handle, cpath, ident))
        payload = broadcast(bytes(ident))
    else:
        payload = broadcast(None)
    if len(payload) != 128:
        raise ValueError("GPUL-CFG-002: the broadcast id must be 128 bytes")
    ident = (C.c_ubyte * 128).from_buffer_copy(payload)
    dev._check(dev._lib.jl_tp_init(dev.handle, cpath, ident, tp.rank, tp.size))


def torch_broadcast(payload: Optional[bytes]) -> bytes:
    """`broadcast` for init_group over an initialised torch.distributed group (CPU or CUDA backend)."""
    import torch
    import torch.distributed as dist
    backend = dist.get_backend()
    device = torch.device("cuda", torch.cuda.current_device()) if "nccl" in backend and "gloo" not in backend \
        else torch.device("cpu")
    t = torch.zeros(128, dtype=torch.uint8, device=device)
    if payload is not None:
        t.copy_(torch.frombuffer(bytearray(payload), dtype=torch.uint8))
    dist.broadcast(t, src=0)
    return bytes(t.cpu().numpy().tobytes())

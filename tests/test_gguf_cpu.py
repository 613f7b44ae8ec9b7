"""The GGUF writer against the native reader, without a GPU: header, metadata and tensor infos
survive the round trip, and malformed files are refused with the reference's error code."""
import struct

import numpy as np
import pytest

import jitllm_b200 as jl
from jitllm_b200.gguf import ALIGNMENT, GGUF_MAGIC, tensor_name

CFG = jl.Configuration(dim=256, hiddenDim=512, numberOfLayers=2, numberOfHeads=4, numberOfKeyValueHeads=2,
                       vocabularySize=512, contextLength=32, rmsNormEps=1e-5, ropeTheta=500000.0)


def _write(tmp_path, cfg=CFG, fmt=jl.GGMLType.Q4_K, name="m.gguf"):
    tensors = jl.synth_model_tensors(cfg, fmt, seed=7)
    path = tmp_path / name
    size = jl.write_gguf(path, cfg, tensors)
    assert size == path.stat().st_size
    return path, tensors


def test_round_trip_of_the_description(built, tmp_path):
    path, tensors = _write(tmp_path)
    with jl.GgufFile(path) as g:
        cfg, n = g.describe()
    import dataclasses
    assert dataclasses.replace(cfg, rmsNormEps=CFG.rmsNormEps) == CFG
    assert cfg.rmsNormEps == pytest.approx(CFG.rmsNormEps, rel=1e-6)  # stored as binary32
    assert n == len(tensors)


def test_tied_embeddings_are_detected(built, tmp_path):
    tied = jl.Configuration(dim=256, hiddenDim=512, numberOfLayers=1, numberOfHeads=4, numberOfKeyValueHeads=2,
                            vocabularySize=256, contextLength=16, tiedEmbeddings=True)
    path, _ = _write(tmp_path, tied, jl.GGMLType.Q8_0, "tied.gguf")
    with jl.GgufFile(path) as g:
        cfg, _ = g.describe()
    assert cfg.tiedEmbeddings and cfg.ropeTheta == pytest.approx(500000.0)


def test_layout_is_what_the_format_says(built, tmp_path):
    path, tensors = _write(tmp_path)
    raw = path.read_bytes()
    magic, version, n_tensors, n_kv = struct.unpack_from("<IIQQ", raw, 0)
    assert (magic, version, n_tensors) == (GGUF_MAGIC, 3, len(tensors)) and n_kv >= 10
    # the last tensor's bytes sit, padded, at the end of the file
    (role, layer), (_, data) = list(tensors.items())[-1]
    blob = np.ascontiguousarray(data).view(np.uint8).tobytes()
    padded = len(blob) + (-len(blob)) % ALIGNMENT
    assert raw[len(raw) - padded:len(raw) - padded + len(blob)] == blob
    assert tensor_name(role, layer).encode() in raw[:65536]


def test_malformed_files_are_refused(built, tmp_path):
    path, _ = _write(tmp_path)
    raw = bytearray(path.read_bytes())
    bad_magic = tmp_path / "bad_magic.gguf"
    bad_magic.write_bytes(b"XXXX" + bytes(raw[4:]))
    with pytest.raises(ValueError, match="GPUL-CFG-002"):
        jl.GgufFile(bad_magic)
    truncated = tmp_path / "short.gguf"
    truncated.write_bytes(bytes(raw[:len(raw) // 2]))  # tensor data cut off
    with pytest.raises(ValueError, match="outside the file"):
        jl.GgufFile(truncated)
    header_cut = tmp_path / "header_cut.gguf"
    header_cut.write_bytes(bytes(raw[:100]))
    with pytest.raises(ValueError, match="malformed"):
        jl.GgufFile(header_cut)
    with pytest.raises(ValueError, match="cannot open"):
        jl.GgufFile(tmp_path / "absent.gguf")


def test_tensor_infos_that_overflow_64_bits_are_refused(built, tmp_path):
    """Dimensions or an offset chosen so that offset + rows * row bytes wraps around 2^64 and lands
    back inside the file must not pass the bounds check."""
    path, tensors = _write(tmp_path)
    raw = bytearray(path.read_bytes())
    (role, layer), _ = list(tensors.items())[-1]
    name = tensor_name(role, layer).encode()
    at = raw.index(struct.pack("<Q", len(name)) + name) + 8 + len(name)
    (n_dims,) = struct.unpack_from("<I", raw, at)
    dims_at, type_at = at + 4, at + 4 + 8 * n_dims
    off_at = type_at + 4
    huge_offset = bytearray(raw)
    struct.pack_into("<Q", huge_offset, off_at, 0xFFFFFFFFFFFFFF00)  # aligned, and wraps when the size is added
    p1 = tmp_path / "huge_offset.gguf"
    p1.write_bytes(bytes(huge_offset))
    with pytest.raises(ValueError, match="outside the file"):
        jl.GgufFile(p1)
    if n_dims >= 2:
        huge_rows = bytearray(raw)
        struct.pack_into("<Q", huge_rows, dims_at + 8, 1 << 62)  # rows * row bytes wraps
        p2 = tmp_path / "huge_rows.gguf"
        p2.write_bytes(bytes(huge_rows))
        with pytest.raises(ValueError, match="outside the file"):
            jl.GgufFile(p2)

"""The byte accounting behind the roofline figures: algorithmic bytes per launch and per decode step
for the named architectures, checked against hand arithmetic (weights once per step, block formats at
34/32, 18/32 and 144/256 bytes per element)."""
import importlib.util
from pathlib import Path

import pytest

import jitllm_b200 as jl

spec = importlib.util.spec_from_file_location("bench", Path(__file__).resolve().parent.parent / "bench.py")
bench = importlib.util.module_from_spec(spec)
spec.loader.exec_module(bench)


def _cfg(arch):
    d = bench.ARCHS[arch]
    return jl.Configuration(dim=d[0], hiddenDim=d[1], numberOfLayers=d[2], numberOfHeads=d[3],
                            numberOfKeyValueHeads=d[4], vocabularySize=d[5], contextLength=d[6], tiedEmbeddings=d[7])


def test_weight_bytes_per_decode_step():
    assert bench.model_bytes(_cfg("8b"), "Q4_K") == pytest.approx(4.221e9, rel=1e-3)   # 7 504 658 432 elements
    assert bench.model_bytes(_cfg("8b"), "Q8_0") == pytest.approx(7.974e9, rel=1e-3)
    assert bench.model_bytes(_cfg("70b"), "Q4_K") == pytest.approx(39.09e9, rel=1e-3)  # 69 501 714 432 elements
    assert bench.model_bytes(_cfg("1b"), "Q8_0") == pytest.approx(1.313e9, rel=1e-3)   # tied: embedding counted once


def test_bytes_per_launch_of_the_8b_layer_shapes():
    cfg = _cfg("8b")
    want = {0: 14.20e6, 1: 9.47e6, 2: 66.13e6, 3: 33.10e6, 4: 296.03e6}
    for op, mb in want.items():
        assert bench.op_bytes(cfg, "Q4_K", op) == pytest.approx(mb, rel=2e-3), op


def test_tensor_parallel_shards_divide_the_bytes():
    cfg = _cfg("70b")
    for op in range(5):
        whole, eighth = bench.op_bytes(cfg, "Q4_K", op), bench.op_bytes(cfg, "Q4_K", op, 8)
        assert eighth < whole / 7.5  # weights divide by eight, the activation vector does not

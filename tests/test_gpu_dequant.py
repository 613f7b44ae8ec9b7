"""Dequantised weights are bit-exact against the oracle (and against the committed fixture of
java.util.Random-seeded blocks from the reference's decode tests)."""
from pathlib import Path

import numpy as np
import pytest

import jitllm_b200 as jl
from jitllm_b200 import GGMLType

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).parent / "golden"


@pytest.mark.parametrize("name,t", [("q4_0", GGMLType.Q4_0), ("q4_k", GGMLType.Q4_K), ("q8_0", GGMLType.Q8_0)])
def test_java_seeded_blocks_decode_bit_exactly(dev, name, t):
    fx = np.load(GOLDEN / "java_random_blocks.npz")
    raw, want = fx[name + "_raw"], fx[name + "_f32_bits"]
    got = dev.dequantize(t, raw, want.size).view(np.uint32)
    nan = np.isnan(want.view(np.float32))
    assert np.array_equal(got[~nan], want[~nan])
    assert np.array_equal(np.isnan(got.view(np.float32)), nan)


def test_q4_0_specified_layout(dev):
    raw = np.zeros(18, dtype=np.uint8)
    raw[1], raw[2], raw[3] = 0x40, 0x0F, 0x80
    out = dev.dequantize(GGMLType.Q4_0, raw, 32)
    assert (out[0], out[16], out[1], out[17]) == (14.0, -16.0, -16.0, 0.0)


@pytest.mark.parametrize("t", [GGMLType.Q8_0, GGMLType.Q4_0, GGMLType.Q4_K])
def test_synthetic_weights_decode_bit_exactly(dev, oracle, t):
    n = 4096 * 512
    raw = jl.synth_tensor(t, n, seed=3)
    assert np.array_equal(dev.dequantize(t, raw, n).view(np.uint32), oracle.dequant(t, raw, n).view(np.uint32))


@pytest.mark.parametrize("t", [GGMLType.Q8_0, GGMLType.Q4_0, GGMLType.Q4_K])
def test_random_payloads_including_extreme_scales(dev, oracle, t):
    rng = np.random.default_rng(17)
    raw = rng.integers(0, 256, size=t.type_size * 64, dtype=np.uint8)
    n = 64 * t.block_size
    got, want = dev.dequantize(t, raw, n), oracle.dequant(t, raw, n)
    nan = np.isnan(want)
    assert np.array_equal(got.view(np.uint32)[~nan], want.view(np.uint32)[~nan])
    assert np.array_equal(np.isnan(got), nan)


def test_empty_and_ragged_inputs(dev):
    assert dev.dequantize(GGMLType.Q8_0, np.zeros(0, dtype=np.uint8), 0).size == 0
    with pytest.raises(ValueError, match="whole number"):
        dev.dequantize(GGMLType.Q4_K, np.zeros(144, dtype=np.uint8), 100)
    with pytest.raises(ValueError, match="GGML type"):
        dev.dequantize(GGMLType.F16, np.zeros(64, dtype=np.uint8), 32)

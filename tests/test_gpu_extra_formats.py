"""Q4_1, Q5_K and Q6_K on the device: decoded weights bit-exact against the oracle, the stand-alone mat-vec within
the per-matmul bound of the other formats (relative L2 <= 1e-3; the sums are binary32 in a different order from
the reference's sequential loop, which in practice gives ~1e-6)."""
import numpy as np
import pytest

import jitllm_b200 as jl
from jitllm_b200 import GGMLType
from tests.util import random_blocks, rel_l2

pytestmark = pytest.mark.gpu
EXTRA = [GGMLType.Q4_1, GGMLType.Q5_K, GGMLType.Q6_K]


def _same_bits(got, want):
    nan = np.isnan(want)
    return np.array_equal(got.view(np.uint32)[~nan], want.view(np.uint32)[~nan]) and np.array_equal(np.isnan(got), nan)


def test_q4_1_known_answers(dev):
    raw = np.zeros(20, dtype=np.uint8)
    raw[0:2] = np.frombuffer(np.float16(0.25).tobytes(), dtype=np.uint8)
    raw[2:4] = np.frombuffer(np.float16(-1.5).tobytes(), dtype=np.uint8)
    nib = np.arange(32) % 16
    raw[4:20] = nib[:16] | (nib[16:] << 4)
    assert np.array_equal(dev.dequantize(GGMLType.Q4_1, raw, 32), (0.25 * nib - 1.5).astype(np.float32))


@pytest.mark.parametrize("t", EXTRA)
def test_decode_bit_exactly(dev, oracle, t):
    rng = np.random.default_rng(40 + int(t))
    blocks = 4096
    n = blocks * t.block_size
    sane = random_blocks(t, blocks, rng)
    assert _same_bits(dev.dequantize(t, sane, n), oracle.dequant(int(t), sane, n))
    wild = rng.integers(0, 256, size=blocks * t.type_size, dtype=np.uint8)  # infinite and NaN scales included
    assert _same_bits(dev.dequantize(t, wild, n), oracle.dequant(int(t), wild, n))


@pytest.mark.parametrize("t", EXTRA)
@pytest.mark.parametrize("rows,cols,n", [(4096, 4096, 1), (1000, 14336, 1), (37, 256, 1), (512, 2048, 3), (300, 1024, 5), (256, 4096, 9),
                                         (64, 14336, 4), (128, 6144, 2), (96, 16384, 1), (40, 16640, 1), (70, 768, 2), (33, 4352, 1), (700, 2048, 40), (257, 1024, 130),
                                         (129, 256, 8), (50, 768, 5), (31, 1280, 7)])
def test_matvec_against_the_oracle(dev, oracle, t, rows, cols, n):
    rng = np.random.default_rng(rows + cols + int(t))
    w = random_blocks(t, rows * cols // t.block_size, rng)
    x = rng.standard_normal((n, cols)).astype(np.float32)
    got = dev.matmul(t, w, rows, cols, x if n > 1 else x[0])
    want = oracle.matmul(int(t), w, x if n > 1 else x[0], rows, cols)
    assert got.shape == want.shape
    assert rel_l2(got, want) <= 1e-3
    # Fewer than eight rows go, row by row, through the model's own mat-vec kernel: 16-bit fixed-point activations
    # per block (~3e-5). A wrong nibble is ~1e-1.
    fused = n < 8
    # Eight or more rows: the tensor-core kernel (binary16 weights and activation parts, ~3e-4).
    tensor_core = n >= 8
    assert fused != tensor_core
    assert rel_l2(got, want) <= (6e-4 if tensor_core else 1e-4)


@pytest.mark.parametrize("t", EXTRA)
def test_device_resident_matvec_repeats_bit_identically(dev, oracle, t):
    rng = np.random.default_rng(5)
    rows, cols = 2048, 4096
    w = random_blocks(t, rows * cols // t.block_size, rng)
    x = rng.standard_normal(cols).astype(np.float32)
    a = dev.matmul(t, w, rows, cols, x)
    b = dev.matmul(t, w, rows, cols, x)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_tensor_parallel_models_refuse_the_extra_formats():
    """One GPU runs such tensors through the row path (tests/test_gpu_mixed_formats.py); a shard of a tensor-parallel
    model does not take them."""
    cfg = jl.Configuration(dim=512, hiddenDim=1024, numberOfLayers=1, numberOfHeads=4, numberOfKeyValueHeads=2,
                           vocabularySize=256, contextLength=32)
    with jl.Device(0) as own:
        model = jl.B200Model(own, cfg, tp=jl.TensorParallel(rank=0, size=2))
        raw = np.zeros(256 * 512 // 256 * 210, dtype=np.uint8)  # this rank's half of the query rows
        with pytest.raises(ValueError, match="GPUL-CFG-002: unsupported.*on one GPU"):
            model.uploadTensor(jl.TensorRole.ATTENTION_QUERY, 0, GGMLType.Q6_K, raw, presharded=True)


def test_too_wide_rows_are_refused(dev):
    """The mat-vec kernel keeps a row's activation in sixteen chunks of 2048 columns."""
    t = GGMLType.Q6_K
    cols = 32768 + 256
    raw = np.zeros(cols // 256 * 210, dtype=np.uint8)
    with pytest.raises(ValueError, match="GPUL-CFG-002"):
        dev.matmul(t, raw, 1, cols, np.zeros(cols, dtype=np.float32))

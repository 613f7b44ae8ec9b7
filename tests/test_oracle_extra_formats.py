"""Pins the CPU oracle's Q4_1, Q5_K and Q6_K decoders and dot products.

Sources (paths under src/test/java/org/beehive/jitllm/ of the reference):
  tensor/Q4_1FloatTensorTest.java:52-71            nibbles i % 16, d = 0.25, m = -1.5 -> 0.25 * q - 1.5
  tensor/Q4_1FloatTensorTest.java:80-123           vectorised dot against element-wise reading, four spans
  backend/tornado/kernels/Q6_KDp4aAccelTest.java:52-95   recipe: d = 0x2C00, byte scales +-(1 + (row + i) % 7),
                                                   raw value (e + row) % 64 written at element e
  backend/tornado/kernels/Q5_KDp4aAccelTest.java:60-92   recipe: payload patterns 0x00 / 0xFF / 0xAA / 0x55 / random
Each recipe is rebuilt here from its description; the expected values come from a closed form or from the
independent numpy decoders of tests/np_formats.py, never from the oracle itself."""
import numpy as np
import pytest

from tests import np_formats
from tests.util import random_blocks

Q4_1, Q5_K, Q6_K = 3, 13, 14
SIZES = {Q4_1: (20, 32), Q5_K: (176, 256), Q6_K: (210, 256)}


def _same_bits(got, want):
    nan = np.isnan(want)
    return np.array_equal(got.view(np.uint32)[~nan], want.view(np.uint32)[~nan]) and np.array_equal(np.isnan(got), nan)


def test_q4_1_known_answers(oracle):
    raw = np.zeros(20, dtype=np.uint8)
    raw[0:2] = np.frombuffer(np.float16(0.25).tobytes(), dtype=np.uint8)
    raw[2:4] = np.frombuffer(np.float16(-1.5).tobytes(), dtype=np.uint8)
    nib = np.arange(32) % 16
    raw[4:20] = nib[:16] | (nib[16:] << 4)
    out = oracle.dequant(Q4_1, raw, 32)
    assert np.array_equal(out, (0.25 * nib - 1.5).astype(np.float32))


def _q6k_recipe_rows():
    """256 rows of one super-block: row r holds raw value (e + r) % 64 at element e."""
    raw = np.zeros((256, 210), dtype=np.uint8)
    raw[:, 208], raw[:, 209] = 0x00, 0x2C  # 0.0625
    rows = np.arange(256)[:, None]
    i = np.arange(16)[None, :]
    mag = 1 + (rows + i) % 7
    raw[:, 192:208] = np.where(i % 2 == 0, mag, -mag).astype(np.int8).view(np.uint8)
    for e in range(256):
        value = (e + rows[:, 0]) % 64
        half, group, pos = e // 128, (e % 128) // 32, e % 32
        at = half * 64 + (group & 1) * 32 + pos
        if group >= 2:
            raw[:, at] = (raw[:, at] & 0x0F) | ((value & 0xF) << 4)
        else:
            raw[:, at] = (raw[:, at] & 0xF0) | (value & 0xF)
        qh = 128 + half * 32 + pos
        raw[:, qh] = (raw[:, qh] & (0xFF ^ (3 << (2 * group)))) | (((value >> 4) & 3) << (2 * group))
    return raw


def test_q6_k_every_quantum_of_the_reference_recipe(oracle):
    raw = _q6k_recipe_rows()
    got = oracle.dequant(Q6_K, raw.reshape(-1), 256 * 256).reshape(256, 256)
    rows = np.arange(256)[:, None]
    e = np.arange(256)[None, :]
    scale_index = e // 16  # the sixteen scales are in element order
    mag = 1 + (rows + scale_index) % 7
    scale = np.where(scale_index % 2 == 0, mag, -mag)
    want = (0.0625 * scale * ((e + rows) % 64 - 32)).astype(np.float32)  # exact in binary32
    assert np.array_equal(got, want)


def test_q5_k_adversarial_patterns(oracle):
    rng = np.random.default_rng(20260913)
    blocks = 48
    raw = rng.integers(0, 256, size=(blocks, 176), dtype=np.uint8)
    for b in range(blocks):
        if b % 4 != 3:
            raw[b, :] = [0x00, 0xFF, 0xAA, 0x55][b % 4]
        d = 0.0 if b % 9 == 0 else 2.0 ** (-14 + b % 12) * 0.031
        dmin = 0.0 if b % 7 == 0 else 2.0 ** (-13 + b % 10) * 0.017
        d, dmin = (-d if b % 3 == 0 else d), (-dmin if b % 5 == 0 else dmin)
        raw[b, 0:2] = np.frombuffer(np.float16(d).tobytes(), dtype=np.uint8)
        raw[b, 2:4] = np.frombuffer(np.float16(dmin).tobytes(), dtype=np.uint8)
    got = oracle.dequant(Q5_K, raw.reshape(-1), blocks * 256)
    assert _same_bits(got, np_formats.dequant_q5_k(raw.reshape(-1)))


@pytest.mark.parametrize("t", [Q4_1, Q5_K, Q6_K])
def test_random_blocks_decode_like_an_independent_restatement(oracle, t):
    rng = np.random.default_rng(100 + t)
    bb, be = SIZES[t]
    raw = rng.integers(0, 256, size=64 * bb, dtype=np.uint8)  # every byte random: infinities and NaNs included
    assert _same_bits(oracle.dequant(t, raw, 64 * be), np_formats.DEQUANT[t](raw))
    sane = random_blocks(t, 64, rng)
    assert _same_bits(oracle.dequant(t, sane, 64 * be), np_formats.DEQUANT[t](sane))
    for i in (0, 1, 31, 32, 255, 256, 64 * be - 1):
        assert oracle.get_float(t, sane, i) == np_formats.DEQUANT[t](sane)[i]


@pytest.mark.parametrize("t", [Q4_1, Q5_K, Q6_K])
@pytest.mark.parametrize("bits", [0, 128, 256])
def test_matmul_agrees_with_float64(oracle, t, bits):
    rng = np.random.default_rng(7 + t)
    rows, cols = 24, 1024
    bb, be = SIZES[t]
    w = random_blocks(t, rows * cols // be, rng)
    x = rng.standard_normal(cols).astype(np.float32)
    want = np_formats.DEQUANT[t](w).reshape(rows, cols).astype(np.float64) @ x.astype(np.float64)
    L = oracle.lib()
    old = L.orc_get_vector_bits()
    try:
        L.orc_set_vector_bits(bits)
        got = oracle.matmul(t, w, x, rows, cols)
    finally:
        L.orc_set_vector_bits(old)
    assert np.all(np.abs(got - want) <= np.maximum(1e-4, np.abs(want) * 1e-5) * 4)

"""The tensor-core (tcgen05) matrix-matrix path against the oracle's batch matmul
(FloatTensor.matmul(context, that[], out[], ...)): per-matmul relative L2 <= 1e-3 is the stated
bar. Weights are rounded to fp16 after an element-exact fp32 decode and activations are carried
as fp16 hi+lo, so ~3e-4 is expected."""
import numpy as np
import pytest

import jitllm_b200 as jl
from jitllm_b200 import GGMLType
from tests.util import rel_l2

pytestmark = pytest.mark.gpu
BAR = 1e-3
EXPECT = 6e-4
FORMATS = [GGMLType.Q8_0, GGMLType.Q4_0, GGMLType.Q4_K]


@pytest.mark.parametrize("t", FORMATS)
@pytest.mark.parametrize("rows,cols,n", [(128, 256, 8), (256, 512, 16), (200, 768, 9), (384, 1024, 33),
                                         (1000, 2048, 64), (130, 256, 130), (512, 1792, 200)])
def test_small_and_ragged_tiles(dev, oracle, t, rows, cols, n):
    w = jl.synth_tensor(t, rows * cols, seed=rows + cols + n)
    x = np.random.default_rng(n).standard_normal((n, cols)).astype(np.float32)
    got, want = dev.matmul(t, w, rows, cols, x), oracle.matmul(t, w, x, rows, cols)
    assert got.shape == (n, rows)
    err = rel_l2(got, want)
    assert err < BAR and err < EXPECT, err
    # every row individually, so a misplaced tile cannot hide in the aggregate
    per_row = np.linalg.norm(got - want, axis=1) / np.linalg.norm(want, axis=1)
    assert per_row.max() < BAR, per_row.max()


@pytest.mark.parametrize("t", FORMATS)
@pytest.mark.parametrize("rows,cols,n", [(4096, 4096, 32), (14336, 4096, 8), (4096, 14336, 32)])
def test_sweep_shapes(dev, oracle, t, rows, cols, n):
    w = jl.synth_tensor(t, rows * cols, seed=rows + n + int(t))
    x = np.random.default_rng(3).standard_normal((n, cols)).astype(np.float32)
    got, want = dev.matmul(t, w, rows, cols, x), oracle.matmul(t, w, x, rows, cols)
    err = rel_l2(got, want)
    assert err < BAR and err < EXPECT, err


def test_prefill_sized_batch_q8_0(dev, oracle):
    rows, cols, n, t = 4096, 4096, 512, GGMLType.Q8_0
    w = jl.synth_tensor(t, rows * cols, seed=17)
    x = np.random.default_rng(5).standard_normal((n, cols)).astype(np.float32)
    got = dev.matmul(t, w, rows, cols, x)
    sample = [0, 1, 127, 128, 255, 300, 511]
    want = oracle.matmul(t, w, x[sample], rows, cols)
    assert rel_l2(got[sample], want) < EXPECT
    # linearity at full size: W(a + b) = W a + W b up to the operand rounding
    y2 = dev.matmul(t, w, rows, cols, x[:64] + x[64:128])
    assert rel_l2(y2, got[:64] + got[64:128]) < BAR


def test_wide_activations_do_not_overflow_fp16(dev, oracle):
    rows, cols, n, t = 256, 1024, 16, GGMLType.Q4_K
    w = jl.synth_tensor(t, rows * cols, seed=19)
    x = (np.random.default_rng(6).standard_normal((n, cols)) * 300.0).astype(np.float32)
    got, want = dev.matmul(t, w, rows, cols, x), oracle.matmul(t, w, x, rows, cols)
    assert rel_l2(got, want) < EXPECT


def test_tall_product_goes_in_token_slabs(dev, oracle):
    """More output tiles than arrival counters (1002 row tiles x 18 token tiles): the launch is cut into
    token slabs; sampled rows against the oracle and two slabs' boundary rows included."""
    rows, cols, n, t = 128256, 256, 1100, GGMLType.Q4_0
    w = jl.synth_tensor(t, rows * cols, seed=23)
    x = np.random.default_rng(7).standard_normal((n, cols)).astype(np.float32)
    got = dev.matmul(t, w, rows, cols, x)
    assert got.shape == (n, rows)
    sample = [0, 63, 64, 1023, 1024, 1025, 1099]
    want = oracle.matmul(t, w, x[sample], rows, cols)
    assert rel_l2(got[sample], want) < EXPECT


@pytest.mark.parametrize("t", FORMATS)
def test_widest_sweep_batch(dev, oracle, t):
    """N = 2048, the widest batch of the standalone sweep, on the 14336 x 4096 shape: sampled token
    rows against the oracle (the full product is 120 G multiply-adds on the CPU), rows on either side
    of token-tile boundaries among them."""
    rows, cols, n = 14336, 4096, 2048
    w = jl.synth_tensor(t, rows * cols, seed=29 + int(t))
    x = np.random.default_rng(8).standard_normal((n, cols)).astype(np.float32)
    got = dev.matmul(t, w, rows, cols, x)
    assert got.shape == (n, rows)
    sample = [0, 127, 128, 1023, 1024, 1900, 2047]
    want = oracle.matmul(t, w, x[sample], rows, cols)
    err = rel_l2(got[sample], want)
    assert err < BAR and err < EXPECT, err
    assert np.all(np.isfinite(got))

"""The allocation-free entry point (jl_gemv_argmax_static) against the ordinary device-resident
matrix-vector entry point (jl_gemv_dev), through the C ABI, twice in a row.

Some callers of this library cannot allocate device memory at call time: a serving loop that
carved up its memory once at start-up, code inside a CUDA stream capture, a host that lends the
library buffers from its own pool. For them the kernel's cross-CTA scratch lives in a static
array inside the library; this test checks that the variant gives the same numbers as the
existing path, that the array's left-over contents from one call do not disturb the next, and
that sizes beyond the stated maximum are refused.

Collected last on purpose (file name), so a run that stops at the first failure has already run
every other test. It must also pass alone in a fresh process."""
import ctypes as C

import numpy as np
import pytest

import jitllm_b200 as jl
from jitllm_b200 import GGMLType

pytestmark = pytest.mark.gpu


def _run_static(dev, t, rows, cols, w_dev, x_dev, y_dev, tok_dev, norm_dev=None, eps=0.0):
    lib = dev._lib
    rc = lib.jl_gemv_argmax_static(int(t), rows, cols, C.c_void_p(w_dev), C.c_void_p(x_dev),
                                   C.c_void_p(norm_dev) if norm_dev else None, C.c_float(eps),
                                   C.c_void_p(y_dev), C.c_void_p(tok_dev), lib.jl_stream(dev.handle))
    return rc, lib.jl_static_last_error().decode()


@pytest.mark.parametrize("t", [GGMLType.Q4_K, GGMLType.Q8_0])
def test_static_scratch_variant_matches_the_allocating_entry_point(dev, t):
    rows, cols = 3000, 2048
    w = jl.synth_tensor(t, rows * cols, seed=123)
    mat = dev.upload_matrix(t, w, rows, cols)          # existing entry point's weight handle
    w_dev = dev.alloc(w.nbytes)                        # the caller's own buffer for the new one
    dev.h2d(w_dev, w)
    x_dev, y_ref_dev, y_dev, tok_dev = dev.alloc(cols * 4), dev.alloc(rows * 4), dev.alloc(rows * 4), dev.alloc(4)
    rng = np.random.default_rng(5)
    try:
        for call in range(2):                          # two calls in a row share the static array
            x = rng.standard_normal(cols).astype(np.float32)
            dev.h2d(x_dev, x)
            mat.matmul_dev(x_dev, 1, y_ref_dev)
            rc, msg = _run_static(dev, t, rows, cols, w_dev, x_dev, y_dev, tok_dev)
            assert rc == 0, msg
            dev.synchronize()
            y_ref, y, tok = np.empty(rows, np.float32), np.empty(rows, np.float32), np.empty(1, np.int32)
            dev.d2h(y_ref, y_ref_dev)
            dev.d2h(y, y_dev)
            dev.d2h(tok, tok_dev)
            assert np.array_equal(y, y_ref), f"call {call}: outputs differ"   # same kernel, same bits
            assert int(tok[0]) == int(np.argmax(y_ref)), f"call {call}: arg-max differs"
    finally:
        for p in (w_dev, x_dev, y_ref_dev, y_dev, tok_dev):
            dev.free(p)
        mat.close()


def test_static_variant_rejects_what_it_cannot_hold(dev):
    buf = dev.alloc(1 << 16)
    try:
        rc, msg = _run_static(dev, GGMLType.Q4_K, 8, 256 * 1024, buf, buf, buf, buf)   # needs > one SM of shared memory
        assert rc != 0 and "unsupported" in msg
        rc, msg = _run_static(dev, GGMLType.Q4_K, 8, 100, buf, buf, buf, buf)
        assert rc != 0 and "multiple of 256" in msg
        rc, msg = _run_static(dev, 1, 8, 256, buf, buf, buf, buf)
        assert rc != 0 and "GGML type" in msg
    finally:
        dev.free(buf)

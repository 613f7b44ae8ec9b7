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


@pytest.mark.parametrize("t", [GGMLType.Q4_K, GGMLType.Q8_0, GGMLType.Q4_0])
def test_static_scratch_variant_matches_the_allocating_entry_point(dev, oracle, t):
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
            assert dev._lib.jl_static_status(dev._lib.jl_stream(dev.handle)) == 0   # no wait ran out
            y_ref, y, tok = np.empty(rows, np.float32), np.empty(rows, np.float32), np.empty(1, np.int32)
            dev.d2h(y_ref, y_ref_dev)
            dev.d2h(y, y_dev)
            dev.d2h(tok, tok_dev)
            assert np.array_equal(y, y_ref), f"call {call}: outputs differ"   # same kernel, same bits
            assert int(tok[0]) == int(np.argmax(y_ref)), f"call {call}: arg-max differs"
            want = oracle.matmul(t, w, x, rows, cols)  # and the oracle agrees, at the mat-vec tolerance
            assert np.linalg.norm(y - want) / np.linalg.norm(want) < 1e-4
    finally:
        for p in (w_dev, x_dev, y_ref_dev, y_dev, tok_dev):
            dev.free(p)
        mat.close()


def test_static_variant_with_the_rmsnorm_folded_in(dev, oracle):
    """norm_w_dev / rms_eps: the input is RMS-normalised first, as the vocabulary projection of a
    decode step does; checked against the oracle's rmsNorm + matmul on two calls in a row."""
    t, rows, cols, eps = GGMLType.Q4_K, 1500, 1024, 1e-5
    w = jl.synth_tensor(t, rows * cols, seed=321)
    w_dev, x_dev, g_dev, y_dev, tok_dev = (dev.alloc(w.nbytes), dev.alloc(cols * 4), dev.alloc(cols * 4),
                                           dev.alloc(rows * 4), dev.alloc(4))
    dev.h2d(w_dev, w)
    rng = np.random.default_rng(7)
    try:
        for call in range(2):
            x = (3.0 * rng.standard_normal(cols)).astype(np.float32)
            g = (1.0 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
            dev.h2d(x_dev, x)
            dev.h2d(g_dev, g)
            rc, msg = _run_static(dev, t, rows, cols, w_dev, x_dev, y_dev, tok_dev, norm_dev=g_dev, eps=eps)
            assert rc == 0, msg
            assert dev._lib.jl_static_status(dev._lib.jl_stream(dev.handle)) == 0
            y, tok = np.empty(rows, np.float32), np.empty(1, np.int32)
            dev.d2h(y, y_dev)
            dev.d2h(tok, tok_dev)
            want = oracle.matmul(t, w, oracle.rmsnorm(x, g, eps), rows, cols)
            assert np.linalg.norm(y - want) / np.linalg.norm(want) < 1e-4, f"call {call}"
            assert int(tok[0]) == int(np.argmax(y)), f"call {call}: arg-max differs"
    finally:
        for p in (w_dev, x_dev, g_dev, y_dev, tok_dev):
            dev.free(p)


def test_static_variant_rejects_what_it_cannot_hold(dev):
    buf = dev.alloc(1 << 16)
    try:
        rc, msg = _run_static(dev, GGMLType.Q4_K, 8, 256 * 1024, buf, buf, buf, buf)   # more columns than a CTA stages
        assert rc != 0 and "unsupported" in msg
        rc, msg = _run_static(dev, GGMLType.Q4_K, 8, 100, buf, buf, buf, buf)
        assert rc != 0 and "multiple of 256" in msg
        rc, msg = _run_static(dev, 1, 8, 256, buf, buf, buf, buf)
        assert rc != 0 and "GGML type" in msg
        # Misaligned pointers are refused on the host, before anything is launched.
        rc, msg = _run_static(dev, GGMLType.Q4_K, 8, 256, buf + 4, buf, buf, buf)
        assert rc != 0 and "16-byte aligned" in msg
        rc, msg = _run_static(dev, GGMLType.Q4_K, 8, 256, buf, buf + 8, buf, buf)
        assert rc != 0 and "16-byte aligned" in msg
        rc, msg = _run_static(dev, GGMLType.Q4_K, 8, 256, buf, buf, buf, buf, norm_dev=buf + 4, eps=1e-5)
        assert rc != 0 and "16-byte aligned" in msg
        rc, msg = _run_static(dev, GGMLType.Q4_K, 8, 256, buf, buf, buf + 2, buf)
        assert rc != 0 and "4-byte aligned" in msg
    finally:
        dev.free(buf)


def test_device_resident_entry_point_refuses_misaligned_vectors(dev):
    t, rows, cols = GGMLType.Q8_0, 16, 256
    mat = dev.upload_matrix(t, jl.synth_tensor(t, rows * cols, seed=1), rows, cols)
    buf = dev.alloc(1 << 14)
    try:
        with pytest.raises(ValueError, match="16-byte aligned"):
            mat.matmul_dev(buf + 4, 1, buf + 4096)
        with pytest.raises(ValueError, match="16-byte aligned"):
            mat.matmul_dev(buf, 1, buf + 4096 + 8)
    finally:
        dev.free(buf)
        mat.close()

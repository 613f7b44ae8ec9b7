"""Host-side mirror of the reference interfaces: argument checks and the synthetic encoders."""
import numpy as np
import pytest

import jitllm_b200 as jl
from jitllm_b200 import GGMLType


def test_batch_slots_is_fixed_width():
    b = jl.BatchSlots([True, False, True], [1, 2, 3], [0, 0, 5], [0, 1, 2])
    assert b.width() == 3 and b.activeCount() == 2
    with pytest.raises(ValueError, match="a batch is fixed width"):
        jl.BatchSlots([True], [1, 2], [0], [0])


def test_kv_storage_request_rejects_non_positive_dimensions():
    jl.KvStorageRequest(8, 4, 2, 16, 2, 128)
    with pytest.raises(ValueError, match="every key/value pool dimension must be positive"):
        jl.KvStorageRequest(0, 4, 2, 16, 2, 128)


def test_ggml_geometry():
    assert (GGMLType.Q8_0.block_size, GGMLType.Q8_0.type_size) == (32, 34)
    assert (GGMLType.Q4_0.block_size, GGMLType.Q4_0.type_size) == (32, 18)
    assert (GGMLType.Q4_K.block_size, GGMLType.Q4_K.type_size) == (256, 144)
    assert GGMLType.Q4_K.byte_size_for(4096 * 4096) == 9437184


def test_configuration_shapes():
    c = jl.Configuration(4096, 14336, 32, 32, 8, 128256, 4096)
    assert c.headSize == 128 and c.kvDim == 1024
    assert c.matrix_shape(jl.TensorRole.ATTENTION_KEY) == (1024, 4096)
    assert c.matrix_shape(jl.TensorRole.FFN_DOWN) == (4096, 14336)


@pytest.mark.parametrize("t,tol", [(GGMLType.Q8_0, 0.008), (GGMLType.Q4_0, 0.11), (GGMLType.Q4_K, 0.10)])
def test_encoders_round_trip_through_the_oracle_decoder(built, oracle, t, tol):
    n = 256 * 64
    x = (np.random.default_rng(5).standard_normal(n) * 0.02).astype(np.float32)
    raw = jl.quantize(t, x)
    assert raw.size == t.byte_size_for(n)
    back = oracle.dequant(t, raw, n)
    assert np.linalg.norm(back - x) / np.linalg.norm(x) < tol


def test_synthetic_tensors_are_seeded_normal_and_reproducible(built, oracle):
    a = jl.synth_tensor(GGMLType.Q8_0, 256 * 256, seed=7)
    b = jl.synth_tensor(GGMLType.Q8_0, 256 * 256, seed=7, threads=1)
    c = jl.synth_tensor(GGMLType.Q8_0, 256 * 256, seed=8)
    assert np.array_equal(a, b) and not np.array_equal(a, c)
    v = oracle.dequant(GGMLType.Q8_0, a, 256 * 256)
    assert abs(float(v.mean())) < 5e-4 and abs(float(v.std()) - 0.02) < 5e-4
    with pytest.raises(ValueError):
        jl.synth_tensor(GGMLType.Q4_K, 100, seed=1)


def test_rope_tables_match_the_oracle_tables(built, oracle):
    cr, ci = jl.precomputeFreqsCis(64, 128, 500000.0)
    ocr = np.empty_like(cr)
    oci = np.empty_like(ci)
    oracle.lib().orc_rope_tables(64, 128, 500000.0, ocr.ctypes.data, oci.ctypes.data)
    # double cos/sin may differ in the last bit between libm and numpy: tables agree to 1 ulp
    assert np.max(np.abs(cr - ocr)) <= 2 ** -23 and np.max(np.abs(ci - oci)) <= 2 ** -23

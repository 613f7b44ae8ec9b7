"""A synthetic GGUF file written to disk, loaded by the native reader and decoded on the GPU, against
the oracle fed the same tensors: the file path gives the same logits as the in-memory upload path."""
import numpy as np
import pytest

import jitllm_b200 as jl

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fmt,tied", [(jl.GGMLType.Q4_K, False), (jl.GGMLType.Q8_0, True)])
def test_gguf_file_decodes_like_the_oracle(dev, oracle, tmp_path, fmt, tied):
    cfg = jl.Configuration(dim=256, hiddenDim=512, numberOfLayers=2, numberOfHeads=4, numberOfKeyValueHeads=2,
                           vocabularySize=1024, contextLength=64, tiedEmbeddings=tied)
    tensors = jl.synth_model_tensors(cfg, fmt, seed=77, std=0.05)
    path = tmp_path / "model.gguf"
    jl.write_gguf(path, cfg, tensors)
    om = oracle.Model(cfg, tensors)
    cr, ci = om.rope_tables()
    model = jl.load_model_gguf(dev, path, maxBatch=1, rope_cos=cr, rope_sin=ci)
    import dataclasses
    assert dataclasses.replace(model.config, rmsNormEps=cfg.rmsNormEps) == cfg  # eps is stored as binary32
    kv = model.createKvStorage(jl.KvStorageRequest(4, 4, 1, 16, cfg.numberOfLayers, cfg.kvDim))
    kv.publishBlockTable(np.arange(4, dtype=np.int32))
    boundary = jl.B200InvocationBoundary(model)
    for pos, tok in enumerate(np.random.default_rng(1).integers(0, cfg.vocabularySize, size=10)):
        want = om.forward(int(tok), pos)
        got = boundary.invoke(int(tok), pos)
        assert float(np.max(np.abs(got.logits - want))) < 2e-3
        assert got.sampledToken == int(np.argmax(want))
    kv.close()


def test_native_rope_tables_match_the_host_formula(dev, oracle, tmp_path):
    cfg = jl.Configuration(dim=256, hiddenDim=512, numberOfLayers=1, numberOfHeads=4, numberOfKeyValueHeads=2,
                           vocabularySize=512, contextLength=32)
    tensors = jl.synth_model_tensors(cfg, jl.GGMLType.Q4_0, seed=78, std=0.05)
    path = tmp_path / "rope.gguf"
    jl.write_gguf(path, cfg, tensors)
    om = oracle.Model(cfg, tensors)
    model = jl.load_model_gguf(dev, path)  # tables computed by the reader
    kv = model.createKvStorage(jl.KvStorageRequest(2, 2, 1, 16, cfg.numberOfLayers, cfg.kvDim))
    kv.publishBlockTable(np.arange(2, dtype=np.int32))
    boundary = jl.B200InvocationBoundary(model)
    for pos, tok in enumerate([3, 99, 410, 7]):
        want = om.forward(tok, pos)
        got = boundary.invoke(tok, pos)
        assert float(np.max(np.abs(got.logits - want))) < 2e-3
    kv.close()


def test_mixed_precision_file_loads_and_decodes(dev, oracle, tmp_path):
    """A file whose value / down / output matrices are Q6_K, Q5_K or Q4_1 (as mixed-precision files are) through
    the native reader: the same logits as the oracle fed the same tensors."""
    from tests.test_gpu_mixed_formats import _mixed
    cfg = jl.Configuration(dim=256, hiddenDim=512, numberOfLayers=3, numberOfHeads=4, numberOfKeyValueHeads=2,
                           vocabularySize=1024, contextLength=64)
    tensors = jl.synth_model_tensors(cfg, jl.GGMLType.Q4_K, seed=79, std=0.05)
    tensors.update(_mixed(cfg, 900))
    path = tmp_path / "mixed.gguf"
    jl.write_gguf(path, cfg, tensors)
    om = oracle.Model(cfg, tensors)
    cr, ci = om.rope_tables()
    model = jl.load_model_gguf(dev, path, maxBatch=1, rope_cos=cr, rope_sin=ci)
    kv = model.createKvStorage(jl.KvStorageRequest(4, 4, 1, 16, cfg.numberOfLayers, cfg.kvDim))
    kv.publishBlockTable(np.arange(4, dtype=np.int32))
    boundary = jl.B200InvocationBoundary(model)
    for pos, tok in enumerate(np.random.default_rng(2).integers(0, cfg.vocabularySize, size=10)):
        want = om.forward(int(tok), pos)
        got = boundary.invoke(int(tok), pos)
        assert float(np.max(np.abs(got.logits - want))) < 6e-3
        assert got.sampledToken == int(np.argmax(want))
    kv.close()

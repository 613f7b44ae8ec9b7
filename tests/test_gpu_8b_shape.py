"""The headline shape, compared and not only timed: two layers with the Llama-3-8B layer geometry
(dim 4096, FFN 14336, 32 query / 8 KV heads of 128, full 128256-row vocabulary), Q4_K, a few
teacher-forced steps against the oracle -- the same bounds the reference applies between its CPU
and GPU paths (src/test/java/org/beehive/jitllm/golden/CpuGpuParity.java:60-82): logits within
1e-2, the greedy token identical."""
import numpy as np
import pytest

import jitllm_b200 as jl
from jitllm_b200 import GGMLType

pytestmark = pytest.mark.gpu


def test_two_layers_of_the_8b_geometry_match_the_oracle(dev, oracle):
    cfg = jl.Configuration(dim=4096, hiddenDim=14336, numberOfLayers=2, numberOfHeads=32, numberOfKeyValueHeads=8,
                           vocabularySize=128256, contextLength=256)
    tensors = jl.synth_model_tensors(cfg, GGMLType.Q4_K, seed=11)
    om = oracle.Model(cfg, tensors)
    cr, ci = om.rope_tables()
    model = jl.load_model(dev, cfg, tensors, cr, ci)
    kv = model.createKvStorage(jl.KvStorageRequest(16, 16, 1, 16, cfg.numberOfLayers, cfg.kvDim))
    kv.publishBlockTable(np.arange(16, dtype=np.int32))
    kv.fill(0x7E00)
    bound = jl.B200InvocationBoundary(model)
    toks = np.random.default_rng(6).integers(0, cfg.vocabularySize, size=5)
    for pos, tok in enumerate(toks):
        want = om.forward(int(tok), pos)
        got = bound.invoke(int(tok), pos)
        assert np.all(np.isfinite(got.logits))
        err = float(np.max(np.abs(got.logits - want)))
        assert err < 1e-2, (pos, err)
        top2 = np.sort(want)[-2:]
        if top2[1] - top2[0] > 2e-2:
            assert got.sampledToken == int(np.argmax(want)), pos
        assert got.sampledToken == int(np.argmax(got.logits))
    kv.close()

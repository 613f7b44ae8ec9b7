"""The oracle's forwardJava against an independent numpy statement, on the synthetic model recipe
of the reference's LlamaCpuOperationEquivalenceTest (dim 64, hidden 128, 4 layers, 4 heads over
2 KV heads, vocab 48, context 32, weights (nextFloat - 0.5) * 0.5 from java.util.Random in the
constructor order of LlamaStandardWeights, rope tables random too). Bit-identical logits and
caches are demanded, as that test demands of the reference's two statements."""
import numpy as np
import pytest

from tests.javarand import JavaRandom
from tests.np_forward import NpLlama

DIM, HIDDEN, LAYERS, HEADS, KV_HEADS, VOCAB, CONTEXT, EPS = 64, 128, 4, 4, 2, 48, 32, 1e-5
KV_DIM, HEAD = DIM * KV_HEADS // HEADS, DIM // HEADS


def _tensor(rnd, n):
    return np.array([(rnd.next_float() - np.float32(0.5)) * np.float32(0.5) for _ in range(n)], dtype=np.float32)


def _weights(seed):
    r = JavaRandom(seed)
    many = lambda n: [_tensor(r, n) for _ in range(LAYERS)]
    w = {}
    w["emb"] = _tensor(r, VOCAB * DIM)
    w["att_norm"] = many(DIM)
    w["wq"] = many(DIM * DIM)
    w["wk"] = many(KV_DIM * DIM)
    w["wv"] = many(KV_DIM * DIM)
    w["wo"] = many(DIM * DIM)
    w["ffn_norm"] = many(DIM)
    w["w1"] = many(HIDDEN * DIM)
    w["w2"] = many(DIM * HIDDEN)
    w["w3"] = many(HIDDEN * DIM)
    w["final_norm"] = _tensor(r, DIM)
    w["cr"] = _tensor(r, CONTEXT * (HEAD // 2))
    w["ci"] = _tensor(r, CONTEXT * (HEAD // 2))
    w["wcls"] = _tensor(r, VOCAB * DIM)
    return w


class _Cfg:
    dim, hiddenDim, numberOfLayers, numberOfHeads, numberOfKeyValueHeads = DIM, HIDDEN, LAYERS, HEADS, KV_HEADS
    vocabularySize, contextLength, rmsNormEps, ropeTheta = VOCAB, CONTEXT, EPS, 10000.0
    headSize, kvDim = HEAD, KV_DIM


def _oracle_model(oracle, w):
    F32 = 0
    t = {(0, -1): (F32, w["emb"]), (10, -1): (F32, w["final_norm"]), (11, -1): (F32, w["wcls"])}
    for l in range(LAYERS):
        for role, key in ((1, "att_norm"), (2, "wq"), (3, "wk"), (4, "wv"), (5, "wo"), (6, "ffn_norm"),
                          (7, "w1"), (8, "w3"), (9, "w2")):
            t[(role, l)] = (F32, w[key][l])
    m = oracle.Model(_Cfg, t)
    m.set_rope_tables(w["cr"], w["ci"])
    return m


def _np_model(w):
    cfg = dict(dim=DIM, hidden=HIDDEN, layers=LAYERS, heads=HEADS, kv_heads=KV_HEADS, vocab=VOCAB, ctx=CONTEXT,
               eps=EPS, head=HEAD, kv_dim=KV_DIM)
    return NpLlama(cfg, w)


def test_forward_pass_is_bit_identical_to_the_independent_statement(oracle):
    w = _weights(20260831)
    a, b = _oracle_model(oracle, w), _np_model(w)
    for pos, tok in enumerate([7, 3, 41, 0, 19, 5, 33, 12]):
        la, lb = a.forward(tok, pos), b.forward(tok, pos)
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32)), f"logits differ at position {pos}"


def test_key_value_caches_agree(oracle):
    w = _weights(4242)
    a, b = _oracle_model(oracle, w), _np_model(w)
    toks = [2, 30, 11, 8, 25]
    for pos, tok in enumerate(toks):
        a.forward(tok, pos)
        b.forward(tok, pos)
    for l in range(LAYERS):
        for pos in range(len(toks)):
            assert np.array_equal(a.kcache(l, pos), b.kc[l, pos].view(np.uint16))
            assert np.array_equal(a.vcache(l, pos), b.vc[l, pos].view(np.uint16))


def test_synthetic_model_produces_real_output(oracle):
    w = _weights(1)
    logits = _oracle_model(oracle, w).forward(5, 0)
    assert np.all(np.isfinite(logits)) and np.any(logits != logits[0])


@pytest.mark.parametrize("bits", [0, 128, 256])
def test_vector_modes_agree_within_rounding(oracle, bits):
    """Q8_0/Q4_0 dots in the scalar, 128-bit and 256-bit summation orders differ only by
    rounding; Q4_K always takes the scalar path (Q4_KFloatTensor.java:125-127)."""
    import jitllm_b200 as jl
    L = oracle.lib()
    rows, cols = 8, 1024
    x = np.random.default_rng(3).standard_normal(cols).astype(np.float32)
    try:
        for t in (jl.GGMLType.Q8_0, jl.GGMLType.Q4_0, jl.GGMLType.Q4_K):
            wq = jl.synth_tensor(t, rows * cols, seed=11)
            L.orc_set_vector_bits(0)
            base = oracle.matmul(t, wq, x, rows, cols)
            L.orc_set_vector_bits(bits)
            got = oracle.matmul(t, wq, x, rows, cols)
            if t == jl.GGMLType.Q4_K or bits == 0:
                assert np.array_equal(base, got)
            else:
                assert np.linalg.norm(base - got) / np.linalg.norm(base) < 1e-6
    finally:
        L.orc_set_vector_bits(0)

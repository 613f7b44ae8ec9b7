"""Device-side temperature / top-p sampling (jl_sample) against the oracle's restatement of the reference's
sampler chain, through the C ABI: the same logits (a real decode step's), the same random number.

Tolerance, stated: the reference adds its cumulative distribution sequentially in fp32 (128 256 additions at the
full vocabulary leave a rounding error around 1e-5, more than the width of one token of a flat distribution),
the device adds exactly (fixed point). So the tokens are required to be identical where the oracle reports the
random number at least 1e-5 away from every boundary, and otherwise the device's token must be the one whose
interval of the cumulative distribution computed in float64 contains the scaled random number to within 3e-5
of the sampled mass. Small vocabularies must agree exactly."""
import ctypes as C

import numpy as np
import pytest

import jitllm_b200 as jl
from jitllm_b200 import GGMLType

pytestmark = pytest.mark.gpu


def _model(dev, vocab, width, std=0.05, seed=3):
    cfg = jl.Configuration(dim=256, hiddenDim=512, numberOfLayers=1, numberOfHeads=4, numberOfKeyValueHeads=2,
                           vocabularySize=vocab, contextLength=64)
    tensors = jl.synth_model_tensors(cfg, GGMLType.Q8_0, seed=seed, std=std)
    cr, ci = jl.precomputeFreqsCis(cfg.contextLength, cfg.headSize, cfg.ropeTheta)
    model = jl.load_model(dev, cfg, tensors, cr, ci, maxBatch=width)
    kv = model.createKvStorage(jl.KvStorageRequest(4 * width, 4, width, 16, cfg.numberOfLayers, cfg.kvDim))
    kv.publishBlockTable(np.arange(4 * width, dtype=np.int32))
    return cfg, model, kv


def _within_float64_interval(logits, temperature, topp, u, got, eps=3e-5):
    """Is `got` the token a float64 evaluation of the chain picks, give or take eps of the sampled mass?"""
    s = (logits.astype(np.float32) / np.float32(temperature)).astype(np.float32)
    e = np.exp((s - s.max()).astype(np.float64)).astype(np.float32).astype(np.float64)
    p = e / e.sum()
    n = p.size
    if topp <= 0 or topp >= 1:
        cdf = np.cumsum(p)
        lo = cdf[got - 1] if got > 0 else 0.0
        return lo - eps <= u <= cdf[got] + eps
    cutoff = (1.0 - topp) / (n - 1)
    order = np.lexsort((np.arange(n), -p))          # largest first, ties by index
    order = order[p[order] >= cutoff * (1 - 1e-6)]
    cum = np.cumsum(p[order])
    last = int(np.searchsorted(cum, topp, side="right"))
    last = min(last, len(order) - 1)
    where = np.nonzero(order == got)[0]
    if len(where) == 0 or where[0] > last + 1:      # one past the end: the nucleus boundary itself is within rounding
        return False
    k = int(where[0])
    for mass in (cum[last], cum[min(last + 1, len(cum) - 1)], cum[max(last - 1, 0)]):
        r = u * mass
        lo = cum[k - 1] if k > 0 else 0.0
        if lo - eps * mass <= r <= cum[k] + eps * mass:
            return True
    return False



def _step_and_sample(dev, model, width, tokens, temperature, topp, u, active=None):
    ex = jl.B200BatchExecutor(model)
    act = [True] * width if active is None else active
    _, logits = ex.decodeStep(jl.BatchSlots(act, tokens, [0] * width, list(range(width))), wantLogits=True)
    # the same step again (same inputs, same position): its logits stay on the device for jl_sample
    ex.decodeStep(jl.BatchSlots(act, tokens, [0] * width, list(range(width))))
    out = np.empty(width, dtype=np.int32)
    uu = np.ascontiguousarray(u, dtype=np.float32)
    dev._check(dev._lib.jl_sample(dev.handle, width, C.c_float(temperature), C.c_float(topp), uu.ctypes.data, out.ctypes.data))
    return logits, out


@pytest.mark.parametrize("vocab", [1000, 128256])
@pytest.mark.parametrize("topp", [0.0, 0.9, 0.5])
def test_tokens_match_the_reference_chain(dev, oracle, vocab, topp):
    width = 8
    cfg, model, kv = _model(dev, vocab, width, std=0.3)
    rng = np.random.default_rng(vocab + int(topp * 10))
    mismatches = total = 0
    for rounds in range(3):
        tokens = [int(v) for v in rng.integers(0, vocab, size=width)]
        u = [np.float32(int(rng.random() * (1 << 24)) / (1 << 24)) for _ in range(width)]
        temperature = float(rng.choice([0.7, 1.0, 1.5]))
        logits, got = _step_and_sample(dev, model, width, tokens, temperature, topp, u)
        for b in range(width):
            want, margin = oracle.sample(logits[b], temperature, topp, float(u[b]))
            total += 1
            if int(got[b]) != want:
                mismatches += 1
                assert margin < 1e-5, (b, int(got[b]), want, margin)
                assert _within_float64_interval(logits[b], temperature, topp, float(u[b]), int(got[b])), (b, int(got[b]), want)
    if vocab == 1000:
        assert mismatches == 0, f"{mismatches} of {total}"
    kv.close()


def test_peaked_rows_ties_and_inactive_rows(dev, oracle):
    """Rows of logits written by hand into the device buffer are not possible through the ABI, so the peaked
    case comes from a low temperature (T = 0.05 makes one token carry nearly all the mass: the nucleus is one
    element), and inactive rows must come back as -1 whatever their random number."""
    width, vocab = 4, 5000
    cfg, model, kv = _model(dev, vocab, width, std=0.3)
    tokens = [5, 6, 7, 8]
    u = [np.float32(0.999), np.float32(0.5), np.float32(0.0), np.float32(0.25)]
    logits, got = _step_and_sample(dev, model, width, tokens, 0.05, 0.9, u, active=[True, False, True, True])
    assert got[1] == -1
    for b in (0, 2, 3):
        want, margin = oracle.sample(logits[b], 0.05, 0.9, float(u[b]))
        assert int(got[b]) == want, (b, int(got[b]), want, margin)
    kv.close()


def test_refusals(dev):
    width = 2
    cfg, model, kv = _model(dev, 1000, width)
    out = np.empty(width, dtype=np.int32)
    u = np.array([0.5, 0.5], dtype=np.float32)
    lib = dev._lib
    # no decode before it
    rc = lib.jl_sample(dev.handle, width, C.c_float(1.0), C.c_float(0.9), u.ctypes.data, out.ctypes.data)
    assert rc != 0 and b"must follow a jl_decode" in lib.jl_last_error(dev.handle)
    ex = jl.B200BatchExecutor(model)
    ex.decodeStep(jl.BatchSlots([True, True], [1, 2], [0, 0], [0, 1]))
    rc = lib.jl_sample(dev.handle, width, C.c_float(0.0), C.c_float(0.9), u.ctypes.data, out.ctypes.data)
    assert rc != 0 and b"temperature must be positive" in lib.jl_last_error(dev.handle)
    bad = np.array([0.5, 1.0], dtype=np.float32)
    rc = lib.jl_sample(dev.handle, width, C.c_float(1.0), C.c_float(0.9), bad.ctypes.data, out.ctypes.data)
    assert rc != 0 and b"outside [0, 1)" in lib.jl_last_error(dev.handle)
    rc = lib.jl_sample(dev.handle, width, C.c_float(1.0), C.c_float(0.9), u.ctypes.data, out.ctypes.data)
    assert rc == 0
    # the rows were consumed: a second draw needs a new step
    rc = lib.jl_sample(dev.handle, width, C.c_float(1.0), C.c_float(0.9), u.ctypes.data, out.ctypes.data)
    assert rc != 0
    kv.close()


def test_sampler_object_through_the_executor(dev, oracle):
    width, vocab = 3, 2000
    cfg, model, kv = _model(dev, vocab, width, std=0.3)
    ex = jl.B200BatchExecutor(model)
    sampler = jl.Sampler.selectSampler(vocab, 0.8, 0.95, rngSeed=11)
    twin = jl.Sampler.selectSampler(vocab, 0.8, 0.95, rngSeed=11)   # the same stream of random numbers
    slots = jl.BatchSlots([True] * width, [3, 4, 5], [0] * width, list(range(width)))
    _, logits = ex.decodeStep(slots, wantLogits=True)
    got = ex.decodeStep(slots, sampler=sampler)
    for b in range(width):
        want, margin = oracle.sample(logits[b], 0.8, 0.95, float(twin.nextFloat()))
        assert int(got[b]) == want or margin < 1e-5
    assert jl.Sampler.selectSampler(vocab, 0.0, 0.95, rngSeed=1).greedy
    kv.close()

"""The oracle's sampler chain (inference/sampler/Sampler.java:63-110 restated in C) on cases small enough to
work out by hand, and against a direct numpy transcription of ToppSampler / CategoricalSampler on random rows.
The reference ships no test vectors for its samplers: these are the pins this path has."""
import numpy as np
import pytest

from oracle import binding as oracle


def _numpy_chain(logits, temperature, topp, u):
    """Straight transcription: divide, softmax (float32, sequential sum), then the two samplers."""
    s = (logits.astype(np.float32) / np.float32(temperature)).astype(np.float32)
    e = np.exp((s - s.max()).astype(np.float64)).astype(np.float32)
    total = np.float32(0)
    for v in e:
        total = np.float32(total + v)
    p = (e / total).astype(np.float32)
    n = p.size
    if topp <= 0 or topp >= 1:
        cdf = np.float32(0)
        for i in range(n):
            cdf = np.float32(cdf + p[i])
            if np.float32(u) < cdf:
                return i
        return n - 1
    cutoff = np.float32((np.float32(1.0) - np.float32(topp)) / np.float32(n - 1))
    cand = [i for i in range(n) if p[i] >= cutoff]
    cand.sort(key=lambda i: (-p[i], i))
    cum, last = np.float32(0), len(cand) - 1
    for k, i in enumerate(cand):
        cum = np.float32(cum + p[i])
        if cum > np.float32(topp):
            last = k
            break
    r = np.float32(np.float32(u) * cum)
    cdf = np.float32(0)
    for k in range(last + 1):
        cdf = np.float32(cdf + p[cand[k]])
        if r < cdf:
            return cand[k]
    return cand[last]


def test_hand_worked_categorical():
    logits = np.log(np.array([0.5, 0.3, 0.15, 0.05], dtype=np.float32))
    for u, want in ((0.0, 0), (0.49, 0), (0.51, 1), (0.79, 1), (0.81, 2), (0.96, 3)):
        assert oracle.sample(logits, 1.0, 0.0, u)[0] == want
        assert oracle.sample(logits, 1.0, 1.0, u)[0] == want   # topp >= 1 also means categorical


def test_hand_worked_nucleus():
    logits = np.log(np.array([0.5, 0.3, 0.15, 0.05], dtype=np.float32))
    # topp 0.7: 0.5 alone does not exceed it, 0.5 + 0.3 does: nucleus {0, 1}, mass 0.8, r = 0.8 u
    for u, want in ((0.0, 0), (0.6, 0), (0.63, 1), (0.99, 1)):
        assert oracle.sample(logits, 1.0, 0.7, u)[0] == want
    # topp 0.4: the largest alone exceeds it
    for u in (0.0, 0.5, 0.99):
        assert oracle.sample(logits, 1.0, 0.4, u)[0] == 0
    # a low temperature sharpens: at T = 0.25 the first token holds 0.5^4 / (sum of 4th powers) = 0.877
    assert oracle.sample(logits, 0.25, 0.0, 0.87)[0] == 0
    assert oracle.sample(logits, 0.25, 0.0, 0.88)[0] == 1


def test_temperature_zero_is_first_argmax():
    logits = np.array([1.0, 3.0, 3.0, -2.0], dtype=np.float32)
    assert oracle.sample(logits, 0.0, 0.9, 0.5)[0] == 1


@pytest.mark.parametrize("topp", [0.0, 0.5, 0.9, 0.95])
def test_against_numpy_transcription(topp):
    rng = np.random.default_rng(int(topp * 100) + 3)
    for case in range(40):
        n = int(rng.integers(2, 400))
        logits = (rng.standard_normal(n) * rng.choice([0.5, 2.0, 6.0])).astype(np.float32)
        t = float(rng.choice([0.5, 0.8, 1.0, 1.3]))
        u = float(np.float32(int(rng.random() * (1 << 24)) / (1 << 24)))
        assert oracle.sample(logits, t, topp, u)[0] == _numpy_chain(logits, t, topp, u), (case, n, t, u)

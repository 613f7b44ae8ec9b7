"""Attention at the key counts the benchmark configurations run at, against the oracle fed token
by token. The key/value pools are poisoned with binary16 NaN first, as the reference's own
verification runs do (docs/architecture/verification.md:427-431): a read of any page the sequence
has not written turns the logits into NaN.

Covered here and nowhere else: more than 1024 keys for one sequence (several clusters per KV head
whose results meet in global memory), a chunked prompt of 1500 tokens, and a launch whose CTAs see
more pages than the kernel keeps page bases for in shared memory (one-token pages, eight rows)."""
import numpy as np
import pytest

import jitllm_b200 as jl
from jitllm_b200 import GGMLType

pytestmark = pytest.mark.gpu
LOGIT_BAR = 1e-2


def _config(heads, kv_heads, head, ctx):
    return jl.Configuration(dim=heads * head, hiddenDim=768, numberOfLayers=2, numberOfHeads=heads,
                            numberOfKeyValueHeads=kv_heads, vocabularySize=1024, contextLength=ctx)


@pytest.mark.parametrize("t", [GGMLType.Q4_K, GGMLType.Q8_0])
def test_one_sequence_long_prompt_then_decode(dev, oracle, t):
    cfg = _config(heads=4, kv_heads=1, head=128, ctx=4096)
    tensors = jl.synth_model_tensors(cfg, t, seed=5, std=0.05)
    om = oracle.Model(cfg, tensors)
    cr, ci = om.rope_tables()
    model = jl.load_model(dev, cfg, tensors, cr, ci)
    bps = cfg.contextLength // 16
    kv = model.createKvStorage(jl.KvStorageRequest(bps, bps, 1, 16, cfg.numberOfLayers, cfg.kvDim))
    kv.publishBlockTable(np.random.default_rng(1).permutation(bps).astype(np.int32))  # scattered pages
    kv.fill(0x7E00)
    P, steps = 1500, 24
    toks = np.random.default_rng(2).integers(0, cfg.vocabularySize, size=P + steps)
    bound = jl.B200InvocationBoundary(model, kvSlot=0)
    bound.prefill([int(v) for v in toks[:P]], 0)
    for pos in range(P):
        om.forward_no_logits(int(toks[pos]), pos)
    worst = 0.0
    for pos in range(P, P + steps):
        want = om.forward(int(toks[pos]), pos)
        got = bound.invoke(int(toks[pos]), pos)
        assert np.all(np.isfinite(got.logits)), pos  # nothing read from a poisoned page
        worst = max(worst, float(np.max(np.abs(got.logits - want))))
        assert got.sampledToken == int(np.argmax(got.logits))
    assert worst < LOGIT_BAR, worst
    kv.close()


def test_wide_batch_with_more_pages_than_the_page_cache(dev, oracle):
    """Eight sequences of about 1150 tokens on one-token pages: every CTA walks more pages than it
    keeps bases for, so the table is consulted directly for the rest."""
    cfg = _config(heads=8, kv_heads=8, head=64, ctx=1280)
    t = GGMLType.Q8_0
    tensors = jl.synth_model_tensors(cfg, t, seed=9, std=0.05)
    width, P, steps = 8, 1140, 6
    model = jl.load_model(dev, cfg, tensors, *oracle.Model(cfg, tensors).rope_tables(), maxBatch=width)
    bps = cfg.contextLength
    kv = model.createKvStorage(jl.KvStorageRequest(width * bps, bps, width, 1, cfg.numberOfLayers, cfg.kvDim))
    kv.publishBlockTable(np.random.default_rng(3).permutation(width * bps).astype(np.int32))
    kv.fill(0x7E00)
    rng = np.random.default_rng(4)
    prompts = rng.integers(0, cfg.vocabularySize, size=(width, P + steps))
    seqs = []
    for b in range(width):
        jl.B200InvocationBoundary(model, kvSlot=b, copyLogits=False).prefill([int(v) for v in prompts[b, :P]], 0)
        om = oracle.Model(cfg, tensors)
        for pos in range(P):
            om.forward_no_logits(int(prompts[b, pos]), pos)
        seqs.append(om)
    ex = jl.B200BatchExecutor(model)
    worst = 0.0
    for s in range(steps):
        pos = P + s
        toks = [int(prompts[b, pos]) for b in range(width)]
        out, logits = ex.decodeStep(jl.BatchSlots([True] * width, toks, [pos] * width, list(range(width))), wantLogits=True)
        for b in range(width):
            want = seqs[b].forward(toks[b], pos)
            assert np.all(np.isfinite(logits[b])), (s, b)
            worst = max(worst, float(np.max(np.abs(logits[b] - want))))
    assert worst < LOGIT_BAR, worst
    kv.close()


@pytest.mark.parametrize("heads,kv_heads,head", [(8, 1, 64), (4, 2, 64), (2, 2, 128)])
def test_prompt_tiles_ragged_and_continued(dev, oracle, heads, kv_heads, head):
    """The tiled prompt attention on ragged chunks: a 37-token prompt (two and a bit 16-row blocks), then a
    second prompt call of 150 tokens that continues the same sequence at position 37 (its rows attend to
    keys of the first call), for query-head groups of 8, 2 and 1 per KV head; checked through the logits of
    the decode steps that follow and through the key rows in the pages."""
    cfg = _config(heads=heads, kv_heads=kv_heads, head=head, ctx=256)
    t = GGMLType.Q8_0
    tensors = jl.synth_model_tensors(cfg, t, seed=21, std=0.05)
    om = oracle.Model(cfg, tensors)
    model = jl.load_model(dev, cfg, tensors, *om.rope_tables())
    bps = cfg.contextLength // 16
    kv = model.createKvStorage(jl.KvStorageRequest(bps, bps, 1, 16, cfg.numberOfLayers, cfg.kvDim))
    kv.publishBlockTable(np.random.default_rng(3).permutation(bps).astype(np.int32))
    kv.fill(0x7E00)
    first, second, steps = 37, 150, 6
    toks = np.random.default_rng(4).integers(0, cfg.vocabularySize, size=first + second + steps)
    bound = jl.B200InvocationBoundary(model, kvSlot=0)
    bound.prefill([int(v) for v in toks[:first]], 0)
    bound.prefill([int(v) for v in toks[first:first + second]], first)
    for pos in range(first + second):
        om.forward_no_logits(int(toks[pos]), pos)
    for layer in range(cfg.numberOfLayers):
        for pos in (0, 36, 37, 100, first + second - 1):
            got = kv.readRow("k", 0, layer, pos).view(np.float16).astype(np.float32)   # binary16 bit patterns
            want = om.kcache(layer, pos).view(np.float16).astype(np.float32)
            assert np.all(np.isfinite(got))
            assert float(np.max(np.abs(got - want))) <= 4e-3 * float(np.max(np.abs(want))), (layer, pos)
    for pos in range(first + second, first + second + steps):
        want = om.forward(int(toks[pos]), pos)
        got = bound.invoke(int(toks[pos]), pos)
        assert np.all(np.isfinite(got.logits)), pos
        assert float(np.max(np.abs(got.logits - want))) < LOGIT_BAR
    kv.close()


@pytest.mark.parametrize("heads,kv_heads,head", [(8, 2, 64), (4, 1, 128), (2, 2, 128), (8, 1, 64)])
def test_batch_attention_kernel_on_ragged_batches(oracle, monkeypatch, heads, kv_heads, head):
    """The tensor-core decode attention for wide batches (one CTA per row and KV head, query heads as the rows
    of the MMA tile), forced on for a narrow batch: eight sequences at different depths (1 to 130 keys: fewer
    keys than one tile, exact multiples of a tile, several ring turns), one inactive row, poisoned pool,
    scattered pages, four steps each; logits against the oracle fed token by token, and the keys the kernel
    itself appends are read back."""
    monkeypatch.setenv("JITLLM_B200_BATCH_ATTN_MIN_PAIRS", "1")
    cfg = _config(heads=heads, kv_heads=kv_heads, head=head, ctx=192)
    t = GGMLType.Q8_0
    tensors = jl.synth_model_tensors(cfg, t, seed=33, std=0.05)
    width, steps = 8, 4
    depths = [1, 5, 31, 32, 33, 64, 100, 130]
    with jl.Device(0) as dev:
        oms = [oracle.Model(cfg, tensors) for _ in range(width)]
        model = jl.load_model(dev, cfg, tensors, *oms[0].rope_tables(), maxBatch=width)
        bps = cfg.contextLength // 16
        kv = model.createKvStorage(jl.KvStorageRequest(width * bps, bps, width, 16, cfg.numberOfLayers, cfg.kvDim))
        kv.publishBlockTable(np.random.default_rng(5).permutation(width * bps).astype(np.int32))
        kv.fill(0x7E00)
        rng = np.random.default_rng(6)
        for b in range(width):
            prompt = [int(v) for v in rng.integers(0, cfg.vocabularySize, size=depths[b])]
            jl.B200InvocationBoundary(model, kvSlot=b, copyLogits=False).prefill(prompt, 0)
            for pos, tok in enumerate(prompt):
                oms[b].forward_no_logits(tok, pos)
        ex = jl.B200BatchExecutor(model)
        positions = list(depths)
        active = [True] * width
        active[3] = False
        for step in range(steps):
            toks = [int(v) for v in rng.integers(0, cfg.vocabularySize, size=width)]
            out, logits = ex.decodeStep(jl.BatchSlots(active, toks, positions, list(range(width))), wantLogits=True)
            for b in range(width):
                if not active[b]:
                    assert out[b] == -1
                    continue
                want = oms[b].forward(toks[b], positions[b])
                assert np.all(np.isfinite(logits[b])), (step, b)
                assert float(np.max(np.abs(logits[b] - want))) < LOGIT_BAR, (step, b)
                got_k = kv.readRow("k", b, cfg.numberOfLayers - 1, positions[b]).view(np.float16).astype(np.float32)
                want_k = oms[b].kcache(cfg.numberOfLayers - 1, positions[b]).view(np.float16).astype(np.float32)
                assert float(np.max(np.abs(got_k - want_k))) <= 4e-3 * float(np.max(np.abs(want_k))), (step, b)
                positions[b] += 1
        kv.close()

"""The decode step through the C ABI against the oracle's forwardJava on small synthetic models:
logits within 1e-2 max-abs (stated bar; ~1e-5 expected), identical greedy tokens, identical KV
pages up to binary16 rounding of nearly-equal inputs."""
import numpy as np
import pytest

import jitllm_b200 as jl
from jitllm_b200 import GGMLType
from tests.util import Pair, rel_l2, small_config

pytestmark = pytest.mark.gpu
FORMATS = [GGMLType.Q8_0, GGMLType.Q4_0, GGMLType.Q4_K]
LOGIT_BAR = 1e-2
TENSOR_CORE_LOGIT_EXPECT = 6e-3  # batches of four or more rows: binary16 weight rounding on top
LOGIT_EXPECT = 4e-3  # 16-bit activations in every mat-vec plus binary16 K/V rounding flips: measured up to 2.4e-3


def _half_close(a_bits, b_bits, ulps=1, abs_frac=2e-5):
    a = a_bits.view(np.float16).astype(np.float32)
    b = b_bits.view(np.float16).astype(np.float32)
    same = a_bits == b_bits
    # Values that differ must be neighbours in binary16, or -- for elements that are tiny next to
    # the rest of the row, where the fp32 inputs themselves differ by ~1e-5 of the row scale --
    # within that absolute distance.
    tol = np.maximum(np.abs(a), 2.0 ** -14) * 2.0 ** -10 * ulps
    tol = np.maximum(tol, abs_frac * float(np.max(np.abs(b))))
    return bool(np.all(same | (np.abs(a - b) <= tol))), float(np.mean(same))


@pytest.mark.parametrize("t", FORMATS)
@pytest.mark.parametrize("head", [64, 128])
def test_teacher_forced_logits_and_kv(dev, oracle, t, head):
    cfg = small_config(layers=2, ctx=64, head=head)
    p = Pair(dev, oracle, cfg, t, seed=21 + head, std=0.05)
    tokens = np.random.default_rng(5).integers(0, cfg.vocabularySize, size=40)
    for pos, tok in enumerate(tokens):
        want = p.oracle_model.forward(int(tok), pos)
        res = p.boundary.invoke(int(tok), pos)
        err = float(np.max(np.abs(res.logits - want)))
        assert err < LOGIT_BAR and err < LOGIT_EXPECT, (pos, err)
        assert res.sampledToken == int(np.argmax(want)) == jl.argmax(res.logits)
        # K/V pages: the device's k and v differ from the oracle's by ~2e-5 relative (the mat-vec
        # holds its input as 16-bit fixed point per block), so they round to the same binary16 value
        # except when they straddle a rounding boundary (about one element in ten in layer 0); a
        # flipped element is one binary16 ulp away and perturbs deeper layers at the 5e-5 level, so
        # deeper layers flip more often. Every element must be within one ulp; most must be identical.
        for l in range(cfg.numberOfLayers):
            for which, cache in (("k", p.oracle_model.kcache), ("v", p.oracle_model.vcache)):
                # layer 0 sees bit-identical inputs and differs by the mat-vec's own error (1e-4 of the
                # row scale at most); deeper layers inherit upstream noise on top
                ok, frac = _half_close(p.kv.readRow(which, 0, l, pos), cache(l, pos),
                                       abs_frac=1e-4 if l == 0 else 1e-3)
                assert ok, (which, l, pos)
                assert frac > (0.75 if l == 0 else 0.3), (which, l, pos, frac)
    # per-operation buffers of the last step
    for name, n in (("q", cfg.dim), ("k", cfg.kvDim), ("v", cfg.kvDim), ("hb", cfg.hiddenDim)):
        if name in ("q", "k"):
            continue  # the oracle rotates q and k in place; the device keeps them un-rotated
        assert rel_l2(p.model.debugRead(name), p.oracle_model.buffer(name, n)) < 5e-4


@pytest.mark.parametrize("t", FORMATS)
def test_greedy_tokens_identical(dev, oracle, t):
    cfg = small_config(layers=3, ctx=96, tied=True)
    p = Pair(dev, oracle, cfg, t, seed=77, std=0.05)
    prompt = [int(v) for v in np.random.default_rng(8).integers(0, cfg.vocabularySize, size=8)]
    cpu, gpu, gaps = [], [], []
    tok_c = tok_g = None
    for pos in range(72):
        feed_c = prompt[pos] if pos < len(prompt) else tok_c
        feed_g = prompt[pos] if pos < len(prompt) else tok_g
        logits = p.oracle_model.forward(feed_c, pos)
        tok_c = int(np.argmax(logits))
        top2 = np.partition(logits, -2)[-2:]
        gaps.append(float(top2[1] - top2[0]))
        tok_g = p.boundary.invoke(feed_g, pos).sampledToken
        cpu.append(tok_c)
        gpu.append(tok_g)
    assert cpu == gpu, f"first divergence at {next(i for i, (a, b) in enumerate(zip(cpu, gpu)) if a != b)}, min top-2 gap {min(gaps):.3g}"


def test_paged_block_table_remapping_and_unmapped_entries(dev, oracle):
    cfg = small_config(layers=2, ctx=64)
    bps = 4
    # slot 0 -> physical blocks in scrambled order, slot 1 unmapped (scratch), slot 2 -> the rest
    table = np.array([5, 2, 7, 0, -1, -1, -1, -1, 1, 3, 4, 6], dtype=np.int32)
    p = Pair(dev, oracle, cfg, GGMLType.Q4_K, seed=31, max_batch=1, slots=3, block_table=table, total_blocks=8, std=0.05)
    toks = np.random.default_rng(2).integers(0, cfg.vocabularySize, size=36)
    bound = jl.B200InvocationBoundary(p.model, kvSlot=2)
    for pos, tok in enumerate(toks):
        want = p.oracle_model.forward(int(tok), pos)
        got = bound.invoke(int(tok), pos)
        assert float(np.max(np.abs(got.logits - want))) < LOGIT_EXPECT
    with pytest.raises(ValueError, match="block table shape changed"):
        p.kv.publishBlockTable(np.zeros(5, dtype=np.int32))
    with pytest.raises(ValueError, match="outside the pool"):
        p.kv.publishBlockTable(np.full(12, 99, dtype=np.int32))


def test_batched_decode_matches_independent_sequences(dev, oracle):
    cfg = small_config(layers=2, ctx=64)
    width = 4
    p = Pair(dev, oracle, cfg, GGMLType.Q8_0, seed=41, max_batch=width, std=0.05)
    seqs = [p.new_oracle_sequence() for _ in range(width)]
    rng = np.random.default_rng(3)
    positions = [0, 0, 0, 0]
    # ragged: rows advance at different rates, one row goes inactive half way
    for step in range(24):
        active = [True, step % 2 == 0, step < 10, True]
        toks = [int(v) for v in rng.integers(0, cfg.vocabularySize, size=width)]
        out, logits = p.executor.decodeStep(jl.BatchSlots(active, toks, positions, [0, 1, 2, 3]), wantLogits=True)
        for b in range(width):
            if not active[b]:
                assert out[b] == -1
                continue
            want = seqs[b].forward(toks[b], positions[b])
            # width 4 runs on the tensor-core path: weights rounded once to binary16 (rel-L2 ~3e-4
            # per product), so the logits sit inside the 1e-2 bar but above the mat-vec path's level
            err = float(np.max(np.abs(logits[b] - want)))
            assert err < LOGIT_BAR and err < TENSOR_CORE_LOGIT_EXPECT, (step, b, err)
            top2 = np.sort(want)[-2:]
            if top2[1] - top2[0] > 2 * TENSOR_CORE_LOGIT_EXPECT:
                assert out[b] == int(np.argmax(want))
            positions[b] += 1
    assert p.executor.maxBatchSize() == width


def test_prefill_then_decode_equals_token_by_token(dev, oracle):
    cfg = small_config(layers=2, ctx=64)
    p = Pair(dev, oracle, cfg, GGMLType.Q4_0, seed=51, std=0.05)
    prompt = [int(v) for v in np.random.default_rng(4).integers(0, cfg.vocabularySize, size=20)]
    for pos, tok in enumerate(prompt[:-1]):
        p.oracle_model.forward_no_logits(tok, pos)
    want = p.oracle_model.forward(prompt[-1], len(prompt) - 1)
    p.boundary.prefill(prompt[:-1], 0)
    got = p.boundary.invoke(prompt[-1], len(prompt) - 1)
    assert float(np.max(np.abs(got.logits - want))) < LOGIT_EXPECT
    assert got.sampledToken == int(np.argmax(want))


def test_argmax_ties_take_the_first_index(dev, oracle):
    """All-zero activations cannot happen, but identical embedding rows can: rows 10 and 20 of a
    tied embedding are made identical, so their logits tie exactly and index 10 must win."""
    cfg = small_config(layers=1, ctx=32, tied=True, vocab=512)
    tensors = jl.synth_model_tensors(cfg, GGMLType.Q8_0, seed=61, std=0.05)
    t, emb = tensors[(jl.TensorRole.TOKEN_EMBEDDING, -1)]
    rb = cfg.dim // 32 * 34
    emb = emb.copy()
    big = jl.quantize(GGMLType.Q8_0, np.full(cfg.dim, 3.0, dtype=np.float32) * np.sign(np.random.default_rng(1).standard_normal(cfg.dim)).astype(np.float32))
    emb[10 * rb:11 * rb] = big
    emb[20 * rb:21 * rb] = big
    tensors[(jl.TensorRole.TOKEN_EMBEDDING, -1)] = (t, emb)
    om = oracle.Model(cfg, tensors)
    cr, ci = om.rope_tables()
    model = jl.load_model(dev, cfg, tensors, cr, ci)
    kv = model.createKvStorage(jl.KvStorageRequest(2, 2, 1, 16, cfg.numberOfLayers, cfg.kvDim))
    kv.publishBlockTable(np.arange(2, dtype=np.int32))
    res = jl.B200InvocationBoundary(model).invoke(10, 0)
    want = om.forward(10, 0)
    assert int(np.argmax(want)) == res.sampledToken
    if want[10] == want[20] == want.max():
        assert res.sampledToken == 10


def test_lifecycle_and_argument_errors(dev, oracle):
    cfg = small_config(layers=1, ctx=32)
    model = jl.B200Model(dev, cfg)
    ex = jl.B200BatchExecutor(model)
    with pytest.raises(jl.IllegalStateError, match="jl_model_finalize"):
        ex.decodeStep(jl.BatchSlots([True], [1], [0], [0]))
    with pytest.raises(jl.IllegalStateError, match="missing"):
        model.finalize()
    with pytest.raises(ValueError, match="expects"):
        dev._check(dev._lib.jl_upload_tensor(dev.handle, 2, 0, 8, 5, 256, np.zeros(5 * 272, dtype=np.uint8).ctypes.data, 5 * 272))
    p = Pair(dev, oracle, cfg, GGMLType.Q8_0, seed=1)
    with pytest.raises(ValueError, match="outside vocabulary"):
        p.executor.decodeStep(jl.BatchSlots([True], [cfg.vocabularySize], [0], [0]))
    with pytest.raises(ValueError, match="position"):
        p.executor.decodeStep(jl.BatchSlots([True], [1], [cfg.contextLength], [0]))
    with pytest.raises(ValueError, match="fixed width"):
        p.executor.decodeStep(jl.BatchSlots([True, True], [1, 1], [0, 0], [0, 1]))
    with pytest.raises(ValueError, match="head_dim"):
        jl.B200Model(dev, jl.Configuration(256, 512, 1, 8, 8, 512, 32))


def test_device_resident_generation_equals_host_driven_steps(dev, oracle):
    cfg = small_config(layers=2, ctx=96)
    width = 2
    p = Pair(dev, oracle, cfg, GGMLType.Q4_K, seed=71, max_batch=width, std=0.05)
    seqs = [p.new_oracle_sequence() for _ in range(width)]
    first = [5, 900]
    hist = p.executor.generate(jl.BatchSlots([True, True], first, [0, 0], [0, 1]), 40)
    assert hist.shape == (40, width)
    for b in range(width):
        tok = first[b]
        for step in range(40):
            tok = int(np.argmax(seqs[b].forward(tok, step)))
            assert hist[step, b] == tok, (b, step)
    with pytest.raises(ValueError, match="run past context"):
        p.executor.generate(jl.BatchSlots([True, True], first, [90, 0], [0, 1]), 10)


@pytest.mark.parametrize("t", FORMATS)
def test_chunked_prefill_on_the_tensor_core_path(dev, oracle, t):
    """A 40-token prompt goes through the matrix-matrix pipeline (one chunk), then decode steps:
    logits after the prompt must agree with the oracle fed token by token. fp16 weight rounding in
    the tensor-core operands is the extra error source here (per-matmul bar 1e-3)."""
    cfg = small_config(layers=2, ctx=96)
    p = Pair(dev, oracle, cfg, t, seed=91, std=0.05)
    prompt = [int(v) for v in np.random.default_rng(12).integers(0, cfg.vocabularySize, size=41)]
    for pos, tok in enumerate(prompt[:-1]):
        p.oracle_model.forward_no_logits(tok, pos)
    p.boundary.prefill(prompt[:-1], 0)
    for l in range(cfg.numberOfLayers):
        for pos in (0, 17, 39):
            ok, _ = _half_close(p.kv.readRow("k", 0, l, pos), p.oracle_model.kcache(l, pos), abs_frac=4e-3)
            assert ok, ("k", l, pos)
    tok = prompt[-1]
    for pos in range(40, 48):
        want = p.oracle_model.forward(tok, pos)
        got = p.boundary.invoke(tok, pos)
        assert float(np.max(np.abs(got.logits - want))) < LOGIT_BAR
        assert rel_l2(got.logits, want) < 2e-3
        tok = int(np.argmax(want))


def test_wide_batch_decode_on_the_tensor_core_path(dev, oracle):
    cfg = small_config(layers=2, ctx=64)
    width = 16
    p = Pair(dev, oracle, cfg, GGMLType.Q4_K, seed=93, max_batch=width, std=0.05)
    seqs = [p.new_oracle_sequence() for _ in range(width)]
    rng = np.random.default_rng(13)
    positions = [0] * width
    for step in range(6):
        active = [not (b == 5 and step >= 3) for b in range(width)]
        toks = [int(v) for v in rng.integers(0, cfg.vocabularySize, size=width)]
        out, logits = p.executor.decodeStep(jl.BatchSlots(active, toks, positions, list(range(width))), wantLogits=True)
        for b in range(width):
            if not active[b]:
                assert out[b] == -1
                continue
            want = seqs[b].forward(toks[b], positions[b])
            assert float(np.max(np.abs(logits[b] - want))) < LOGIT_BAR
            assert rel_l2(logits[b], want) < 2e-3
            top2 = np.partition(want, -2)[-2:]
            if top2[1] - top2[0] > 5e-3:
                assert out[b] == int(np.argmax(want))
            positions[b] += 1


@pytest.mark.parametrize("width", [2, 4])
def test_two_slots_share_the_physical_blocks_of_a_common_prefix(dev, oracle, width):
    """Prefix sharing as the reference's PrefixCache hands it out (runtime/kv/PrefixCache.java,
    BATCHED_DECODE.md:245-265): slots whose block tables point at the same physical blocks for the
    prompt they have in common. The prefix is written once, through slot 0; every slot then decodes
    its own continuation into blocks of its own and must match an oracle sequence that saw prefix +
    continuation. Width 2 runs the mat-vec path, width 4 the tensor-core path."""
    cfg = small_config(layers=2, ctx=64)
    bps, prefix = 4, 32                           # two full 16-token blocks are shared
    table = np.full(width * bps, jl.UNMAPPED, dtype=np.int32)
    for b in range(width):
        table[b * bps:b * bps + 2] = [0, 1]       # the shared physical blocks
        table[b * bps + 2:b * bps + 4] = [2 + 2 * b, 3 + 2 * b]
    p = Pair(dev, oracle, cfg, GGMLType.Q4_K, seed=71, max_batch=width, slots=width, block_table=table,
             total_blocks=2 + 2 * width, std=0.05)
    rng = np.random.default_rng(12)
    common = [int(v) for v in rng.integers(0, cfg.vocabularySize, size=prefix)]
    p.boundary.prefill(common, 0)                 # slot 0 writes blocks 0 and 1 for everybody
    seqs = [p.new_oracle_sequence() for _ in range(width)]
    for om in seqs:
        for pos, tok in enumerate(common):
            om.forward_no_logits(tok, pos)
    bar = LOGIT_EXPECT if width < 4 else TENSOR_CORE_LOGIT_EXPECT
    for step in range(10):
        toks = [int(v) for v in rng.integers(0, cfg.vocabularySize, size=width)]
        pos = prefix + step
        out, logits = p.executor.decodeStep(jl.BatchSlots([True] * width, toks, [pos] * width, list(range(width))),
                                            wantLogits=True)
        for b in range(width):
            want = seqs[b].forward(toks[b], pos)
            assert float(np.max(np.abs(logits[b] - want))) < bar, (step, b)
    # the shared blocks still hold what slot 0 wrote: nobody's continuation touched them
    for b in range(1, width):
        for which in ("k", "v"):
            assert np.array_equal(p.kv.readRow(which, b, 0, prefix - 1), p.kv.readRow(which, 0, 0, prefix - 1))

"""Shared helpers for the parity tests."""
import numpy as np

import jitllm_b200 as jl


def rel_l2(got: np.ndarray, want: np.ndarray) -> float:
    return float(np.linalg.norm(got.astype(np.float64) - want.astype(np.float64)) /
                 max(np.linalg.norm(want.astype(np.float64)), 1e-30))


def small_config(layers=2, ctx=64, vocab=1024, tied=False, head=64):
    if head == 64:
        return jl.Configuration(dim=256, hiddenDim=512, numberOfLayers=layers, numberOfHeads=4,
                                numberOfKeyValueHeads=2, vocabularySize=vocab, contextLength=ctx,
                                tiedEmbeddings=tied)
    return jl.Configuration(dim=512, hiddenDim=768, numberOfLayers=layers, numberOfHeads=4,
                            numberOfKeyValueHeads=1, vocabularySize=vocab, contextLength=ctx,
                            tiedEmbeddings=tied)


class Pair:
    """The same synthetic model on the oracle and on the GPU, sharing weight bytes and RoPE tables."""

    def __init__(self, dev, oracle, config, ggml_type, seed, max_batch=1, slots=None, block_tokens=16,
                 block_table=None, total_blocks=None, std=0.02, replace=None):
        self.config = config
        self.tensors = jl.synth_model_tensors(config, ggml_type, seed, std=std)
        for key, value in (replace or {}).items():  # {(role, layer): (type, bytes)}: tensors in another format
            assert key in self.tensors
            self.tensors[key] = value
        self.oracle_model = oracle.Model(config, self.tensors)
        cr, ci = self.oracle_model.rope_tables()
        self.model = jl.load_model(dev, config, self.tensors, cr, ci, maxBatch=max_batch)
        slots = slots or max_batch
        bps = (config.contextLength + block_tokens - 1) // block_tokens
        total = total_blocks or slots * bps
        self.kv = self.model.createKvStorage(jl.KvStorageRequest(total, bps, slots, block_tokens,
                                                                 config.numberOfLayers, config.kvDim))
        if block_table is None:
            block_table = np.arange(slots * bps, dtype=np.int32)
        self.kv.publishBlockTable(block_table)
        self.executor = jl.B200BatchExecutor(self.model)
        self.boundary = jl.B200InvocationBoundary(self.model, kvSlot=0)
        self._oracle = oracle

    def new_oracle_sequence(self):
        return self._oracle.Model(self.config, self.tensors)


def random_blocks(t, n_blocks, rng, scale=0.01):
    """Random payload bytes with block scales of a sane magnitude (a fully random fp16 scale is often
    infinite or NaN, which tests nothing but overflow in a dot product)."""
    t = jl.GGMLType(t)
    return jl.random_blocks(t, n_blocks * t.block_size, int(rng.integers(0, 2**31)), scale)

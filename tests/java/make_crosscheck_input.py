"""Writes the input file of QuantizedForwardCrossCheck.java: a tiny seeded Llama in GGUF blocks.

    python tests/java/make_crosscheck_input.py {Q8_0|Q4_0|Q4_K} out.bin

Layout (little endian): "JLXC", dim, hidden, layers, heads, kv heads, vocab, context, GGML type,
token count (int32 each), eps, theta (float32), the tokens (int32), then every tensor's bytes, each
starting on a 32-byte boundary, in the order LlamaStandardWeights' constructor takes them:
embedding; per layer attention norm, wq, wk, wv, wo, FFN norm, w1 (gate), w2 (down), w3 (up);
final norm; RoPE cos; RoPE sin; output matrix. The RoPE tables are the oracle's, so both sides use
the same bits (the reference reads them from the weights, as here)."""
import struct
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

import jitllm_b200 as jl  # noqa: E402
from oracle import binding as oracle  # noqa: E402

CONFIG = dict(dim=256, hiddenDim=512, numberOfLayers=3, numberOfHeads=4, numberOfKeyValueHeads=2,
              vocabularySize=512, contextLength=32, rmsNormEps=1e-5, ropeTheta=10000.0)
TOKENS = [7, 3, 41, 0, 19, 5, 33, 12, 400, 77, 1, 255]
SEED = 20260831


def build(fmt_name):
    cfg = jl.Configuration(**CONFIG)
    fmt = jl.GGMLType[fmt_name]
    tensors = jl.synth_model_tensors(cfg, fmt, SEED, std=0.05)
    om = oracle.Model(cfg, tensors)
    cr, ci = om.rope_tables()
    return cfg, fmt, tensors, om, cr, ci


def write(fmt_name, path):
    cfg, fmt, tensors, om, cr, ci = build(fmt_name)
    R = jl.TensorRole
    blob = bytearray()
    blob += struct.pack("<10i", 0x43584C4A, cfg.dim, cfg.hiddenDim, cfg.numberOfLayers, cfg.numberOfHeads,
                        cfg.numberOfKeyValueHeads, cfg.vocabularySize, cfg.contextLength, int(fmt), len(TOKENS))
    blob += struct.pack("<2f", cfg.rmsNormEps, cfg.ropeTheta)
    blob += struct.pack("<%di" % len(TOKENS), *TOKENS)

    def put(arr):
        nonlocal blob
        blob += b"\0" * ((-len(blob)) % 32)
        blob += np.ascontiguousarray(arr).view(np.uint8).tobytes()

    put(tensors[(R.TOKEN_EMBEDDING, -1)][1])
    for l in range(cfg.numberOfLayers):
        for role in (R.ATTENTION_NORM, R.ATTENTION_QUERY, R.ATTENTION_KEY, R.ATTENTION_VALUE, R.ATTENTION_OUTPUT,
                     R.FFN_NORM, R.FFN_GATE, R.FFN_DOWN, R.FFN_UP):
            put(tensors[(role, l)][1])
    put(tensors[(R.OUTPUT_NORM, -1)][1])
    put(cr.astype(np.float32))
    put(ci.astype(np.float32))
    put(tensors[(R.OUTPUT, -1)][1] if (R.OUTPUT, -1) in tensors else tensors[(R.TOKEN_EMBEDDING, -1)][1])
    Path(path).write_bytes(bytes(blob))
    return len(blob)


if __name__ == "__main__":
    if len(sys.argv) != 3:
        sys.exit(__doc__)
    print(write(sys.argv[1], sys.argv[2]), "bytes")

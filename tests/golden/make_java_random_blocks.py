"""Regenerates tests/golden/java_random_blocks.npz: the byte blocks the reference's decode tests
draw from java.util.Random (Q4_0DecodeTest seed 20260908, Q4_KDecodeTest seed 20260904; Q8_0 reuses
the latter seed) and the oracle's element-exact decode of them as raw binary32 bit patterns.

Run from the repository root:  python tests/golden/make_java_random_blocks.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import binding  # noqa: E402
from tests.javarand import JavaRandom  # noqa: E402

out = {}
for name, fmt, seed, blocks, bb, be in (("q4_0", 2, 20260908, 16, 18, 32), ("q4_k", 12, 20260904, 8, 144, 256),
                                        ("q8_0", 8, 20260904, 16, 34, 32)):
    raw = JavaRandom(seed).next_bytes(blocks * bb)
    out[name + "_raw"] = raw
    out[name + "_f32_bits"] = binding.dequant(fmt, raw, blocks * be).view(np.uint32)
np.savez_compressed(Path(__file__).parent / "java_random_blocks.npz", **out)
print("wrote", Path(__file__).parent / "java_random_blocks.npz")

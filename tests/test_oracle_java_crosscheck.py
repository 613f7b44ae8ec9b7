"""The oracle's logits against jitLLM's own CPU path, when somebody with a JDK has produced them.

tests/java/QuantizedForwardCrossCheck.java runs InferenceCore.forwardJava of the reference over a
tiny seeded model in GGUF blocks (tests/java/make_crosscheck_input.py writes its input) and leaves
the raw bits of every logit in tests/java/crosscheck_<format>.logits. No JDK exists where this
repository is built, so those files are absent and the comparison is skipped; the input writer and
the oracle side are exercised regardless, so that the recipe cannot rot."""
import importlib.util
from pathlib import Path

import numpy as np
import pytest

HERE = Path(__file__).resolve().parent / "java"
spec = importlib.util.spec_from_file_location("make_crosscheck_input", HERE / "make_crosscheck_input.py")
maker = importlib.util.module_from_spec(spec)
spec.loader.exec_module(maker)


@pytest.mark.parametrize("fmt", ["Q8_0", "Q4_0", "Q4_K"])
def test_input_file_and_oracle_logits(tmp_path, fmt):
    size = maker.write(fmt, tmp_path / "in.bin")
    assert size == (tmp_path / "in.bin").stat().st_size and size > 100_000
    cfg, _, _, om, _, _ = maker.build(fmt)
    logits = [om.forward(tok, pos) for pos, tok in enumerate(maker.TOKENS)]
    assert all(np.all(np.isfinite(v)) for v in logits) and np.ptp(logits[-1]) > 0
    produced = HERE / f"crosscheck_{fmt.lower()}.logits"
    if not produced.exists():
        pytest.skip("no JDK here: QuantizedForwardCrossCheck has not been run, nothing to compare with")
    lines = produced.read_text().split("\n")
    for pos, want in enumerate(logits):
        got = np.array([int(h, 16) for h in lines[pos].split()], dtype=np.uint32).view(np.float32)
        assert got.shape == want.shape
        # bit for bit except where glibc and the JVM round exp() differently in the last place
        assert np.max(np.abs(got - want)) <= 1e-6 * max(1.0, float(np.max(np.abs(want)))), pos

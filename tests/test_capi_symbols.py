"""The C-ABI library loads and exports every function include/jitllm_b200.h declares (no compute
calls: this runs without a GPU)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "jitllm_b200.h"


def _declared():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(jl_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_entry_points():
    names = _declared()
    for must in ("jl_init", "jl_destroy", "jl_last_error", "jl_model_create", "jl_upload_tensor", "jl_upload_rope",
                 "jl_kv_create", "jl_kv_publish_block_table", "jl_decode", "jl_prefill", "jl_dequant", "jl_gemv"):
        assert must in names


def test_library_exports_every_declared_symbol(built):
    from jitllm_b200 import _lib
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in _declared():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_python_binding_covers_the_header(built):
    from jitllm_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared()
    _lib.load()


def test_no_silent_cpu_fallback(built):
    """Without a CUDA device the library refuses to initialise and says why."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import jitllm_b200 as jl
    with pytest.raises(RuntimeError, match="no usable CUDA device"):
        jl.Device(0)


def test_product_package_never_imports_the_oracle():
    for py in (ROOT / "jitllm_b200").rglob("*.py"):
        text = py.read_text()
        assert "oracle" not in text.replace("no CPU fallback", ""), f"{py} mentions the oracle"
    for src in (ROOT / "jitllm_b200" / "csrc").rglob("*"):
        if src.is_file():
            assert "jl_oracle" not in src.read_text(), f"{src} includes the oracle"

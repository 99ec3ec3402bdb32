"""The C-ABI library builds for sm_100a, loads without a GPU and exports every symbol
that include/litedsa_b200.h declares (no compute calls here)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _declared_functions():
    text = (ROOT / "include" / "litedsa_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(litedsa_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_operators():
    names = _declared_functions()
    for must in ("litedsa_union_qm", "litedsa_masked_mla_fp8", "litedsa_abi_version"):
        assert must in names


def test_library_exports_every_declared_symbol(built_lib):
    from litetopk_b200 import _lib
    names = _declared_functions()
    assert sorted(_lib.SIGNATURES) == names, "ctypes table and header disagree"
    for n in names:
        assert getattr(built_lib, n) is not None
    assert built_lib.litedsa_abi_version() >= 1
    assert b"shape" in built_lib.litedsa_error_string(2)


def test_no_cpu_fallback_when_library_missing(monkeypatch, tmp_path):
    from litetopk_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "missing.so")
    with pytest.raises(ImportError):
        _lib.lib()


def test_python_api_rejects_cpu_tensors(built_lib):
    import torch
    from litetopk_b200 import api
    with pytest.raises(ValueError):
        api.union_qm(torch.zeros((4, 64), dtype=torch.int32), 2)
    with pytest.raises(TypeError):
        api.union_qm(torch.zeros((4, 64), dtype=torch.int64), 2)


def test_host_buffer_entry_validates_without_a_gpu(built_lib):
    import torch
    from litetopk_b200 import api
    q = torch.zeros((4, 64, 576), dtype=torch.bfloat16)
    idx = torch.zeros((4, 64), dtype=torch.int32)
    kv_cpu = torch.zeros((128, 576), dtype=torch.uint8)
    with pytest.raises(ValueError, match="CUDA"):          # the cache must live on a GPU: no CPU path
        api.sparse_prefill_host(q, kv_cpu, idx, 0.1)


def test_product_code_never_imports_the_oracle():
    for f in (ROOT / "litetopk_b200").rglob("*.py"):
        src = f.read_text()
        assert not re.search(r"^\s*(from|import)\s+oracle\b", src, flags=re.M), f

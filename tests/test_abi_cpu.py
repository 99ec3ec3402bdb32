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
    assert built_lib.litedsa_abi_version() >= 3
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


def test_entry_points_reject_bad_arguments_before_any_cuda_call(built_lib):
    # argument and shape rules are checked on the host first, so these calls need no GPU;
    # the pointers are fake but never dereferenced
    from litetopk_b200 import _lib
    L = built_lib
    P = 0x1000        # 16-byte aligned non-null
    ARG, SHAPE, UNSUP = _lib.ERR_ARG, _lib.ERR_SHAPE, _lib.ERR_UNSUPPORTED
    # union: null output, T != ng * G, cap not a multiple of 128, k not a multiple of 4
    assert L.litedsa_union_qm(P, None, P, P, None, None, 4, 64, 2, 128, 2, 0, 0, 1, 1024, 0, None) == ARG
    assert L.litedsa_union_qm(P, P, P, P, None, None, 5, 64, 2, 128, 2, 0, 0, 1, 1024, 0, None) == SHAPE
    assert L.litedsa_union_qm(P, P, P, P, None, None, 4, 50, 2, 100, 2, 0, 0, 1, 1024, 0, None) == SHAPE
    assert L.litedsa_union_qm(P, P, P, P, None, None, 128, 2, 1, 256, 128, 0, 0, 1, 1024, 0, None) == SHAPE
    # attention: null q, topk not a multiple of 128, heads not dividing 128, misaligned base
    ok = dict(sm=0.1, os=1.0)
    assert L.litedsa_masked_mla_fp8(None, P, P, ok["sm"], ok["os"], None, P, 64, P, None, P,
                                    2, 128, 128, 576, 576, 128, None) == ARG
    assert L.litedsa_masked_mla_fp8(P, P, P, ok["sm"], ok["os"], None, P, 64, P, None, P,
                                    2, 128, 100, 576, 576, 128, None) == SHAPE
    assert L.litedsa_masked_mla_fp8(P, P, P, ok["sm"], ok["os"], None, P, 48, P, None, P,
                                    2, 128, 128, 576, 576, 128, None) == SHAPE
    assert L.litedsa_masked_mla_fp8(P + 8, P, P, ok["sm"], ok["os"], None, P, 64, P, None, P,
                                    2, 128, 128, 576, 576, 128, None) == UNSUP
    # extended form: neither mask given, q_group_div not dividing the tile count
    assert L.litedsa_masked_mla_fp8_ex(P, P, P, ok["sm"], ok["os"], None, None, 64, P, None, P,
                                       2, 128, 128, 576, 576, 128, None, None, 1, 0, 0, 0, 0, None) == ARG
    assert L.litedsa_masked_mla_fp8_ex(P, P, P, ok["sm"], ok["os"], None, P, 64, P, None, P,
                                       3, 128, 128, 576, 576, 128, None, None, 2, 0, 0, 0, 0, None) == SHAPE
    # in-place addressing: a head pitch that is not a multiple of 16 bytes
    assert L.litedsa_masked_mla_fp8_ex(P, P, P, ok["sm"], ok["os"], None, P, 64, P, None, P,
                                       2, 128, 128, 576, 576, 128, None, None, 1, 64 * 584, 584, 0, 0,
                                       None) == UNSUP
    # allocation-free form: every rule is checked before its scratch is touched
    na = L.litedsa_masked_mla_fp8_kv656_noalloc
    assert na(P, P, P, ok["sm"], ok["os"], None, P, 64, None, None, P, 2, 128, 128, 576, 128, None, None) == ARG
    assert na(P, P, P, ok["sm"], ok["os"], None, P, 64, P, None, P, 2, 128, 100, 576, 128, None, None) == SHAPE
    assert na(P, P, P, ok["sm"], ok["os"], None, P, 48, P, None, P, 2, 128, 128, 576, 128, None, None) == SHAPE
    assert na(P + 8, P, P, ok["sm"], ok["os"], None, P, 64, P, None, P, 2, 128, 128, 576, 128, None, None) == UNSUP
    assert na(P, P, P, ok["sm"], ok["os"], None, P, 64, P, None, P, 2, 65537, 128, 576, 128, None, None) == UNSUP
    # bf16 operators: missing range arrays, width other than 512 / 576, list not in 64-key blocks
    assert L.litedsa_dsv4_masked_mla_bf16(P, P, P, None, P, P, P, 0.1, 64, P, P, None,
                                          2, 128, 128, 512, 512, 512, 128, 0, 0, 0, 0, None, 0, None) == ARG
    assert L.litedsa_dsv4_masked_mla_bf16(P, P, P, P, P, P, P, 0.1, 64, P, P, None,
                                          2, 128, 128, 500, 512, 512, 128, 0, 0, 0, 0, None, 0, None) == SHAPE
    assert L.litedsa_dsv4_masked_mla_bf16(P, P, P, P, P, P, P, 0.1, 64, P, P, None,
                                          2, 128, 96, 512, 512, 512, 96, 0, 0, 0, 0, None, 0, None) == SHAPE
    # a workspace too small for the tiles (16 + 16 * ng bytes) is rejected before any CUDA call
    assert L.litedsa_dsv4_masked_mla_bf16(P, P, P, P, P, P, P, 0.1, 64, P, P, None,
                                          2, 128, 128, 512, 512, 512, 128, 0, 0, 0, 0, P, 32, None) == SHAPE
    assert L.litedsa_masked_mla_bf16(P, P, P, 0.1, None, None, 64, P, None, P,
                                     2, 128, 128, 576, 576, 576, 128, None, None) == ARG
    assert L.litedsa_masked_mla_bf16(P, P, P, 0.1, None, P, 64, P, None, P,
                                     2, 128, 64, 576, 576, 576, 64, None, None) == SHAPE
    assert L.litedsa_dequant_kv656(P, P, 16, 1000, None) == SHAPE
    # KV-split merge: null output, max arrays given on one side only, div not dividing ng, div > 32,
    # misaligned rows
    mg = L.litedsa_merge_kv_splits
    assert mg(P, P, None, None, None, P, None, 4, 2, None) == ARG
    assert mg(P, P, P, None, P, P, None, 4, 2, None) == ARG
    assert mg(P, P, None, None, P, P, None, 5, 2, None) == SHAPE
    assert mg(P, P, None, None, P, P, None, 66, 33, None) == UNSUP
    assert mg(P + 8, P, None, None, P, P, None, 4, 2, None) == UNSUP
    # multi-destination form: destination count out of range, null destination
    outs = (ctypes.c_void_p * 9)(*([P] * 9))
    assert L.litedsa_masked_mla_fp8_multi(P, P, P, ok["sm"], ok["os"], None, P, 64, outs, 9, None, P,
                                          2, 128, 128, 576, 576, 128, None) == SHAPE
    outs2 = (ctypes.c_void_p * 2)(P, None)
    assert L.litedsa_masked_mla_fp8_multi(P, P, P, ok["sm"], ok["os"], None, P, 64, outs2, 2, None, P,
                                          2, 128, 128, 576, 576, 128, None) == ARG
    # DSv4: queries outside the cache, heads not dividing 128
    assert L.litedsa_dsv4_c128a_bf16(P, None, P, 4, 64, 0, 4, 0, 128, 128, 0.1, None, P, P,
                                     576, 576, 576, 0, 0, 0, 0, None) == SHAPE
    assert L.litedsa_dsv4_c128a_bf16(P, None, P, 1, 48, 0, 64, 0, 128, 128, 0.1, None, P, P,
                                     576, 576, 576, 0, 0, 0, 0, None) == SHAPE


def test_host_pipeline_chunk_schedule():
    """Chunks of sparse_prefill_host: cover [0, T) once, tile-aligned cuts, short first / last chunk."""
    from litetopk_b200.api import _chunk_schedule
    for T, chunk, G in [(8192, 512, 2), (8192, 512, 8), (100, 512, 2), (2048, 512, 2), (2050, 512, 2),
                        (2046, 512, 2), (4100, 512, 4), (1, 512, 1), (3000, 512, 8), (65536, 512, 8)]:
        b = _chunk_schedule(T, chunk, G)
        assert b[0] == 0 and b[-1] == T
        assert all(x < y for x, y in zip(b, b[1:]))
        assert all(x % G == 0 for x in b[:-1])
        assert max(y - x for x, y in zip(b, b[1:])) <= chunk
        if T >= 4 * chunk:
            assert b[1] - b[0] <= chunk // 4 and b[-1] - b[-2] <= chunk // 4

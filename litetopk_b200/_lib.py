"""ctypes binding of liblitedsa_b200.so (the C ABI declared in include/litedsa_b200.h).

There is no CPU or PyTorch fallback: if the library is missing or a symbol cannot be
resolved, importing `lib()` raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_int64, c_uint64, c_float, c_void_p, c_char_p
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "_C" / "liblitedsa_b200.so"

OK, ERR_ARG, ERR_SHAPE, ERR_UNSUPPORTED, ERR_CUDA, ERR_TIMEOUT = range(6)

# name -> (restype, argtypes); must list every function of include/litedsa_b200.h
SIGNATURES = {
    "litedsa_abi_version": (c_int, []),
    "litedsa_error_string": (c_char_p, [c_int]),
    "litedsa_union_qm": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int64,
                                 c_int, c_void_p]),
    "litedsa_masked_mla_fp8": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_float, c_void_p,
                                       c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                       c_int, c_int, c_int64, c_int64, c_int64, c_void_p]),
    "litedsa_masked_mla_fp8_ex": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_float, c_void_p,
                                          c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int,
                                          c_int, c_int, c_int64, c_int64, c_int64, c_void_p,
                                          c_void_p, c_int, c_int64, c_int64, c_int64, c_int64,
                                          c_void_p]),
    "litedsa_masked_mla_fp8_multi": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_float,
                                             c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
                                             c_void_p, c_int, c_int, c_int, c_int64, c_int64,
                                             c_int64, c_void_p]),
    "litedsa_attn_status": (c_int, [c_void_p, c_int]),
    "litedsa_set_wait_limit_ns": (c_int, [c_uint64, c_void_p]),
    "litedsa_selftest_wait_timeout": (c_int, [c_uint64, c_void_p]),
    "litedsa_quantize_e4m3": (c_int, [c_void_p, c_void_p, c_int64, c_float, c_void_p]),
    "litedsa_repack_kv656": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_float, c_void_p,
                                     c_void_p]),
    "litedsa_masked_mla_fp8_kv656_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_float,
                                                     c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                                     c_void_p, c_int, c_int, c_int, c_int64, c_int64,
                                                     c_void_p, c_void_p]),
    "litedsa_dsv4_c128a_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                        c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_int64,
                                        c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_void_p]),
    "litedsa_dsv4_status": (c_int, [c_void_p, c_int]),
    "litedsa_dsv4_masked_mla_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_float, c_int, c_void_p, c_void_p, c_void_p,
                                             c_int, c_int, c_int, c_int, c_int64, c_int64, c_int64,
                                             c_int64, c_int64, c_int64, c_int64, c_void_p, c_int64,
                                             c_void_p]),
    "litedsa_masked_mla_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p,
                                        c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                        c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p]),
    "litedsa_dequant_kv656": (c_int, [c_void_p, c_void_p, c_int, c_int64, c_void_p]),
    "litedsa_merge_kv_splits": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_int, c_int, c_void_p]),
    "litedsa_bf16_status": (c_int, [c_void_p, c_int]),
    "litedsa_probe_mma_tflops": (c_int, [c_int, c_int, c_int, c_void_p]),
    "litedsa_index_logits_fp8": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                         c_int, c_int, c_int64, c_int64, c_void_p]),
    "litedsa_topk_select": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int64,
                                    c_void_p]),
    "litedsa_index_status": (c_int, [c_void_p, c_int]),
}

_lib = None


class LiteDSAError(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        msg = lib().litedsa_error_string(code).decode() if _lib is not None else str(code)
        super().__init__(f"{where}: {msg} (code {code})")


def lib() -> ctypes.CDLL:
    """Load the library once.  Raises if it has not been built (python -m litetopk_b200.build)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} not found: build the CUDA library with `python -m litetopk_b200.build` "
                "(there is no CPU fallback)")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)      # AttributeError if the symbol is missing
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(code: int, where: str) -> None:
    if code != OK:
        raise LiteDSAError(code, where)

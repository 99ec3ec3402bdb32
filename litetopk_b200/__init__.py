"""litetopk_b200: the LiteDSA sparse-attention hot path (union_qm + masked FP8 MLA prefill)
for NVIDIA B200 (sm_100a), behind the reference module's operator API.

Hand-written CUDA kernels reached through a C ABI (include/litedsa_b200.h); this package
is the thin Python host side.  There is no CPU fallback.
"""
from .api import (attn_status, dsv4_c128a_bf16, dsv4_status, masked_mla_fp8,  # noqa: F401
                  masked_mla_fp8_out, quantize_e4m3,
                  repack_kv656, sparse_prefill, union_qm, union_qm_out)
from . import synth  # noqa: F401

__all__ = ["union_qm", "union_qm_out", "masked_mla_fp8", "masked_mla_fp8_out", "sparse_prefill",
           "quantize_e4m3", "repack_kv656", "attn_status", "synth"]

"""litetopk_b200: the LiteDSA sparse-attention hot path (union_qm + masked FP8 MLA prefill)
for NVIDIA B200 (sm_100a), behind the reference module's operator API.

Hand-written CUDA kernels reached through a C ABI (include/litedsa_b200.h); this package
is the thin Python host side.  There is no CPU fallback.
"""
from .api import (attn_status, bf16_status, dequant_kv656, dsv4_c128a_bf16,  # noqa: F401
                  index_logits_fp8, index_status, lite_topk, topk_select,
                  dsv4_masked_mla_bf16_out, dsv4_status, masked_mla_bf16_out, masked_mla_fp8,
                  masked_mla_fp8_out, merge_kv_splits, prepare_kv, quantize_e4m3, repack_kv656, sparse_prefill,
                  sparse_prefill_host, union_qm, union_qm_out)
from . import synth  # noqa: F401

__all__ = ["union_qm", "union_qm_out", "masked_mla_fp8", "masked_mla_fp8_out", "masked_mla_bf16_out",
           "dsv4_c128a_bf16", "dsv4_masked_mla_bf16_out", "sparse_prefill", "sparse_prefill_host",
           "prepare_kv", "merge_kv_splits", "quantize_e4m3", "repack_kv656", "dequant_kv656", "attn_status",
           "bf16_status", "dsv4_status", "index_logits_fp8", "topk_select", "lite_topk",
           "index_status", "synth"]

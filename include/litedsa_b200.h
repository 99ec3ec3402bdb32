/*
 * litedsa_b200 -- C ABI of the B200 (sm_100a) LiteDSA sparse-attention hot path.
 *
 * One shared library (liblitedsa_b200.so), plain pointers and sizes, no C++ or
 * framework types in any signature.  Every function
 *   - takes DEVICE pointers unless a parameter says "host",
 *   - is asynchronous on the CUDA stream passed as `stream` (a cudaStream_t cast to
 *     void*; NULL = the legacy default stream),
 *   - allocates nothing on the device unless its comment says otherwise,
 *   - never throws, traps or exits: it returns one of the LITEDSA_* codes below.
 * Outputs are caller-owned, destination-passing, exactly as in the reference
 * operators these entry points replace.
 */
#ifndef LITEDSA_B200_H_
#define LITEDSA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  LITEDSA_OK = 0,
  LITEDSA_ERR_ARG = 1,         /* null pointer / inconsistent optional arguments   */
  LITEDSA_ERR_SHAPE = 2,       /* a shape rule of the operator is violated         */
  LITEDSA_ERR_UNSUPPORTED = 3, /* valid request this build cannot serve            */
  LITEDSA_ERR_CUDA = 4,        /* a CUDA runtime / driver call failed              */
  LITEDSA_ERR_TIMEOUT = 5      /* a device-side bounded wait expired (status word) */
};

/* Version of this ABI (bumped on any signature change). */
int litedsa_abi_version(void);

/* Human-readable text for a LITEDSA_* code (static storage). */
const char* litedsa_error_string(int code);

/*
 * Per-tile union + query-major membership bitmask.
 * Replaces the reference operator
 *   union_qm(topk_indices, u_phys, counts, memb_qm, req_pg, block_table, block_size, seq_space)
 * (kernels/b200/dsa/litedsa.cu:31-75, kernel kernels/b200/dsa/litedsa_union.cuh:34-184).
 *
 *   topk_indices [T, k]  int32, logical positions, -1 (or >= seq_space) = invalid
 *   u_phys       [ng, cap] int32 out: ascending union, physical slots; live prefix = counts[g]
 *   counts       [ng]    int32 out
 *   memb_qm      [ng, G, cap/32] uint32 out: bit r of row (g, q) <=> rank r in token q's list
 *   req_pg       [ng]    int32 request id per tile, or NULL together with block_table
 *   block_table  [bt_rows, bt_blocks] int32 logical block -> physical block, or NULL
 *                (identity: physical slot == logical position)
 * Shape rules (as the reference): T == ng*G, cap == G*k, cap % 128 == 0, G <= 16,
 * G*cap/32 <= 16384, 0 < seq_space <= 2^20 and a multiple of 1024.  Additionally
 * k % 4 == 0.
 * fill_tail == 0: words beyond the live prefixes are left untouched (the reference's
 * overwrite contract, litedsa_union.cuh:22-25); != 0: u_phys tail := -1, mask tail := 0.
 */
int litedsa_union_qm(const int32_t* topk_indices, int32_t* u_phys, int32_t* counts,
                     uint32_t* memb_qm, const int32_t* req_pg, const int32_t* block_table,
                     int T, int k, int ng, int cap, int G, int bt_rows, int bt_blocks,
                     int block_size, int64_t seq_space, int fill_tail, void* stream);

/*
 * Masked FP8 MLA prefill over the per-tile union list.
 * Replaces the reference operator
 *   masked_mla_fp8(q, kv, indices, sm_scale, out_scale, topk_length, memb_qm, h_per_q,
 *                  out, max_logits, lse)
 * (kernels/b200/dsa/litedsa.cu:77-135; kernel litedsa_attention_sm100.cuh:1832-2479),
 * same argument order; tensor shapes/strides are passed as integers.
 *
 *   q8       [ng, 128, 576] e4m3; row r of a tile = token r / h_per_q, head r % h_per_q;
 *            q_row_stride = bytes between consecutive rows (576 when dense, multiple of 16)
 *   kv8      [s_kv, 576] e4m3, kv_row_stride bytes between rows (multiple of 16)
 *   indices  [ng, topk] int32 physical KV slots in ascending rank order,
 *            indices_row_stride = elements between tiles (multiple of 4)
 *   topk_length [ng] int32 live entries per tile (NULL: topk for every tile)
 *   memb_qm  [ng, 128/h_per_q, topk/32] uint32 membership bits (bit r <=> rank r)
 *   out      [ng, 128, 512] bf16 = out_scale * softmax(sm_scale * q.k) @ kv8[:, :512]
 *   max_logits [ng, 128] fp32 (natural-log units) or NULL;  lse [ng, 128] fp32
 *   debug_dump  NULL in production (bring-up aid: raw S / O of tile 0)
 * Rules: topk % 128 == 0; h_per_q divides 128; 128 / h_per_q <= 16; bases 16-byte aligned.
 * A row with no valid key gets out = 0, lse = +inf, max_logits = -inf.
 */
int litedsa_masked_mla_fp8(const void* q8, const void* kv8, const int32_t* indices,
                           float sm_scale, float out_scale, const int32_t* topk_length,
                           const uint32_t* memb_qm, int h_per_q, void* out, float* max_logits,
                           float* lse, int ng, int s_kv, int topk, int64_t q_row_stride,
                           int64_t kv_row_stride, int64_t indices_row_stride,
                           float* debug_dump, void* stream);

/*
 * litedsa_masked_mla_fp8 with the all-gather of a query-sharded multi-GPU run folded into
 * the kernel's epilogue.  Every output box is written to n_outs (1..8) destinations with
 * TMA tile stores: outs[0] is this GPU's [ng, 128, 512] bf16 buffer, outs[1..] are
 * peer-mapped device addresses of the slot this rank owns in each peer's gathered buffer
 * (same shape).  The writes to a peer are complete when this kernel has completed; the
 * caller orders the peers' reads after it (a barrier among the ranks).  No counterpart
 * in the reference, which has no multi-GPU code (its tiles are independent units,
 * kernels/b200/dsa/litedsa_attention_sm100.cuh:1839-1840).
 */
int litedsa_masked_mla_fp8_multi(const void* q8, const void* kv8, const int32_t* indices,
                                 float sm_scale, float out_scale, const int32_t* topk_length,
                                 const uint32_t* memb_qm, int h_per_q, void* const* outs,
                                 int n_outs, float* max_logits, float* lse, int ng, int s_kv,
                                 int topk, int64_t q_row_stride, int64_t kv_row_stride,
                                 int64_t indices_row_stride, void* stream);

/*
 * Synchronous read (and optional reset) of the attention kernels' device status word on
 * the current device.  out4_host[0] = first bounded wait that expired (0 = none),
 * [1] = block, [2] = loop iteration, [3] = launches completed since the last reset.
 * Returns LITEDSA_ERR_TIMEOUT when out4_host[0] != 0.  No counterpart in the reference,
 * whose waits are unbounded (litedsa_attention_sm100.cuh:1965, 2371).
 */
int litedsa_attn_status(int* out4_host, int reset);

/*
 * out_e4m3[i] = e4m3_saturating(in_bf16[i] / scale), i < n.  n % 8 == 0, 16-byte aligned
 * pointers.  Feeds litedsa_masked_mla_fp8 from bf16 queries.  No counterpart in the
 * reference, whose callers hand it e4m3 queries (litedsa_attention_sm100.cuh:2503).
 */
int litedsa_quantize_e4m3(const void* in_bf16, void* out_e4m3, int64_t n, float scale,
                          void* stream);

/*
 * DeepSeek-V3.2 style packed cache rows (656 bytes: 512 e4m3 latent codes | 4 fp32
 * per-128 scales | 64 bf16 rope) -> the 576-byte all-e4m3 row with one scalar scale that
 * litedsa_masked_mla_fp8 (and the reference module, litedsa.cu:82-92) consumes.  Codes
 * are copied, rope is re-encoded as e4m3(rope / scale).  *mismatch_flag (device int32,
 * zeroed by the caller) is set non-zero if some per-128 scale differs from `scale`: such
 * a cache cannot be represented without requantising and must not use this path.
 * out_pitch = bytes between output rows (>= 576, multiple of 16).
 */
int litedsa_repack_kv656(const void* kv656, void* kv576, int s_kv, int64_t out_pitch,
                         float scale, int* mismatch_flag, void* stream);

/*
 * DeepSeek-V4 style packed BF16 attention over two contiguous key ranges.
 * Replaces the reference operator
 *   dsv4_masked_mla_bf16(q, kv, indices, pref, win_lo, win_hi, counts, sm_scale, h_per_q,
 *                        out, lse, attn_sink)            (kernels/b200/dsa/litedsa_dsv4.cu:50-121)
 * for callers whose ranges are contiguous in memory: the gathered union index list and the
 * per-token rank ranges are replaced by the two KV tensors and the first query position.
 * Token t of the call sits at position p = pos0 + t and attends to kv_comp rows
 * [0, min(p / ratio, n_comp)) and kv_raw rows [max(0, p - window + 1), p].
 *
 *   q        [ng, 128, 576] bf16 (row r of a tile = token r / h_per_q, head r % h_per_q)
 *   kv_comp  [n_comp, 576] bf16 (may be NULL when n_comp == 0);  kv_raw [s_raw, 576] bf16
 *   *_row_stride in ELEMENTS (>= 576, multiples of 8); V = the first 512 dims of the same rows
 *   attn_sink [128] fp32 per packed row or NULL: adds exp(sink) to the OUTPUT normaliser only
 *   out [ng, 128, 512] bf16;  lse [ng, 128] fp32 (natural log, without the sink)
 * Requires pos0 + ng * (128 / h_per_q) <= s_raw.
 * The kernel uses all 227 KB of shared memory and needs its dynamic base within 768 bytes of
 * a 1024-byte boundary: the first call on each device launches a one-thread probe and reads
 * its answer back synchronously (make that call outside stream capture); when the base
 * does not fit the call returns LITEDSA_ERR_UNSUPPORTED.
 */
int litedsa_dsv4_c128a_bf16(const void* q, const void* kv_comp, const void* kv_raw, int ng,
                            int h_per_q, int n_comp, int s_raw, int pos0, int window, int ratio,
                            float sm_scale, const float* attn_sink, void* out, float* lse,
                            int64_t q_row_stride, int64_t kc_row_stride, int64_t kr_row_stride,
                            void* stream);

/* Status word of the DSv4 kernel; same meaning and use as litedsa_attn_status. */
int litedsa_dsv4_status(int* out4_host, int reset);

/*
 * Masked FP8 MLA prefill from packed 656-byte cache rows WITHOUT any allocation.
 * This entry point has no counterpart in the reference.  It exists for hosts that are not
 * allowed to call cudaMalloc where attention runs (a runtime that owns all device memory
 * through its own pool, a plugin contract that forbids the callee to allocate, a memory
 * budget frozen at start-up): the temporary 576-byte-row cache that
 * litedsa_repack_kv656 + litedsa_masked_mla_fp8 would need from the caller is a fixed
 * buffer inside the library instead.
 *
 *   kv656   [s_kv, 656] packed rows whose per-128 scales all equal kv_scale
 *   mismatch_flag  device int32 or NULL: set non-zero when some scale differs (result invalid)
 *   every other argument as in litedsa_masked_mla_fp8 (sm_scale multiplies q . k of the CODES,
 *   kv_scale is also the output scale)
 *
 * Limits and rules:
 *   - s_kv <= 65536 rows; longer caches return LITEDSA_ERR_UNSUPPORTED.
 *   - the buffer (about 36 MiB) is part of the library image: every GPU that loads the
 *     library holds it until the process exits.
 *   - the first call on a device looks the buffer's address up; make that call outside
 *     stream capture.
 *   - all calls share the buffer and it keeps the previous call's rows: calls whose GPU
 *     work can overlap (other streams, other threads) race and must be serialised.
 */
int litedsa_masked_mla_fp8_kv656_noalloc(const void* q8, const void* kv656, const int32_t* indices,
                                         float sm_scale, float kv_scale,
                                         const int32_t* topk_length, const uint32_t* memb_qm,
                                         int h_per_q, void* out, float* max_logits, float* lse,
                                         int ng, int s_kv, int topk, int64_t q_row_stride,
                                         int64_t indices_row_stride, int* mismatch_flag,
                                         void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LITEDSA_B200_H_ */

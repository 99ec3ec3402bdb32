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
 * Rules: topk % 128 == 0; h_per_q divides 128; 128 / h_per_q <= 16; bases 16-byte aligned.
 * A row with no valid key gets out = 0, lse = +inf, max_logits = -inf.
 */
int litedsa_masked_mla_fp8(const void* q8, const void* kv8, const int32_t* indices,
                           float sm_scale, float out_scale, const int32_t* topk_length,
                           const uint32_t* memb_qm, int h_per_q, void* out, float* max_logits,
                           float* lse, int ng, int s_kv, int topk, int64_t q_row_stride,
                           int64_t kv_row_stride, int64_t indices_row_stride, void* stream);

/*
 * litedsa_masked_mla_fp8 plus the optional modes that the reference kernel's parameter
 * block carries but its binding leaves switched off (kernels/b200/dsa/litedsa.cu:127-132):
 *   attn_sink [128] fp32 per packed row or NULL: exp(sink) joins the OUTPUT normaliser only,
 *            lse is unchanged (litedsa_attention_sm100.cuh:2127-2133);
 *   topk_length_per_q [ng, 128/h_per_q] int32 or NULL: token q of a tile attends only union
 *            ranks < its bound (a causal prefix of the ascending list); the key-block loop
 *            runs to the LAST token's bound and topk_length is ignored; memb_qm may then be
 *            NULL (litedsa_attention_sm100.cuh:1378-1385, 1846-1851, 1988-1996);
 *   q_group_div >= 1: that many consecutive tiles (slices of one long union list) share ONE
 *            Q tile, so q8 is [ng / q_group_div, 128, 576]; the outputs stay per tile and the
 *            caller merges them with their lse (litedsa_attention_sm100.cuh:1383-1385, 1909).
 *   q_token_stride, q_head_stride, out_token_stride, out_head_stride (ELEMENTS; 0 = the dense
 *            packed layout): in-place addressing of q and out inside [T, H_padded, d] tensors
 *            that hold h_per_q real heads per token.  Row r of tile g is then read at
 *            q8 + (g*G + r / h_per_q) * q_token_stride + (r % h_per_q) * q_head_stride and
 *            written likewise into out, so a tensor-parallel caller needs neither the pack
 *            copy of q nor the unpack copy of out that the reference's packed path pays
 *            (kernels/b200/dsa/DSV4_ZEROCOPY_PLAN.md:12-22, 50-76: planned there, not built).
 *            Pitches must be multiples of 16 bytes; lse / max_logits stay packed [ng, 128].
 */
int litedsa_masked_mla_fp8_ex(const void* q8, const void* kv8, const int32_t* indices,
                              float sm_scale, float out_scale, const int32_t* topk_length,
                              const uint32_t* memb_qm, int h_per_q, void* out, float* max_logits,
                              float* lse, int ng, int s_kv, int topk, int64_t q_row_stride,
                              int64_t kv_row_stride, int64_t indices_row_stride,
                              const float* attn_sink, const int32_t* topk_length_per_q,
                              int q_group_div, int64_t q_token_stride, int64_t q_head_stride,
                              int64_t out_token_stride, int64_t out_head_stride, void* stream);

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
 * Synchronous read (and optional reset) of the FP8 attention kernels' device status block
 * on the current device.  out4_host[0] = first bounded wait that expired since the last
 * reset (0 = none), [1] = its block, [2] = its loop iteration, [3] = launches completed
 * since the last reset.  Returns LITEDSA_ERR_TIMEOUT when out4_host[0] != 0.
 * The record is STICKY: it stays until a call with reset != 0, so a caller that polls it
 * after a batch of launches learns that one of them gave up (that launch's outputs are
 * invalid).  An expired wait ends only its own launch: every launch carries its own epoch,
 * and later launches run normally without a reset.  Entry points themselves stay
 * asynchronous and return LITEDSA_OK at enqueue time.  No counterpart in the reference,
 * whose waits are unbounded (litedsa_attention_sm100.cuh:1965, 2371).
 */
int litedsa_attn_status(int* out4_host, int reset);

/*
 * Limit of one device-side wait for all later launches of this process, in nanoseconds
 * (0 restores the default, 2 s).  *previous_ns (may be NULL) receives the old value.
 */
int litedsa_set_wait_limit_ns(uint64_t limit_ns, uint64_t* previous_ns);

/*
 * Self-test of the bounded wait (for test suites).  Launches a one-warp kernel that waits,
 * with the given limit (1 ns .. 1 s), on an mbarrier nobody arrives on, and synchronises.
 * The wait must give up and the kernel return normally: *returned_device (device int32)
 * becomes 2 (1 would mean the wait succeeded), the FP8 status block records the site, and
 * the function returns LITEDSA_ERR_TIMEOUT -- the expected outcome.  Nothing hangs, traps
 * or faults.  Reset the status block afterwards (litedsa_attn_status(NULL, 1)).
 */
int litedsa_selftest_wait_timeout(uint64_t limit_ns, int* returned_device);

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
 * q_token_stride, q_head_stride, out_token_stride, out_head_stride (ELEMENTS; 0 = the dense
 * packed layout) address q and out in place inside [T, H_padded, d] tensors with h_per_q real
 * heads per token (see litedsa_masked_mla_fp8_ex; kernels/b200/dsa/DSV4_ZEROCOPY_PLAN.md:50-76).
 * The kernel uses all 227 KB of shared memory and needs its dynamic base within 768 bytes of
 * a 1024-byte boundary: the first call on each device launches a one-thread probe and reads
 * its answer back synchronously (make that call outside stream capture); when the base
 * does not fit the call returns LITEDSA_ERR_UNSUPPORTED.
 */
int litedsa_dsv4_c128a_bf16(const void* q, const void* kv_comp, const void* kv_raw, int ng,
                            int h_per_q, int n_comp, int s_raw, int pos0, int window, int ratio,
                            float sm_scale, const float* attn_sink, void* out, float* lse,
                            int64_t q_row_stride, int64_t kc_row_stride, int64_t kr_row_stride,
                            int64_t q_token_stride, int64_t q_head_stride, int64_t out_token_stride,
                            int64_t out_head_stride, void* stream);

/* Status block of the DSv4 kernel; same meaning and use as litedsa_attn_status. */
int litedsa_dsv4_status(int* out4_host, int reset);

/*
 * The reference's DSv4 operator with its own argument list:
 *   dsv4_masked_mla_bf16(q, kv, indices, pref, win_lo, win_hi, counts, sm_scale, h_per_q,
 *                        out, lse, attn_sink)
 * (kernels/b200/dsa/litedsa_dsv4.cu:50-121, export litedsa_dsv4_binding.cu:17-18; kernel
 * litedsa_attention_sm100_dsv4.cuh:1849-2485), tensor shapes/strides passed as integers.
 *
 *   q        [ng, 128, d] bf16 (row r of a tile = token r / h_per_q, head r % h_per_q)
 *   kv       [s_kv, d] bf16 flat workspace; V = the first 512 dims of the same rows
 *   indices  [ng, topk] int32 rows of kv in ascending rank order (-1 / out of range = skipped)
 *   pref, win_lo, win_hi [ng, 128/h_per_q] int32: token q of tile g attends the union ranks
 *            r < pref  or  win_lo <= r < win_hi   (litedsa_attention_sm100_dsv4.cuh:1824-1829,
 *            2015-2025), and only r < counts[g]
 *   counts   [ng] int32 live entries of each tile's list
 *   attn_sink [128] fp32 per packed row or NULL: joins the OUTPUT normaliser only
 *   out [ng, 128, 512] bf16;  lse [ng, 128] fp32 (natural log, without the sink)
 *   d = 512 (the reference's only width) or 576; topk % 64 == 0; strides in ELEMENTS
 *   (q/kv: >= d, multiples of 8; indices: >= topk); q / kv / out 16-byte aligned.
 *   q_token_stride, q_head_stride, out_token_stride, out_head_stride (ELEMENTS; 0 = the dense
 *   packed layout): q and out addressed in place inside [T, H_padded, d] tensors with
 *   h_per_q real heads per token, as in litedsa_masked_mla_fp8_ex -- the zero-copy form the
 *   reference planned for this operator (kernels/b200/dsa/DSV4_ZEROCOPY_PLAN.md:50-76).
 *   workspace, workspace_bytes: NULL / 0, or a caller-owned device buffer of at least
 *   16 + 16 * ng bytes (16-byte aligned).  With a workspace the library first classifies every
 *   tile's index list ON THE DEVICE: when all of them are two contiguous ascending runs of rows
 *   (the packed prefix + sliding window lists this operator exists for) the attention runs in
 *   a kernel that reads K and V with plain tiled TMA loads instead of gathering rows; otherwise
 *   the gather kernel runs.  Both kernels are enqueued and one of them returns at once, so
 *   there is no host synchronisation and the results are the same to rounding (block
 *   boundaries of the online softmax differ).  The workspace may be reused by later calls on
 *   the same stream.
 * With d = 576 or a workspace the first call on a device reads a one-thread probe back
 * synchronously (dynamic shared-memory alignment): make that call outside stream capture.
 */
int litedsa_dsv4_masked_mla_bf16(const void* q, const void* kv, const int32_t* indices,
                                 const int32_t* pref, const int32_t* win_lo,
                                 const int32_t* win_hi, const int32_t* counts, float sm_scale,
                                 int h_per_q, void* out, float* lse, const float* attn_sink,
                                 int ng, int s_kv, int topk, int d, int64_t q_row_stride,
                                 int64_t kv_row_stride, int64_t indices_row_stride,
                                 int64_t q_token_stride, int64_t q_head_stride,
                                 int64_t out_token_stride, int64_t out_head_stride,
                                 void* workspace, int64_t workspace_bytes, void* stream);

/*
 * masked_mla_fp8's bf16 twin for KV caches that have no single-scale all-e4m3 form (per-128
 * scales that differ, bf16 rope -- the DeepSeek-V3.2 cache row): bf16 q and a bf16 KV
 * workspace (see litedsa_dequant_kv656), the union list and query-major membership mask of
 * litedsa_union_qm.  Argument order of masked_mla_fp8 (kernels/b200/dsa/litedsa.cu:77-80)
 * without out_scale; numerics of the reference's bf16 kernel (64-key blocks, bf16 P,
 * litedsa_attention_sm100_dsv4.cuh:2072-2083), accurate to bf16 rounding.
 *
 *   q [ng, 128, d] bf16, kv [s_kv, d] bf16 (d = 576 or 512; V = first 512 dims), strides in
 *   ELEMENTS; indices [ng, topk] int32; topk_length [ng] or NULL; memb_qm [ng, G, topk/32];
 *   out [ng, 128, 512] bf16; max_logits [ng, 128] or NULL; lse [ng, 128]; attn_sink [128] or
 *   NULL.  topk % 128 == 0.
 */
int litedsa_masked_mla_bf16(const void* q, const void* kv, const int32_t* indices, float sm_scale,
                            const int32_t* topk_length, const uint32_t* memb_qm, int h_per_q,
                            void* out, float* max_logits, float* lse, int ng, int s_kv, int topk,
                            int d, int64_t q_row_stride, int64_t kv_row_stride,
                            int64_t indices_row_stride, const float* attn_sink, void* stream);

/*
 * Packed 656-byte cache rows (512 e4m3 codes | 4 fp32 per-128 scales | 64 bf16 rope) ->
 * bf16 rows [s_kv, 576]: latent = code x the scale of its 128-dim chunk, rope copied.
 * out_pitch = BYTES between output rows (>= 1152, multiple of 16).  The reference's bf16
 * operator consumes such a "flat dequantised workspace" (litedsa_dsv4.cu:40-48).
 */
int litedsa_dequant_kv656(const void* kv656, void* kv_bf16, int s_kv, int64_t out_pitch,
                          void* stream);

/*
 * Merge of KV-split attention outputs: the q_group_div consecutive tiles that shared one Q tile
 * in litedsa_masked_mla_fp8_ex are combined with their lse into the attention over the whole
 * union list.  The reference carries q_group_div in its kernel and leaves the merge to the
 * caller (kernels/b200/dsa/litedsa_attention_sm100.cuh:1383-1385, 1909).
 *
 *   out_parts [ng, 128, 512] bf16, lse_parts [ng, 128] fp32 (+inf = a part without keys),
 *   max_parts [ng, 128] or NULL; attn_sink [128] or NULL: the array the attention call got
 *   (a part is normalised by its own row sum plus the sink, lse excludes the sink);
 *   out [ng / q_group_div, 128, 512] bf16, lse [ng / q_group_div, 128], max_logits likewise
 *   or NULL (given exactly when max_parts is).  q_group_div <= 32; out_parts and out 16-byte
 *   aligned.  A row all of whose parts are empty gets out = 0, lse = +inf.
 */
int litedsa_merge_kv_splits(const void* out_parts, const float* lse_parts, const float* max_parts,
                            const float* attn_sink, void* out, float* lse, float* max_logits,
                            int ng, int q_group_div, void* stream);

/* Status block of the bf16 gather kernel; same meaning and use as litedsa_attn_status. */
int litedsa_bf16_status(int* out4_host, int reset);

/*
 * Measurement aid: the dense tcgen05 tensor-core rate of the current device in TFLOP/s,
 * measured by a kernel that only issues MMAs from shared memory on every SM pair
 * (synchronous, a few milliseconds).  kind 0 = FP8 e4m3 (kind::f8f6f4), 1 = bf16
 * (kind::f16); m_pair = 256 (128 rows per CTA of a pair: the peak shape) or 128 (64 rows
 * per CTA: the attention kernels' shape); N = 256; iters = MMAs per pair (multiple of 8,
 * >= 64).  *tflops_out is a HOST double.  The benchmark's FP8 roofline denominator comes
 * from here.  No counterpart in the reference.
 */
int litedsa_probe_mma_tflops(int kind, int m_pair, int iters, double* tflops_out);

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

/*
 * The step before the union: index logits and top-k selection, producing the
 * `topk_indices [T, k] i32` tensor that litedsa_union_qm takes
 * (kernels/b200/dsa/litedsa.cu:31-33).  The reference repository removed its own indexer
 * (README.md:3-6), so these two entry points have NO counterpart there; they implement the
 * published FP8 form of the DeepSeek-V3.2 lightning indexer:
 *
 *   logit[t, s] = k_scale[s] * sum_h weights[t, h] * relu(q_idx8[t, h, :] . k_idx8[s, :])
 *
 * for the T query tokens at positions q_pos0 .. q_pos0 + T - 1 and the keys s <= position.
 *   q_idx8   [T, Hi, 128] e4m3 codes, dense, Hi in {32, 64, 128}
 *   k_idx8   [S, 128] e4m3 codes, rows k_row_stride bytes apart (multiple of 16)
 *   weights  [T, Hi] fp32 (head weight x query scale x softmax scale)
 *   k_scale  [S] fp32 or NULL (1.0)
 *   logits   [T, logits_row_stride] fp32.  All S entries of every row are written: the
 *            logit for s <= q_pos0 + t, -inf beyond the token's position (litedsa_topk_select
 *            never reads those).
 * Asynchronous on `stream`; bounded waits report through litedsa_index_status.
 */
int litedsa_index_logits_fp8(const void* q_idx8, const void* k_idx8, const float* weights,
                             const float* k_scale, float* logits, int T, int Hi, int S, int q_pos0,
                             long long k_row_stride, long long logits_row_stride, void* stream);

/*
 * Exact top-k of every row of `logits`: topk_idx[t, :] = the k positions i < len(t) with the
 * largest values; ties at the k-th value go to the smaller positions; NaN sorts below every
 * number.  The selected SET is exact and reproducible; the order inside a row is fixed for a
 * given input but not specified (the union operator does not depend on it).  Rows with
 * len(t) <= k list 0 .. len(t) - 1 and are padded with -1 at the end.  len(t) = lengths[t] (clamped to [0, S]) or, when lengths is NULL,
 * min(S, q_pos0 + t + 1) (causal).  No allocation, no host synchronisation.
 */
int litedsa_topk_select(const float* logits, const int32_t* lengths, int32_t* topk_idx, int T, int S,
                        int k, int q_pos0, long long logits_row_stride, void* stream);

/* Status block of the index-logits kernel; same layout and return rule as litedsa_attn_status. */
int litedsa_index_status(int* out4_host, int reset);

#ifdef __cplusplus
}
#endif
#endif /* LITEDSA_B200_H_ */

// The step before the union: index logits and top-k selection (sm_100a).
//
// The reference repository no longer carries its indexer ("The repository-local LiteTopK
// indexer and standalone MS MARCO top-k kernels have been removed", README.md:3-6); what its
// attention path consumes is the result, `topk_indices [T, k] i32` with -1 padding
// (kernels/b200/dsa/litedsa.cu:31-33).  This file produces that tensor from the published
// formulation of the DeepSeek-V3.2 lightning indexer in its FP8 form:
//
//   logit[t, s] = k_scale[s] * sum_h  weights[t, h] * relu( q8[t, h, :] . k8[s, :] )     (s <= pos(t))
//   topk_idx[t, :] = the k positions s <= pos(t) with the largest logits (all of them and -1
//                    padding when fewer than k exist)
//
// with q8 [T, Hi, 128] and k8 [S, 128] e4m3 codes, weights [T, Hi] fp32 (head weight x query
// scale x softmax scale), k_scale [S] fp32 and pos(t) = q_pos0 + t.  Nothing here has a
// counterpart in the reference to be checked against; the CPU oracle restates the formula.
//
// index_logits_kernel (tensor-bound): the product is computed TRANSPOSED, keys on the M axis,
// so that the head sum of a (token, key) pair is a sum along one accumulator row, i.e. inside
// one thread.  One CTA owns 2 x 256 / Hi tokens: their q rows are the B operand of two
// N = 256 accumulators (512 TMEM columns); the K tiles (128 keys x 128 bytes, TMA, four
// stages) are the A operand and are streamed once per CTA, up to the causal bound of its
// last token.  While the tensor core fills one accumulator, four warps drain the other:
// tcgen05.ld, relu, multiply by the head weight, add; then x k_scale, causal mask, and 128
// consecutive fp32 logits per token leave each warp as coalesced stores.
//
// topk_select_kernel (memory-bound): one CTA per token row.  Exact radix select (11 + 11 + 10
// bits of the order-preserving integer image of the fp32 logits) over the row held in shared
// memory, then one ordered emission pass: the output is ascending in position, ties at the
// k-th value are resolved towards the smaller position, so the result is deterministic.
#include "common.cuh"
#include "tensor_map.cuh"

namespace lt {
namespace idx {

// ------------------------------------------------------------------ index logits
constexpr int kThreads = 384;
constexpr int kKeyTile = 128;             // keys per MMA (M)
constexpr int kCols = 256;                // (token, head) columns per accumulator (N)
constexpr int kDim = 128;                 // index head dim = bytes per row
constexpr int kStages = 4;
constexpr uint32_t kQTile = kCols * kDim;       // 32 KB
constexpr uint32_t kKTile = kKeyTile * kDim;    // 16 KB
constexpr uint32_t kOffQ = 0;
constexpr uint32_t kOffK = kOffQ + 2 * kQTile;
constexpr uint32_t kOffW = kOffK + kStages * kKTile;
constexpr uint32_t kOffBar = kOffW + 2 * kCols * 4;
constexpr uint32_t kSmem = kOffBar + 256 + 1024;   // + alignment slack

struct Bars {
  uint64_t q_full, k_full[kStages], k_free[kStages], acc_full[2], acc_free[2];
  uint32_t tmem_base;
};
static_assert(sizeof(Bars) <= 256, "barrier block too large");

struct LogitParams {
  const float* weights;     // [T, Hi]
  const float* k_scale;     // [S] or null (1.0)
  float* logits;            // [T, ld]
  int T, Hi, S, q_pos0;
  long long ld;
  int epoch;
  unsigned long long wait_limit_ns;
};

enum { kSiteQFull = 1, kSiteKFull, kSiteKFree, kSiteAccFull, kSiteAccFree };

__device__ int g_status[8];

template <int HI>
__global__ void __launch_bounds__(kThreads, 1)
index_logits_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const LogitParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (sbase - raw);
  float* wsm = reinterpret_cast<float*>(sm + kOffW);
  Bars& bar = *reinterpret_cast<Bars*>(sm + kOffBar);
  const Waiter wt{g_status, p.epoch, p.wait_limit_ns};

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  constexpr int tpa = kCols / HI;               // tokens per accumulator
  const int tok0 = blockIdx.x * 2 * tpa;        // first token of this CTA
  const int tok_end = min(p.T, tok0 + 2 * tpa);
  // key tiles up to the causal bound of the CTA's last token
  const int pos_max = p.q_pos0 + tok_end - 1;
  const int n_tiles = min((p.S + kKeyTile - 1) / kKeyTile, pos_max / kKeyTile + 1);

  if (threadIdx.x == 0) {
    mbar_init(&bar.q_full, 1);
    for (int i = 0; i < kStages; ++i) { mbar_init(&bar.k_full[i], 1); mbar_init(&bar.k_free[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bar.acc_full[i], 1); mbar_init(&bar.acc_free[i], 4); }
    fence_mbar_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
  }
  // head weights of the CTA's tokens: column c of accumulator a is row tok0 * Hi + 256 a + c
  for (int i = threadIdx.x; i < 2 * kCols; i += kThreads) {
    const long long r = (long long)tok0 * HI + i;
    wsm[i] = r < (long long)p.T * HI ? __ldg(p.weights + r) : 0.f;
  }
  __syncthreads();
  if (warp == 2) {
    tmem_alloc_cta(&bar.tmem_base, 512);
    tmem_relinquish_cta();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bar.tmem_base;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      const uint64_t pol_keep = l2_policy_evict_last(), pol_stream = l2_policy_evict_first();
      mbar_arrive_expect_tx(&bar.q_full, 2 * kQTile);
      tma_load_2d_hint(sbase + kOffQ, &map_q, 0, tok0 * HI, &bar.q_full, pol_stream);
      tma_load_2d_hint(sbase + kOffQ + kQTile, &map_q, 0, tok0 * HI + kCols, &bar.q_full, pol_stream);
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % kStages;
        if (j >= kStages && !mbar_wait(&bar.k_free[s], ((j / kStages) & 1) ^ 1, wt, kSiteKFree, j)) break;
        mbar_arrive_expect_tx(&bar.k_full[s], kKTile);
        tma_load_2d_hint(sbase + kOffK + s * kKTile, &map_k, 0, j * kKeyTile, &bar.k_full[s], pol_keep);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue (one thread)
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(0, 0, false, false, kKeyTile, kCols);
      bool ok = mbar_wait(&bar.q_full, 0, wt, kSiteQFull, 0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % kStages;
        ok = mbar_wait(&bar.k_full[s], (j / kStages) & 1, wt, kSiteKFull, j);
        if (!ok) break;
        const uint64_t ad = umma_desc(sbase + kOffK + s * kKTile, 16, 1024, kSwz128);
        for (int a = 0; a < 2 && ok; ++a) {
          // accumulator a still holds tile j-1 until its four warps have read it
          if (j > 0) ok = mbar_wait(&bar.acc_free[a], (j - 1) & 1, wt, kSiteAccFree, j);
          if (!ok) break;
          tc_fence_after();
          const uint64_t bd = umma_desc(sbase + kOffQ + a * kQTile, 16, 1024, kSwz128);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            mma_f8_cta(tmem + a * kCols, ad + 2 * kk, bd + 2 * kk, idesc, kk ? 1u : 0u);
          mma_commit_cta(&bar.acc_full[a]);
        }
        mma_commit_cta(&bar.k_free[s]);     // both accumulators have read the K tile
      }
    }
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- accumulator drain
    const int a = (warp - 4) >> 2;                      // which accumulator
    const int q4 = warp & 3;                            // TMEM lane quarter of this warp
    const int krow = 32 * q4 + lane;                    // key row of the tile = TMEM lane
    const uint32_t tcol = tmem + ((uint32_t)(32 * q4) << 16) + a * kCols;
    const float* w = wsm + a * kCols;
    const int t_base = tok0 + a * tpa;
    for (int j = 0; j < n_tiles; ++j) {
      if (!mbar_wait(&bar.acc_full[a], j & 1, wt, kSiteAccFull, j)) break;
      __syncwarp();
      tc_fence_after();
      float acc[tpa];
#pragma unroll
      for (int i = 0; i < tpa; ++i) acc[i] = 0.f;
      float x[2][32];
      tmem_ld32(tcol, x[0]);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        tmem_wait_ld();
        if (c < 7) tmem_ld32(tcol + 32 * (c + 1), x[(c + 1) & 1]);
        const float* xc = x[c & 1];
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 w4 = *reinterpret_cast<const float4*>(w + 32 * c + i);
          sum = fmaf(fmaxf(xc[i], 0.f), w4.x, sum);
          sum = fmaf(fmaxf(xc[i + 1], 0.f), w4.y, sum);
          sum = fmaf(fmaxf(xc[i + 2], 0.f), w4.z, sum);
          sum = fmaf(fmaxf(xc[i + 3], 0.f), w4.w, sum);
        }
        acc[(32 * c) / HI] += sum;   // a 32-column chunk never straddles two tokens (HI >= 32)
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.acc_free[a]);
      // scale, causal mask, store: lanes of a warp hold 32 consecutive keys
      const int s_key = j * kKeyTile + krow;
      if (s_key < p.S) {
        const float ks = p.k_scale ? __ldg(p.k_scale + s_key) : 1.f;
#pragma unroll
        for (int tt = 0; tt < tpa; ++tt) {
          const int t = t_base + tt;
          if (t >= p.T) continue;
          const float v = s_key <= p.q_pos0 + t ? acc[tt] * ks : -INFINITY;
          p.logits[(long long)t * p.ld + s_key] = v;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    __syncwarp();
    tmem_dealloc_cta(tmem, 512);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(&g_status[3], 1);
}

// ------------------------------------------------------------------ top-k selection
constexpr int kSelThreads = 512;
constexpr int kBins = 2048;
constexpr int kMaxSmemRow = 49152;       // keys of a row held in shared memory (192 KB)

struct SelParams {
  const float* logits;      // [T, ld]
  const int32_t* lengths;   // [T] valid prefix per row, or null: min(S, q_pos0 + t + 1)
  int32_t* out;             // [T, k]
  int T, S, k, q_pos0;
  long long ld;
};

// order-preserving map fp32 -> u32 (NaN sorts lowest)
__device__ __forceinline__ uint32_t okey(float f) {
  if (f != f) return 0u;
  const uint32_t b = __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

template <bool kSmemRow>
__global__ void __launch_bounds__(kSelThreads)
topk_select_kernel(const SelParams p) {
  extern __shared__ __align__(16) uint32_t rowkeys[];
  __shared__ uint32_t hist[kBins];
  __shared__ uint32_t warp_tot[kSelThreads / 32];
  __shared__ uint32_t sel_bin, sel_rem;
  __shared__ uint32_t wgt[kSelThreads / 32], weq[kSelThreads / 32];

  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int n = p.lengths ? min(max(p.lengths[t], 0), p.S) : min(p.S, max(p.q_pos0 + t + 1, 0));
  int32_t* out = p.out + (long long)t * p.k;
  const float* row = p.logits + (long long)t * p.ld;
  if (n <= p.k) {            // everything valid is selected
    for (int i = tid; i < p.k; i += kSelThreads) out[i] = i < n ? i : -1;
    return;
  }
  if (kSmemRow) {
    for (int i = tid; i < n; i += kSelThreads) rowkeys[i] = okey(__ldg(row + i));
    __syncthreads();
  }
  auto key_at = [&](int i) -> uint32_t { return kSmemRow ? rowkeys[i] : okey(__ldg(row + i)); };

  // three digits, most significant first: (shift, bits) = (21, 11), (10, 11), (0, 10)
  uint32_t prefix = 0, prefix_mask = 0, rem = (uint32_t)p.k;
#pragma unroll 1
  for (int pass = 0; pass < 3; ++pass) {
    const int shift = pass == 0 ? 21 : (pass == 1 ? 10 : 0);
    const uint32_t dmask = pass == 2 ? 0x3FFu : 0x7FFu;
    for (int i = tid; i < kBins; i += kSelThreads) hist[i] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += kSelThreads) {
      const uint32_t u = key_at(i);
      if ((u & prefix_mask) == prefix) atomicAdd(&hist[(u >> shift) & dmask], 1u);
    }
    __syncthreads();
    // thread i owns bins 4i .. 4i+3; suffix sums from the top: find the bin b with
    // count(bins > b) < rem <= count(bins >= b)
    const uint32_t h0 = hist[4 * tid], h1 = hist[4 * tid + 1], h2 = hist[4 * tid + 2], h3 = hist[4 * tid + 3];
    const uint32_t mine = h0 + h1 + h2 + h3;
    uint32_t incl = mine;                    // inclusive suffix sum within the warp (towards higher lanes)
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t v = __shfl_down_sync(0xffffffffu, incl, off);
      if (lane + off < 32) incl += v;
    }
    if (lane == 0) warp_tot[wid] = incl;
    __syncthreads();
    uint32_t above = 0;                      // elements in bins owned by higher threads
    for (int w = wid + 1; w < kSelThreads / 32; ++w) above += warp_tot[w];
    above += incl - mine;
    if (above < rem && rem <= above + mine) {          // the crossing is in my four bins
      uint32_t a = above;
      int b = 4 * tid + 3;
      if (a + h3 >= rem) { b = 4 * tid + 3; }
      else if ((a += h3, a + h2 >= rem)) { b = 4 * tid + 2; }
      else if ((a += h2, a + h1 >= rem)) { b = 4 * tid + 1; }
      else { a += h1; b = 4 * tid; }
      sel_bin = (uint32_t)b;
      sel_rem = rem - a;
    }
    __syncthreads();
    prefix |= sel_bin << shift;
    prefix_mask |= dmask << shift;
    rem = sel_rem;
    __syncthreads();
  }
  // prefix = the k-th largest key; rem = how many elements equal to it are taken (smallest
  // positions first).  Ordered emission: warp w owns a contiguous segment of the row.
  const uint32_t kth = prefix;
  const int seg = (((n + kSelThreads / 32 - 1) / (kSelThreads / 32)) + 31) & ~31;
  const int s0 = min(wid * seg, n), s1 = min(s0 + seg, n);
  uint32_t cgt = 0, ceq = 0;
  for (int i = s0 + lane; i < s1; i += 32) {
    const uint32_t u = key_at(i);
    cgt += u > kth;
    ceq += u == kth;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    cgt += __shfl_xor_sync(0xffffffffu, cgt, off);
    ceq += __shfl_xor_sync(0xffffffffu, ceq, off);
  }
  if (lane == 0) { wgt[wid] = cgt; weq[wid] = ceq; }
  __syncthreads();
  uint32_t gt_run = 0, eq_run = 0;
  for (int w = 0; w < wid; ++w) { gt_run += wgt[w]; eq_run += weq[w]; }
  const uint32_t lt_mask = (1u << lane) - 1u;
  for (int i0 = s0; i0 < s1; i0 += 32) {
    const int i = i0 + lane;
    const uint32_t u = i < s1 ? key_at(i) : 0u;
    const bool gt = i < s1 && u > kth, eq = i < s1 && u == kth;
    const uint32_t bg = __ballot_sync(0xffffffffu, gt), be = __ballot_sync(0xffffffffu, eq);
    const uint32_t gt_before = gt_run + __popc(bg & lt_mask);
    const uint32_t eq_before = eq_run + __popc(be & lt_mask);
    if (gt || (eq && eq_before < rem)) {
      const uint32_t slot = gt_before + min(eq_before, rem);
      if (slot < (uint32_t)p.k) out[slot] = i;
    }
    gt_run += __popc(bg);
    eq_run += __popc(be);
  }
}

}  // namespace idx
}  // namespace lt

// Index logits of T query tokens at positions q_pos0 .. q_pos0 + T - 1 against S keys.
//   q_idx8  [T, Hi, 128] e4m3 codes, dense; Hi in {32, 64, 128}
//   k_idx8  [S, 128] e4m3 codes, rows k_row_stride bytes apart (multiple of 16)
//   weights [T, Hi] fp32;  k_scale [S] fp32 or null (1.0)
//   logits  [T, logits_row_stride] fp32: entries s <= q_pos0 + t are written, entries beyond a
//           token's position inside the processed tiles are -inf, later ones are left untouched
// No counterpart in the reference (its indexer was removed); asynchronous on `stream`.
extern "C" int litedsa_index_logits_fp8(const void* q_idx8, const void* k_idx8, const float* weights,
                                        const float* k_scale, float* logits, int T, int Hi, int S,
                                        int q_pos0, long long k_row_stride,
                                        long long logits_row_stride, void* stream) {
  using namespace lt;
  using namespace lt::idx;
  if (!q_idx8 || !k_idx8 || !weights || !logits) return LITEDSA_ERR_ARG;
  if (T <= 0 || S <= 0 || q_pos0 < 0) return LITEDSA_ERR_SHAPE;
  if (Hi != 32 && Hi != 64 && Hi != 128) return LITEDSA_ERR_UNSUPPORTED;
  if (logits_row_stride < S || k_row_stride < kDim || k_row_stride % 16) return LITEDSA_ERR_SHAPE;
  if (((uintptr_t)q_idx8 | (uintptr_t)k_idx8) & 15) return LITEDSA_ERR_UNSUPPORTED;
  if ((long long)T * Hi > 0x7fffffffLL) return LITEDSA_ERR_UNSUPPORTED;
  CUtensorMap map_q, map_k;
  if (!make_map_2d(&map_q, q_idx8, CU_TENSOR_MAP_DATA_TYPE_UINT8, kDim, (uint64_t)T * Hi, kDim, kDim, kCols) ||
      !make_map_2d(&map_k, k_idx8, CU_TENSOR_MAP_DATA_TYPE_UINT8, kDim, (uint64_t)S,
                   (uint64_t)k_row_stride, kDim, kKeyTile))
    return LITEDSA_ERR_CUDA;
  LogitParams p;
  p.weights = weights; p.k_scale = k_scale; p.logits = logits;
  p.T = T; p.Hi = Hi; p.S = S; p.q_pos0 = q_pos0; p.ld = logits_row_stride;
  p.epoch = next_launch_epoch(); p.wait_limit_ns = wait_limit_ns();
  auto kern = Hi == 32 ? index_logits_kernel<32> : (Hi == 64 ? index_logits_kernel<64> : index_logits_kernel<128>);
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem) != cudaSuccess)
    return LITEDSA_ERR_CUDA;
  const int tok_per_cta = 2 * (kCols / Hi);
  const int grid = (T + tok_per_cta - 1) / tok_per_cta;
  kern<<<grid, kThreads, kSmem, reinterpret_cast<cudaStream_t>(stream)>>>(map_q, map_k, p);
  return cudaGetLastError() == cudaSuccess ? LITEDSA_OK : LITEDSA_ERR_CUDA;
}

// Exact top-k per row of `logits`: topk_idx[t, :] = the k positions i < len(t) with the largest
// values, ascending in position, ties at the k-th value resolved towards smaller positions;
// rows with len(t) <= k list 0 .. len(t) - 1 and are padded with -1.  len(t) = lengths[t], or
// min(S, q_pos0 + t + 1) when lengths is null (causal).  NaN sorts below every number.
// The output is what the union operator takes as topk_indices
// (kernels/b200/dsa/litedsa.cu:31-33).  No allocation; asynchronous on `stream`.
extern "C" int litedsa_topk_select(const float* logits, const int32_t* lengths, int32_t* topk_idx,
                                   int T, int S, int k, int q_pos0, long long logits_row_stride,
                                   void* stream) {
  using namespace lt::idx;
  if (!logits || !topk_idx) return LITEDSA_ERR_ARG;
  if (T <= 0 || S <= 0 || k <= 0 || logits_row_stride < S) return LITEDSA_ERR_SHAPE;
  SelParams p;
  p.logits = logits; p.lengths = lengths; p.out = topk_idx;
  p.T = T; p.S = S; p.k = k; p.q_pos0 = q_pos0; p.ld = logits_row_stride;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (S <= kMaxSmemRow) {
    const size_t smem = (size_t)S * 4;
    if (cudaFuncSetAttribute(topk_select_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return LITEDSA_ERR_CUDA;
    topk_select_kernel<true><<<T, kSelThreads, smem, st>>>(p);
  } else {
    topk_select_kernel<false><<<T, kSelThreads, 0, st>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? LITEDSA_OK : LITEDSA_ERR_CUDA;
}

// Status block of the index-logits kernel (same layout as litedsa_attn_status).
extern "C" int litedsa_index_status(int* out4_host, int reset) {
  using namespace lt::idx;
  if (out4_host && cudaMemcpyFromSymbol(out4_host, g_status, sizeof(int) * 4) != cudaSuccess)
    return LITEDSA_ERR_CUDA;
  if (reset) {
    const int z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (cudaMemcpyToSymbol(g_status, z, sizeof(z)) != cudaSuccess) return LITEDSA_ERR_CUDA;
  }
  return (out4_host && out4_host[0] != 0) ? LITEDSA_ERR_TIMEOUT : LITEDSA_OK;
}

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
// last token.  While the tensor core fills one accumulator, eight warps drain the other
// (lane quarter x column half): tcgen05.ld, relu, multiply by the head weight, add; then
// x k_scale, causal mask, and 128 consecutive fp32 logits per token leave each warp as
// coalesced stores.
//
// topk_select (memory-bound): exact selection per token row.  Rows up to 32768 entries go
// through persistent CTAs that prefetch the next row with a bulk copy while the current one
// is processed from registers (value-linear histogram, exact ranking of the threshold bin);
// longer rows through a radix select over the order-preserving integer image of the logits.
// Ties at the k-th value are resolved towards the smaller position, so the selected set is
// deterministic; the order inside a row is not specified.
#include "common.cuh"
#include "tensor_map.cuh"

namespace lt {
namespace idx {

// ------------------------------------------------------------------ index logits
constexpr int kThreads = 640;             // TMA, MMA, TMEM warps + 16 drain warps
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

// packed fp32 pair fma (one issue slot for two lanes of work)
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(reinterpret_cast<unsigned long long&>(d))
      : "l"(reinterpret_cast<unsigned long long&>(a)), "l"(reinterpret_cast<unsigned long long&>(b)),
        "l"(reinterpret_cast<unsigned long long&>(c)));
  return d;
}

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
    for (int i = 0; i < 2; ++i) { mbar_init(&bar.acc_full[i], 1); mbar_init(&bar.acc_free[i], 8); }
    fence_mbar_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
  }
  // head weights of the CTA's tokens: column c of accumulator a is row tok0 * Hi + 256 a + c.
  // Halved: the drain computes relu(x) as (x + |x|) / 2 with the division folded in here.
  for (int i = threadIdx.x; i < 2 * kCols; i += kThreads) {
    const long long r = (long long)tok0 * HI + i;
    wsm[i] = r < (long long)p.T * HI ? 0.5f * __ldg(p.weights + r) : 0.f;
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
    // Sixteen warps: accumulator a, column half hf (128 columns = tpa / 2 whole tokens), TMEM
    // lane quarter q4.  relu(x) * w is computed as (x + |x|) * (w / 2): an add with an absolute-
    // value operand and a packed fma, both on the fma pipe (a max would go to the half-rate
    // integer pipe, which then paces the kernel).
    const int dw = warp - 4;
    const int a = dw >> 3, hf = (dw >> 2) & 1;
    const int q4 = warp & 3;                            // TMEM lane quarter of this warp
    const int krow = 32 * q4 + lane;                    // key row of the tile = TMEM lane
    const uint32_t tcol = tmem + ((uint32_t)(32 * q4) << 16) + a * kCols + 128 * hf;
    const float* w = wsm + a * kCols + 128 * hf;
    constexpr int tph = tpa / 2;                        // tokens per column half
    const int t_base = tok0 + a * tpa + hf * tph;
    // Key tiles beyond the causal bound of the CTA's last token are not computed: their entries
    // are -inf for every token of the CTA (this warp's tokens and key rows).  Written first,
    // while the tensor core fills the first accumulators.
    for (int j = n_tiles; j * kKeyTile < p.S; ++j) {
      const int s_key = j * kKeyTile + krow;
      if (s_key < p.S) {
#pragma unroll
        for (int tt = 0; tt < tph; ++tt) {
          const int t = t_base + tt;
          if (t < p.T) p.logits[(long long)t * p.ld + s_key] = -INFINITY;
        }
      }
    }
    for (int j = 0; j < n_tiles; ++j) {
      // this key's scale is fetched before the wait, so its latency hides behind the MMAs
      const int s_key = j * kKeyTile + krow;
      const float ks = (p.k_scale && s_key < p.S) ? __ldg(p.k_scale + s_key) : 1.f;
      if (!mbar_wait(&bar.acc_full[a], j & 1, wt, kSiteAccFull, j)) break;
      __syncwarp();
      tc_fence_after();
      float acc[tph];
      float x[2][32];
      tmem_ld32(tcol, x[0]);
      // two packed fma chains (four independent partial sums), carried over the 32-column chunks
      // of one token and folded when the token's last chunk is done (a chunk never straddles two
      // tokens)
      float2 s0 = make_float2(0.f, 0.f), s1 = make_float2(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        tmem_wait_ld();
        if (c < 3) tmem_ld32(tcol + 32 * (c + 1), x[(c + 1) & 1]);
        const float* xc = x[c & 1];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 w4 = *reinterpret_cast<const float4*>(w + 32 * c + i);
          s0 = fma2(make_float2(xc[i] + fabsf(xc[i]), xc[i + 1] + fabsf(xc[i + 1])), make_float2(w4.x, w4.y), s0);
          s1 = fma2(make_float2(xc[i + 2] + fabsf(xc[i + 2]), xc[i + 3] + fabsf(xc[i + 3])),
                    make_float2(w4.z, w4.w), s1);
        }
        if ((32 * (c + 1)) % HI == 0 || c == 3) {
          acc[(32 * c) / HI] = (s0.x + s0.y) + (s1.x + s1.y);
          s0 = make_float2(0.f, 0.f);
          s1 = make_float2(0.f, 0.f);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar.acc_free[a]);
      // scale, causal mask, store: lanes of a warp hold 32 consecutive keys
      if (s_key < p.S) {
#pragma unroll
        for (int tt = 0; tt < tph; ++tt) {
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
constexpr int kBins = 2048;
constexpr int kMaxSmemRow = 49152;       // keys of a row held in shared memory (192 KB)
constexpr int kCandCap = 4096;           // keys of the threshold bin kept in shared memory

struct SelParams {
  const float* logits;      // [T, ld]
  const int32_t* lengths;   // [T] valid prefix per row, or null: min(S, q_pos0 + t + 1)
  int32_t* out;             // [T, k]
  int T, S, k, q_pos0;
  long long ld;
  int epoch;
  unsigned long long wait_limit_ns;
};

// order-preserving map fp32 -> u32 (NaN sorts lowest, -0 and +0 share one key) and its inverse
__device__ __forceinline__ uint32_t okey(float f) {
  if (f != f) return 0u;
  const uint32_t b = f == 0.f ? 0u : __float_as_uint(f);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float okey_inv(uint32_t u) {
  return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}

struct SelShared {
  uint32_t hist[kBins];
  uint32_t cand[kCandCap];
  uint32_t wa[32], wb[32];
  uint32_t sel_bin, sel_rem, n_cand, kth, ties;
};

// block-wide max / min of two values (all threads get the result); ends with a barrier
template <int NT>
__device__ __forceinline__ void block_max_min(SelShared& sh, uint32_t& vmax, uint32_t& vmin) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    vmax = max(vmax, __shfl_xor_sync(0xffffffffu, vmax, off));
    vmin = min(vmin, __shfl_xor_sync(0xffffffffu, vmin, off));
  }
  if (lane == 0) { sh.wa[wid] = vmax; sh.wb[wid] = vmin; }
  __syncthreads();
  uint32_t a = lane < NT / 32 ? sh.wa[lane] : 0u, b = lane < NT / 32 ? sh.wb[lane] : 0xffffffffu;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    a = max(a, __shfl_xor_sync(0xffffffffu, a, off));
    b = min(b, __shfl_xor_sync(0xffffffffu, b, off));
  }
  vmax = a; vmin = b;
  __syncthreads();
}

// Block-wide: given hist[0 .. kBins) and `rem`, find the bin b with count(bins > b) < rem <=
// count(bins >= b); returns b and the rank inside the bin (rem - count(bins > b)).  Thread i
// owns kBins / NT consecutive bins.  Ends with a barrier; hist may be reused afterwards.
template <int NT>
__device__ __forceinline__ uint32_t find_bin(SelShared& sh, uint32_t rem, uint32_t* rem_out) {
  constexpr int BPT = kBins / NT;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  uint32_t h[BPT], mine = 0;
#pragma unroll
  for (int i = 0; i < BPT; ++i) { h[i] = sh.hist[BPT * tid + i]; mine += h[i]; }
  uint32_t incl = mine;                      // inclusive suffix sum within the warp (towards higher lanes)
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t v = __shfl_down_sync(0xffffffffu, incl, off);
    if (lane + off < 32) incl += v;
  }
  if (lane == 0) sh.wa[wid] = incl;
  __syncthreads();
  // suffix sum over the warp totals (every warp computes it; NT / 32 <= 32 entries)
  uint32_t wt = lane < NT / 32 ? sh.wa[lane] : 0u, wsuf = wt;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t v = __shfl_down_sync(0xffffffffu, wsuf, off);
    if (lane + off < 32) wsuf += v;
  }
  const uint32_t above_warps = __shfl_sync(0xffffffffu, wsuf - wt, wid);   // totals of the higher warps
  uint32_t above = above_warps + incl - mine;                             // + higher lanes of my warp
  if (above < rem && rem <= above + mine) {  // the crossing is in my bins: walk them from the top
    int b = BPT - 1;
#pragma unroll
    for (int i = BPT - 1; i > 0; --i)
      if (b == i && above + h[i] < rem) { above += h[i]; b = i - 1; }
    sh.sel_bin = (uint32_t)(BPT * tid + b);
    sh.sel_rem = rem - above;
  }
  __syncthreads();
  *rem_out = sh.sel_rem;
  const uint32_t bsel = sh.sel_bin;
  __syncthreads();
  return bsel;
}

// Block-wide exact radix select over m keys get(0 .. m): the rem-th largest key and how many
// keys equal to it belong to the top rem.  Digits of up to 11 bits, most significant first,
// starting at the highest bit in which kmax and kmin (the range of the keys) differ.
template <int NT, class Get>
__device__ __forceinline__ uint32_t radix_kth(SelShared& sh, Get get, int m, uint32_t kmax, uint32_t kmin,
                                              uint32_t rem, uint32_t* ties_out) {
  const int tid = threadIdx.x;
  const int top = kmax == kmin ? -1 : 31 - __clz(kmax ^ kmin);
  uint32_t prefix_mask = top < 0 ? 0xffffffffu : (top >= 31 ? 0u : ~((2u << top) - 1u));
  uint32_t prefix = kmax & prefix_mask;
  int hi = top;                              // highest bit not yet decided
#pragma unroll 1
  while (hi >= 0) {
    const int bits = min(11, hi + 1);
    const int shift = hi + 1 - bits;
    const uint32_t dmask = (1u << bits) - 1u;
    for (int i = tid; i < kBins; i += NT) sh.hist[i] = 0;
    __syncthreads();
    for (int i = tid; i < m; i += NT) {
      const uint32_t u = get(i);
      if ((u & prefix_mask) == prefix) atomicAdd(&sh.hist[(u >> shift) & dmask], 1u);
    }
    __syncthreads();
    const uint32_t b = find_bin<NT>(sh, rem, &rem);
    prefix |= b << shift;
    prefix_mask |= dmask << shift;
    hi = shift - 1;
  }
  *ties_out = rem;
  return prefix;
}

// Block-wide ordered emission: out[slot] = i for every selected position i, ascending, where
// selected = key > kth, or key == kth and fewer than `ties` equal keys precede it.  Warp w owns
// a contiguous segment of the row; slot = #greater before i + min(#equal before i, ties).
template <int NT, class Get>
__device__ __forceinline__ void emit_ordered(SelShared& sh, Get key_at, int n, uint32_t kth, uint32_t ties,
                                             int32_t* out, int k) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int seg = (((n + NT / 32 - 1) / (NT / 32)) + 31) & ~31;
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
  __syncthreads();
  if (lane == 0) { sh.wa[wid] = cgt; sh.wb[wid] = ceq; }
  __syncthreads();
  uint32_t gt_run = 0, eq_run = 0;
  for (int w = 0; w < wid; ++w) { gt_run += sh.wa[w]; eq_run += sh.wb[w]; }
  const uint32_t lt_mask = (1u << lane) - 1u;
  for (int i0 = s0; i0 < s1; i0 += 32) {
    const int i = i0 + lane;
    const uint32_t u = i < s1 ? key_at(i) : 0u;
    const bool gt = i < s1 && u > kth, eq = i < s1 && u == kth;
    const uint32_t bg = __ballot_sync(0xffffffffu, gt), be = __ballot_sync(0xffffffffu, eq);
    const uint32_t gt_before = gt_run + __popc(bg & lt_mask);
    const uint32_t eq_before = eq_run + __popc(be & lt_mask);
    if (gt || (eq && eq_before < ties)) {
      const uint32_t slot = gt_before + min(eq_before, ties);
      if (slot < (uint32_t)k) out[slot] = i;
    }
    gt_run += __popc(bg);
    eq_run += __popc(be);
  }
}

// One CTA per row, rows of any length and alignment: the exact bitwise radix select over the
// row's order-preserving keys (kept in shared memory when they fit, re-read from memory by
// every pass otherwise) and the ordered emission.  This is the path for logits tensors whose
// rows are not 16-byte aligned; aligned rows go through the streaming kernels below, which fall
// back to the same two steps whenever their fast path does not apply.
constexpr int kGenericThreads = 1024;
template <bool kSmemRow>
__global__ void __launch_bounds__(kGenericThreads)
topk_select_kernel(const SelParams p) {
  constexpr int NT = kGenericThreads;
  extern __shared__ __align__(16) uint32_t rowkeys[];
  __shared__ SelShared sh;
  const int t = blockIdx.x, tid = threadIdx.x;
  const int n = p.lengths ? min(max(p.lengths[t], 0), p.S) : min(p.S, max(p.q_pos0 + t + 1, 0));
  int32_t* out = p.out + (long long)t * p.k;
  const float* row = p.logits + (long long)t * p.ld;
  if (n <= p.k) {            // everything valid is selected
    for (int i = tid; i < p.k; i += NT) out[i] = i < n ? i : -1;
    return;
  }
  uint32_t kmax = 0u, kmin = 0xffffffffu;
  for (int i = tid; i < n; i += NT) {
    const uint32_t u = okey(__ldg(row + i));
    if (kSmemRow) rowkeys[i] = u;
    kmax = max(kmax, u);
    kmin = min(kmin, u);
  }
  block_max_min<NT>(sh, kmax, kmin);         // barrier: the shared-memory row is complete
  auto key_at = [&](int i) -> uint32_t { return kSmemRow ? rowkeys[i] : okey(__ldg(row + i)); };
  uint32_t ties = 0;
  const uint32_t kth = radix_kth<NT>(sh, key_at, n, kmax, kmin, (uint32_t)p.k, &ties);
  emit_ordered<NT>(sh, key_at, n, kth, ties, out, p.k);
}

constexpr int kSurvCap = 8192;           // survivors of the sampled filter kept in shared memory

// block-wide float max / min (NaN operands are ignored); all threads get the result
template <int NT>
__device__ __forceinline__ void block_fmax_fmin(float* red_a, float* red_b, float& vmax, float& vmin) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, off));
    vmin = fminf(vmin, __shfl_xor_sync(0xffffffffu, vmin, off));
  }
  if (lane == 0) { red_a[wid] = vmax; red_b[wid] = vmin; }
  __syncthreads();
  float a = lane < NT / 32 ? red_a[lane] : -INFINITY, b = lane < NT / 32 ? red_b[lane] : INFINITY;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, off));
    b = fminf(b, __shfl_xor_sync(0xffffffffu, b, off));
  }
  vmax = a; vmin = b;
  __syncthreads();
}

// Block-wide, second half of a row for the streaming kernels.  The m_s survivors of the filter
// sit in shared memory (values sval, positions spos).  fast: the filter kept at least k and at
// most kSurvCap entries.  Steps: exact selection among the survivors (value-linear histogram,
// threshold bin, its keys ranked by counting), then every survivor >= the k-th value is written
// out (thread i owns a contiguous run of survivor slots; one block-wide exclusive scan).  When
// the fast path does not apply -- or stops applying: NaN / infinite values, a single value,
// more threshold-bin keys than threads, a tie at the k-th value that must be cut by position --
// the row is finished exactly from memory: bitwise radix select (unless the k-th value is
// already known) and ordered emission.
template <int NT, class PosT>
__device__ __forceinline__ void finish_row(SelShared& sh, float* red_a, float* red_b, uint32_t* eq_total,
                                           const float* sval, const PosT* spos, uint32_t m_s, bool fast,
                                           const float* row, int n, int k, int32_t* out) {
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  uint32_t kth = 0, ties = 0;
  bool have_kth = false;
  if (fast) {
    float vmax = -INFINITY, vmin = INFINITY, chk = 0.f;
    for (uint32_t i = tid; i < m_s; i += NT) {
      const float v = sval[i];
      vmax = fmaxf(vmax, v); vmin = fminf(vmin, v); chk = fmaf(v, 0.f, chk);
    }
    const bool any_odd = __syncthreads_or(chk != chk);
    block_fmax_fmin<NT>(red_a, red_b, vmax, vmin);
    const float range = vmax - vmin;
    if (!any_odd && range > 0.f && range <= 3.0e38f) {
      const float sc = 2047.f / range;
      auto bin_of = [&](float v) -> uint32_t {
        return __float_as_uint(fmaf(v - vmin, sc, 8388608.f)) & 0xFFFu;
      };
      for (int i = tid; i < kBins; i += NT) sh.hist[i] = 0;
      __syncthreads();
      for (uint32_t i = tid; i < m_s; i += NT) atomicAdd(&sh.hist[bin_of(sval[i])], 1u);
      __syncthreads();
      uint32_t rem = 0;
      const uint32_t b = find_bin<NT>(sh, (uint32_t)k, &rem);
      for (uint32_t i = tid; i < m_s; i += NT) {
        const float v = sval[i];
        if (bin_of(v) == b) {
          const uint32_t c = atomicAdd(&sh.n_cand, 1u);
          if (c < (uint32_t)NT) sh.cand[c] = okey(v);
        }
      }
      __syncthreads();
      const uint32_t m = sh.n_cand;
      if (m <= (uint32_t)NT) {
        if (tid < (int)m) {
          const uint32_t mine = sh.cand[tid];
          uint32_t gtc = 0, eqc = 0;
          for (uint32_t j = 0; j < m; ++j) {
            const uint32_t o = sh.cand[j];
            gtc += o > mine;
            eqc += o == mine;
          }
          if (gtc < rem && rem <= gtc + eqc) { sh.kth = mine; sh.ties = rem - gtc; *eq_total = eqc; }
        }
        __syncthreads();
        kth = sh.kth; ties = sh.ties;
        have_kth = true;
        if (ties != *eq_total) fast = false;      // the tie at the k-th value must be cut by position
      } else {
        fast = false;
      }
      __syncthreads();
    } else {
      fast = false;
    }
  }
  if (fast) {
    const float kv = okey_inv(kth);
    const uint32_t per = (m_s + NT - 1) / NT;
    const uint32_t i0 = min((uint32_t)tid * per, m_s), i1 = min(i0 + per, m_s);
    uint32_t cnt = 0;
    for (uint32_t i = i0; i < i1; ++i) cnt += sval[i] >= kv;
    uint32_t inc = cnt;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t a = __shfl_up_sync(0xffffffffu, inc, off);
      if (lane >= off) inc += a;
    }
    if (lane == 31) sh.wa[wid] = inc;
    __syncthreads();
    uint32_t wtot = lane < NT / 32 ? sh.wa[lane] : 0u, ws = wtot;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const uint32_t a = __shfl_up_sync(0xffffffffu, ws, off);
      if (lane >= off) ws += a;
    }
    uint32_t o = __shfl_sync(0xffffffffu, ws - wtot, wid) + inc - cnt;
    for (uint32_t i = i0; i < i1; ++i)
      if (sval[i] >= kv) {
        if (o < (uint32_t)k) out[o] = (int32_t)spos[i];
        ++o;
      }
  } else {
    auto key_mem = [&](int i) -> uint32_t { return okey(__ldg(row + i)); };
    if (!have_kth) {
      uint32_t kmax = 0u, kmin = 0xffffffffu;
      for (int i = tid; i < n; i += NT) {
        const uint32_t u = key_mem(i);
        kmax = max(kmax, u);
        kmin = min(kmin, u);
      }
      block_max_min<NT>(sh, kmax, kmin);
      kth = radix_kth<NT>(sh, key_mem, n, kmax, kmin, (uint32_t)k, &ties);
    }
    emit_ordered<NT>(sh, key_mem, n, kth, ties, out, k);
  }
}

// Block-wide: a filter threshold from 2048 samples smp[4] per thread of a row of n entries.
// With q = k / n the expected number of samples above the k-th value is 2048 q; four standard
// deviations and a few bins above that, the sample rank r gives a value that at least k
// elements of the row exceed (probability of the opposite about 3e-5 per row; that case and
// every other surprise take the exact path).  -inf when no useful threshold exists.
template <int NT>
__device__ __forceinline__ float sampled_threshold(SelShared& sh, float* red_a, float* red_b,
                                                   const float (&smp)[4], int n, int k) {
  float smax = fmaxf(fmaxf(smp[0], smp[1]), fmaxf(smp[2], smp[3]));
  float smin = fminf(fminf(smp[0], smp[1]), fminf(smp[2], smp[3]));
  block_fmax_fmin<NT>(red_a, red_b, smax, smin);
  const float srange = smax - smin;
  const float qf = (float)k / (float)n, mean = 2048.f * qf;
  const uint32_t r = (uint32_t)ceilf(mean + 4.f * sqrtf(mean * (1.f - qf)) + 8.f);
  float t_lo = -INFINITY;
  if (srange > 0.f && srange <= 3.0e38f && r < 2048u) {
    const float sc = 2047.f / srange;
    for (int i = threadIdx.x; i < kBins; i += NT) sh.hist[i] = 0;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (smp[i] == smp[i]) atomicAdd(&sh.hist[__float_as_uint(fmaf(smp[i] - smin, sc, 8388608.f)) & 0xFFFu], 1u);
    __syncthreads();
    uint32_t rem_s = 0;
    const uint32_t b = find_bin<NT>(sh, r, &rem_s);
    if (b > 1u) t_lo = smin + (float)(b - 2u) / sc;       // two bins below: rounding-safe lower edge
  }
  return t_lo;
}

// Rows of at most 512 * EPT entries, 16-byte aligned: persistent CTAs, one row at a time.
// The row arrives in shared memory by ONE bulk copy (no registers, no threads involved), is
// moved into REGISTERS as fp32 values -- thread i owns the 16-byte quads i, i + 512, ... -- and
// the next row's copy is issued at once, so it lands while this row is being processed.
// Selection without sorting and without touching most elements more than once:
//   1. 2048 evenly spaced samples of the row give a threshold that, with overwhelming
//      probability, a little more than k elements exceed;
//   2. one compare per element builds the survivors' positional masks (block-wide scan);
//   3. the ~1.3 k survivors' positions go to shared memory, their values are re-read;
//   4. among them: value-linear histogram (bin = the low bits of fma(v - min, 2047 / range,
//      2^23): no float-to-int conversion), suffix scan, the few keys of the threshold bin ranked
//      exactly by counting;
//   5. survivors >= the k-th value are written out (block-wide scan of per-thread counts).
// The output order is fixed but not ascending.  Whatever the fast path does not cover -- too
// few or too many survivors, NaN or infinite values, a single value, more threshold-bin keys
// than threads, a tie at the k-th value that must be cut by position -- is finished by the
// exact bitwise radix select and the ordered emission over the row re-read from memory.
constexpr int kStreamThreads = 512;
enum { kSiteSelRow = 11 };

template <int EPT>
__global__ void __launch_bounds__(kStreamThreads, 1)
topk_select_stream_kernel(const SelParams p) {
  constexpr int NT = kStreamThreads, NQ = EPT / 4;
  extern __shared__ __align__(16) float rowbuf[];      // the row | survivor values | survivor positions
  float* sval = rowbuf + ((p.S + 3) & ~3);
  uint16_t* spos = reinterpret_cast<uint16_t*>(sval + kSurvCap);
  __shared__ SelShared sh;
  __shared__ __align__(8) uint64_t row_bar;
  __shared__ float red_a[NT / 32], red_b[NT / 32];
  __shared__ uint32_t eq_total;
  const Waiter wt{g_status, p.epoch, p.wait_limit_ns};
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  auto len_of = [&](int t) -> int {
    return p.lengths ? min(max(p.lengths[t], 0), p.S) : min(p.S, max(p.q_pos0 + t + 1, 0));
  };
  // rows that need a selection are fetched; the others are written directly
  auto fetch = [&](int t) {       // thread 0 only
    const int n = len_of(t);
    if (n > p.k) {
      const uint32_t bytes = (uint32_t)(((n + 3) & ~3) * 4);
      mbar_arrive_expect_tx(&row_bar, bytes);
      bulk_load_1d(smem_u32(rowbuf), p.logits + (long long)t * p.ld, bytes, &row_bar);
    }
  };
  if (tid == 0) {
    mbar_init(&row_bar, 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (tid == 0 && (int)blockIdx.x < p.T) fetch(blockIdx.x);
  uint32_t phase = 0;

  for (int t = blockIdx.x; t < p.T; t += gridDim.x) {
    const int n = len_of(t);
    int32_t* out = p.out + (long long)t * p.k;
    const int t_next = t + gridDim.x;
    if (n <= p.k) {            // everything valid is selected; no copy was issued for this row
      for (int i = tid; i < p.k; i += NT) out[i] = i < n ? i : -1;
      if (tid == 0 && t_next < p.T) fetch(t_next);
      continue;
    }
    const bool landed = mbar_wait(&row_bar, phase, wt, kSiteSelRow, t);
    phase ^= 1;
    // ---- registers: quad q of this thread holds positions 4 * (q * NT + tid) .. + 3.  Quads
    // [0, nfull) are entirely below n for every thread; the next one may be cut; the rest is empty.
    float vr[EPT];
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
      const float4 v = 4 * (q * NT + tid) < n ? reinterpret_cast<const float4*>(rowbuf)[q * NT + tid]
                                              : make_float4(0.f, 0.f, 0.f, 0.f);
      vr[4 * q] = v.x; vr[4 * q + 1] = v.y; vr[4 * q + 2] = v.z; vr[4 * q + 3] = v.w;
    }
    const int nfull = n / (4 * NT);                 // block-uniform
    // 2048 samples of the row, evenly spaced over its positions (read while the row is still
    // in shared memory): they place the threshold of the filter below
    float smp[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) smp[i] = rowbuf[(int)(((long long)(4 * tid + i) * n) >> 11)];
    auto live = [&](int q, int c) -> bool { return q < nfull || 4 * (q * NT + tid) + c < n; };
    fence_proxy_async_smem();      // these reads are ordered before the next bulk write
    if (tid == 0) sh.n_cand = 0;
    const bool all_landed = __syncthreads_and(landed);
    if (tid == 0 && t_next < p.T) fetch(t_next);
    if (!all_landed) continue;     // a wait ran out: the status word says so (block-uniform decision)

    const float* row = p.logits + (long long)t * p.ld;
    bool fast = true;                // block-uniform: the fast path still applies

    // ---- 1. a threshold from the sample; short rows skip the filter: everything survives
    float t_lo = -INFINITY;
    if (n > kSurvCap / 2) t_lo = sampled_threshold<NT>(sh, red_a, red_b, smp, n, p.k);

    // ---- 2. filter: one 4-bit mask per quad (kept for the extraction below), survivor count,
    // block-wide exclusive scan
    unsigned long long selm = 0ull;
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
      uint32_t m4;
      if (q < nfull) {
        m4 = (uint32_t)(vr[4 * q] >= t_lo) | ((uint32_t)(vr[4 * q + 1] >= t_lo) << 1) |
             ((uint32_t)(vr[4 * q + 2] >= t_lo) << 2) | ((uint32_t)(vr[4 * q + 3] >= t_lo) << 3);
      } else {
        m4 = 0;
#pragma unroll
        for (int c = 0; c < 4; ++c) m4 |= (uint32_t)(live(q, c) && vr[4 * q + c] >= t_lo) << c;
      }
      selm |= (unsigned long long)m4 << (4 * q);
    }
    const uint32_t nsel = __popcll(selm);
    uint32_t slot = 0, m_s = 0;
    {
      const uint32_t cnt = nsel;
      uint32_t inc = cnt;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const uint32_t a = __shfl_up_sync(0xffffffffu, inc, off);
        if (lane >= off) inc += a;
      }
      if (lane == 31) sh.wa[wid] = inc;
      __syncthreads();
      uint32_t wtot = lane < NT / 32 ? sh.wa[lane] : 0u, ws = wtot;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const uint32_t a = __shfl_up_sync(0xffffffffu, ws, off);
        if (lane >= off) ws += a;
      }
      slot = __shfl_sync(0xffffffffu, ws - wtot, wid) + inc - cnt;
      m_s = __shfl_sync(0xffffffffu, ws, NT / 32 - 1);
      __syncthreads();
    }
    if (m_s < (uint32_t)p.k || m_s > (uint32_t)kSurvCap) fast = false;   // too few (threshold too high) / too many

    if (fast) {
      // ---- 3. survivors: values and positions out of the registers into shared memory; about
      // one element in ten survives, so most quads are skipped on their mask nibble
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        const uint32_t m4 = (uint32_t)(selm >> (4 * q)) & 15u;
        if (m4) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
            if (m4 & (1u << c)) {
              sval[slot] = vr[4 * q + c];
              spos[slot] = (uint16_t)(4 * (q * NT + tid) + c);
              ++slot;
            }
        }
      }
      __syncthreads();
    }
    finish_row<NT>(sh, red_a, red_b, &eq_total, sval, spos, m_s, fast, row, n, p.k, out);
    __syncthreads();               // sh.* is reused by the next row
  }
}


// Rows of any length, 16-byte aligned: persistent CTAs; a row streams through two 64 KB
// shared-memory buffers (bulk copies, two chunks in flight, running across rows), its 2048
// samples are read from memory first.  Per chunk a thread filters 32 elements straight out of
// shared memory (count, block-wide scan, survivors appended to the list); after the last chunk
// the survivors are finished like in the register kernel above.
constexpr int kChunk = 16384;            // floats per chunk
enum { kSiteSelChunk = 12 };

__global__ void __launch_bounds__(kStreamThreads, 1)
topk_select_chunked_kernel(const SelParams p) {
  constexpr int NT = kStreamThreads, NQ = kChunk / 4 / NT;
  extern __shared__ __align__(16) float cbuf[];       // 2 chunks | survivor values | survivor positions
  float* sval = cbuf + 2 * kChunk;
  uint32_t* spos = reinterpret_cast<uint32_t*>(sval + kSurvCap);
  __shared__ SelShared sh;
  __shared__ __align__(8) uint64_t bar[2];
  __shared__ float red_a[NT / 32], red_b[NT / 32];
  __shared__ uint32_t eq_total;
  const Waiter wt{g_status, p.epoch, p.wait_limit_ns};
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  auto len_of = [&](int t) -> int {
    return p.lengths ? min(max(p.lengths[t], 0), p.S) : min(p.S, max(p.q_pos0 + t + 1, 0));
  };
  auto chunks_of = [&](int n) -> int { return (n + kChunk - 1) / kChunk; };
  // fetch cursor (thread 0): next (row, chunk) to request and its running chunk number
  int tf = blockIdx.x, cf = 0;
  uint32_t gf = 0;
  auto skip_short = [&]() { while (tf < p.T && len_of(tf) <= p.k) tf += gridDim.x; };
  auto fetch_next = [&]() {       // thread 0 only
    if (tf >= p.T) return;
    const int n = len_of(tf);
    const int start = cf * kChunk;
    const uint32_t bytes = (uint32_t)(min(kChunk, ((n + 3) & ~3) - start) * 4);
    uint64_t* b = &bar[gf & 1];
    mbar_arrive_expect_tx(b, bytes);
    bulk_load_1d(smem_u32(cbuf + (gf & 1) * kChunk), p.logits + (long long)tf * p.ld + start, bytes, b);
    ++gf;
    if (++cf == chunks_of(n)) { cf = 0; tf += gridDim.x; skip_short(); }
  };
  if (tid == 0) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    fence_mbar_init();
    skip_short();
    fetch_next();
    fetch_next();
  }
  __syncthreads();
  uint32_t gc = 0;                 // running number of the next chunk to consume

  for (int t = blockIdx.x; t < p.T; t += gridDim.x) {
    const int n = len_of(t);
    int32_t* out = p.out + (long long)t * p.k;
    if (n <= p.k) {            // everything valid is selected; nothing was fetched for this row
      for (int i = tid; i < p.k; i += NT) out[i] = i < n ? i : -1;
      continue;
    }
    const float* row = p.logits + (long long)t * p.ld;
    // 2048 evenly spaced samples, read from memory while the first chunk lands
    float smp[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) smp[i] = __ldg(row + (int)(((long long)(4 * tid + i) * n) >> 11));
    if (tid == 0) sh.n_cand = 0;
    float t_lo = -INFINITY;
    if (n > kSurvCap / 2) t_lo = sampled_threshold<NT>(sh, red_a, red_b, smp, n, p.k);
    else __syncthreads();

    bool fast = true;
    uint32_t m_run = 0;
    const int nch = chunks_of(n);
    for (int c = 0; c < nch; ++c, ++gc) {
      const bool landed = mbar_wait(&bar[gc & 1], (gc >> 1) & 1, wt, kSiteSelChunk, c);
      const float4* buf = reinterpret_cast<const float4*>(cbuf + (gc & 1) * kChunk);
      const int start = c * kChunk;
      // this thread's 8 quads of the chunk: positions start + 4 * (q * NT + tid) .. + 3
      float4 v[NQ];
      uint32_t cnt = 0;
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        const int pos = start + 4 * (q * NT + tid);
        v[q] = pos < n ? buf[q * NT + tid] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        if (pos + 3 >= n) {      // the row's last quad may be cut: entries beyond n never survive
          if (pos + 1 >= n) v[q].y = NAN;
          if (pos + 2 >= n) v[q].z = NAN;
          if (pos + 3 >= n) v[q].w = NAN;
          if (pos >= n) v[q].x = NAN;
        }
        cnt += (v[q].x >= t_lo) + (v[q].y >= t_lo) + (v[q].z >= t_lo) + (v[q].w >= t_lo);
      }
      fence_proxy_async_smem();    // these reads are ordered before the next bulk write of the buffer
      // block-wide exclusive scan of the counts (its barrier also frees the buffer)
      uint32_t inc = cnt;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const uint32_t a = __shfl_up_sync(0xffffffffu, inc, off);
        if (lane >= off) inc += a;
      }
      if (lane == 31) sh.wa[wid] = inc;
      const bool all_landed = __syncthreads_and(landed);
      if (tid == 0) fetch_next();
      uint32_t wtot = lane < NT / 32 ? sh.wa[lane] : 0u, ws = wtot;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const uint32_t a = __shfl_up_sync(0xffffffffu, ws, off);
        if (lane >= off) ws += a;
      }
      uint32_t slot = m_run + __shfl_sync(0xffffffffu, ws - wtot, wid) + inc - cnt;
      const uint32_t total = __shfl_sync(0xffffffffu, ws, NT / 32 - 1);
      if (!all_landed || m_run + total > (uint32_t)kSurvCap) fast = false;   // block-uniform
      if (fast) {
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
          const uint32_t pos = (uint32_t)(start + 4 * (q * NT + tid));
          if (v[q].x >= t_lo) { sval[slot] = v[q].x; spos[slot] = pos; ++slot; }
          if (v[q].y >= t_lo) { sval[slot] = v[q].y; spos[slot] = pos + 1; ++slot; }
          if (v[q].z >= t_lo) { sval[slot] = v[q].z; spos[slot] = pos + 2; ++slot; }
          if (v[q].w >= t_lo) { sval[slot] = v[q].w; spos[slot] = pos + 3; ++slot; }
        }
      }
      m_run += total;
      __syncthreads();             // sh.wa is reused by the next chunk's scan
    }
    if (m_run < (uint32_t)p.k) fast = false;       // the threshold was too high
    finish_row<NT>(sh, red_a, red_b, &eq_total, sval, spos, m_run, fast, row, n, p.k, out);
    __syncthreads();               // sh.* is reused by the next row
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
// values (order inside a row unspecified), ties at the k-th value resolved towards smaller
// positions; rows with len(t) <= k list 0 .. len(t) - 1 and are padded with -1.  len(t) = lengths[t], or
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
  p.epoch = lt::next_launch_epoch(); p.wait_limit_ns = lt::wait_limit_ns();
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // rows up to 32768 entries live in registers (512 threads x 64 or 32 consecutive positions,
  // transposed through shared memory); longer rows stay in shared memory up to 49152 entries
  // and are re-read from memory by every pass beyond that
  const size_t smem = (((size_t)S + 3) & ~(size_t)3) * 4;      // whole 16-byte quads
  auto launch = [&](auto kern, int threads, size_t dyn) -> int {
    if (dyn && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn) != cudaSuccess)
      return LITEDSA_ERR_CUDA;
    kern<<<T, threads, dyn, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? LITEDSA_OK : LITEDSA_ERR_CUDA;
  };
  const bool aligned = (logits_row_stride & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0;
  if (aligned && S <= kStreamThreads * 64) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = T < sms ? T : sms;
    auto kern = S <= kStreamThreads * 32 ? topk_select_stream_kernel<32> : topk_select_stream_kernel<64>;
    const size_t dyn = smem + (size_t)kSurvCap * 6;      // + survivor values (fp32) and positions (u16)
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn) != cudaSuccess)
      return LITEDSA_ERR_CUDA;
    kern<<<grid, kStreamThreads, dyn, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? LITEDSA_OK : LITEDSA_ERR_CUDA;
  }
  if (aligned) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const size_t dyn = (size_t)2 * kChunk * 4 + (size_t)kSurvCap * 8;
    if (cudaFuncSetAttribute(topk_select_chunked_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)dyn) != cudaSuccess)
      return LITEDSA_ERR_CUDA;
    topk_select_chunked_kernel<<<T < sms ? T : sms, kStreamThreads, dyn, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? LITEDSA_OK : LITEDSA_ERR_CUDA;
  }
  if (S <= kMaxSmemRow) return launch(topk_select_kernel<true>, kGenericThreads, smem);
  return launch(topk_select_kernel<false>, kGenericThreads, 0);
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

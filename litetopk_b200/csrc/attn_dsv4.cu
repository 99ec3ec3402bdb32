// DeepSeek-V4 style packed BF16 attention over two contiguous key ranges (sm_100a).
//
// Every query token at position p attends to the compressed-prefix entries
// [0, p / ratio) of a small compressed KV and to the raw sliding window
// [p - window + 1, p]; G = 128 / h adjacent tokens are packed into one 128-row tile.
// The reference's DSv4 operator (kernels/b200/dsa/litedsa_dsv4.cu:50-121, kernel
// kernels/b200/dsa/litedsa_attention_sm100_dsv4.cuh:1849-2485) expresses the same mask as
// two ranges per token in the rank space of a gathered union list (range_mask32,
// litedsa_attention_sm100_dsv4.cuh:1824-1829) and gathers rows with TMA gather4.  Here the
// ranges are used directly: both key segments are contiguous in memory, so K and V tiles
// come from plain tiled TMA loads (13 per 64-key block per CTA instead of 2 x 36 gathers),
// no index list exists, and the mask is two comparisons per column.
//
// Organisation: cluster of 2 CTAs per tile (64 query rows each), 64-key blocks, bf16
// tcgen05 cta_group::2 MMAs (S = Q K^T over 576 dims: 36 K-steps of 16; O += P V: two
// N = 256 halves x 4 K-steps), S double-buffered in TMEM, O in TMEM, base-2 online softmax
// with the same lazy running-max policy as the FP8 kernel, P stored as bf16 (no pre-scale,
// litedsa_attention_sm100_dsv4.cuh:2072-2083), optional per-row attention sink in the
// output normaliser only (:2138-2157).
#include "common.cuh"
#include "tensor_map.cuh"

namespace lt {
namespace dsv4 {

constexpr int kThreads = 320;                         // 4 softmax warps, 1 TMA warp, 1 MMA warp, 4 epilogue warps
constexpr int kWarpEpi0 = 6;
constexpr int kBlockKeys = 64;
constexpr int kD = 576, kDV = 512;
constexpr int kQChunks = 9;                           // 64 bf16 = 128 bytes per chunk
constexpr uint32_t kQChunkBytes = 64 * 128;           // 64 rows
constexpr uint32_t kQBytes = kQChunks * kQChunkBytes; // 73728
constexpr uint32_t kKChunkBytes = 32 * 128;           // 32 keys per CTA
constexpr uint32_t kKStage = kQChunks * kKChunkBytes; // 36864
constexpr uint32_t kVChunkBytes = 64 * 128;           // 64 keys x 64 dims
constexpr uint32_t kVStage = 4 * kVChunkBytes;        // 64 keys x 256 dims = 32768
constexpr uint32_t kPBytes = 64 * 64 * 2;             // 64 rows x 64 keys bf16
constexpr uint32_t kOffQ = 0;
constexpr uint32_t kOffK = kOffQ + kQBytes;
constexpr uint32_t kOffV = kOffK + 2 * kKStage;
constexpr uint32_t kOffP = kOffV + 2 * kVStage;
constexpr uint32_t kOffStage = kOffP + kPBytes;       // 221184: 4 x 2 KB output staging slices (epilogue warps)
constexpr uint32_t kOffMisc = kOffStage + 4 * 2048;
constexpr uint32_t kMiscBytes = 2304;
constexpr uint32_t kSmemUsed = kOffMisc + kMiscBytes;
constexpr uint32_t kSmem = 232448;                    // all of it: 768 bytes of alignment slack remain
static_assert(kSmem <= 232448, "shared-memory plan exceeds the 227 KB per-CTA limit");

constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemO = 0, kTmemS0 = 256, kTmemS1 = 288;   // S: 32 columns per buffer

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kMInit = -1e30f;
constexpr float kRescaleThreshold = 6.0f;

struct Misc {
  uint64_t q_full, k_full[2], v_full[2], s_free[2], p_ready;   // used in the leader CTA
  uint64_t qk_done[2], pv_done[2];                             // every CTA (one phase per stage use)
  uint64_t q_free;                                             // every CTA: the tile's QK^T are complete
  uint64_t o_free;                                             // leader CTA: O has been read out of TMEM
  uint64_t epi_ready;                                          // every CTA: the tile's row scales are published
  uint32_t tmem_base, pad;
  float xbuf[3][128];   // [block parity | 2 = end-of-tile row-sum merge][lane]
  float oscale[2][64];  // [tile parity][row]: 1 / normaliser, 0 for rows without a key
};
static_assert(sizeof(Misc) <= kMiscBytes, "Misc too large");

struct Params {
  __nv_bfloat16* out;        // [ng, 128, 512]
  float* lse;                // [ng, 128]
  const float* sink;         // [128] per packed row, or null
  int ng, n_comp, s_raw, G, h_per_q, pos0, window, ratio;
  float scale_log2;
  int epoch;                          // this launch's epoch for the bounded waits
  unsigned long long wait_limit_ns;
  // rank mode (the reference operator's argument list, litedsa_dsv4.cu:50-55, when every
  // tile's gathered index list is two contiguous runs of rows of one flat KV workspace):
  // runs[tile] = (first row of run 0, its length, first row of run 1, its length); a token may
  // attend the list ranks  rank < pref  or  win_lo <= rank < win_hi  (rank < counts)
  const int4* runs;          // [ng] or null (position mode)
  const int32_t* pref;       // [ng, G]
  const int32_t* win_lo;     // [ng, G]
  const int32_t* win_hi;     // [ng, G]
  const int32_t* counts;     // [ng] or null
  // the launch runs only if *gate == gate_value (null: always); lets the host enqueue this
  // kernel and the gather kernel back to back and have the device pick one of them
  const int* gate;
  int gate_value;
};

enum { kSiteQ = 101, kSiteKFull, kSiteVFull, kSiteQkDone, kSitePvDone, kSiteSFree, kSitePReady,
       kSiteKFree, kSiteVFree, kSitePFree, kSiteEpi, kSiteQFree, kSiteOFree, kSiteSmem };

// status block of the DSv4 kernel (layout: see Waiter in common.cuh)
__device__ int g_status[8];

// key segments of a tile: compressed blocks first, then window blocks
struct TilePlan {
  int p0, pref_max, wlo, count_w, nbc, nb, row_c;   // row_c: first row of the first segment
};
template <bool kRank>
__device__ __forceinline__ TilePlan plan_tile(const Params& p, int tile) {
  TilePlan t;
  if (kRank) {
    const int4 r = __ldg(p.runs + tile);
    t.p0 = 0;
    t.row_c = r.x; t.pref_max = max(r.y, 0);
    t.wlo = r.z;   t.count_w = max(r.w, 0);
  } else {
    t.p0 = p.pos0 + tile * p.G;
    const int plast = t.p0 + p.G - 1;
    t.row_c = 0;
    t.pref_max = min(plast / p.ratio, p.n_comp);
    t.wlo = max(0, t.p0 - p.window + 1);
    t.count_w = plast - t.wlo + 1;
  }
  t.nbc = (t.pref_max + kBlockKeys - 1) / kBlockKeys;
  t.nb = t.nbc + (t.count_w + kBlockKeys - 1) / kBlockKeys;
  if (t.nb == 0) t.nb = 1;      // an empty list: one fully masked block keeps the pipeline uniform
  return t;
}
// bits [0, x) of a 32-bit word (x may be negative or beyond 32)
__device__ __forceinline__ uint32_t low_bits(int x) {
  return x <= 0 ? 0u : (x >= 32 ? 0xffffffffu : ((1u << x) - 1u));
}

__device__ __forceinline__ void mma_f16_elect(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, pe;\n\tsetp.ne.b32 p, %4, 0;\n\telect.sync _|pe, 0xffffffff;\n\t"
      "@pe tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <bool kRank>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
dsv4_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kc32,
            const __grid_constant__ CUtensorMap map_kr32, const __grid_constant__ CUtensorMap map_kc64,
            const __grid_constant__ CUtensorMap map_kr64,
            const __grid_constant__ CUtensorMap map_out, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (sbase - raw);
  Misc& ms = *reinterpret_cast<Misc*>(sm + kOffMisc);
  const Waiter wt{g_status, p.epoch, p.wait_limit_ns};
  // device-side choice between this kernel and the gather kernel (uniform across the grid)
  if (p.gate != nullptr && *reinterpret_cast<const volatile int*>(p.gate) != p.gate_value) return;
  // the plan leaves less than 1024 bytes for aligning the base: refuse to run (uniformly, in
  // both CTAs, before any barrier exists) if this launch's base needs more
  if ((sbase - raw) + kSmemUsed > kSmem) {
    if (threadIdx.x == 0) wt.fail(kSiteSmem, 0);
    return;
  }

  // Persistent: each cluster walks tiles cid, cid + #clusters, ...  Stages, buffers and
  // barrier phases are indexed by the cluster-wide running block number kb, so the next
  // tile's Q / K / V loads and first QK^T overlap the previous tile's epilogue.
  const uint32_t cta = cluster_ctarank();
  const int cid = blockIdx.x >> 1, ncl = gridDim.x >> 1;
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(&ms.q_full, 1);
    mbar_init(&ms.p_ready, 8);
    mbar_init(&ms.q_free, 1);
    mbar_init(&ms.o_free, 8);
    mbar_init(&ms.epi_ready, 4);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ms.k_full[i], 1);
      mbar_init(&ms.v_full[i], 1);
      mbar_init(&ms.s_free[i], 8);
      mbar_init(&ms.qk_done[i], 1);
      mbar_init(&ms.pv_done[i], 1);
    }
    fence_mbar_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_kc32);
    tma_prefetch_desc(&map_kr32);
    tma_prefetch_desc(&map_kc64);
    tma_prefetch_desc(&map_kr64);
    tma_prefetch_desc(&map_out);
  }
  __syncthreads();
  cluster_sync_all();
  if (warp == 5) {
    tmem_alloc_pair(&ms.tmem_base, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ms.tmem_base;

  if (warp < 4) {
    // ------------------------------------------------------------ softmax + epilogue
    const int tl = threadIdx.x;                   // TMEM lane
    const int r = tl & 63, h = tl >> 6;           // row of this CTA, key half (32 columns)
    const int row = (int)cta * 64 + r;
    const int q = row / p.h_per_q;                // token of the tile this row belongs to
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const float c = p.scale_log2;
    const uint32_t a_s_free[2] = {mapa(smem_u32(&ms.s_free[0]), 0), mapa(smem_u32(&ms.s_free[1]), 0)};
    const uint32_t a_p_ready = mapa(smem_u32(&ms.p_ready), 0);
    int kb0 = 0, it = 0;
   for (int tile = cid; tile < p.ng; tile += ncl) {
    const TilePlan tp = plan_tile<kRank>(p, tile);
    const int nb = tp.nb;
    int pref_q, lo_q, hi_q;
    if (kRank) {
      // list ranks this token may attend: rank < pref_q, or lo_q <= rank < hi_q (all < cnt)
      const int cnt = p.counts ? min(max(__ldg(p.counts + tile), 0), tp.pref_max + tp.count_w)
                               : tp.pref_max + tp.count_w;
      const size_t tq = (size_t)tile * p.G + q;
      pref_q = min(__ldg(p.pref + tq), cnt);
      lo_q = __ldg(p.win_lo + tq);
      hi_q = min(__ldg(p.win_hi + tq), cnt);
    } else {
      const int pq = tp.p0 + q;
      pref_q = min(pq / p.ratio, p.n_comp);
      lo_q = max(pq - p.window + 1, 0) - tp.wlo;   // window-rank range of this token
      hi_q = pq - tp.wlo + 1;
    }
    float m = kMInit, li = 0.f, real_m = -INFINITY;

    for (int k = 0; k < nb; ++k) {
      const int kb = kb0 + k;
      const int s = kb & 1;
      const uint32_t ph = (kb >> 1) & 1;
      mbar_wait(&ms.qk_done[s], ph, wt, kSiteQkDone, k);
      tc_fence_after();
      float sv[32];
      tmem_ld32(tmem + lane_base + (s ? kTmemS1 : kTmemS0), sv);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(a_s_free[s]);

      float cur = -INFINITY;
      if (kRank) {
        // columns this thread holds: 32 consecutive list ranks starting at `off`, of which the
        // first `lim` exist in this segment; valid = existing and in one of the token's two
        // rank ranges -- one 32-bit mask per block
        const bool seg0 = k < tp.nbc;
        const int base = (seg0 ? k : k - tp.nbc) * kBlockKeys + 32 * h;
        const int lim = (seg0 ? tp.pref_max : tp.count_w) - base;
        const int off = (seg0 ? 0 : tp.pref_max) + base;
        const uint32_t vm = low_bits(lim) & (low_bits(pref_q - off) | (low_bits(hi_q - off) & ~low_bits(lo_q - off)));
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          sv[j] = ((vm >> j) & 1u) ? sv[j] : -INFINITY;
          cur = fmaxf(cur, sv[j]);
        }
      } else {
        // columns this thread holds: keys [32h, 32h+32) of the block, as a contiguous valid range
        int v_lo, v_hi;
        if (k < tp.nbc) {                       // compressed block: rank = 64k + j < pref_q
          v_lo = 0;
          v_hi = pref_q - (k * kBlockKeys + 32 * h);
        } else {                                // window block: lo_q <= 64(k-nbc) + j < hi_q
          const int base = (k - tp.nbc) * kBlockKeys + 32 * h;
          v_lo = lo_q - base;
          v_hi = hi_q - base;
        }
        v_lo = max(v_lo, 0);
        v_hi = min(v_hi, 32);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          sv[j] = (j >= v_lo && j < v_hi) ? sv[j] : -INFINITY;
          cur = fmaxf(cur, sv[j]);
        }
      }
      cur *= c;
      ms.xbuf[kb & 1][tl] = cur;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      cur = fmaxf(cur, ms.xbuf[kb & 1][tl ^ 64]);
      real_m = fmaxf(real_m, cur);
      const bool rescale = __any_sync(0xffffffffu, cur - m > kRescaleThreshold);
      float new_m = m, scale_old = 1.f;
      if (rescale) {
        new_m = fmaxf(cur, m);
        scale_old = fast_exp2(m - new_m);
      }
      m = new_m;
      li *= scale_old;

      uint32_t pk[16];
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        const float p0 = fast_exp2(fmaf(sv[j], c, -new_m));
        const float p1 = fast_exp2(fmaf(sv[j + 1], c, -new_m));
        li += p0 + p1;
        __nv_bfloat162 b2 = __floats2bfloat162_rn(p0, p1);
        pk[j >> 1] = *reinterpret_cast<uint32_t*>(&b2);
      }
      // the single P buffer was last read by the PV of the previous block (of this or the
      // previous tile)
      if (kb >= 1) mbar_wait(&ms.pv_done[(kb - 1) & 1], ((kb - 1) >> 1) & 1, wt, kSitePFree, k);
      // P: [64 rows][64 keys] bf16, K-major core matrices: 8-key group cg at cg*1024 + row*16
      uint8_t* pdst = sm + kOffP + (4 * h) * 1024 + r * 16;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        *reinterpret_cast<uint4*>(pdst + i * 1024) =
            make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
      if (rescale && k > 0) {
        tc_fence_after();                      // PV(k-1) completion was awaited above
        float o[32];
#pragma unroll 1
        for (int cc = 0; cc < 8; ++cc) {
          const uint32_t ocol = tmem + lane_base + kTmemO + cc * 32;
          tmem_ld32(ocol, o);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] *= scale_old;
          tmem_st32(ocol, o);
        }
        tmem_wait_st();
        tc_fence_before();
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(a_p_ready);
    }

    // epilogue
    ms.xbuf[2][tl] = li;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    li += ms.xbuf[2][tl ^ 64];
    if (real_m == -INFINITY) { li = 0.f; m = -INFINITY; }
    const size_t grow = (size_t)tile * 128 + row;
    if (h == 0) {
      float l = __logf(li) + m * kLn2;
      if (!(li > 0.f)) l = INFINITY;
      p.lse[grow] = l;
    }
    // hand the tile over to the epilogue warps: all they need is 1 / normaliser per row
    float denom = li;
    if (p.sink != nullptr && li > 0.f) denom += fast_exp2(__ldg(p.sink + row) * kLog2e - m);
    if (h == 0) ms.oscale[it & 1][r] = (li > 0.f) ? __fdividef(1.0f, denom) : 0.f;
    __syncwarp();
    if (lane == 0) mbar_arrive(&ms.epi_ready);
    kb0 += nb;
    ++it;
   }
  } else if (warp == 4) {
    // ------------------------------------------------------------ TMA producer (tiled loads)
    if (lane == 0) {
      const uint32_t a_q_full = mapa(smem_u32(&ms.q_full), 0);
      const uint32_t a_k_full[2] = {mapa(smem_u32(&ms.k_full[0]), 0), mapa(smem_u32(&ms.k_full[1]), 0)};
      const uint32_t a_v_full[2] = {mapa(smem_u32(&ms.v_full[0]), 0), mapa(smem_u32(&ms.v_full[1]), 0)};
      const uint64_t pol_stream = l2_policy_evict_first();     // q streams through once
      int kb0 = 0, it = 0;
      for (int tile = cid; tile < p.ng; tile += ncl, ++it) {
        const TilePlan tp = plan_tile<kRank>(p, tile);
        const int nb = tp.nb;
        // the previous tile's Q must have been consumed by its last QK^T
        if (it > 0) mbar_wait(&ms.q_free, (it - 1) & 1, wt, kSiteQFree, it);
        if (cta == 0) mbar_arrive_expect_tx(&ms.q_full, 2 * kQBytes);
        // this CTA's 64 rows of the tile = (token, head) pairs starting at row 64 cta
        for (int j = 0; j < kQChunks; ++j)
          tma_load_3d_pair_hint(sbase + kOffQ + j * kQChunkBytes, &map_q, 64 * j,
                                (64 * (int)cta) % p.h_per_q, tile * p.G + (64 * (int)cta) / p.h_per_q,
                                a_q_full, pol_stream);
        for (int k = 0; k < nb; ++k) {
          const int kb = kb0 + k;
          const int s = kb & 1;
          const uint32_t ph = (kb >> 1) & 1;
          const bool comp = k < tp.nbc;
          const int row0 = comp ? tp.row_c + k * kBlockKeys : tp.wlo + (k - tp.nbc) * kBlockKeys;
          const CUtensorMap* m32 = comp ? &map_kc32 : &map_kr32;
          const CUtensorMap* m64 = comp ? &map_kc64 : &map_kr64;
          if (kb >= 2) mbar_wait(&ms.qk_done[s], ph ^ 1, wt, kSiteKFree, k);   // K stage free
          if (cta == 0) mbar_arrive_expect_tx(&ms.k_full[s], 2 * kKStage);
          for (int j = 0; j < kQChunks; ++j)
            tma_load_2d_pair(sbase + kOffK + s * kKStage + j * kKChunkBytes, m32, 64 * j,
                             row0 + 32 * (int)cta, a_k_full[s]);
          // V stage s was last read by the PV of block kb-2
          if (kb >= 2) mbar_wait(&ms.pv_done[s], ph ^ 1, wt, kSiteVFree, k);
          if (cta == 0) mbar_arrive_expect_tx(&ms.v_full[s], 2 * kVStage);
          for (int j = 0; j < 4; ++j)
            tma_load_2d_pair(sbase + kOffV + s * kVStage + j * kVChunkBytes, m64,
                             256 * (int)cta + 64 * j, row0, a_v_full[s]);
        }
        kb0 += nb;
      }
    }
  } else if (warp >= kWarpEpi0) {
    // ------------------------------------------------------------ epilogue warps
    // O out of TMEM, x 1 / normaliser, bf16, TMA tile stores -- while the softmax warps already
    // work on the next tile.  A warp reads the TMEM lanes of its quarter (warp % 4): rows r of
    // key half h, all 256 columns in 8 rounds of 32 dims.  A round (32 rows x 64 bytes,
    // 64-byte swizzle: the 16-byte stores of eight consecutive rows hit distinct banks) is
    // staged in the warp's own 2 KB slice and one lane hands the box to TMA.
    const int tl = ((warp & 3) << 5) | lane;
    const int r = tl & 63, h = tl >> 6;
    const uint32_t ocol = tmem + ((uint32_t)((warp & 3) * 32) << 16) + kTmemO;
    const uint32_t stage_off = kOffStage + (warp - kWarpEpi0) * 2048;
    uint8_t* st_row = sm + stage_off + (r & 31) * 64;
    const int sw = (r >> 1) & 3;
    const uint32_t a_o_free = mapa(smem_u32(&ms.o_free), 0);
    int kb0 = 0, it = 0;
    for (int tile = cid; tile < p.ng; tile += ncl, ++it) {
      const int nb = plan_tile<kRank>(p, tile).nb;
      const int kbl = kb0 + nb - 1;                 // last block of the tile
      mbar_wait(&ms.epi_ready, it & 1, wt, kSiteEpi, it);
      mbar_wait(&ms.pv_done[kbl & 1], (kbl >> 1) & 1, wt, kSiteEpi, nb);
      tc_fence_after();
      const float oscale = ms.oscale[it & 1][r];
      const uint32_t emask = oscale != 0.f ? 0xffffffffu : 0u;
      // this warp's 32 rows of the tile = (token, head) pairs starting at row r0
      const int r0 = (int)cta * 64 + 32 * (warp & 1);
      const int out_head = r0 % p.h_per_q, out_tok = tile * p.G + r0 / p.h_per_q;
      float ob[2][32];
      tmem_ld32(ocol, ob[0]);
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) {
        float* o = ob[cc & 1];
        tmem_wait_ld();
        if (cc < 7) {
          tmem_ld32(ocol + (cc + 1) * 32, ob[(cc + 1) & 1]);
        } else {
          // O has been read: the next tile's first PV may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(a_o_free);
        }
        uint32_t w[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          __nv_bfloat162 v2 = __floats2bfloat162_rn(o[2 * j] * oscale, o[2 * j + 1] * oscale);
          w[j] = *reinterpret_cast<uint32_t*>(&v2) & emask;      // rows without a key: zeros
        }
        // the previous round's box must have been read out of the slice
        if (lane == 0) bulk_wait_read_all();
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 4; ++j)
          *reinterpret_cast<uint4*>(st_row + ((j ^ sw) << 4)) =
              make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_3d(&map_out, sbase + stage_off, 256 * h + 32 * cc, out_head, out_tok);
          bulk_commit_group();
        }
      }
      kb0 += nb;
    }
    if (lane == 0) bulk_wait_all();   // boxes written before the CTA retires
    tc_fence_before();
  } else if (warp == 5 && cta == 0) {
    // ------------------------------------------------------------ MMA issue (whole warp, elected lane)
    constexpr uint32_t idesc_qk = umma_idesc(1, 1, false, false, 128, 64);
    constexpr uint32_t idesc_pv = umma_idesc(1, 1, false, true, 128, 256);
    const uint32_t a_qk_done_peer[2] = {mapa(smem_u32(&ms.qk_done[0]), 1), mapa(smem_u32(&ms.qk_done[1]), 1)};
    const uint32_t a_pv_done_peer[2] = {mapa(smem_u32(&ms.pv_done[0]), 1), mapa(smem_u32(&ms.pv_done[1]), 1)};
    const uint32_t a_q_free_peer = mapa(smem_u32(&ms.q_free), 1);
    int kb0 = 0, it = 0;
    for (int tile = cid; tile < p.ng; tile += ncl, ++it) {
      const int nb = plan_tile<kRank>(p, tile).nb;
      mbar_wait(&ms.q_full, it & 1, wt, kSiteQ, it);
      __syncwarp();
      for (int k = 0; k <= nb; ++k) {
        if (k < nb) {
          const int kb = kb0 + k;
          const int s = kb & 1;
          const uint32_t ph = (kb >> 1) & 1;
          mbar_wait(&ms.k_full[s], ph, wt, kSiteKFull, k);
          if (kb >= 2) mbar_wait(&ms.s_free[s], ph ^ 1, wt, kSiteSFree, k);
          __syncwarp();
          tc_fence_after();
          const uint32_t d = tmem + (s ? kTmemS1 : kTmemS0);
          const uint64_t ad0 = umma_desc(sbase + kOffQ, 16, 1024, kSwz128);
          const uint64_t bd0 = umma_desc(sbase + kOffK + s * kKStage, 16, 1024, kSwz128);
#pragma unroll
          for (int j = 0; j < kQChunks; ++j) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              mma_f16_elect(d, ad0 + (uint64_t)(j * (kQChunkBytes >> 4) + kk * 2),
                            bd0 + (uint64_t)(j * (kKChunkBytes >> 4) + kk * 2), idesc_qk,
                            (j | kk) ? 1u : 0u);
          }
          mma_commit_pair_elect(smem_u32(&ms.qk_done[s]));
          mma_commit_pair_elect(a_qk_done_peer[s]);
          if (k == nb - 1) {     // the Q tile is no longer needed once these MMAs complete
            mma_commit_pair_elect(smem_u32(&ms.q_free));
            mma_commit_pair_elect(a_q_free_peer);
          }
        }
        if (k > 0) {
          const int kl = k - 1, kb = kb0 + kl;
          const int s = kb & 1;
          mbar_wait(&ms.p_ready, kb & 1, wt, kSitePReady, kl);
          mbar_wait(&ms.v_full[s], (kb >> 1) & 1, wt, kSiteVFull, kl);
          // the tile's first PV overwrites O: the previous tile must have read it out
          if (kl == 0 && it > 0) mbar_wait(&ms.o_free, (it - 1) & 1, wt, kSiteOFree, it);
          __syncwarp();
          tc_fence_after();
          const uint64_t ad0 = umma_desc(sbase + kOffP, 1024, 128, kSwzNone);
          const uint64_t bd0 = umma_desc(sbase + kOffV + s * kVStage, kVChunkBytes, 1024, kSwz128);
#pragma unroll
          for (int nbk = 0; nbk < 2; ++nbk) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              mma_f16_elect(tmem + kTmemO + nbk * 128, ad0 + (uint64_t)(ks * (2048 >> 4)),
                            bd0 + (uint64_t)(nbk * (2 * kVChunkBytes >> 4) + ks * (2048 >> 4)), idesc_pv,
                            (kl | ks) ? 1u : 0u);
          }
          mma_commit_pair_elect(smem_u32(&ms.pv_done[s]));
          mma_commit_pair_elect(a_pv_done_peer[s]);
        }
      }
      kb0 += nb;
    }
  }

  __syncthreads();
  __syncwarp();
  cluster_sync_all();
  if (warp == 5) tmem_dealloc_pair(tmem, kTmemCols);
  if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(&g_status[3], 1);
}

// The kernel's shared-memory plan leaves 768 bytes for aligning its tiles to 1024 bytes.
// Dynamic shared memory of a kernel without static shared memory starts at a fixed offset
// of the CTA's window; this probe (same configuration: no static shared memory, the same
// dynamic size) reports that offset once per device so that the host can refuse to launch
// instead of letting the kernel give up.
__device__ unsigned g_smem_base_mod1024;
__global__ void smem_base_probe() {
  extern __shared__ uint8_t probe_raw[];
  if (threadIdx.x == 0) g_smem_base_mod1024 = smem_u32(probe_raw) & 1023u;
}
static bool smem_alignment_ok() {
  static thread_local int cached_dev = -1;
  static thread_local bool cached = false;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev == cached_dev) return cached;
  bool ok = false;
  unsigned h = 0xffffffffu;
  if (cudaFuncSetAttribute(smem_base_probe, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem) == cudaSuccess) {
    smem_base_probe<<<1, 32, kSmem>>>();
    if (cudaMemcpyFromSymbol(&h, g_smem_base_mod1024, sizeof(unsigned)) == cudaSuccess) {
      const unsigned pad = (1024u - h) & 1023u;
      ok = pad + kSmemUsed <= kSmem;
    }
  }
  cudaGetLastError();
  cached_dev = dev; cached = ok;
  return ok;
}

// how many 2-CTA clusters of this kernel the current device can hold at once
static int max_clusters() {
  static thread_local int cached_dev = -1, cached = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev == cached_dev) return cached;
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int n = sms / 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sms, 1, 1); cfg.blockDim = dim3(kThreads, 1, 1); cfg.dynamicSmemBytes = kSmem;
  cudaLaunchAttribute at;
  at.id = cudaLaunchAttributeClusterDimension;
  at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
  cfg.attrs = &at; cfg.numAttrs = 1;
  int q = 0;
  if (cudaFuncSetAttribute(dsv4_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem) == cudaSuccess &&
      cudaOccupancyMaxActiveClusters(&q, dsv4_kernel<false>, &cfg) == cudaSuccess && q > 0)
    n = q;
  cudaGetLastError();
  cached_dev = dev; cached = n;
  return n;
}

// One warp per tile: is the tile's gathered index list (its first counts[tile] entries) two
// contiguous ascending runs of valid rows?  runs[tile] = (first row of run 0, its length, first
// row of run 1, its length); a tile that is not sets *gate (cleared by the host beforehand) to 1.
__global__ void __launch_bounds__(128)
classify_runs_kernel(const int32_t* __restrict__ indices, long long idx_stride, int topk,
                     const int32_t* __restrict__ counts, int ng, int s_kv, int4* __restrict__ runs,
                     int* __restrict__ gate) {
  const int tile = (int)((blockIdx.x * (unsigned)blockDim.x + threadIdx.x) >> 5), lane = threadIdx.x & 31;
  if (tile >= ng) return;
  const int32_t* row = indices + (size_t)tile * idx_stride;
  const int cnt = min(max(counts ? __ldg(counts + tile) : topk, 0), topk);
  int breaks = 0, first_break = 0x7fffffff, bad = 0;
  for (int j = lane; j < cnt; j += 32) {
    const int v = __ldg(row + j);
    bad |= (v < 0 || v >= s_kv);
    if (j + 1 < cnt && __ldg(row + j + 1) != v + 1) {
      ++breaks;
      first_break = min(first_break, j);
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    breaks += __shfl_xor_sync(0xffffffffu, breaks, off);
    first_break = min(first_break, __shfl_xor_sync(0xffffffffu, first_break, off));
    bad |= __shfl_xor_sync(0xffffffffu, bad, off);
  }
  if (lane == 0) {
    const int l0 = breaks ? first_break + 1 : cnt;
    const int a0 = cnt > 0 ? __ldg(row) : 0;
    const int b0 = l0 < cnt ? __ldg(row + l0) : 0;
    runs[tile] = make_int4(a0, l0, b0, cnt - l0);
    if (bad || breaks > 1) atomicOr(gate, 1);
  }
}

}  // namespace dsv4

// Rank mode of the range kernel for the reference operator's argument list (see
// litedsa_dsv4_masked_mla_bf16): classifies every tile's index list on the device, then enqueues
// the range kernel gated on "every tile is two contiguous runs".  workspace: 16 + 16 * ng bytes
// (gate word, then runs[ng]); the caller enqueues the gather kernel behind it, gated on the
// opposite value, so exactly one of the two does the work -- no host synchronisation.
int dsv4_rank_enqueue(const void* q, const void* kv, const int32_t* indices, const int32_t* pref,
                      const int32_t* win_lo, const int32_t* win_hi, const int32_t* counts,
                      float sm_scale, int h_per_q, void* out, float* lse, const float* attn_sink,
                      int ng, int s_kv, int topk, int d, int64_t q_row_stride, int64_t kv_row_stride,
                      int64_t indices_row_stride, int64_t q_token_stride, int64_t q_head_stride,
                      int64_t out_token_stride, int64_t out_head_stride, void* workspace,
                      cudaStream_t stream) {
  using namespace dsv4;
  int* gate = reinterpret_cast<int*>(workspace);
  int4* runs = reinterpret_cast<int4*>(reinterpret_cast<char*>(workspace) + 16);
  if (!smem_alignment_ok()) return LITEDSA_ERR_UNSUPPORTED;
  if (cudaMemsetAsync(gate, 0, 16, stream) != cudaSuccess) return LITEDSA_ERR_CUDA;
  classify_runs_kernel<<<(ng + 3) / 4, 128, 0, stream>>>(indices, indices_row_stride, topk, counts, ng, s_kv,
                                                         runs, gate);
  const int G = 128 / h_per_q;
  CUtensorMap mq, mk32, mk64, mout;
  const auto BF = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const uint64_t q_hs = (q_head_stride ? (uint64_t)q_head_stride : (uint64_t)q_row_stride) * 2;
  const uint64_t q_ts = q_token_stride ? (uint64_t)q_token_stride * 2 : (uint64_t)h_per_q * q_hs;
  const uint64_t o_hs = (out_head_stride ? (uint64_t)out_head_stride : (uint64_t)kDV) * 2;
  const uint64_t o_ts = out_token_stride ? (uint64_t)out_token_stride * 2 : (uint64_t)h_per_q * o_hs;
  const uint32_t qb_h = (uint32_t)min(h_per_q, 64), ob_h = (uint32_t)min(h_per_q, 32);
  // tensors are declared d columns wide: for d = 512 the kernel's ninth 64-dim chunk lies
  // outside and is zero-filled by TMA, so the 576-dim kernel serves both widths
  if (!make_map_3d(&mq, q, BF, (uint64_t)d, (uint64_t)h_per_q, (uint64_t)ng * G, q_hs, q_ts, 64, qb_h, 64 / qb_h) ||
      !make_map_2d(&mk32, kv, BF, (uint64_t)d, (uint64_t)s_kv, (uint64_t)kv_row_stride * 2, 64, 32) ||
      !make_map_2d(&mk64, kv, BF, (uint64_t)d, (uint64_t)s_kv, (uint64_t)kv_row_stride * 2, 64, 64) ||
      !make_map_3d(&mout, out, BF, kDV, (uint64_t)h_per_q, (uint64_t)ng * G, o_hs, o_ts, 32, ob_h, 32 / ob_h,
                   CU_TENSOR_MAP_SWIZZLE_64B))
    return LITEDSA_ERR_CUDA;
  Params p;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.lse = lse; p.sink = attn_sink;
  p.ng = ng; p.n_comp = 0; p.s_raw = s_kv; p.G = G; p.h_per_q = h_per_q; p.pos0 = 0;
  p.window = 1; p.ratio = 1; p.scale_log2 = sm_scale * kLog2e;
  p.epoch = next_launch_epoch(); p.wait_limit_ns = wait_limit_ns();
  p.runs = runs; p.pref = pref; p.win_lo = win_lo; p.win_hi = win_hi; p.counts = counts;
  p.gate = gate; p.gate_value = 0;
  if (cudaFuncSetAttribute(dsv4_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem) !=
      cudaSuccess)
    return LITEDSA_ERR_CUDA;
  dsv4_kernel<true><<<2 * min(ng, max_clusters()), kThreads, kSmem, stream>>>(mq, mk32, mk32, mk64, mk64, mout, p);
  return cudaGetLastError() == cudaSuccess ? LITEDSA_OK : LITEDSA_ERR_CUDA;
}

namespace dsv4 {
}  // namespace dsv4
}  // namespace lt

// DSv4 packed BF16 attention over (compressed prefix, sliding window).  Replaces the
// reference operator dsv4_masked_mla_bf16 (kernels/b200/dsa/litedsa_dsv4.cu:50-55) for
// callers whose two key ranges are contiguous: instead of a gathered union index list plus
// per-token rank ranges it takes the two KV tensors and the first query position.
extern "C" int litedsa_dsv4_c128a_bf16(const void* q, const void* kv_comp, const void* kv_raw,
                                       int ng, int h_per_q, int n_comp, int s_raw, int pos0,
                                       int window, int ratio, float sm_scale,
                                       const float* attn_sink, void* out, float* lse,
                                       int64_t q_row_stride, int64_t kc_row_stride,
                                       int64_t kr_row_stride, int64_t q_token_stride,
                                       int64_t q_head_stride, int64_t out_token_stride,
                                       int64_t out_head_stride, void* stream) {
  using namespace lt;
  using namespace lt::dsv4;
  if (!q || !kv_raw || !out || !lse) return LITEDSA_ERR_ARG;
  if (n_comp > 0 && !kv_comp) return LITEDSA_ERR_ARG;
  if (ng <= 0 || s_raw <= 0 || n_comp < 0 || pos0 < 0 || window <= 0 || ratio <= 0)
    return LITEDSA_ERR_SHAPE;
  if (h_per_q <= 0 || 128 % h_per_q != 0 || 128 / h_per_q > 16) return LITEDSA_ERR_SHAPE;
  const int G = 128 / h_per_q;
  if ((int64_t)pos0 + (int64_t)ng * G > s_raw) return LITEDSA_ERR_SHAPE;   // queries sit inside the cache
  if (window + G - 1 > 8 * kBlockKeys * 64) return LITEDSA_ERR_UNSUPPORTED;
  // strides are in ELEMENTS (bf16); TMA needs 16-byte aligned bases and pitches
  if (q_row_stride < kD || kr_row_stride < kD || (q_row_stride % 8) || (kr_row_stride % 8) ||
      (n_comp > 0 && (kc_row_stride < kD || (kc_row_stride % 8))))
    return LITEDSA_ERR_UNSUPPORTED;
  if (((uintptr_t)q | (uintptr_t)kv_raw | (uintptr_t)kv_comp | (uintptr_t)out) & 15)
    return LITEDSA_ERR_UNSUPPORTED;
  if (q_token_stride < 0 || q_head_stride < 0 || out_token_stride < 0 || out_head_stride < 0)
    return LITEDSA_ERR_SHAPE;
  if ((q_head_stride && (q_head_stride < kD || q_head_stride % 8)) || q_token_stride % 8 ||
      (out_head_stride && (out_head_stride < kDV || out_head_stride % 8)) || out_token_stride % 8)
    return LITEDSA_ERR_UNSUPPORTED;
  const void* kc = n_comp > 0 ? kv_comp : kv_raw;      // never dereferenced when n_comp == 0
  const uint64_t kc_rows = n_comp > 0 ? (uint64_t)n_comp : 1;
  const int64_t kc_pitch = n_comp > 0 ? kc_row_stride : kr_row_stride;
  CUtensorMap mq, mkc32, mkr32, mkc64, mkr64, mout;
  const auto BF = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  // q and out are addressed as (dim, head, token): row r of a tile is (token r / h, head r % h),
  // which covers the dense packed layout and the in-place layout with padded head slots alike
  const uint64_t q_hs = (q_head_stride ? (uint64_t)q_head_stride : (uint64_t)q_row_stride) * 2;
  const uint64_t q_ts = q_token_stride ? (uint64_t)q_token_stride * 2 : (uint64_t)h_per_q * q_hs;
  const uint64_t o_hs = (out_head_stride ? (uint64_t)out_head_stride : (uint64_t)kDV) * 2;
  const uint64_t o_ts = out_token_stride ? (uint64_t)out_token_stride * 2 : (uint64_t)h_per_q * o_hs;
  const uint32_t qb_h = (uint32_t)min(h_per_q, 64), ob_h = (uint32_t)min(h_per_q, 32);
  if (!make_map_3d(&mq, q, BF, kD, (uint64_t)h_per_q, (uint64_t)ng * G, q_hs, q_ts, 64, qb_h, 64 / qb_h) ||
      !make_map_2d(&mkc32, kc, BF, kD, kc_rows, (uint64_t)kc_pitch * 2, 64, 32) ||
      !make_map_2d(&mkr32, kv_raw, BF, kD, (uint64_t)s_raw, (uint64_t)kr_row_stride * 2, 64, 32) ||
      !make_map_2d(&mkc64, kc, BF, kD, kc_rows, (uint64_t)kc_pitch * 2, 64, 64) ||
      !make_map_2d(&mkr64, kv_raw, BF, kD, (uint64_t)s_raw, (uint64_t)kr_row_stride * 2, 64, 64) ||
      // out leaves as boxes of 32 rows x 32 dims (64 bytes wide, 64-byte swizzle)
      !make_map_3d(&mout, out, BF, kDV, (uint64_t)h_per_q, (uint64_t)ng * G, o_hs, o_ts, 32, ob_h, 32 / ob_h,
                   CU_TENSOR_MAP_SWIZZLE_64B))
    return LITEDSA_ERR_CUDA;
  Params p;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.lse = lse; p.sink = attn_sink;
  p.ng = ng; p.n_comp = n_comp; p.s_raw = s_raw; p.G = G; p.h_per_q = h_per_q; p.pos0 = pos0;
  p.window = window; p.ratio = ratio; p.scale_log2 = sm_scale * kLog2e;
  p.epoch = next_launch_epoch(); p.wait_limit_ns = wait_limit_ns();
  if (!smem_alignment_ok()) return LITEDSA_ERR_UNSUPPORTED;   // first call per device: synchronous probe
  p.runs = nullptr; p.pref = p.win_lo = p.win_hi = p.counts = nullptr; p.gate = nullptr; p.gate_value = 0;
  if (cudaFuncSetAttribute(dsv4_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem) !=
      cudaSuccess)
    return LITEDSA_ERR_CUDA;
  dsv4_kernel<false><<<2 * min(ng, max_clusters()), kThreads, kSmem, reinterpret_cast<cudaStream_t>(stream)>>>(
      mq, mkc32, mkr32, mkc64, mkr64, mout, p);
  return cudaGetLastError() == cudaSuccess ? LITEDSA_OK : LITEDSA_ERR_CUDA;
}

// Status word of the DSv4 kernel (same meaning as litedsa_attn_status).
extern "C" int litedsa_dsv4_status(int* out4_host, int reset) {
  using namespace lt::dsv4;
  if (out4_host && cudaMemcpyFromSymbol(out4_host, g_status, sizeof(int) * 4) != cudaSuccess)
    return LITEDSA_ERR_CUDA;
  if (reset) {
    const int z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (cudaMemcpyToSymbol(g_status, z, sizeof(z)) != cudaSuccess) return LITEDSA_ERR_CUDA;
  }
  return (out4_host && out4_host[0] != 0) ? LITEDSA_ERR_TIMEOUT : LITEDSA_OK;
}

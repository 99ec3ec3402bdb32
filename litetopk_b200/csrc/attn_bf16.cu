// Masked BF16 MLA prefill over a per-tile union list of gathered KV rows (sm_100a).
//
// Two operators of the reference end up here:
//   * dsv4_masked_mla_bf16(q, kv, indices, pref, win_lo, win_hi, counts, sm_scale, h_per_q,
//     out, lse, attn_sink)  (kernels/b200/dsa/litedsa_dsv4.cu:50-121, kernel
//     kernels/b200/dsa/litedsa_attention_sm100_dsv4.cuh:1849-2485): bf16 q / KV rows of 512
//     dims gathered through an ascending index list; row r of a tile attends the union
//     ranks [0, pref) and [win_lo, win_hi) of its token (range_mask32, :1824-1829);
//   * masked_mla_fp8 on a cache whose per-128 scales differ and whose rope part is bf16
//     (the DeepSeek-V3.2 cache row): such a cache has no single-scale all-e4m3 form, so it is
//     dequantised once into a bf16 [s_kv, 576] workspace (litedsa_dequant_kv656) and attended
//     here with the query-major membership mask of union_qm
//     (kernels/b200/dsa/litedsa_union.cuh:147-171) at bf16 accuracy -- the same "flat
//     dequantised workspace" route the reference's own bf16 operator takes
//     (litedsa_dsv4.cu:40-48).
//
// Numerics are the reference bf16 kernel's (litedsa_attention_sm100_dsv4.cuh:2015-2157):
// 64-key blocks in rank order, base-2 online softmax whose running max moves only when a
// row of a 32-row group overshoots it by more than 6, P stored as bf16 without pre-scale,
// fp32 accumulation, optional sink in the output normaliser only.
//
// Organisation: persistent clusters of 2 CTAs (64 query rows each) walking tiles
// cid, cid + #clusters, ...; tcgen05 cta_group::2 kind::f16 MMAs (S = Q K^T: N = 64 keys split
// over the pair; O += P V: two N = 256 halves, value dims split over the pair); S
// double-buffered in TMEM, O in TMEM.  20 warps per CTA:
//   warps 0-3    softmax (thread = TMEM lane: row = lane % 64, key half = lane / 64);
//   warps 4-11   KV row gather: 16-byte cp.async copies written straight into the
//                128-byte-swizzled tile layout (K: own 32 keys x kD dims; V: all 64 keys x this
//                CTA's 256 value dims), two independent ready-driven cursors; warp 4 also
//                loads the Q tile (TMA);
//   warp 12      MMA issue (leader CTA; one elected lane issues);
//   warps 13-14  relay "K / V landed" from the peer CTA to the leader's barriers;
//   warp 15      index-validity bits (index in range and rank < count);
//   warps 16-19  tile epilogue: O out of TMEM, x 1 / normaliser, bf16, TMA tile stores, while
//                the softmax warps already work on the next tile.
// No TMA multicast of any kind.  Every wait is bounded (common.cuh).
#include "common.cuh"
#include "tensor_map.cuh"

namespace lt {
namespace b16 {

constexpr int kThreads = 640;
constexpr int kSoftmaxWarps = 4, kProducerWarps = 8;
constexpr int kWarpProd0 = 4, kWarpMma = 12, kWarpRelayK = 13, kWarpRelayV = 14, kWarpValid = 15,
              kWarpEpi0 = 16;
constexpr int kBlockKeys = 64;
constexpr int kDV = 512;
constexpr uint32_t kQChunkBytes = 64 * 128;           // 64 rows x 64 bf16
constexpr uint32_t kKChunkBytes = 32 * 128;           // 32 keys per CTA
constexpr uint32_t kVChunkBytes = 64 * 128;           // 64 keys x 64 dims
constexpr uint32_t kVStage = 4 * kVChunkBytes;        // 64 keys x 256 dims = 32768
constexpr uint32_t kPBytes = 64 * 64 * 2;             // 64 rows x 64 keys bf16
constexpr uint32_t kStageBytes = 4 * 2048;            // output staging, one 2 KB slice per epilogue warp
constexpr uint32_t kMiscBytes = 2304;

template <int kD>
struct Plan {
  static constexpr int kChunks = kD / 64;                       // 128-byte chunks per row
  static constexpr uint32_t kQBytes = kChunks * kQChunkBytes;   // per CTA
  static constexpr uint32_t kKStage = kChunks * kKChunkBytes;
  static constexpr uint32_t kOffQ = 0;
  static constexpr uint32_t kOffK = kOffQ + kQBytes;
  static constexpr uint32_t kOffV = kOffK + 2 * kKStage;
  static constexpr uint32_t kOffP = kOffV + 2 * kVStage;
  static constexpr uint32_t kOffStage = kOffP + kPBytes;
  static constexpr uint32_t kOffMisc = kOffStage + kStageBytes;
  static constexpr uint32_t kUsed = kOffMisc + kMiscBytes;
  // 576 dims fill the 227 KB to within 768 bytes: the launcher checks the alignment of the
  // dynamic shared-memory base instead of reserving a full 1 KB of slack
  static constexpr uint32_t kSmem = kUsed + 1024 <= 232448 ? kUsed + 1024 : 232448;
  static_assert(kUsed <= 232448, "shared-memory plan exceeds the 227 KB per-CTA limit");
};

constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemO = 0, kTmemS0 = 256, kTmemS1 = 288;   // S: 32 columns per buffer

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kMInit = -1e30f;
constexpr float kRescaleThreshold = 6.0f;

struct Misc {
  // leader CTA only: q_full, k_peer / v_peer (peer's tiles landed), s_free / p_ready
  uint64_t q_full, k_peer[2], v_peer[2], s_free[2], p_ready;
  // every CTA
  uint64_t k_land[2], v_land[2], qk_done[2], pv_done[2], valid_ready[2], valid_free[2];
  uint64_t q_free;                  // the tile's QK^T are complete (Q tile reusable)
  uint64_t o_free;                  // leader CTA: the tile's O has been read out of TMEM
  uint64_t epi_ready;               // the tile's row scales are published
  uint32_t valid[2][2];             // 64 validity bits per stage
  uint32_t tmem_base, pad;
  float xbuf[3][128];               // [block parity | 2 = end-of-tile row-sum merge][lane]
  float oscale[2][64];              // [tile parity][row]: 1 / normaliser, 0 for rows without a key
};
static_assert(sizeof(Misc) <= kMiscBytes, "Misc too large");

struct Params {
  const uint8_t* kv;         // bf16 rows, kv_pitch bytes apart
  long long kv_pitch;
  const int32_t* indices;    // [ng, idx_stride] physical rows in ascending rank order
  long long idx_stride;
  const int32_t* counts;     // [ng] live entries per tile, or null (= cap)
  const uint32_t* memb;      // [ng, G, cap/32] membership bits, or null (range mode)
  const int32_t* pref;       // [ng, G] range mode: rank < pref ...
  const int32_t* win_lo;     // [ng, G] ... or win_lo <= rank < win_hi
  const int32_t* win_hi;
  const float* sink;         // [128] per packed row, or null
  float* lse;                // [ng, 128]
  float* max_logits;         // [ng, 128] or null
  int ng, s_kv, cap, h_per_q, G;
  float scale_log2;
  int epoch;
  unsigned long long wait_limit_ns;
  // the launch runs only if *gate == gate_value (null: always): the device-side choice between
  // this kernel and the range kernel's rank mode
  const int* gate;
  int gate_value;
};

enum { kSiteQ = 201, kSiteKLand, kSiteKPeer, kSiteVLand, kSiteVPeer, kSiteQkDone, kSitePvDone,
       kSiteSFree, kSitePReady, kSiteValidReady, kSiteValidFree, kSiteKFree, kSitePFree, kSiteEpi,
       kSiteRelayK, kSiteRelayV, kSiteQFree, kSiteOFree, kSiteSmem };

// status block of the bf16 gather kernel (layout: see Waiter in common.cuh)
__device__ int g_status[8];

__device__ __forceinline__ void mma_f16_elect(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, pe;\n\tsetp.ne.b32 p, %4, 0;\n\telect.sync _|pe, 0xffffffff;\n\t"
      "@pe tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// bits j of [0, 32) with lo <= j < hi
__device__ __forceinline__ uint32_t range_bits(int lo, int hi) {
  lo = max(lo, 0);
  hi = min(hi, 32);
  if (hi <= lo) return 0u;
  const uint32_t upto_hi = hi >= 32 ? 0xffffffffu : ((1u << hi) - 1u);
  return upto_hi & ~((1u << lo) - 1u);
}

template <int kD>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
masked_mla_bf16_kernel(const __grid_constant__ CUtensorMap map_q,
                       const __grid_constant__ CUtensorMap map_out, const Params p) {
  using PL = Plan<kD>;
  constexpr int kChunks = PL::kChunks;
  constexpr int kRowPieces = kD / 8;                  // 16-byte pieces per KV row
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;      // 128B-swizzle tiles need 1024-byte alignment
  uint8_t* sm = smem_raw + (sbase - raw);
  Misc& ms = *reinterpret_cast<Misc*>(sm + PL::kOffMisc);
  const Waiter wt{g_status, p.epoch, p.wait_limit_ns};
  if (p.gate != nullptr && *reinterpret_cast<const volatile int*>(p.gate) != p.gate_value) return;
  // refuse to run (uniformly, in both CTAs, before any barrier exists) if aligning the base
  // would push the plan past the allocation
  if ((sbase - raw) + PL::kUsed > PL::kSmem) {
    if (threadIdx.x == 0) wt.fail(kSiteSmem, 0);
    return;
  }

  const uint32_t cta = cluster_ctarank();
  const int cid = blockIdx.x >> 1, ncl = gridDim.x >> 1;
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  auto tile_count = [&](int tile) -> int {
    const int c = p.counts ? p.counts[tile] : p.cap;
    return min(max(c, 0), p.cap);
  };
  auto blocks_of = [&](int count) -> int { return max((count + kBlockKeys - 1) / kBlockKeys, 1); };

  if (threadIdx.x == 0) {
    mbar_init(&ms.q_full, 1);
    mbar_init(&ms.p_ready, 8);          // 4 softmax warps x 2 CTAs
    mbar_init(&ms.q_free, 1);
    mbar_init(&ms.o_free, 8);           // 4 epilogue warps x 2 CTAs
    mbar_init(&ms.epi_ready, kSoftmaxWarps);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ms.k_peer[i], 1);
      mbar_init(&ms.v_peer[i], 1);
      mbar_init(&ms.s_free[i], 8);
      mbar_init(&ms.k_land[i], kProducerWarps * 32);   // one async arrival per gather thread
      mbar_init(&ms.v_land[i], kProducerWarps * 32);
      mbar_init(&ms.qk_done[i], 1);
      mbar_init(&ms.pv_done[i], 1);
      mbar_init(&ms.valid_ready[i], 1);
      mbar_init(&ms.valid_free[i], kSoftmaxWarps);
    }
    fence_mbar_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_out);
  }
  __syncthreads();
  cluster_sync_all();
  if (warp == kWarpMma) {
    tmem_alloc_pair(&ms.tmem_base, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ms.tmem_base;

  if (warp < kSoftmaxWarps) {
    // ------------------------------------------------------------ softmax
    const int tl = threadIdx.x;                   // TMEM lane
    const int r = tl & 63, h = tl >> 6;           // row of this CTA, key half (32 columns)
    const int row = (int)cta * 64 + r;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const float c = p.scale_log2;
    const int capw = p.cap >> 5;
    const uint32_t a_s_free[2] = {mapa(smem_u32(&ms.s_free[0]), 0), mapa(smem_u32(&ms.s_free[1]), 0)};
    const uint32_t a_p_ready = mapa(smem_u32(&ms.p_ready), 0);
    int kb0 = 0, it = 0;
    for (int tile = cid; tile < p.ng; tile += ncl) {
      const int nb = blocks_of(tile_count(tile));
      const size_t trow = (size_t)tile * p.G + row / p.h_per_q;     // (tile, token) of this row
      const uint32_t* mrow = p.memb ? p.memb + trow * capw + h : nullptr;
      int pref_q = 0, lo_q = 0, hi_q = 0;
      if (!mrow) {
        pref_q = __ldg(p.pref + trow);
        lo_q = __ldg(p.win_lo + trow);
        hi_q = __ldg(p.win_hi + trow);
      }
      uint32_t mk = mrow ? __ldg(mrow) : 0u;
      float m = kMInit, li = 0.f, real_m = -INFINITY;

      for (int k = 0; k < nb; ++k) {
        const int kb = kb0 + k;
        const int s = kb & 1;
        const uint32_t ph = (kb >> 1) & 1;
        uint32_t mk_next = mk;
        if (mrow && k + 1 < nb) mk_next = __ldg(mrow + (size_t)(k + 1) * 2);
        mbar_wait(&ms.qk_done[s], ph, wt, kSiteQkDone, k);
        tc_fence_after();
        float sv[32];
        tmem_ld32(tmem + lane_base + (s ? kTmemS1 : kTmemS0), sv);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(a_s_free[s]);

        // my 32 columns are the union ranks [64k + 32h, +32)
        uint32_t bits;
        if (mrow) {
          bits = mk;
        } else {
          const int base = k * kBlockKeys + 32 * h;
          bits = range_bits(0, pref_q - base) | range_bits(lo_q - base, hi_q - base);
        }
        mbar_wait(&ms.valid_ready[s], ph, wt, kSiteValidReady, k);
        bits &= ms.valid[s][h];
        __syncwarp();
        if (lane == 0) mbar_arrive(&ms.valid_free[s]);
        mk = mk_next;

        float cur = -INFINITY;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          sv[j] = ((bits >> j) & 1u) ? sv[j] : -INFINITY;
          cur = fmaxf(cur, sv[j]);
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
        uint8_t* pdst = sm + PL::kOffP + (4 * h) * 1024 + r * 16;
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

      // end of tile: merge the two key halves' row sums, publish lse and 1 / normaliser
      ms.xbuf[2][tl] = li;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      li += ms.xbuf[2][tl ^ 64];
      if (real_m == -INFINITY) { li = 0.f; m = -INFINITY; }
      const size_t grow = (size_t)tile * 128 + row;
      if (h == 0) {
        float l = __logf(li) + m * kLn2;
        if (!(li > 0.f)) l = INFINITY;
        p.lse[grow] = l;
        if (p.max_logits) p.max_logits[grow] = real_m * kLn2;
      }
      float denom = li;
      if (p.sink != nullptr && li > 0.f) denom += fast_exp2(__ldg(p.sink + row) * kLog2e - m);
      if (h == 0) ms.oscale[it & 1][r] = (li > 0.f) ? __fdividef(1.0f, denom) : 0.f;
      __syncwarp();
      if (lane == 0) mbar_arrive(&ms.epi_ready);
      kb0 += nb;
      ++it;
    }
  } else if (warp < kWarpProd0 + kProducerWarps) {
    // ------------------------------------------------------------ KV row gather (cp.async) and the Q tile (TMA)
    // Warp pw owns rows [4pw, 4pw+4) of this CTA's 32 keys for the K tile (kD bf16 = kRowPieces
    // 16-byte pieces per row) and rows [8pw, 8pw+8) of the block's 64 keys for the V tile
    // (this CTA's 256 value dims = 32 pieces per row, one row per instruction).
    const int pw = warp - kWarpProd0;
    const uint32_t a_q_full = mapa(smem_u32(&ms.q_full), 0);
    struct Cursor { int tile, k, nb, kb0; };
    auto cur_init = [&](Cursor& cu) {
      cu.tile = cid; cu.k = 0; cu.kb0 = 0;
      cu.nb = cu.tile < p.ng ? blocks_of(tile_count(cu.tile)) : 0;
    };
    auto cur_next = [&](Cursor& cu) {
      if (++cu.k == cu.nb) {
        cu.kb0 += cu.nb; cu.k = 0; cu.tile += ncl;
        cu.nb = cu.tile < p.ng ? blocks_of(tile_count(cu.tile)) : 0;
      }
    };
    Cursor ck, cv;
    cur_init(ck);
    cur_init(cv);
    const uint64_t pol_stream = l2_policy_evict_first();
    // lane l < 4 holds the index of own key 4pw + l (K rows), lane 8 + l (l < 8) of key
    // 8pw + l of the block's 64 keys (V rows)
    const int my_key = lane < 8 ? 32 * (int)cta + 4 * pw + (lane & 3) : 8 * pw + ((lane - 8) & 7);
    auto load_idx = [&](const Cursor& cu) -> int {
      const int v = __ldg(p.indices + (size_t)cu.tile * p.idx_stride + (size_t)cu.k * kBlockKeys + my_key);
      return ((unsigned)v < (unsigned)p.s_kv) ? v : 0;     // out-of-range rows are masked later
    };
    int kidx = 0, vidx = 0;
    if (ck.tile < p.ng) { kidx = load_idx(ck); vidx = load_idx(cv); }
    const uint8_t* kvb = p.kv;
    const long long pitch = p.kv_pitch;
    int q_tile = cid, q_it = 0;
    unsigned long long idle_since = 0;
    unsigned idle_iters = 0;
    bool aborted = false;
    while ((ck.tile < p.ng || cv.tile < p.ng || (pw == 0 && q_tile < p.ng)) && !aborted) {
      bool did = false;
      if (pw == 0 && q_tile < p.ng) {
        // the previous tile's Q must have been consumed by its last QK^T
        const bool okq = q_it == 0 || mbar_test(&ms.q_free, (q_it - 1) & 1);
        if (__all_sync(0xffffffffu, okq)) {
          if (lane == 0) {
            if (cta == 0) mbar_arrive_expect_tx(&ms.q_full, 2 * PL::kQBytes);
            for (int j = 0; j < kChunks; ++j)
              // this CTA's 64 rows of the tile = (token, head) pairs starting at row 64 cta
              tma_load_3d_pair_hint(sbase + PL::kOffQ + j * kQChunkBytes, &map_q, 64 * j,
                                    (64 * (int)cta) % p.h_per_q, q_tile * p.G + (64 * (int)cta) / p.h_per_q,
                                    a_q_full, pol_stream);
          }
          __syncwarp();
          q_tile += ncl;
          ++q_it;
          did = true;
        }
      }
      if (ck.tile < p.ng) {
        const int kb = ck.kb0 + ck.k;
        const int s = kb & 1;
        const uint32_t ph = (kb >> 1) & 1;
        // stage s held block kb-2: its QK^T must have read it
        const bool ok = kb < 2 || mbar_test(&ms.qk_done[s], ph ^ 1);
        if (__all_sync(0xffffffffu, ok)) {
          const uint32_t kst = sbase + PL::kOffK + s * PL::kKStage;
          // 4 rows x kRowPieces pieces, linear id L = 32 i + lane: row L / kRowPieces
#pragma unroll
          for (int i = 0; i < (4 * kRowPieces) / 32; ++i) {
            const int L = 32 * i + lane;
            const int rl = L / kRowPieces, pi = L - rl * kRowPieces;   // constants: shifts / mul
            const int ri = __shfl_sync(0xffffffffu, kidx, rl);
            const int row = 4 * pw + rl;
            const int cj = pi >> 3, cc = pi & 7;
            cp_async16(kst + cj * kKChunkBytes + row * 128 + ((cc ^ (row & 7)) << 4),
                            kvb + (size_t)ri * pitch + 16 * pi);
          }
          cp_async_mbar_arrive_noinc(&ms.k_land[s]);
          cur_next(ck);
          if (ck.tile < p.ng) kidx = load_idx(ck);
          did = true;
        }
      }
      if (cv.tile < p.ng) {
        const int kb = cv.kb0 + cv.k;
        const int s = kb & 1;
        const uint32_t ph = (kb >> 1) & 1;
        // V stage s was last read by the PV of block kb-2
        const bool ok = kb < 2 || mbar_test(&ms.pv_done[s], ph ^ 1);
        if (__all_sync(0xffffffffu, ok)) {
          const uint32_t vst = sbase + PL::kOffV + s * kVStage;
          const int cj = lane >> 3, cc = lane & 7;      // piece `lane` of the row's 512 value bytes
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int ri = __shfl_sync(0xffffffffu, vidx, 8 + i);
            const int row = 8 * pw + i;
            cp_async16(vst + cj * kVChunkBytes + row * 128 + ((cc ^ (row & 7)) << 4),
                            kvb + (size_t)ri * pitch + 512 * (int)cta + 16 * lane);
          }
          cp_async_mbar_arrive_noinc(&ms.v_land[s]);
          cur_next(cv);
          if (cv.tile < p.ng) vidx = load_idx(cv);
          did = true;
        }
      }
      if (did) {
        idle_since = 0;
        idle_iters = 0;
      } else if ((++idle_iters & 63u) != 0) {
        __nanosleep(8);
      } else {
        // the (slow) time-limit and abort check runs once per 64 idle polls
        const unsigned long long now = globaltimer_ns();
        if (idle_since == 0) idle_since = now;
        bool stop = wt.aborting();
        if (now - idle_since > wt.limit_ns) {
          if (lane == 0) wt.fail(kSiteKFree, ck.k);
          stop = true;
        }
        aborted = __any_sync(0xffffffffu, stop);
      }
    }
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------ MMA issue (leader CTA; elected lane)
    if (cta == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(1, 1, false, false, 128, 64);
      constexpr uint32_t idesc_pv = umma_idesc(1, 1, false, true, 128, 256);
      const uint32_t a_qk_done_peer[2] = {mapa(smem_u32(&ms.qk_done[0]), 1), mapa(smem_u32(&ms.qk_done[1]), 1)};
      const uint32_t a_pv_done_peer[2] = {mapa(smem_u32(&ms.pv_done[0]), 1), mapa(smem_u32(&ms.pv_done[1]), 1)};
      const uint32_t a_q_free_peer = mapa(smem_u32(&ms.q_free), 1);
      int kb0 = 0, it = 0;
      for (int tile = cid; tile < p.ng; tile += ncl, ++it) {
        const int nb = blocks_of(tile_count(tile));
        mbar_wait(&ms.q_full, it & 1, wt, kSiteQ, it);
        __syncwarp();
        for (int k = 0; k <= nb; ++k) {
          if (k < nb) {
            const int kb = kb0 + k;
            const int s = kb & 1;
            const uint32_t ph = (kb >> 1) & 1;
            mbar_wait(&ms.k_land[s], ph, wt, kSiteKLand, k);
            mbar_wait(&ms.k_peer[s], ph, wt, kSiteKPeer, k);
            if (kb >= 2) mbar_wait(&ms.s_free[s], ph ^ 1, wt, kSiteSFree, k);
            __syncwarp();
            // the K tile was written by cp.async (generic proxy), the MMA reads it through
            // the async proxy
            fence_proxy_async_smem();
            tc_fence_after();
            const uint32_t d = tmem + (s ? kTmemS1 : kTmemS0);
            const uint64_t ad0 = umma_desc(sbase + PL::kOffQ, 16, 1024, kSwz128);
            const uint64_t bd0 = umma_desc(sbase + PL::kOffK + s * PL::kKStage, 16, 1024, kSwz128);
#pragma unroll
            for (int j = 0; j < kChunks; ++j) {
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
            const uint32_t ph = (kb >> 1) & 1;
            mbar_wait(&ms.p_ready, kb & 1, wt, kSitePReady, kl);
            mbar_wait(&ms.v_land[s], ph, wt, kSiteVLand, kl);
            mbar_wait(&ms.v_peer[s], ph, wt, kSiteVPeer, kl);
            // the tile's first PV overwrites O: the previous tile must have read it out
            if (kl == 0 && it > 0) mbar_wait(&ms.o_free, (it - 1) & 1, wt, kSiteOFree, it);
            __syncwarp();
            fence_proxy_async_smem();
            tc_fence_after();
            const uint64_t ad0 = umma_desc(sbase + PL::kOffP, 1024, 128, kSwzNone);
            const uint64_t bd0 = umma_desc(sbase + PL::kOffV + s * kVStage, kVChunkBytes, 1024, kSwz128);
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
  } else if (warp == kWarpRelayK || warp == kWarpRelayV) {
    // ------------------------------------------------------------ "landed" relays to the leader CTA
    if (cta == 1) {
      const bool is_k = warp == kWarpRelayK;
      const uint32_t a_peer[2] = {mapa(smem_u32(is_k ? &ms.k_peer[0] : &ms.v_peer[0]), 0),
                                  mapa(smem_u32(is_k ? &ms.k_peer[1] : &ms.v_peer[1]), 0)};
      int kb0 = 0;
      for (int tile = cid; tile < p.ng; tile += ncl) {
        const int nb = blocks_of(tile_count(tile));
        for (int k = 0; k < nb; ++k) {
          const int kb = kb0 + k;
          const int s = kb & 1;
          const uint32_t ph = (kb >> 1) & 1;
          mbar_wait(is_k ? &ms.k_land[s] : &ms.v_land[s], ph, wt, is_k ? kSiteRelayK : kSiteRelayV, k);
          fence_proxy_async_smem();     // this CTA's cp.async writes -> the leader's MMA reads
          if (lane == 0) mbar_arrive_cluster_release(a_peer[s]);
        }
        kb0 += nb;
      }
    }
  } else if (warp == kWarpValid) {
    // ------------------------------------------------------------ index-validity bits
    int kb0 = 0;
    for (int tile = cid; tile < p.ng; tile += ncl) {
      const int count = tile_count(tile);
      const int nb = blocks_of(count);
      const int32_t* idx_row = p.indices + (size_t)tile * p.idx_stride;
      int i0 = __ldg(idx_row + lane), i1 = __ldg(idx_row + 32 + lane);
      for (int k = 0; k < nb; ++k) {
        const int kb = kb0 + k;
        const int s = kb & 1;
        const uint32_t ph = (kb >> 1) & 1;
        int n0 = i0, n1 = i1;
        if (k + 1 < nb) {
          n0 = __ldg(idx_row + (size_t)(k + 1) * kBlockKeys + lane);
          n1 = __ldg(idx_row + (size_t)(k + 1) * kBlockKeys + 32 + lane);
        }
        const int rank0 = k * kBlockKeys + lane;
        const uint32_t w0 = __ballot_sync(0xffffffffu, (unsigned)i0 < (unsigned)p.s_kv && rank0 < count);
        const uint32_t w1 = __ballot_sync(0xffffffffu, (unsigned)i1 < (unsigned)p.s_kv && rank0 + 32 < count);
        if (kb >= 2) mbar_wait(&ms.valid_free[s], ph ^ 1, wt, kSiteValidFree, k);
        if (lane == 0) {
          ms.valid[s][0] = w0;
          ms.valid[s][1] = w1;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&ms.valid_ready[s]);
        i0 = n0;
        i1 = n1;
      }
      kb0 += nb;
    }
  } else {
    // ------------------------------------------------------------ epilogue warps
    // O out of TMEM, x 1 / normaliser, bf16, TMA tile stores.  A warp reads the TMEM lanes of
    // its quarter (warp % 4): rows r of key half h, all 256 columns in 8 rounds of 32 dims.  A
    // round (32 rows x 64 bytes, 64-byte swizzle) is staged in the warp's own 2 KB slice and
    // one lane hands the box to TMA.
    const int tl = ((warp & 3) << 5) | lane;
    const int r = tl & 63, h = tl >> 6;
    const uint32_t ocol = tmem + ((uint32_t)((warp & 3) * 32) << 16) + kTmemO;
    const uint32_t stage_off = PL::kOffStage + (warp - kWarpEpi0) * 2048;
    uint8_t* st_row = sm + stage_off + (r & 31) * 64;
    const int sw = (r >> 1) & 3;
    const uint32_t a_o_free = mapa(smem_u32(&ms.o_free), 0);
    int kb0 = 0, it = 0;
    for (int tile = cid; tile < p.ng; tile += ncl, ++it) {
      const int nb = blocks_of(tile_count(tile));
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
  }

  // tear-down: nobody may still be reading TMEM of either CTA when it is released
  __syncthreads();
  __syncwarp();
  cluster_sync_all();
  if (warp == kWarpMma) tmem_dealloc_pair(tmem, kTmemCols);
  if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(&g_status[3], 1);
}

// Offset of the dynamic shared-memory base inside its 1 KB alignment window, measured once
// per device by a one-thread probe launched with the same dynamic size (synchronous on
// first use: make the first call outside stream capture).  The 576-dim plan leaves only
// 768 bytes for aligning its tiles; the launcher refuses instead of letting the kernel give up.
__device__ unsigned g_smem_base_mod1024;
__global__ void smem_base_probe() {
  extern __shared__ __align__(1024) uint8_t probe_raw[];
  if (threadIdx.x == 0) g_smem_base_mod1024 = smem_u32(probe_raw) & 1023u;
}
template <int kD>
static bool smem_alignment_ok() {
  using PL = Plan<kD>;
  if (PL::kUsed + 1024 <= PL::kSmem) return true;     // a full 1 KB of slack: nothing to check
  static thread_local int cached_dev = -1;
  static thread_local bool cached = false;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev == cached_dev) return cached;
  bool ok = false;
  unsigned h = 0xffffffffu;
  if (cudaFuncSetAttribute(smem_base_probe, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PL::kSmem) == cudaSuccess) {
    smem_base_probe<<<1, 32, PL::kSmem>>>();
    if (cudaMemcpyFromSymbol(&h, g_smem_base_mod1024, sizeof(unsigned)) == cudaSuccess) {
      const unsigned pad = (1024u - h) & 1023u;
      ok = pad + PL::kUsed <= PL::kSmem;
    }
  }
  cudaGetLastError();
  cached_dev = dev; cached = ok;
  return ok;
}

template <int kD>
static int max_clusters() {
  static thread_local int cached_dev = -1, cached = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev == cached_dev) return cached;
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int n = sms / 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sms, 1, 1); cfg.blockDim = dim3(kThreads, 1, 1); cfg.dynamicSmemBytes = Plan<kD>::kSmem;
  cudaLaunchAttribute at;
  at.id = cudaLaunchAttributeClusterDimension;
  at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
  cfg.attrs = &at; cfg.numAttrs = 1;
  int q = 0;
  if (cudaFuncSetAttribute(masked_mla_bf16_kernel<kD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)Plan<kD>::kSmem) == cudaSuccess &&
      cudaOccupancyMaxActiveClusters(&q, masked_mla_bf16_kernel<kD>, &cfg) == cudaSuccess && q > 0)
    n = q;
  cudaGetLastError();
  cached_dev = dev; cached = n;
  return n;
}

struct Args {
  const void* q; const void* kv; const int32_t* indices; const int32_t* counts;
  const uint32_t* memb; const int32_t* pref; const int32_t* win_lo; const int32_t* win_hi;
  const float* sink; void* out; float* max_logits; float* lse;
  int ng, s_kv, topk, d, h_per_q;
  int64_t q_row_stride, kv_row_stride, idx_row_stride;     // ELEMENTS
  float sm_scale;
  // in-place addressing of q / out inside [T, H_padded, d] tensors (ELEMENTS, 0 = dense packed)
  int64_t q_token_stride, q_head_stride, out_token_stride, out_head_stride;
  const int* gate = nullptr;      // run only if *gate == 1 (see Params)
};

// argument rules shared by both entry points (no CUDA call)
static int check(const Args& a) {
  if (!a.q || !a.kv || !a.indices || !a.out || !a.lse) return LITEDSA_ERR_ARG;
  if (!a.memb && !(a.pref && a.win_lo && a.win_hi)) return LITEDSA_ERR_ARG;
  if (a.ng <= 0 || a.s_kv <= 0 || a.topk <= 0 || a.topk % kBlockKeys != 0) return LITEDSA_ERR_SHAPE;
  if (a.h_per_q <= 0 || 128 % a.h_per_q != 0 || 128 / a.h_per_q > 16) return LITEDSA_ERR_SHAPE;
  if (a.d != 512 && a.d != 576) return LITEDSA_ERR_SHAPE;
  if (a.memb && a.topk % 128 != 0) return LITEDSA_ERR_SHAPE;        // whole mask words per tile row
  // strides in ELEMENTS (bf16); TMA / 16-byte copies need 16-byte aligned bases and pitches
  if (a.q_row_stride < a.d || a.kv_row_stride < a.d || (a.q_row_stride % 8) || (a.kv_row_stride % 8))
    return LITEDSA_ERR_UNSUPPORTED;
  if (((uintptr_t)a.q | (uintptr_t)a.kv | (uintptr_t)a.out) & 15) return LITEDSA_ERR_UNSUPPORTED;
  if (a.idx_row_stride < a.topk) return LITEDSA_ERR_UNSUPPORTED;
  if (a.q_token_stride < 0 || a.q_head_stride < 0 || a.out_token_stride < 0 || a.out_head_stride < 0)
    return LITEDSA_ERR_SHAPE;
  if ((a.q_head_stride && (a.q_head_stride < a.d || a.q_head_stride % 8)) || a.q_token_stride % 8 ||
      (a.out_head_stride && (a.out_head_stride < kDV || a.out_head_stride % 8)) || a.out_token_stride % 8)
    return LITEDSA_ERR_UNSUPPORTED;
  return LITEDSA_OK;
}

template <int kD>
static int launch(const Args& a, cudaStream_t stream) {
  using PL = Plan<kD>;
  CUtensorMap mq, mout;
  const auto BF = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  // q and out are addressed as (dim, head, token): row r of a tile is (token r / h, head r % h),
  // which covers the dense packed layout and the in-place layout with padded head slots alike
  const int h = a.h_per_q, G = 128 / h;
  const uint64_t q_hs = (a.q_head_stride ? (uint64_t)a.q_head_stride : (uint64_t)a.q_row_stride) * 2;
  const uint64_t q_ts = a.q_token_stride ? (uint64_t)a.q_token_stride * 2 : (uint64_t)h * q_hs;
  const uint64_t o_hs = (a.out_head_stride ? (uint64_t)a.out_head_stride : (uint64_t)kDV) * 2;
  const uint64_t o_ts = a.out_token_stride ? (uint64_t)a.out_token_stride * 2 : (uint64_t)h * o_hs;
  const uint32_t qb_h = (uint32_t)min(h, 64), ob_h = (uint32_t)min(h, 32);
  if (!make_map_3d(&mq, a.q, BF, kD, (uint64_t)h, (uint64_t)a.ng * G, q_hs, q_ts, 64, qb_h, 64 / qb_h) ||
      // out leaves as boxes of 32 rows x 32 dims (64 bytes wide, 64-byte swizzle)
      !make_map_3d(&mout, a.out, BF, kDV, (uint64_t)h, (uint64_t)a.ng * G, o_hs, o_ts, 32, ob_h, 32 / ob_h,
                   CU_TENSOR_MAP_SWIZZLE_64B))
    return LITEDSA_ERR_CUDA;
  Params p;
  p.kv = reinterpret_cast<const uint8_t*>(a.kv); p.kv_pitch = a.kv_row_stride * 2;
  p.indices = a.indices; p.idx_stride = a.idx_row_stride; p.counts = a.counts;
  p.memb = a.memb; p.pref = a.pref; p.win_lo = a.win_lo; p.win_hi = a.win_hi; p.sink = a.sink;
  p.lse = a.lse; p.max_logits = a.max_logits;
  p.ng = a.ng; p.s_kv = a.s_kv; p.cap = a.topk; p.h_per_q = a.h_per_q; p.G = 128 / a.h_per_q;
  p.scale_log2 = a.sm_scale * kLog2e;
  p.epoch = next_launch_epoch(); p.wait_limit_ns = wait_limit_ns();
  p.gate = a.gate; p.gate_value = 1;
  if (!smem_alignment_ok<kD>()) return LITEDSA_ERR_UNSUPPORTED;
  if (cudaFuncSetAttribute(masked_mla_bf16_kernel<kD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)PL::kSmem) != cudaSuccess)
    return LITEDSA_ERR_CUDA;
  masked_mla_bf16_kernel<kD><<<2 * min(a.ng, max_clusters<kD>()), kThreads, PL::kSmem, stream>>>(mq, mout, p);
  return cudaGetLastError() == cudaSuccess ? LITEDSA_OK : LITEDSA_ERR_CUDA;
}

static int run(const Args& a, void* stream) {
  const int rc = check(a);
  if (rc != LITEDSA_OK) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return a.d == 576 ? launch<576>(a, st) : launch<512>(a, st);
}

// One warp per cache row: 512 e4m3 codes x their per-128 fp32 scale -> bf16, the 64 bf16 rope
// values copied behind them.
__global__ void __launch_bounds__(256) dequant_kv656_kernel(const uint8_t* __restrict__ in,
                                                             uint8_t* __restrict__ out, int s_kv,
                                                             long long out_pitch) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < s_kv;
       row += gridDim.x * warps_per_block) {
    const uint8_t* src = in + (size_t)row * 656;
    uint8_t* dst = out + (size_t)row * out_pitch;
    // lane: codes [8 lane, +8) (chunk lane / 16) and [256 + 8 lane, +8) (chunk 2 + lane / 16):
    // two coalesced 256-byte loads in, two coalesced 512-byte stores out
    const uint2 c0 = __ldcs(reinterpret_cast<const uint2*>(src) + lane);
    const uint2 c1 = __ldcs(reinterpret_cast<const uint2*>(src) + 32 + lane);
    const float s0 = __ldg(reinterpret_cast<const float*>(src + 512) + (lane >> 4));
    const float s1 = __ldg(reinterpret_cast<const float*>(src + 512) + 2 + (lane >> 4));
    const uint32_t w[4] = {c0.x, c0.y, c1.x, c1.y};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float sc = j < 2 ? s0 : s1;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const __nv_fp8x2_storage_t two = (__nv_fp8x2_storage_t)((w[j] >> (16 * hh)) & 0xffffu);
        const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(two, __NV_E4M3);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
        __nv_bfloat162 b2 = __floats2bfloat162_rn(f.x * sc, f.y * sc);
        o[2 * j + hh] = *reinterpret_cast<uint32_t*>(&b2);
      }
    }
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    d4[lane] = make_uint4(o[0], o[1], o[2], o[3]);
    d4[32 + lane] = make_uint4(o[4], o[5], o[6], o[7]);
    // rope: 128 bytes = 8 x 16
    if (lane < 8)
      reinterpret_cast<uint4*>(dst + 1024)[lane] = __ldcs(reinterpret_cast<const uint4*>(src + 528) + lane);
  }
}

}  // namespace b16
}  // namespace lt

// The reference's DSv4 operator with its own argument list
//   dsv4_masked_mla_bf16(q, kv, indices, pref, win_lo, win_hi, counts, sm_scale, h_per_q,
//                        out, lse, attn_sink)        (kernels/b200/dsa/litedsa_dsv4.cu:50-121)
// tensor shapes and strides passed as integers.  d = 512 as in the reference, or 576.  The four
// trailing strides (ELEMENTS, 0 = dense packed) address q and out in place inside
// [T, H_padded, d] tensors with h_per_q real heads per token: the zero-copy form the reference
// planned for this operator (kernels/b200/dsa/DSV4_ZEROCOPY_PLAN.md:50-76).
extern "C" int litedsa_dsv4_masked_mla_bf16(const void* q, const void* kv, const int32_t* indices,
                                            const int32_t* pref, const int32_t* win_lo,
                                            const int32_t* win_hi, const int32_t* counts,
                                            float sm_scale, int h_per_q, void* out, float* lse,
                                            const float* attn_sink, int ng, int s_kv, int topk,
                                            int d, int64_t q_row_stride, int64_t kv_row_stride,
                                            int64_t indices_row_stride, int64_t q_token_stride,
                                            int64_t q_head_stride, int64_t out_token_stride,
                                            int64_t out_head_stride, void* workspace,
                                            int64_t workspace_bytes, void* stream) {
  using namespace lt::b16;
  if (!pref || !win_lo || !win_hi || !counts) return LITEDSA_ERR_ARG;
  Args a{q, kv, indices, counts, nullptr, pref, win_lo, win_hi, attn_sink, out, nullptr, lse,
         ng, s_kv, topk, d, h_per_q, q_row_stride, kv_row_stride, indices_row_stride, sm_scale,
         q_token_stride, q_head_stride, out_token_stride, out_head_stride};
  const int rc = check(a);
  if (rc != LITEDSA_OK) return rc;
  // With a workspace the device decides: when every tile's index list is two contiguous runs
  // of rows (the packed prefix + window pattern this operator exists for) the range kernel
  // reads K and V with tiled TMA loads and the gather kernel returns at once; otherwise the
  // range kernel returns at once and the gather kernel does the work.
  if (workspace != nullptr) {
    if (workspace_bytes < 16 + 16 * (int64_t)ng || ((uintptr_t)workspace & 15)) return LITEDSA_ERR_SHAPE;
    const int rc2 = lt::dsv4_rank_enqueue(q, kv, indices, pref, win_lo, win_hi, counts, sm_scale, h_per_q, out,
                                          lse, attn_sink, ng, s_kv, topk, d, q_row_stride, kv_row_stride,
                                          indices_row_stride, q_token_stride, q_head_stride,
                                          out_token_stride, out_head_stride, workspace,
                                          reinterpret_cast<cudaStream_t>(stream));
    if (rc2 != LITEDSA_OK) return rc2;
    a.gate = reinterpret_cast<const int*>(workspace);
  }
  return run(a, stream);
}

// masked_mla_fp8's bf16 twin: the same union list + query-major membership mask
// (kernels/b200/dsa/litedsa.cu:77-80 argument order, minus out_scale) over bf16 q and a bf16
// KV workspace, for caches that have no single-scale all-e4m3 form.
extern "C" int litedsa_masked_mla_bf16(const void* q, const void* kv, const int32_t* indices,
                                       float sm_scale, const int32_t* topk_length,
                                       const uint32_t* memb_qm, int h_per_q, void* out,
                                       float* max_logits, float* lse, int ng, int s_kv, int topk,
                                       int d, int64_t q_row_stride, int64_t kv_row_stride,
                                       int64_t indices_row_stride, const float* attn_sink,
                                       void* stream) {
  using namespace lt::b16;
  if (!memb_qm) return LITEDSA_ERR_ARG;
  Args a{q, kv, indices, topk_length, memb_qm, nullptr, nullptr, nullptr, attn_sink, out, max_logits,
         lse, ng, s_kv, topk, d, h_per_q, q_row_stride, kv_row_stride, indices_row_stride, sm_scale,
         0, 0, 0, 0};
  return run(a, stream);
}

// Packed 656-byte cache rows (512 e4m3 codes | 4 fp32 per-128 scales | 64 bf16 rope) ->
// bf16 rows [s_kv, 576] (latent = code x its chunk's scale, rope copied); out_pitch = bytes
// between output rows (>= 1152, multiple of 16).
extern "C" int litedsa_dequant_kv656(const void* kv656, void* kv_bf16, int s_kv, int64_t out_pitch,
                                     void* stream) {
  using namespace lt::b16;
  if (!kv656 || !kv_bf16) return LITEDSA_ERR_ARG;
  if (s_kv <= 0 || out_pitch < 1152 || out_pitch % 16) return LITEDSA_ERR_SHAPE;
  if (((uintptr_t)kv656 | (uintptr_t)kv_bf16) & 15) return LITEDSA_ERR_UNSUPPORTED;
  const int blocks = min(148 * 8, (s_kv + 7) / 8);
  dequant_kv656_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint8_t*>(kv656), reinterpret_cast<uint8_t*>(kv_bf16), s_kv, out_pitch);
  return cudaGetLastError() == cudaSuccess ? LITEDSA_OK : LITEDSA_ERR_CUDA;
}

// Status block of the bf16 gather kernel (same meaning and use as litedsa_attn_status).
extern "C" int litedsa_bf16_status(int* out4_host, int reset) {
  using namespace lt::b16;
  if (out4_host && cudaMemcpyFromSymbol(out4_host, g_status, sizeof(int) * 4) != cudaSuccess)
    return LITEDSA_ERR_CUDA;
  if (reset) {
    const int z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (cudaMemcpyToSymbol(g_status, z, sizeof(z)) != cudaSuccess) return LITEDSA_ERR_CUDA;
  }
  return (out4_host && out4_host[0] != 0) ? LITEDSA_ERR_TIMEOUT : LITEDSA_OK;
}

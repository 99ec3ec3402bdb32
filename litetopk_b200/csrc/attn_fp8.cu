// Masked FP8 MLA prefill over a per-tile union list (sm_100a, tcgen05 + TMEM + TMA).
//
// What it computes is fixed by the reference operator masked_mla_fp8
// (kernels/b200/dsa/litedsa.cu:77-135, kernel
// kernels/b200/dsa/litedsa_attention_sm100.cuh:1832-2479): for every 128-row tile
// (G = 128 / h_per_q adjacent tokens x h_per_q heads), S = Q8 K8^T over the tile's union
// of KV rows, a per-row validity/membership mask, base-2 online softmax in blocks of
// 128 keys whose running max only moves when some row of a 32-row group overshoots it
// by more than 6, P quantised to e4m3 after a x7 pre-scale, O += P8 V8 (V = the first
// 512 bytes of the same KV rows), out = bf16(O * out_scale / l), lse, max_logits.
// Those numerics are reproduced exactly so the two implementations agree to rounding.
//
// How it is organised here (written from scratch, raw PTX, no CuTe):
//   * one cluster of 2 CTAs per tile; each CTA owns 64 query rows.  Both GEMMs are
//     single tcgen05 cta_group::2 instructions spanning the pair: QK^T splits the 128
//     keys of a block across the CTAs (N split), PV splits the 512 value dims (N split).
//   * 6 warps per CTA: warps 0-3 softmax + epilogue (one TMEM lane per thread),
//     warp 4 = TMA producer (Q tile, row gathers for K and V, index-validity bits),
//     warp 5 = MMA issue (one thread of the leader CTA) and TMEM allocation.
//   * every tile of the 576-byte rows is stored as five 128-byte-swizzled column
//     chunks (the fifth is half zero-filled by TMA bounds handling), so Q, K and V all
//     share one shared-memory geometry and one tensor-map shape.
//   * completion is tracked with mbarriers only; every wait is bounded (common.cuh)
//     and reports through a status word instead of trapping.
//   * no TMA multicast of any kind; the pair is signalled with two plain commits.
#include "common.cuh"
#include "tensor_map.cuh"
#include <cstdlib>

namespace lt {

constexpr int kSoftmaxWarps = 8, kProducerWarps = 8;
constexpr int kWarpMma = 16, kWarpCopy = 17, kWarpRelay = 18, kWarpValid = 19;
constexpr int kAttnThreads = 640;
constexpr int kBlockKeys = 128;                      // keys per softmax block (whole pair)
constexpr int kDQK = 576, kDV = 512;
constexpr int kChunks = 5;                           // 128-byte column chunks per row
constexpr int kChunkBytes = 64 * 128;                // 64 rows x 128 B
constexpr uint32_t kQBytes = kChunks * kChunkBytes;  // 40960 (per CTA)
constexpr uint32_t kKStage = kChunks * kChunkBytes;  // 64 keys x 640 B
constexpr uint32_t kVChunk = 128 * 128;              // 128 keys x 128 B
constexpr uint32_t kVStage = 2 * kVChunk;            // 128 keys x 256 dims
constexpr uint32_t kPBytes = 64 * 128;               // 64 rows x 128 keys e4m3
constexpr uint32_t kOffQ = 0;
constexpr uint32_t kOffK = kOffQ + kQBytes;
constexpr uint32_t kOffV = kOffK + 2 * kKStage;
constexpr uint32_t kOffP = kOffV + 2 * kVStage;
constexpr uint32_t kOffMisc = kOffP + 2 * kPBytes;   // 204800
constexpr uint32_t kMiscBytes = 3072;
constexpr uint32_t kAttnSmem = kOffMisc + kMiscBytes + 1024;  // + alignment slack
static_assert(kAttnSmem <= 232448, "shared-memory plan exceeds the 227 KB per-CTA limit");

constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemO = 0;                        // 256 columns: O (64 rows x 512 dims per CTA)
constexpr uint32_t kTmemS0 = 256, kTmemS1 = 320;      // 64 columns each: S double buffer

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kPScaleLog2 = 2.8073549220576042f;    // log2(7)
constexpr float kPScaleLn = 1.9459101090932196f;      // ln(7)
constexpr float kMInit = -1e30f;
constexpr float kRescaleThreshold = 6.0f;

struct Misc {
  // in the leader CTA only: q_full (both CTAs' Q tiles), k_peer / v_peer (peer's K / V landed),
  // s_free / p_ready (softmax warps of both CTAs)
  uint64_t q_full, k_peer[2], v_peer[2], s_free[2], p_ready[2];
  // in every CTA
  uint64_t k_land[2], v_land[2], k_copied[2], qk_done[2], pv_done[2], valid_ready[2], valid_free[2];
  uint32_t valid[2][4];             // 128 validity bits per stage
  uint32_t tmem_base;
  uint32_t pad;
  float xbuf[2][256];               // row-max exchange (double-buffered); row-sum exchange at the end
};
static_assert(sizeof(Misc) <= kMiscBytes, "Misc too large");

struct AttnParams {
  const uint32_t* memb;      // [ng, G, cap/32]
  const int32_t* indices;    // [ng, idx_stride]
  const int32_t* counts;     // [ng] or null
  __nv_bfloat16* out;        // [ng, 128, 512]
  float* lse;                // [ng, 128]
  float* max_logits;         // [ng, 128] or null
  float* dbg;                // debug dump or null
  int ng, s_kv, cap, h_per_q, G;
  long long idx_stride;
  float scale_log2, out_scale;
  int exp_flags;             // experiment switches (0 in production)
};

// wait sites reported in the status word
enum { kSiteQ = 1, kSiteKLand, kSiteKPeer, kSiteVLand, kSiteVPeer, kSiteQkDone, kSitePvDone,
       kSiteSFree, kSitePReady, kSiteValidReady, kSiteValidFree, kSiteKFree, kSiteKCopied,
       kSiteVFree, kSitePFree, kSiteEpi, kSiteRelayK, kSiteRelayV, kSiteSmemAlign };

// status[0] first failing wait site, [1] block, [2] iteration, [3] launches completed
__device__ int g_attn_status[4];

// bring-up aid: cycle stamps of one tile's roles (role 0 softmax thread 0, 1 producer warp 0,
// 2 MMA thread, 3 copy thread, 4 relay thread), 8 slots per block, written after the S/O dump
#define LT_TS(role, k, slot)                                                              \
  do {                                                                                    \
    if (kDebug && ts_on && (k) < 64) ts[(((role) * 64 + (k)) << 3) + (slot)] = clock64(); \
  } while (0)

template <bool kDebug>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kAttnThreads, 1)
masked_mla_fp8_kernel(const __grid_constant__ CUtensorMap map_q,
                      const __grid_constant__ CUtensorMap map_kv, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;       // 128B-swizzle tiles need 1024-byte alignment
  uint8_t* sm = smem_raw + (sbase - raw);
  Misc& ms = *reinterpret_cast<Misc*>(sm + kOffMisc);
  int* status = g_attn_status;

  const uint32_t cta = cluster_ctarank();
  const int tile = blockIdx.x >> 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int count = p.counts ? p.counts[tile] : p.cap;
  count = min(max(count, 0), p.cap);
  const int nb = max((count + kBlockKeys - 1) / kBlockKeys, 1);
  long long* ts = nullptr;
  bool ts_on = false;
  if (kDebug && p.dbg) {
    ts = reinterpret_cast<long long*>(p.dbg + (size_t)p.cap * 128 + 128 * 512 + 256);
    ts_on = (tile == p.ng / 2) && cta == 0 && lane == 0;
  }

  if (threadIdx.x == 0) {
    mbar_init(&ms.q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ms.k_peer[i], 1);
      mbar_init(&ms.v_peer[i], 1);
      mbar_init(&ms.s_free[i], 2 * kSoftmaxWarps);
      mbar_init(&ms.p_ready[i], 2 * kSoftmaxWarps);
      mbar_init(&ms.k_land[i], 1);
      mbar_init(&ms.v_land[i], 1);
      mbar_init(&ms.k_copied[i], 2);
      mbar_init(&ms.qk_done[i], 1);
      mbar_init(&ms.pv_done[i], 1);
      mbar_init(&ms.valid_ready[i], 1);
      mbar_init(&ms.valid_free[i], kSoftmaxWarps);
    }
    fence_mbar_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_kv);
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
  const uint32_t peer = cta ^ 1u;

  if (warp < kSoftmaxWarps) {
    // ------------------------------------------------------------ softmax + epilogue
    // TMEM lane tl = 32*(warp%4)+lane holds tile row r = tl%64 and key/dim half h = tl/64;
    // the two warps sharing a lane quarter split that half's 64 columns (ch = warp/4).
    const int t = threadIdx.x;                    // 0..255
    const int tl = ((warp & 3) << 5) | lane;
    const int r = tl & 63, h = tl >> 6, ch = warp >> 2;
    const int part = 2 * h + ch;                  // which 32-key quarter of the block
    const int row = (int)cta * 64 + r;            // row of the 128-row tile
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const int capw = p.cap >> 5;
    const uint32_t* mrow = p.memb + ((size_t)tile * p.G + row / p.h_per_q) * capw + part;
    uint32_t mk = __ldg(mrow);
    const float c = p.scale_log2;
    float m = kMInit, li = 0.f, real_m = -INFINITY;
    const uint32_t a_s_free[2] = {mapa(smem_u32(&ms.s_free[0]), 0), mapa(smem_u32(&ms.s_free[1]), 0)};
    const uint32_t a_p_ready[2] = {mapa(smem_u32(&ms.p_ready[0]), 0), mapa(smem_u32(&ms.p_ready[1]), 0)};
    const int xi = part * 64 + r;                 // slot in the exchange buffer

    for (int k = 0; k < nb; ++k) {
      const int s = k & 1;
      const uint32_t ph = (k >> 1) & 1;
      uint32_t mk_next = mk;
      if (k + 1 < nb) mk_next = __ldg(mrow + (size_t)(k + 1) * 4);

      if (warp == 0) LT_TS(0, k, 0);
      mbar_wait(&ms.qk_done[s], ph, status, kSiteQkDone, k);
      if (warp == 0) LT_TS(0, k, 1);
      tc_fence_after();
      float sv[32];
      tmem_ld32(tmem + lane_base + (s ? kTmemS1 : kTmemS0) + 32 * ch, sv);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(a_s_free[s]);

      if (kDebug && p.dbg && tile == 0) {
        float* d = p.dbg + ((size_t)k * 128 + row) * 128 + 32 * part;
#pragma unroll
        for (int j = 0; j < 32; ++j) d[j] = sv[j];
      }

      mbar_wait(&ms.valid_ready[s], ph, status, kSiteValidReady, k);
      const uint32_t bits = ms.valid[s][part] & mk;
      __syncwarp();
      if (lane == 0) mbar_arrive(&ms.valid_free[s]);
      mk = mk_next;
      if (warp == 0) LT_TS(0, k, 2);

      float cur = -INFINITY;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        sv[j] = ((bits >> j) & 1u) ? sv[j] : -INFINITY;
        cur = fmaxf(cur, sv[j]);
      }
      cur *= c;
      float* xb = ms.xbuf[k & 1];
      xb[xi] = cur;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      cur = fmaxf(fmaxf(xb[r], xb[64 + r]), fmaxf(xb[128 + r], xb[192 + r]));
      if (warp == 0) LT_TS(0, k, 3);
      real_m = fmaxf(real_m, cur);
      const bool rescale = __any_sync(0xffffffffu, cur - m > kRescaleThreshold);
      float new_m = m, scale_old = 1.f;
      if (rescale) {
        new_m = fmaxf(cur, m);
        scale_old = fast_exp2(m - new_m);
      }
      m = new_m;
      li *= scale_old;

      const float nm = -new_m + kPScaleLog2;
      uint32_t pk[8];
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float2 d0, d1;
        d0.x = fast_exp2(fmaf(sv[j], c, nm));
        d0.y = fast_exp2(fmaf(sv[j + 1], c, nm));
        d1.x = fast_exp2(fmaf(sv[j + 2], c, nm));
        d1.y = fast_exp2(fmaf(sv[j + 3], c, nm));
        li += d0.x + d0.y;
        li += d1.x + d1.y;
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(d0, __NV_SATFINITE, __NV_E4M3);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(d1, __NV_SATFINITE, __NV_E4M3);
        pk[j >> 2] = lo | (hi << 16);
      }
      if (warp == 0) LT_TS(0, k, 4);
      // P buffer s was last read by PV(k-2)
      if (k >= 2) mbar_wait(&ms.pv_done[s], ph ^ 1, status, kSitePFree, k);
      if (warp == 0) LT_TS(0, k, 5);
      uint8_t* pdst = sm + kOffP + s * kPBytes + (2 * part) * 1024 + r * 16;
      *reinterpret_cast<uint4*>(pdst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      *reinterpret_cast<uint4*>(pdst + 1024) = make_uint4(pk[4], pk[5], pk[6], pk[7]);

      if (rescale && k > 0) {
        // O still holds blocks [0, k): needs PV(k-1) complete
        mbar_wait(&ms.pv_done[(k - 1) & 1], ((k - 1) >> 1) & 1, status, kSitePvDone, k);
        tc_fence_after();
        float o[32];
#pragma unroll 1
        for (int cc = 0; cc < 4; ++cc) {
          const uint32_t ocol = tmem + lane_base + kTmemO + ch * 128 + cc * 32;
          tmem_ld32(ocol, o);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] *= scale_old;
          tmem_st32(ocol, o);
        }
        tmem_wait_st();
        tc_fence_before();
      }
      if (warp == 0) LT_TS(0, k, 6);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(a_p_ready[s]);
      if (warp == 0) LT_TS(0, k, 7);
    }

    // epilogue
    float* xb = ms.xbuf[nb & 1];
    xb[xi] = li;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    li = (xb[r] + xb[64 + r]) + (xb[128 + r] + xb[192 + r]);
    if (real_m == -INFINITY) { li = 0.f; m = -INFINITY; }
    const size_t grow = (size_t)tile * 128 + row;
    if (part == 0) {
      float l = __logf(li) - kPScaleLn + m * kLn2;
      if (!(li > 0.f)) l = INFINITY;
      p.lse[grow] = l;
      if (p.max_logits) p.max_logits[grow] = real_m * kLn2;
    }
    mbar_wait(&ms.pv_done[(nb - 1) & 1], ((nb - 1) >> 1) & 1, status, kSiteEpi, nb);
    tc_fence_after();
    const bool empty = !(li > 0.f);
    const float oscale = empty ? 0.f : __fdividef(p.out_scale, li);
    __nv_bfloat16* orow = p.out + grow * kDV + 256 * h + 128 * ch;
    float o[32];
#pragma unroll 1
    for (int cc = 0; cc < 4; ++cc) {
      tmem_ld32(tmem + lane_base + kTmemO + ch * 128 + cc * 32, o);
      tmem_wait_ld();
      if (kDebug && p.dbg && tile == 0) {
        float* d = p.dbg + (size_t)p.cap * 128 + (size_t)row * 512 + 256 * h + 128 * ch + cc * 32;
#pragma unroll
        for (int j = 0; j < 32; ++j) d[j] = o[j];
      }
      uint32_t w[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float a = empty ? 0.f : o[2 * j] * oscale;
        const float b = empty ? 0.f : o[2 * j + 1] * oscale;
        __nv_bfloat162 v2 = __floats2bfloat162_rn(a, b);
        w[j] = *reinterpret_cast<uint32_t*>(&v2);
      }
      uint4* dst = reinterpret_cast<uint4*>(orow + cc * 32);
#pragma unroll
      for (int j = 0; j < 4; ++j) dst[j] = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
    }
    if (kDebug && p.dbg && tile == 0 && part == 0) {
      float* d = p.dbg + (size_t)p.cap * 128 + 128 * 512;
      d[row] = m;
      d[128 + row] = li;
    }
    tc_fence_before();
  } else if (warp < kSoftmaxWarps + kProducerWarps) {
    // ------------------------------------------------------------ TMA producers (K rows, Q tile)
    // warp pw gathers row quads pw and pw+8 of this CTA's 64 keys, all five column chunks
    if (lane == 0) {
      const int pw = warp - kSoftmaxWarps;
      if (pw == 0) {
        if (cta == 0) mbar_arrive_expect_tx(&ms.q_full, 2 * kQBytes);
        const uint32_t a_q_full = mapa(smem_u32(&ms.q_full), 0);
        for (int j = 0; j < kChunks; ++j)
          tma_load_2d_pair(sbase + kOffQ + j * kChunkBytes, &map_q, 128 * j,
                           tile * 128 + (int)cta * 64, a_q_full);
      }
      const int32_t* idx_row = p.indices + (size_t)tile * p.idx_stride + 64 * cta + 4 * pw;
      int4 c0 = __ldg(reinterpret_cast<const int4*>(idx_row));
      int4 c1 = __ldg(reinterpret_cast<const int4*>(idx_row + 32));
      for (int k = 0; k < nb; ++k) {
        const int s = k & 1;
        const uint32_t ph = (k >> 1) & 1;
        int4 n0 = c0, n1 = c1;
        if (k + 1 < nb) {
          n0 = __ldg(reinterpret_cast<const int4*>(idx_row + (size_t)(k + 1) * kBlockKeys));
          n1 = __ldg(reinterpret_cast<const int4*>(idx_row + (size_t)(k + 1) * kBlockKeys + 32));
        }
        if (pw == 0) LT_TS(1, k, 0);
        if (k >= 2) {
          // stage s held block k-2: QK(k-2) must have read it and its V copies must be out
          mbar_wait(&ms.qk_done[s], ph ^ 1, status, kSiteKFree, k);
          mbar_wait(&ms.k_copied[s], ph ^ 1, status, kSiteKCopied, k);
        }
        if (pw == 0) LT_TS(1, k, 1);
        if ((p.exp_flags & 1) && k >= 2) {
          if (pw == 0) mbar_arrive(&ms.k_land[s]);
          c0 = n0; c1 = n1;
          continue;
        }
        if (pw == 0) mbar_arrive_expect_tx(&ms.k_land[s], kKStage);
        const uint32_t bar = smem_u32(&ms.k_land[s]);
        const uint32_t dst = sbase + kOffK + s * kKStage + (uint32_t)pw * 512;
#pragma unroll
        for (int j = 0; j < kChunks; ++j) {
          tma_gather4(dst + j * kChunkBytes, &map_kv, 128 * j, c0, bar);
          tma_gather4(dst + j * kChunkBytes + 4096, &map_kv, 128 * j, c1, bar);
        }
        if (pw == 0) LT_TS(1, k, 2);
        c0 = n0; c1 = n1;
      }
    }
  } else if (warp == kWarpMma) {
    // ------------------------------------------------------------ MMA issue (leader CTA only)
    if (cta == 0 && lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(0, 0, false, false, 128, 128);
      constexpr uint32_t idesc_pv = umma_idesc(0, 0, false, true, 128, 256);
      const uint32_t a_qk_done_peer[2] = {mapa(smem_u32(&ms.qk_done[0]), 1), mapa(smem_u32(&ms.qk_done[1]), 1)};
      const uint32_t a_pv_done_peer[2] = {mapa(smem_u32(&ms.pv_done[0]), 1), mapa(smem_u32(&ms.pv_done[1]), 1)};
      mbar_wait(&ms.q_full, 0, status, kSiteQ, 0);
      // S = Q K^T of block k into S buffer k%2 (needs K stage k%2 on both CTAs, buffer drained)
      auto issue_qk = [&](int k) {
        const int s = k & 1;
        const uint32_t ph = (k >> 1) & 1;
        LT_TS(2, k, 0);
        mbar_wait(&ms.k_land[s], ph, status, kSiteKLand, k);
        mbar_wait(&ms.k_peer[s], ph, status, kSiteKPeer, k);
        LT_TS(2, k, 1);
        if (k >= 2) mbar_wait(&ms.s_free[s], ph ^ 1, status, kSiteSFree, k);
        LT_TS(2, k, 2);
        tc_fence_after();
        const uint32_t d = tmem + (s ? kTmemS1 : kTmemS0);
        const uint32_t qb = sbase + kOffQ, kb = sbase + kOffK + s * kKStage;
#pragma unroll
        for (int j = 0; j < kChunks; ++j) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            if (j * 128 + kk * 32 >= kDQK) break;
            const uint64_t ad = umma_desc(qb + j * kChunkBytes + kk * 32, 16, 1024, kSwz128);
            const uint64_t bd = umma_desc(kb + j * kChunkBytes + kk * 32, 16, 1024, kSwz128);
            mma_f8_pair(d, ad, bd, idesc_qk, (j | kk) ? 1u : 0u);
          }
        }
        mma_commit_pair(smem_u32(&ms.qk_done[s]));
        mma_commit_pair(a_qk_done_peer[s]);
        LT_TS(2, k, 3);
      };
      // QK runs ahead of PV: S(k+1) is produced while the softmax warps work on block k.
      // Issue order: QK(0), QK(1), PV(0), QK(2), PV(1), QK(3), ...
      issue_qk(0);
      if (nb > 1) issue_qk(1);
      for (int kb_ = 0; kb_ < nb; ++kb_) {
        const int s = kb_ & 1;
        const uint32_t ph = (kb_ >> 1) & 1;
        LT_TS(2, kb_, 4);
        mbar_wait(&ms.p_ready[s], ph, status, kSitePReady, kb_);
        LT_TS(2, kb_, 5);
        mbar_wait(&ms.v_land[s], ph, status, kSiteVLand, kb_);
        mbar_wait(&ms.v_peer[s], ph, status, kSiteVPeer, kb_);
        LT_TS(2, kb_, 6);
        tc_fence_after();
        const uint32_t pb = sbase + kOffP + s * kPBytes, vb = sbase + kOffV + s * kVStage;
#pragma unroll
        for (int nbk = 0; nbk < 2; ++nbk) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint64_t ad = umma_desc(pb + ks * 2048, 1024, 128, kSwzNone);
            const uint64_t bd = umma_desc(vb + nbk * kVChunk + ks * 4096, kVChunk, 1024, kSwz128);
            mma_f8_pair(tmem + kTmemO + nbk * 128, ad, bd, idesc_pv, (kb_ | ks) ? 1u : 0u);
          }
        }
        mma_commit_pair(smem_u32(&ms.pv_done[s]));
        mma_commit_pair(a_pv_done_peer[s]);
        LT_TS(2, kb_, 7);
        if (kb_ + 2 < nb) issue_qk(kb_ + 2);
      }
    }
  } else if (warp == kWarpCopy) {
    // ------------------------------------------------------------ V operand = copies of K chunks
    // The value dims of a key are the first 512 bytes of the row the K gather already
    // fetched.  Chunk pair {2d, 2d+1} of this CTA's 64 keys goes to rows [64*cta, +64) of
    // CTA d's V stage: two copies stay local, two cross to the peer over DSMEM.
    if (lane == 0) {
      const uint32_t a_k_peer[2] = {mapa(smem_u32(&ms.k_peer[0]), 0), mapa(smem_u32(&ms.k_peer[1]), 0)};
      for (int k = 0; k < nb; ++k) {
        const int s = k & 1;
        const uint32_t ph = (k >> 1) & 1;
        LT_TS(3, k, 0);
        mbar_wait(&ms.k_land[s], ph, status, kSiteRelayK, k);
        LT_TS(3, k, 1);
        if (cta == 1) mbar_arrive_cluster(a_k_peer[s]);
        if (k >= 2) mbar_wait(&ms.pv_done[s], ph ^ 1, status, kSiteVFree, k);   // V stage s free
        LT_TS(3, k, 2);
        if ((p.exp_flags & 2) && k >= 2) {
          mbar_arrive(&ms.v_land[s]);
          continue;
        }
        mbar_arrive_expect_tx(&ms.v_land[s], kVStage);
        const uint32_t src = sbase + kOffK + s * kKStage;
        const uint32_t vdst = sbase + kOffV + s * kVStage + cta * (64 * 128);
        const uint32_t vbar = smem_u32(&ms.v_land[s]);
#pragma unroll
        for (uint32_t d = 0; d < 2; ++d) {
#pragma unroll
          for (uint32_t nbk = 0; nbk < 2; ++nbk)
            bulk_copy_s2s(mapa(vdst + nbk * kVChunk, d), src + (2 * d + nbk) * kChunkBytes,
                          kChunkBytes, mapa(vbar, d));
        }
        LT_TS(3, k, 3);
      }
    }
  } else if (warp == kWarpRelay) {
    // ------------------------------------------------------------ "V landed" relay
    if (lane == 0) {
      const uint32_t a_v_peer[2] = {mapa(smem_u32(&ms.v_peer[0]), 0), mapa(smem_u32(&ms.v_peer[1]), 0)};
      for (int k = 0; k < nb; ++k) {
        const int s = k & 1;
        const uint32_t ph = (k >> 1) & 1;
        mbar_wait(&ms.v_land[s], ph, status, kSiteRelayV, k);
        LT_TS(4, k, 0);
        // all four copies INTO this CTA are done: tell both CTAs' producers (K stages are
        // sources of those copies) and, from the peer, the MMA thread
        mbar_arrive_cluster(mapa(smem_u32(&ms.k_copied[s]), 0));
        mbar_arrive_cluster(mapa(smem_u32(&ms.k_copied[s]), 1));
        if (cta == 1) mbar_arrive_cluster(a_v_peer[s]);
      }
    }
  } else {
    // ------------------------------------------------------------ index-validity bits
    const int32_t* idx_row = p.indices + (size_t)tile * p.idx_stride;
    int4 cur = __ldg(reinterpret_cast<const int4*>(idx_row) + lane);
    for (int k = 0; k < nb; ++k) {
      const int s = k & 1;
      const uint32_t ph = (k >> 1) & 1;
      int4 nxt = cur;
      if (k + 1 < nb) nxt = __ldg(reinterpret_cast<const int4*>(idx_row + (size_t)(k + 1) * kBlockKeys) + lane);
      const int rank0 = k * kBlockKeys + lane * 4;
      auto ok = [&](int idx, int rk) -> uint32_t {
        return (idx >= 0 && idx < p.s_kv && rk < count) ? 1u : 0u;
      };
      const uint32_t nib = ok(cur.x, rank0) | (ok(cur.y, rank0 + 1) << 1) |
                           (ok(cur.z, rank0 + 2) << 2) | (ok(cur.w, rank0 + 3) << 3);
      if (k >= 2) mbar_wait(&ms.valid_free[s], ph ^ 1, status, kSiteValidFree, k);
      const uint32_t nib_hi = __shfl_down_sync(0xffffffffu, nib, 1);
      if ((lane & 1) == 0)
        reinterpret_cast<uint8_t*>(&ms.valid[s][0])[lane >> 1] = (uint8_t)(nib | (nib_hi << 4));
      __syncwarp();
      if (lane == 0) mbar_arrive(&ms.valid_ready[s]);
      cur = nxt;
    }
  }
  (void)peer;

  // tear-down: nobody may still be reading TMEM of either CTA when it is released
  __syncthreads();
  __syncwarp();
  cluster_sync_all();
  if (warp == kWarpMma) tmem_dealloc_pair(tmem, kTmemCols);
  if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(&status[3], 1);
}

static int launch_fp8(const void* q8, const void* kv8, const int32_t* indices, float sm_scale,
                      float out_scale, const int32_t* counts, const uint32_t* memb, int h_per_q,
                      void* out, float* max_logits, float* lse, int ng, int s_kv, int topk,
                      long long q_row_stride, long long kv_row_stride, long long idx_row_stride,
                      float* dbg, cudaStream_t stream) {
  CUtensorMap map_q, map_kv;
  if (!make_map_2d(&map_q, q8, CU_TENSOR_MAP_DATA_TYPE_UINT8, kDQK, (uint64_t)ng * 128,
                   (uint64_t)q_row_stride, 128, 64))
    return LITEDSA_ERR_CUDA;
  if (!make_map_2d(&map_kv, kv8, CU_TENSOR_MAP_DATA_TYPE_UINT8, kDQK, (uint64_t)s_kv,
                   (uint64_t)kv_row_stride, 128, 1))
    return LITEDSA_ERR_CUDA;
  AttnParams p;
  p.memb = memb; p.indices = indices; p.counts = counts;
  p.out = reinterpret_cast<__nv_bfloat16*>(out); p.lse = lse; p.max_logits = max_logits;
  p.dbg = dbg;
  p.ng = ng; p.s_kv = s_kv; p.cap = topk; p.h_per_q = h_per_q; p.G = 128 / h_per_q;
  p.idx_stride = idx_row_stride;
  p.scale_log2 = sm_scale * kLog2e; p.out_scale = out_scale;
  { const char* e = getenv("LITEDSA_EXP"); p.exp_flags = e ? atoi(e) : 0; }
  auto kern = dbg ? masked_mla_fp8_kernel<true> : masked_mla_fp8_kernel<false>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kAttnSmem) !=
      cudaSuccess)
    return LITEDSA_ERR_CUDA;
  kern<<<2 * ng, kAttnThreads, kAttnSmem, stream>>>(map_q, map_kv, p);
  return cudaGetLastError() == cudaSuccess ? LITEDSA_OK : LITEDSA_ERR_CUDA;
}

}  // namespace lt

// Masked FP8 MLA prefill; replaces the reference operator
//   masked_mla_fp8(q, kv, indices, sm_scale, out_scale, topk_length, memb_qm, h_per_q,
//                  out, max_logits, lse)            (kernels/b200/dsa/litedsa.cu:77-135)
// with the same argument order and meaning; tensor shapes and strides are integers.
extern "C" int litedsa_masked_mla_fp8(const void* q8, const void* kv8, const int32_t* indices,
                                      float sm_scale, float out_scale,
                                      const int32_t* topk_length, const uint32_t* memb_qm,
                                      int h_per_q, void* out, float* max_logits, float* lse,
                                      int ng, int s_kv, int topk, int64_t q_row_stride,
                                      int64_t kv_row_stride, int64_t indices_row_stride,
                                      float* debug_dump, void* stream) {
  using namespace lt;
  if (!q8 || !kv8 || !indices || !memb_qm || !out || !lse) return LITEDSA_ERR_ARG;
  // shape rules of the reference launcher (litedsa.cu:82-98)
  if (ng <= 0 || s_kv <= 0 || topk <= 0 || topk % 128 != 0) return LITEDSA_ERR_SHAPE;
  if (h_per_q <= 0 || 128 % h_per_q != 0 || 128 / h_per_q > 16) return LITEDSA_ERR_SHAPE;
  // TMA needs 16-byte aligned bases and row pitches
  if (q_row_stride < kDQK || kv_row_stride < kDQK || q_row_stride % 16 || kv_row_stride % 16)
    return LITEDSA_ERR_UNSUPPORTED;
  if (((uintptr_t)q8 | (uintptr_t)kv8 | (uintptr_t)indices | (uintptr_t)out) & 15)
    return LITEDSA_ERR_UNSUPPORTED;
  if (indices_row_stride < topk || indices_row_stride % 4) return LITEDSA_ERR_UNSUPPORTED;
  return launch_fp8(q8, kv8, indices, sm_scale, out_scale, topk_length, memb_qm, h_per_q, out,
                    max_logits, lse, ng, s_kv, topk, q_row_stride, kv_row_stride,
                    indices_row_stride, debug_dump, reinterpret_cast<cudaStream_t>(stream));
}

// Synchronous read (and optional reset) of the device status word of the attention
// kernels on the current device: out[0] = first wait site that expired (0 = none),
// out[1] = block, out[2] = iteration, out[3] = launches completed since the last reset.
extern "C" int litedsa_attn_status(int* out4_host, int reset) {
  using namespace lt;
  if (out4_host &&
      cudaMemcpyFromSymbol(out4_host, g_attn_status, sizeof(int) * 4) != cudaSuccess)
    return LITEDSA_ERR_CUDA;
  if (reset) {
    const int z[4] = {0, 0, 0, 0};
    if (cudaMemcpyToSymbol(g_attn_status, z, sizeof(z)) != cudaSuccess) return LITEDSA_ERR_CUDA;
  }
  return (out4_host && out4_host[0] != 0) ? LITEDSA_ERR_TIMEOUT : LITEDSA_OK;
}

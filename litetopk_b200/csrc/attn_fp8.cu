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
//   * persistent: one cluster of 2 CTAs per SM pair walks tiles cid, cid + #clusters, ...;
//     each CTA owns 64 query rows.  Both GEMMs are single tcgen05 cta_group::2 instructions
//     spanning the pair: QK^T splits the 128 keys of a block across the CTAs (N split), PV
//     splits the 512 value dims (N split).
//   * 24 warps per CTA:
//       warps 0-7   softmax, two groups of four warps on alternate key blocks (one TMEM lane
//                   per thread, 64 S columns each);
//       warps 8-15  KV row gather with 16-byte cp.async copies written straight into the
//                   128-byte-swizzled tile layout (K: own 64 keys x 576 bytes; V: all 128 keys
//                   x this CTA's 256 value bytes) and the Q tile (TMA);
//       warp 16     MMA issue (leader CTA; whole warp polls, one elected lane issues);
//       warps 17-18 relay "K / V landed" from the peer CTA to the leader's barriers;
//       warp 19     index-validity bits;
//       warps 20-23 tile epilogue: O out of TMEM, x out_scale / l, bf16, staged per warp and
//                   written with TMA tile stores while the softmax warps already work on the
//                   next tile.
//   * Q and K tiles are four 128-byte-swizzled column chunks per 64 rows plus a compact
//     64-byte-swizzled chunk for the 64 rope bytes; V tiles two MN-major chunks per 128 keys.
//   * the 512 latent dims of every Q tile are moved from shared memory into TENSOR MEMORY once
//     per tile (by the epilogue warps) and the QK^T MMAs read them from there (A operand in
//     TMEM); only the rope chunk of Q stays in shared memory.
//   * completion is tracked with mbarriers only; every wait is bounded (common.cuh) and
//     reports through a status word instead of trapping.
//   * no TMA multicast of any kind; the pair is signalled with two plain commits.
#include "common.cuh"
#include "tensor_map.cuh"


namespace lt {
constexpr unsigned kIdleCheckEvery = 64;   // idle polls between two time-limit checks (power of two)
constexpr unsigned kIdleSleepNs = 8;       // back-off of an idle poll


constexpr int kSoftmaxWarps = 8, kProducerWarps = 8;
constexpr int kWarpMma = 16, kWarpCopy = 17, kWarpRelay = 18, kWarpValid = 19, kWarpEpi0 = 20;
constexpr int kEpiWarps = 4;
constexpr int kAttnThreads = 768;
constexpr int kBlockKeys = 128;                      // keys per softmax block (whole pair)
constexpr int kDQK = 576, kDV = 512;
constexpr int kChunkBytes = 64 * 128;                // 64 rows x 128 B (dims 128j .. 128j+127)
constexpr int kRopeChunkBytes = 64 * 64;             // 64 rows x 64 B (dims 512 .. 575), 64-byte swizzle
constexpr uint32_t kQBytes = 4 * kChunkBytes + kRopeChunkBytes;  // 36864 (per CTA)
constexpr uint32_t kKStage = kQBytes;                // 64 keys x 576 B
constexpr uint32_t kVChunk = 128 * 128;              // 128 keys x 128 B
constexpr uint32_t kVStage = 2 * kVChunk;            // 128 keys x 256 dims
constexpr uint32_t kPBytes = 64 * 128;               // 64 rows x 128 keys e4m3
constexpr uint32_t kMiscBytes = 7168;
constexpr uint32_t kStageBytes = 4 * 4096;           // staged epilogue: one 4 KB slice per epilogue warp

// Shared-memory plan: two K stages, two V stages, two P buffers, own output staging.  (A third
// K stage fits only with a single P buffer and staging aliased onto the Q tile; measured
// slower: the single P buffer then waits for PVs whose V tile landed late.)
constexpr int kKStages = 2;
struct Plan {
  static constexpr int kPBufs = 2;
  static constexpr uint32_t kOffQ = 0;
  static constexpr uint32_t kOffK = kOffQ + kQBytes;
  static constexpr uint32_t kOffV = kOffK + kKStages * kKStage;
  static constexpr uint32_t kOffP = kOffV + 2 * kVStage;
  static constexpr uint32_t kOffMisc = kOffP + kPBufs * kPBytes;
  static constexpr uint32_t kOffStage = kOffMisc + kMiscBytes;
  static constexpr uint32_t kSmem = kOffStage + kStageBytes + 1024;   // + alignment slack
  static_assert(kOffV % 1024 == 0 && kOffP % 1024 == 0, "swizzled tiles need 1024-byte alignment");
  static_assert(kSmem <= 232448, "shared-memory plan exceeds the 227 KB per-CTA limit");
};

constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemO = 0;                        // 256 columns: O (64 rows x 512 dims per CTA)
constexpr uint32_t kTmemS0 = 256, kTmemS1 = 320;      // 64 columns each: S double buffer
constexpr uint32_t kTmemQ = 384;                      // 128 columns: the 512 latent dims of Q (e4m3, 4 per column)

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kPScaleLog2 = 2.8073549220576042f;    // log2(7)
constexpr float kPScaleLn = 1.9459101090932196f;      // ln(7)
constexpr float kMInit = -1e30f;
constexpr float kRescaleThreshold = 6.0f;

struct Misc {
  // in the leader CTA only: k_peer / v_peer (peer's K / V landed), s_free / p_ready (softmax
  // warps of both CTAs)
  uint64_t k_peer[3], v_peer[2], s_free[2], p_ready[2];
  // in every CTA.  qk_done is indexed by the running block number modulo 6: one barrier tells
  // the softmax group of block kb (S buffer kb % 2) and the gather warps (K stage kb % 2 or
  // kb % 3) that QK^T(kb) is complete, and none is reused before both have looked at it.
  uint64_t k_land[3], v_land[2], qk_done[6], pv_done[2], valid_ready[2], valid_free[2];
  uint64_t m_pub[2];                // running max of block k published by softmax group k%2
  uint64_t q_land;                  // every CTA: this CTA's Q tile has landed in shared memory
  uint64_t qt_ready;                // leader CTA: Q's latent part is in tensor memory in both CTAs
  uint64_t q_free;                  // all QK^T of the current tile are complete (Q tile reusable)
  uint64_t o_free;                  // leader CTA: the tile's O has been read out of TMEM
  uint64_t epi_ready;               // the tile's row scales are published (softmax warps)
  uint32_t valid[2][4];             // 128 validity bits per stage
  uint32_t tmem_base;
  uint32_t pad;
  float xbuf[2][2][128];            // [group][parity][lane]: row-max exchange between key halves
  float mshare[2][128];             // [group][lane]: running max after the group's latest block
  float fin[3][256];                // end of tile: row sums, true maxima, last running max
  float oscale[2][64];              // [tile parity][row]: out_scale / l, 0 for rows without a key
};
static_assert(sizeof(Misc) <= kMiscBytes, "Misc too large");

constexpr int kMaxOutputs = 8;
// tensor maps of the output destinations: this GPU's buffer and, in a sharded run, the
// peers' gathered buffers (peer-mapped addresses written with plain TMA tile stores)
struct OutMaps { CUtensorMap m[kMaxOutputs]; };

struct AttnParams {
  const uint32_t* memb;      // [ng, G, cap/32], or null when len_per_q replaces it
  const int32_t* len_per_q;  // [ng, G] per-token causal prefix bound on the union ranks, or null
  const float* sink;         // [128] per packed row (natural-log units), or null
  int q_group_div;           // this many consecutive tiles share one Q tile (KV split)
  const uint8_t* kv;         // [s_kv, kv_pitch] e4m3 rows (576 bytes used)
  long long kv_pitch;        // bytes between KV rows
  const int32_t* indices;    // [ng, idx_stride]
  const int32_t* counts;     // [ng] or null
  __nv_bfloat16* out;        // [ng, 128, 512]
  float* lse;                // [ng, 128]
  float* max_logits;         // [ng, 128] or null
  int ng, s_kv, cap, h_per_q, G;
  int n_out;                 // destinations of every output box (1 + peers that hold a copy)
  long long idx_stride;
  float scale_log2, out_scale;
  int epoch;                          // this launch's epoch for the bounded waits
  unsigned long long wait_limit_ns;
};

// wait sites reported in the status word
enum { kSiteQ = 1, kSiteKLand, kSiteKPeer, kSiteVLand, kSiteVPeer, kSiteQkDone, kSitePvDone,
       kSiteSFree, kSitePReady, kSiteValidReady, kSiteValidFree, kSiteKFree, kSiteKCopied,
       kSiteVFree, kSitePFree, kSiteEpi, kSiteRelayK, kSiteRelayV, kSiteMPub, kSiteMmaIdle, kSiteQFree, kSiteOFree, kSiteSelfTest };

// status block of the FP8 attention kernels (layout: see Waiter in common.cuh)
__device__ int g_attn_status[8];

// a running block number's K stage / phase and its qk_done barrier / phase
struct BlockIdx {
  int ks, kph, b6, b6ph;
  __device__ __forceinline__ explicit BlockIdx(int kb) {
    ks = kb % kKStages; kph = (kb / kKStages) & 1;
    b6 = kb % 6; b6ph = (kb / 6) & 1;
  }
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kAttnThreads, 1)
masked_mla_fp8_kernel(const __grid_constant__ CUtensorMap map_q,
                      const __grid_constant__ CUtensorMap map_q_rope,
                      const __grid_constant__ OutMaps omaps, const AttnParams p) {
  using PL = Plan;
  constexpr uint32_t kOffQ = PL::kOffQ, kOffK = PL::kOffK, kOffV = PL::kOffV, kOffP = PL::kOffP,
                     kOffMisc = PL::kOffMisc, kOffStage = PL::kOffStage;
  constexpr int kPBufs = PL::kPBufs;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;       // 128B-swizzle tiles need 1024-byte alignment
  uint8_t* sm = smem_raw + (sbase - raw);
  Misc& ms = *reinterpret_cast<Misc*>(sm + kOffMisc);
  const Waiter wt{g_attn_status, p.epoch, p.wait_limit_ns};

  // Persistent: each cluster walks tiles cid, cid + #clusters, ...  Every role runs the same
  // tile loop; stages, buffers and barrier phases are indexed by the cluster-wide running
  // block number kb, so the next tile's Q / K / V loads and first QK^T overlap the previous
  // tile's last softmax blocks and its epilogue.
  const uint32_t cta = cluster_ctarank();
  const int cid = blockIdx.x >> 1, ncl = gridDim.x >> 1;
  // broadcast so the compiler knows the role index is warp-uniform
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  // live union entries of a tile; with per-token prefix bounds the block loop runs to the LAST
  // token's bound (litedsa_attention_sm100.cuh:1846-1851)
  auto tile_count = [&](int tile) -> int {
    const int c = p.len_per_q ? p.len_per_q[(size_t)tile * p.G + (p.G - 1)]
                              : (p.counts ? p.counts[tile] : p.cap);
    return min(max(c, 0), p.cap);
  };
  auto blocks_of = [&](int count) -> int { return max((count + kBlockKeys - 1) / kBlockKeys, 1); };

  if (threadIdx.x == 0) {
    mbar_init(&ms.q_land, 1);
    mbar_init(&ms.qt_ready, 2 * kEpiWarps);
    mbar_init(&ms.q_free, 1);
    mbar_init(&ms.o_free, 2 * kEpiWarps);
    mbar_init(&ms.epi_ready, kSoftmaxWarps);
    for (int i = 0; i < 3; ++i) {
      mbar_init(&ms.k_peer[i], 1);
      mbar_init(&ms.k_land[i], kProducerWarps * 32);        // one async arrival per gather thread
    }
    for (int i = 0; i < 6; ++i) mbar_init(&ms.qk_done[i], 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ms.v_peer[i], 1);
      mbar_init(&ms.s_free[i], 8);        // 4 warps of one softmax group x 2 CTAs
      mbar_init(&ms.p_ready[i], 8);
      mbar_init(&ms.v_land[i], kProducerWarps * 32);        // one async arrival per gather thread
      mbar_init(&ms.pv_done[i], 1);
      mbar_init(&ms.valid_ready[i], 1);
      mbar_init(&ms.valid_free[i], 4);
      mbar_init(&ms.m_pub[i], 4);
    }
    fence_mbar_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_q_rope);
    for (int d = 0; d < p.n_out; ++d) tma_prefetch_desc(&omaps.m[d]);
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
    // ------------------------------------------------------------ softmax + epilogue
    // Two groups of four warps work on alternate key blocks (group g: blocks with kb % 2 == g),
    // so two blocks are in flight and the latencies of one chain (TMEM load, exchanges,
    // fences) hide behind the other.  Within a group, thread = TMEM lane tl: tile row
    // r = tl % 64, key half h = tl / 64 (64 S columns each).  The only state that crosses
    // groups is the running max m, handed over through shared memory right after each
    // block's row maxima are known; the row sum l is kept per group relative to the m of the
    // group's latest block and merged at the end of the tile.
    const int g = warp >> 2;                      // softmax group = block parity it serves
    const int tl = ((warp & 3) << 5) | lane;
    const int r = tl & 63, h = tl >> 6;
    const int row = (int)cta * 64 + r;            // row of the 128-row tile
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const int capw = p.cap >> 5;
    const float c = p.scale_log2;
    const uint32_t a_s_free = mapa(smem_u32(&ms.s_free[g]), 0);
    const uint32_t a_p_ready = mapa(smem_u32(&ms.p_ready[g]), 0);
    const uint32_t scol = tmem + lane_base + (g ? kTmemS1 : kTmemS0);
    int kb0 = 0, it = 0;

    for (int tile = cid; tile < p.ng; tile += ncl) {
      const int nb = blocks_of(tile_count(tile));
      const size_t trow = (size_t)tile * p.G + row / p.h_per_q;     // (tile, token) of this row
      const uint32_t* mrow = p.memb ? p.memb + trow * capw + 2 * h : nullptr;
      // per-token causal prefix: this row may attend union ranks < row_bound
      const int row_bound = p.len_per_q ? __ldg(p.len_per_q + trow) : 0x7fffffff;
      float m_mine = kMInit;      // the running max my row sum is relative to
      float li = 0.f, real_m = -INFINITY;
      const int k_first = (g - kb0) & 1;          // first local block with (kb0 + k) % 2 == g
      uint2 mk = make_uint2(~0u, ~0u);
      if (mrow && k_first < nb) mk = __ldcs(reinterpret_cast<const uint2*>(mrow + (size_t)k_first * 4));

      for (int k = k_first; k < nb; k += 2) {
        const int kb = kb0 + k;
        const uint32_t ph = (kb >> 1) & 1;
        uint2 mk_next = mk;
        if (mrow && k + 2 < nb) mk_next = __ldcs(reinterpret_cast<const uint2*>(mrow + (size_t)(k + 2) * 4));

        {
          const BlockIdx bi(kb);
          mbar_wait(&ms.qk_done[bi.b6], bi.b6ph, wt, kSiteQkDone, k);
        }
        __syncwarp();      // lanes leave the wait loop one by one: re-converge before .aligned ops
        tc_fence_after();
        float sv[64];
        tmem_ld32(scol, sv);
        tmem_ld32(scol + 32, sv + 32);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(a_s_free);

        mbar_wait(&ms.valid_ready[g], ph, wt, kSiteValidReady, k);
        uint32_t v0 = ms.valid[g][2 * h] & mk.x, v1 = ms.valid[g][2 * h + 1] & mk.y;
        if (p.len_per_q) {     // ranks of my 64 columns: [128k + 64h, +64)
          const int n = min(max(row_bound - (k * kBlockKeys + 64 * h), 0), 64);
          const unsigned long long pm = n >= 64 ? ~0ull : ((1ull << n) - 1ull);
          v0 &= (uint32_t)pm;
          v1 &= (uint32_t)(pm >> 32);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&ms.valid_free[g]);
        mk = mk_next;

        float cur = -INFINITY;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          sv[j] = ((v0 >> j) & 1u) ? sv[j] : -INFINITY;
          sv[32 + j] = ((v1 >> j) & 1u) ? sv[32 + j] : -INFINITY;
          cur = fmaxf(cur, fmaxf(sv[j], sv[32 + j]));
        }
        cur *= c;
        float* xb = ms.xbuf[g][ph];
        xb[tl] = cur;
        if (g == 0) asm volatile("bar.sync 1, 128;" ::: "memory");
        else asm volatile("bar.sync 2, 128;" ::: "memory");
        cur = fmaxf(cur, xb[tl ^ 64]);
        real_m = fmaxf(real_m, cur);
        // running max after block k-1 of this tile comes from the other group
        float m_prev = kMInit;
        if (k > 0) {
          mbar_wait(&ms.m_pub[g ^ 1], ((kb - 1) >> 1) & 1, wt, kSiteMPub, k);
          m_prev = ms.mshare[g ^ 1][tl];
        }
        const bool rescale = __any_sync(0xffffffffu, cur - m_prev > kRescaleThreshold);
        const float new_m = rescale ? fmaxf(cur, m_prev) : m_prev;
        ms.mshare[g][tl] = new_m;
        __syncwarp();
        if (lane == 0) mbar_arrive(&ms.m_pub[g]);
        li *= fast_exp2(m_mine - new_m);
        m_mine = new_m;

        const float nm = -new_m + kPScaleLog2;
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 64; j += 4) {
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
        // the P buffer was last read by the PV of block kb-2 (two buffers) or kb-1 (one)
        if (kPBufs == 2) {
          if (kb >= 2) mbar_wait(&ms.pv_done[g], ph ^ 1, wt, kSitePFree, k);
        } else {
          if (kb >= 1) mbar_wait(&ms.pv_done[g ^ 1], ((kb - 1) >> 1) & 1, wt, kSitePFree, k);
        }
        uint8_t* pdst = sm + kOffP + (kPBufs == 2 ? g : 0) * kPBytes + (4 * h) * 1024 + r * 16;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          *reinterpret_cast<uint4*>(pdst + i * 1024) =
              make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);

        if (rescale && k > 0) {
          // O holds blocks [0, k) relative to m_prev: bring it to new_m once PV(k-1) is complete
          mbar_wait(&ms.pv_done[g ^ 1], ((kb - 1) >> 1) & 1, wt, kSitePvDone, k);
          __syncwarp();      // lanes leave the wait loop one by one: re-converge before .aligned ops
          tc_fence_after();
          const float f = fast_exp2(m_prev - new_m);
          float o[32];
#pragma unroll 1
          for (int cc = 0; cc < 8; ++cc) {
            const uint32_t ocol = tmem + lane_base + kTmemO + cc * 32;
            tmem_ld32(ocol, o);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] *= f;
            tmem_st32(ocol, o);
          }
          tmem_wait_st();
          tc_fence_before();
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(a_p_ready);
      }

      // end of tile: merge the two groups' row sums (each relative to its own latest running max)
      const int t = threadIdx.x;                    // 0..255 = g*128 + tl
      ms.fin[0][t] = li;
      ms.fin[1][t] = real_m;
      ms.fin[2][t] = m_mine;
      asm volatile("bar.sync 3, 256;" ::: "memory");
      const int kbl = kb0 + nb - 1;                 // last block of the tile
      const int last_g = kbl & 1;
      float m = ms.fin[2][last_g * 128 + tl];       // running max after the last block
      float lsum = 0.f;
      real_m = -INFINITY;
      // fixed summation order (even local blocks first, whichever group served them), so a
      // tile's result does not depend on the blocks its cluster processed before
      const int g_even = kb0 & 1;
#pragma unroll
      for (int gi = 0; gi < 2; ++gi) {
        const int gg = gi ^ g_even;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int o = gg * 128 + hh * 64 + r;
          lsum += ms.fin[0][o] * fast_exp2(ms.fin[2][o] - m);
          real_m = fmaxf(real_m, ms.fin[1][o]);
        }
      }
      li = lsum;
      if (real_m == -INFINITY) { li = 0.f; m = -INFINITY; }
      const size_t grow = (size_t)tile * 128 + row;
      if (g == 0 && h == 0) {
        float l = __logf(li) - kPScaleLn + m * kLn2;
        if (!(li > 0.f)) l = INFINITY;
        p.lse[grow] = l;
        if (p.max_logits) p.max_logits[grow] = real_m * kLn2;
      }
      // Hand the tile over to the gather warps, which read O out of TMEM, scale it and store
      // it while these warps already work on the next tile: all they need is 1 / l per row.
      if (g == 0 && h == 0) {
        // the sink joins the OUTPUT normaliser only (in l's units: x 7, relative to m)
        float denom = li;
        if (p.sink != nullptr && li > 0.f) denom += fast_exp2(__ldg(p.sink + row) * kLog2e - m + kPScaleLog2);
        ms.oscale[it & 1][r] = (li > 0.f) ? __fdividef(p.out_scale, denom) : 0.f;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&ms.epi_ready);
      kb0 += nb;
      ++it;
    }
  } else if (warp < kSoftmaxWarps + kProducerWarps) {
    // ------------------------------------------------------------ KV row gather (cp.async) and the Q tile (TMA)
    // The union rows are fetched with 16-byte cp.async copies issued by all 256 threads of
    // these eight warps: fire-and-forget, any number of blocks in flight, destination written
    // directly in the 128-byte-swizzled tile layout, completion reported to an mbarrier by an
    // asynchronous arrival.  (TMA gather4 was measured at one instruction per ~8.5 ns per SM,
    // i.e. ~1 us per block for this tile shape: it, not the tensor pipe, set the pace.)
    // Warp pw owns rows [8pw, 8pw+8) of this CTA's 64 keys (K tile: all 576 bytes, nine copies
    // per lane) and rows [16pw, 16pw+16) of the block's 128 keys (V tile: this CTA's 256 value
    // bytes, eight copies per lane).  K and V streams have different stage-free conditions
    // (QK^T done vs PV done), so each warp advances two independent cursors and issues
    // whichever is ready; neither tile is derived from the other, so no stage waits on a copy.
    const int pw = warp - kSoftmaxWarps;
    struct Cursor { int tile, it, k, nb, kb0; };
    auto cur_init = [&](Cursor& c) {
      c.tile = cid; c.it = 0; c.k = 0; c.kb0 = 0;
      c.nb = c.tile < p.ng ? blocks_of(tile_count(c.tile)) : 0;
    };
    auto cur_next = [&](Cursor& c) {
      if (++c.k == c.nb) {
        c.kb0 += c.nb; c.k = 0; c.tile += ncl; ++c.it;
        c.nb = c.tile < p.ng ? blocks_of(tile_count(c.tile)) : 0;
      }
    };
    Cursor ck, cv;   // K gather, V gather
    cur_init(ck);
    cur_init(cv);
    // q and out stream through once (evict-first TMA traffic), and so do the index lists and
    // membership words (streaming loads): they must not push the re-read KV rows out of L2
    const uint64_t pol_stream = l2_policy_evict_first();
    // lane l < 16 holds the index of own key 8pw + l%8 (K tile rows), lane l >= 16 of key
    // 16pw + l - 16 of the block's 128 keys (V tile rows)
    const int my_key = lane < 16 ? 64 * (int)cta + 8 * pw + (lane & 7) : 16 * pw + (lane - 16);
    auto load_idx = [&](const Cursor& c) -> int {
      const int v = __ldcs(p.indices + (size_t)c.tile * p.idx_stride + (size_t)c.k * kBlockKeys + my_key);
      return ((unsigned)v < (unsigned)p.s_kv) ? v : 0;     // out-of-range rows are masked later
    };
    // The indices of a block are loaded right after the previous block's gather has been issued
    // (one block ahead), so a cold index line from HBM is in flight while that gather lands.
    int kidx = 0, vidx = 0;
    if (ck.tile < p.ng) { kidx = load_idx(ck); vidx = load_idx(cv); }
    const uint8_t* kvb = p.kv;
    const long long pitch = p.kv_pitch;
    const int cj = lane >> 3, cc = lane & 7;       // latent piece `lane`: chunk cj, 16-byte slot cc
    int q_tile = cid, q_it = 0;                    // next Q tile to request (warp 0 only)
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
            mbar_arrive_expect_tx(&ms.q_land, kQBytes);
            // this CTA's 64 rows of the tile = (token, head) pairs starting at row 64 cta
            const int qh = (64 * (int)cta) % p.h_per_q;
            const int qt = (q_tile / p.q_group_div) * p.G + (64 * (int)cta) / p.h_per_q;
            for (int j = 0; j < 4; ++j)
              tma_load_3d_hint(sbase + kOffQ + j * kChunkBytes, &map_q, 128 * j, qh, qt, &ms.q_land, pol_stream);
            tma_load_3d_hint(sbase + kOffQ + 4 * kChunkBytes, &map_q_rope, 512, qh, qt, &ms.q_land, pol_stream);
          }
          __syncwarp();
          q_tile += ncl;
          ++q_it;
          did = true;
        }
      }
      if (ck.tile < p.ng) {
        const int kb = ck.kb0 + ck.k;
        const BlockIdx bi(kb);
        const int s = bi.ks;
        // stage s held block kb - kKStages: its QK^T must have read it
        bool ok = true;
        if (kb >= kKStages) {
          const BlockIdx prev(kb - kKStages);
          ok = mbar_test(&ms.qk_done[prev.b6], prev.b6ph);
        }
        if (__all_sync(0xffffffffu, ok)) {
          const uint32_t kst = sbase + kOffK + s * kKStage;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int ri = __shfl_sync(0xffffffffu, kidx, i);
            const int row = 8 * pw + i;
            cp_async16(kst + cj * kChunkBytes + row * 128 + ((cc ^ (row & 7)) << 4),
                       kvb + (size_t)ri * pitch + 16 * lane);
          }
          {
            const int ri = __shfl_sync(0xffffffffu, kidx, lane >> 2);
            const int row = 8 * pw + (lane >> 2);
            // rope bytes: compact 64-byte rows, 64-byte swizzle (16-byte unit ^ ((row / 2) % 4))
            cp_async16(kst + 4 * kChunkBytes + row * 64 + (((lane & 3) ^ ((row >> 1) & 3)) << 4),
                       kvb + (size_t)ri * pitch + 512 + 16 * (lane & 3));
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
          const uint32_t vst = sbase + kOffV + s * kVStage;
          // lane: row 16pw + 2i + lane/16 of the block's 128 keys, 16-byte piece lane%16 of this
          // CTA's 256 value bytes
          const int pc = lane & 15, nbk = pc >> 3, c8 = pc & 7;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rloc = 2 * i + (lane >> 4);
            const int ri = __shfl_sync(0xffffffffu, vidx, 16 + rloc);
            const int row = 16 * pw + rloc;
            cp_async16(vst + nbk * kVChunk + row * 128 + ((c8 ^ (row & 7)) << 4),
                       kvb + (size_t)ri * pitch + 256 * cta + 16 * pc);
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
      } else if ((++idle_iters & (kIdleCheckEvery - 1)) != 0) {
        __nanosleep(kIdleSleepNs);
      } else {
        // the (slow) time-limit and abort check runs once per kIdleCheckEvery idle polls
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
  } else {
   if (warp == kWarpMma) {
    // ------------------------------------------------------------ MMA issue (leader CTA only)
    if (cta == 0) {   // the whole warp runs this loop; one elected lane issues
      constexpr uint32_t idesc_qk = umma_idesc(0, 0, false, false, 128, 128);
      constexpr uint32_t idesc_pv = umma_idesc(0, 0, false, true, 128, 256);
      const uint32_t a_qk_done0 = smem_u32(&ms.qk_done[0]), a_qk_done0_peer = mapa(a_qk_done0, 1);
      const uint32_t a_pv_done_peer[2] = {mapa(smem_u32(&ms.pv_done[0]), 1), mapa(smem_u32(&ms.pv_done[1]), 1)};
      const uint32_t a_q_free_peer = mapa(smem_u32(&ms.q_free), 1);
      // S = Q K^T of block kb into S buffer kb%2
      // The K / V tiles were written by cp.async (generic proxy) and are read by the tensor core
      // through the async proxy: a cross-proxy fence sits between "landed" and the MMA.
      // descriptor high words: 128-byte swizzle (8-row groups 1024 B apart) for the four latent
      // chunks, 64-byte swizzle (8-row groups 512 B apart) for the compact rope chunk
      const uint32_t hi128 = (uint32_t)(umma_desc(0, 16, 1024, kSwz128) >> 32);
      const uint32_t hi64 = (uint32_t)(umma_desc(0, 16, 512, kSwz64) >> 32);
      auto issue_qk = [&](int k, int kb, const BlockIdx& bi) {
        fence_proxy_async_smem();
        tc_fence_after();
        const uint32_t d = tmem + ((kb & 1) ? kTmemS1 : kTmemS0);
        const uint32_t a_rope_lo = (uint32_t)umma_desc(sbase + kOffQ + 4 * kChunkBytes, 16, 512, kSwz64);
        const uint32_t b_lo = (uint32_t)umma_desc(sbase + kOffK + bi.ks * kKStage, 16, 1024, kSwz128);
        mma_f8_pair_qk18(d, idesc_qk, tmem + kTmemQ, b_lo, hi128, hi64, a_rope_lo);
        mma_commit_pair_elect(a_qk_done0 + 8u * (uint32_t)bi.b6);
        mma_commit_pair_elect(a_qk_done0_peer + 8u * (uint32_t)bi.b6);
      };
      auto issue_pv = [&](int k, int kb) {
        const int s = kb & 1;
        fence_proxy_async_smem();
        tc_fence_after();
        const uint64_t ad = umma_desc(sbase + kOffP + (kPBufs == 2 ? s : 0) * kPBytes, 1024, 128, kSwzNone);
        const uint64_t bd = umma_desc(sbase + kOffV + s * kVStage, kVChunk, 1024, kSwz128);
        mma_f8_pair_pv8(tmem + kTmemO, idesc_pv, (uint32_t)ad, (uint32_t)bd, (uint32_t)(ad >> 32),
                        (uint32_t)(bd >> 32), k ? 1u : 0u);
        mma_commit_pair_elect(smem_u32(&ms.pv_done[s]));
        mma_commit_pair_elect(a_pv_done_peer[s]);
      };
      int kb0 = 0, it = 0;
      bool aborted = false;
      for (int tile = cid; tile < p.ng && !aborted; tile += ncl, ++it) {
        const int nb = blocks_of(tile_count(tile));
        mbar_wait(&ms.qt_ready, it & 1, wt, kSiteQ, it);
        __syncwarp();
        // Ready-driven issue: whichever of "next QK" (its K stage landed on both CTAs and its S
        // buffer drained) and "next PV" (its P written, its V stage landed on both CTAs, and for
        // the tile's first PV the previous tile's O read out) is ready goes first.
        int qk_i = 0, pv_i = 0;
        unsigned long long idle_since = 0;
        unsigned idle_iters = 0;
        while (pv_i < nb && !aborted) {
          bool did = false;
          {
            const int kb = kb0 + pv_i;
            const int s = kb & 1;
            const uint32_t ph = (kb >> 1) & 1;
            // lanes poll independently: act only on what every lane has seen (keeps the warp converged)
            const bool ok = pv_i < qk_i && mbar_test(&ms.p_ready[s], ph) && mbar_test(&ms.v_land[s], ph) &&
                            mbar_test(&ms.v_peer[s], ph) &&
                            (pv_i > 0 || it == 0 || mbar_test(&ms.o_free, (it - 1) & 1));
            if (__all_sync(0xffffffffu, ok)) {
              issue_pv(pv_i, kb);
              ++pv_i;
              did = true;
            }
          }
          if (qk_i < nb) {
            const int kb = kb0 + qk_i;
            const BlockIdx bi(kb);
            const int s = kb & 1;
            const uint32_t ph = (kb >> 1) & 1;
            const bool ok = mbar_test(&ms.k_land[bi.ks], bi.kph) && mbar_test(&ms.k_peer[bi.ks], bi.kph) &&
                            (kb < 2 || mbar_test(&ms.s_free[s], ph ^ 1));
            if (__all_sync(0xffffffffu, ok)) {
              issue_qk(qk_i, kb, bi);
              ++qk_i;
              if (qk_i == nb) {      // the Q tile is no longer needed once these MMAs complete
                mma_commit_pair_elect(smem_u32(&ms.q_free));
                mma_commit_pair_elect(a_q_free_peer);
              }
              did = true;
            }
          }
          if (did) {
            idle_since = 0;
            idle_iters = 0;
          } else if ((++idle_iters & (kIdleCheckEvery - 1)) != 0) {
            __nanosleep(kIdleSleepNs);
          } else {
            const unsigned long long now = globaltimer_ns();
            if (idle_since == 0) idle_since = now;
            bool stop = wt.aborting();
            if (now - idle_since > wt.limit_ns) {
              if (lane == 0) wt.fail(kSiteMmaIdle, pv_i);
              stop = true;
            }
            aborted = __any_sync(0xffffffffu, stop);
          }
        }
        kb0 += nb;
      }
    }
  } else if (warp >= kWarpEpi0) {
    // ------------------------------------------------------------ epilogue warps
    // O out of TMEM, x out_scale / l, bf16, TMA tile stores -- while the softmax warps already
    // work on the next tile.  A warp reads the TMEM lanes of its quarter (warp % 4): rows r of
    // key half h, dims [256h, 256h + 256) in 8 rounds of 32 dims.  Two rounds are staged as one
    // box of 32 rows x 128 bytes in the warp's 4 KB slice (128-byte swizzle: the 16-byte stores
    // of eight consecutive rows hit distinct banks) and one lane hands the box to TMA:
    // full-line asynchronous writes, no barrier wider than the warp.
    const int ew = warp - kWarpEpi0;
    const int e_tl = ((warp & 3) << 5) | lane, e_r = e_tl & 63, e_h = e_tl >> 6;
    const uint32_t e_ocol = tmem + ((uint32_t)((warp & 3) * 32) << 16) + kTmemO;
    const uint32_t a_o_free = mapa(smem_u32(&ms.o_free), 0);
    const uint32_t a_qt_ready = mapa(smem_u32(&ms.qt_ready), 0);
    const uint64_t pol_stream = l2_policy_evict_first();
    // These warps also move the latent part of every Q tile from shared memory (where TMA put
    // it) into tensor memory, where the QK^T MMAs read it: lane = row (e_r, duplicated in lanes
    // 64-127 as the 64-rows-per-CTA form of the instruction wants), chunk j -> 32 columns.  The
    // tile's Q lands when the previous tile's last QK^T has completed, i.e. shortly before that
    // tile's epilogue starts: transfer Q(t + 1), then write out O(t).
    auto transfer_q = [&](int q_it) {
      mbar_wait(&ms.q_land, q_it & 1, wt, kSiteQ, q_it);
      __syncwarp();      // lanes leave the wait loop one by one: re-converge before .aligned ops
      const uint8_t* qrow = sm + kOffQ + e_r * 128;
#pragma unroll 1
      for (int j = 0; j < 4; ++j) {
        uint32_t v[32];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const uint4 t = *reinterpret_cast<const uint4*>(qrow + j * kChunkBytes + ((u ^ (e_r & 7)) << 4));
          v[4 * u] = t.x; v[4 * u + 1] = t.y; v[4 * u + 2] = t.z; v[4 * u + 3] = t.w;
        }
        tmem_st32(tmem + ((uint32_t)((warp & 3) * 32) << 16) + kTmemQ + 32 * j, reinterpret_cast<const float*>(v));
      }
      tmem_wait_st();
      tc_fence_before();
      fence_proxy_async_smem();      // these reads are ordered before the next TMA write of the tile
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(a_qt_ready);
    };
    int kb0 = 0, it = 0;
    if (cid < p.ng) transfer_q(0);
    for (int tile = cid; tile < p.ng; tile += ncl, ++it) {
      const int nb = blocks_of(tile_count(tile));
      const int kbl = kb0 + nb - 1;                // last block of the tile
      if (tile + ncl < p.ng) transfer_q(it + 1);
      // the row scales are published and the tile's last PV has completed
      mbar_wait(&ms.epi_ready, it & 1, wt, kSiteEpi, it);
      mbar_wait(&ms.pv_done[kbl & 1], (kbl >> 1) & 1, wt, kSiteEpi, nb);
      __syncwarp();      // lanes leave the wait loop one by one: re-converge before .aligned ops
      tc_fence_after();
      const float oscale = ms.oscale[it & 1][e_r];
      const uint32_t emask = oscale != 0.f ? 0xffffffffu : 0u;
      // this warp's 32 rows of the tile = (token, head) pairs starting at row r0
      const int r0 = (int)cta * 64 + 32 * (warp & 1);
      const int out_head = r0 % p.h_per_q, out_tok = tile * p.G + r0 / p.h_per_q;
      float ob[2][32];
      tmem_ld32(e_ocol, ob[0]);
#pragma unroll
      for (int cc = 0; cc < 8; ++cc) {
        float* o = ob[cc & 1];
        tmem_wait_ld();
        if (cc < 7) {
          tmem_ld32(e_ocol + (cc + 1) * 32, ob[(cc + 1) & 1]);
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
          w[j] = *reinterpret_cast<uint32_t*>(&v2) & emask;    // rows without a valid key: zeros
        }
        {
          // two rounds make one box of 32 rows x 128 bytes (128-byte swizzle) in the warp's 4 KB
          // slice; before the first of them the previous box must have been read out
          if ((cc & 1) == 0) {
            if (lane == 0) bulk_wait_read_all();
            __syncwarp();
          }
          const uint32_t slice = kOffStage + (uint32_t)ew * 4096;
          uint8_t* st_row = sm + slice + (e_r & 31) * 128;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(st_row + (((4 * (cc & 1) + j) ^ (e_r & 7)) << 4)) =
                make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
          if (cc & 1) {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              for (int d = 0; d < p.n_out; ++d)
                tma_store_3d_hint(&omaps.m[d], sbase + slice, 256 * e_h + 64 * (cc >> 1), out_head, out_tok, pol_stream);
              bulk_commit_group();
            }
          }
        }
      }
      kb0 += nb;
    }
    if (lane == 0) bulk_wait_all();   // output boxes written before the CTA retires
    tc_fence_before();
  } else if (warp == kWarpCopy || warp == kWarpRelay) {
    // ------------------------------------------------------------ "landed" relays to the leader CTA
    // The MMA thread lives in the leader CTA and can only wait on its own barriers: in the
    // peer CTA warp 17 forwards "K tile landed" and warp 18 "V tile landed".
    if (cta == 1) {
      const bool is_k = warp == kWarpCopy;
      const uint32_t a_peer0 = mapa(smem_u32(is_k ? &ms.k_peer[0] : &ms.v_peer[0]), 0);
      int kb0 = 0;
      for (int tile = cid; tile < p.ng; tile += ncl) {
        const int nb = blocks_of(tile_count(tile));
        for (int k = 0; k < nb; ++k) {
          const int kb = kb0 + k;
          const BlockIdx bi(kb);
          const int s = is_k ? bi.ks : (kb & 1);
          const uint32_t ph = is_k ? (uint32_t)bi.kph : (uint32_t)((kb >> 1) & 1);
          mbar_wait(is_k ? &ms.k_land[s] : &ms.v_land[s], ph, wt, is_k ? kSiteRelayK : kSiteRelayV, k);
          fence_proxy_async_smem();     // this CTA's cp.async writes -> the leader's MMA reads
          if (lane == 0) mbar_arrive_cluster_release(a_peer0 + 8u * (uint32_t)s);
        }
        kb0 += nb;
      }
    }
  } else {
    // ------------------------------------------------------------ index-validity bits (warp kWarpValid)
    static_assert(kWarpValid == kWarpRelay + 1 && kWarpValid + 1 == kWarpEpi0, "role layout");
    int kb0 = 0;
    for (int tile = cid; tile < p.ng; tile += ncl) {
      const int count = tile_count(tile);
      const int nb = blocks_of(count);
      const int32_t* idx_row = p.indices + (size_t)tile * p.idx_stride;
      int4 cur = __ldcs(reinterpret_cast<const int4*>(idx_row) + lane);
      for (int k = 0; k < nb; ++k) {
        const int kb = kb0 + k;
        const int s = kb & 1;
        const uint32_t ph = (kb >> 1) & 1;
        int4 nxt = cur;
        if (k + 1 < nb) nxt = __ldcs(reinterpret_cast<const int4*>(idx_row + (size_t)(k + 1) * kBlockKeys) + lane);
        const int rank0 = k * kBlockKeys + lane * 4;
        auto ok = [&](int idx, int rk) -> uint32_t {
          return (idx >= 0 && idx < p.s_kv && rk < count) ? 1u : 0u;
        };
        const uint32_t nib = ok(cur.x, rank0) | (ok(cur.y, rank0 + 1) << 1) |
                             (ok(cur.z, rank0 + 2) << 2) | (ok(cur.w, rank0 + 3) << 3);
        if (kb >= 2) mbar_wait(&ms.valid_free[s], ph ^ 1, wt, kSiteValidFree, k);
        const uint32_t nib_hi = __shfl_down_sync(0xffffffffu, nib, 1);
        if ((lane & 1) == 0)
          reinterpret_cast<uint8_t*>(&ms.valid[s][0])[lane >> 1] = (uint8_t)(nib | (nib_hi << 4));
        __syncwarp();
        if (lane == 0) mbar_arrive(&ms.valid_ready[s]);
        cur = nxt;
      }
      kb0 += nb;
    }
  }
  }

  // tear-down: nobody may still be reading TMEM of either CTA when it is released
  __syncthreads();
  __syncwarp();
  cluster_sync_all();
  if (warp == kWarpMma) tmem_dealloc_pair(tmem, kTmemCols);
  if (blockIdx.x == 0 && threadIdx.x == 0) atomicAdd(&g_attn_status[3], 1);
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
  cfg.gridDim = dim3(sms, 1, 1); cfg.blockDim = dim3(kAttnThreads, 1, 1); cfg.dynamicSmemBytes = Plan::kSmem;
  cudaLaunchAttribute at; at.id = cudaLaunchAttributeClusterDimension; at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
  cfg.attrs = &at; cfg.numAttrs = 1;
  int q = 0;
  if (cudaFuncSetAttribute(masked_mla_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)Plan::kSmem) == cudaSuccess &&
      cudaOccupancyMaxActiveClusters(&q, masked_mla_fp8_kernel, &cfg) == cudaSuccess && q > 0)
    n = q;
  cudaGetLastError();
  cached_dev = dev; cached = n;
  return n;
}

static int launch_fp8_t(const CUtensorMap& map_q, const CUtensorMap& map_q_rope, const OutMaps& omaps,
                        const AttnParams& p, cudaStream_t stream) {
  using PL = Plan;
  auto kern = masked_mla_fp8_kernel;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PL::kSmem) != cudaSuccess)
    return LITEDSA_ERR_CUDA;
  kern<<<2 * min(p.ng, max_clusters()), kAttnThreads, PL::kSmem, stream>>>(
      map_q, map_q_rope, omaps, p);
  return cudaGetLastError() == cudaSuccess ? LITEDSA_OK : LITEDSA_ERR_CUDA;
}

static int launch_fp8(const Fp8Args& a, void* const* outs, int n_out, cudaStream_t stream) {
  CUtensorMap map_q, map_q_rope;
  OutMaps omaps;
  // q and out are addressed as (dim, head, token): row r of a tile is (token r / h, head r % h),
  // which covers the dense packed layout and the in-place layout with padded head slots alike.
  // out is stored as boxes of 32 rows x 64 dims (128 bytes wide, 128-byte swizzle); only the
  // destinations in use are encoded, the unused slots repeat the first map
  const int h = a.h_per_q, G = 128 / h;
  const int qdiv = a.q_group_div > 0 ? a.q_group_div : 1;
  const uint64_t q_hs = a.q_head_stride ? (uint64_t)a.q_head_stride : (uint64_t)a.q_row_stride;
  const uint64_t q_ts = a.q_token_stride ? (uint64_t)a.q_token_stride : (uint64_t)h * q_hs;
  const uint64_t o_hs = (a.out_head_stride ? (uint64_t)a.out_head_stride : (uint64_t)kDV) * 2;
  const uint64_t o_ts = a.out_token_stride ? (uint64_t)a.out_token_stride * 2 : (uint64_t)h * o_hs;
  const uint32_t ob_h = (uint32_t)min(h, 32);
  for (int d = 0; d < n_out; ++d)
    if (!make_map_3d(&omaps.m[d], outs[d], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, kDV, (uint64_t)h,
                     (uint64_t)a.ng * G, o_hs, o_ts, 64, ob_h, 32 / ob_h, CU_TENSOR_MAP_SWIZZLE_128B))
      return LITEDSA_ERR_CUDA;
  for (int d = n_out; d < kMaxOutputs; ++d) omaps.m[d] = omaps.m[0];
  // Q per CTA: four boxes of 128 bytes x 64 rows (128-byte swizzle) and the rope box of 64 bytes
  // x 64 rows (64-byte swizzle)
  const uint32_t qb_h = (uint32_t)min(h, 64);
  if (!make_map_3d(&map_q, a.q8, CU_TENSOR_MAP_DATA_TYPE_UINT8, kDQK, (uint64_t)h,
                   (uint64_t)(a.ng / qdiv) * G, q_hs, q_ts, 128, qb_h, 64 / qb_h) ||
      !make_map_3d(&map_q_rope, a.q8, CU_TENSOR_MAP_DATA_TYPE_UINT8, kDQK, (uint64_t)h,
                   (uint64_t)(a.ng / qdiv) * G, q_hs, q_ts, 64, qb_h, 64 / qb_h, CU_TENSOR_MAP_SWIZZLE_64B))
    return LITEDSA_ERR_CUDA;
  AttnParams p;
  p.memb = a.memb_qm; p.len_per_q = a.topk_length_per_q; p.sink = a.attn_sink; p.q_group_div = qdiv;
  p.indices = a.indices; p.counts = a.topk_length;
  p.kv = reinterpret_cast<const uint8_t*>(a.kv8); p.kv_pitch = a.kv_row_stride;
  p.out = reinterpret_cast<__nv_bfloat16*>(outs[0]); p.n_out = n_out; p.lse = a.lse;
  p.max_logits = a.max_logits;
  p.ng = a.ng; p.s_kv = a.s_kv; p.cap = a.topk; p.h_per_q = a.h_per_q; p.G = 128 / a.h_per_q;
  p.idx_stride = a.indices_row_stride;
  p.scale_log2 = a.sm_scale * kLog2e; p.out_scale = a.out_scale;
  p.epoch = next_launch_epoch(); p.wait_limit_ns = wait_limit_ns();
  return launch_fp8_t(map_q, map_q_rope, omaps, p, stream);
}

// Host-side argument rules shared by every FP8 attention entry point: the reference
// launcher's shape rules (kernels/b200/dsa/litedsa.cu:82-98) plus the alignment TMA needs.
// No CUDA call is made here.
int check_fp8_args(const Fp8Args& a) {
  if (!a.q8 || !a.kv8 || !a.indices || !a.lse) return LITEDSA_ERR_ARG;
  if (!a.memb_qm && !a.topk_length_per_q) return LITEDSA_ERR_ARG;   // one of the two masks
  if (a.ng <= 0 || a.s_kv <= 0 || a.topk <= 0 || a.topk % 128 != 0) return LITEDSA_ERR_SHAPE;
  if (a.h_per_q <= 0 || 128 % a.h_per_q != 0 || 128 / a.h_per_q > 16) return LITEDSA_ERR_SHAPE;
  if (a.q_group_div < 1 || a.ng % a.q_group_div != 0) return LITEDSA_ERR_SHAPE;
  // TMA needs 16-byte aligned bases and row pitches
  if (a.q_row_stride < kDQK || a.kv_row_stride < kDQK || a.q_row_stride % 16 || a.kv_row_stride % 16)
    return LITEDSA_ERR_UNSUPPORTED;
  if (((uintptr_t)a.q8 | (uintptr_t)a.kv8 | (uintptr_t)a.indices) & 15) return LITEDSA_ERR_UNSUPPORTED;
  if (a.indices_row_stride < a.topk || a.indices_row_stride % 4) return LITEDSA_ERR_UNSUPPORTED;
  // in-place addressing: TMA wants 16-byte multiples for every pitch
  if (a.q_token_stride < 0 || a.q_head_stride < 0 || a.out_token_stride < 0 || a.out_head_stride < 0)
    return LITEDSA_ERR_SHAPE;
  if ((a.q_head_stride && (a.q_head_stride < kDQK || a.q_head_stride % 16)) || a.q_token_stride % 16 ||
      (a.out_head_stride && (a.out_head_stride < kDV || a.out_head_stride % 8)) || a.out_token_stride % 8)
    return LITEDSA_ERR_UNSUPPORTED;
  return LITEDSA_OK;
}

int run_fp8(const Fp8Args& a, void* const* outs, int n_outs, void* stream) {
  int rc = check_fp8_args(a);
  if (rc != LITEDSA_OK) return rc;
  if (!outs || n_outs < 1 || n_outs > kMaxOutputs) return n_outs < 1 || n_outs > kMaxOutputs ? LITEDSA_ERR_SHAPE : LITEDSA_ERR_ARG;
  for (int d = 0; d < n_outs; ++d) {
    if (!outs[d]) return LITEDSA_ERR_ARG;
    if ((uintptr_t)outs[d] & 15) return LITEDSA_ERR_UNSUPPORTED;
  }
  return launch_fp8(a, outs, n_outs, reinterpret_cast<cudaStream_t>(stream));
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
                                      void* stream) {
  using namespace lt;
  if (!memb_qm || !out) return LITEDSA_ERR_ARG;
  Fp8Args a{q8, kv8, indices, sm_scale, out_scale, topk_length, memb_qm, h_per_q, max_logits, lse,
            ng, s_kv, topk, q_row_stride, kv_row_stride, indices_row_stride, nullptr, nullptr, 1};
  void* outs[1] = {out};
  return run_fp8(a, outs, 1, stream);
}

// The operator with the optional modes of the reference kernel's parameter block that its
// binding leaves switched off (litedsa.cu:127-132): attn_sink [128] per packed row joins the
// output normaliser (litedsa_attention_sm100.cuh:2127-2133); topk_length_per_q [ng, G] bounds
// each token to a causal prefix of the union ranks and may replace memb_qm (:1378-1385,
// :1988-1996); q_group_div consecutive tiles share one Q tile (KV split, :1383-1385, :1909).
// q_token_stride / q_head_stride / out_token_stride / out_head_stride (ELEMENTS, 0 = dense packed)
// address q and out in place inside [T, H_padded, d] tensors that hold h_per_q real heads per
// token, which removes the pack / unpack copies around the kernel
// (kernels/b200/dsa/DSV4_ZEROCOPY_PLAN.md:12-22, 50-76).
extern "C" int litedsa_masked_mla_fp8_ex(const void* q8, const void* kv8, const int32_t* indices,
                                         float sm_scale, float out_scale,
                                         const int32_t* topk_length, const uint32_t* memb_qm,
                                         int h_per_q, void* out, float* max_logits, float* lse,
                                         int ng, int s_kv, int topk, int64_t q_row_stride,
                                         int64_t kv_row_stride, int64_t indices_row_stride,
                                         const float* attn_sink, const int32_t* topk_length_per_q,
                                         int q_group_div, int64_t q_token_stride,
                                         int64_t q_head_stride, int64_t out_token_stride,
                                         int64_t out_head_stride, void* stream) {
  using namespace lt;
  if (!out) return LITEDSA_ERR_ARG;
  Fp8Args a{q8, kv8, indices, sm_scale, out_scale, topk_length, memb_qm, h_per_q, max_logits, lse,
            ng, s_kv, topk, q_row_stride, kv_row_stride, indices_row_stride, attn_sink,
            topk_length_per_q, q_group_div, q_token_stride, q_head_stride, out_token_stride,
            out_head_stride};
  void* outs[1] = {out};
  return run_fp8(a, outs, 1, stream);
}

// The same operator with the all-gather of a sharded run folded into its epilogue: every
// output box is written to n_outs destinations with plain TMA tile stores -- outs[0] is
// this GPU's buffer, outs[1..] are the peers' copies (peer-mapped device addresses of the
// slot this rank owns in each peer's gathered buffer).  The reference has no multi-GPU path.
extern "C" int litedsa_masked_mla_fp8_multi(const void* q8, const void* kv8, const int32_t* indices,
                                            float sm_scale, float out_scale,
                                            const int32_t* topk_length, const uint32_t* memb_qm,
                                            int h_per_q, void* const* outs, int n_outs,
                                            float* max_logits, float* lse, int ng, int s_kv,
                                            int topk, int64_t q_row_stride, int64_t kv_row_stride,
                                            int64_t indices_row_stride, void* stream) {
  using namespace lt;
  if (!memb_qm || !outs) return LITEDSA_ERR_ARG;
  Fp8Args a{q8, kv8, indices, sm_scale, out_scale, topk_length, memb_qm, h_per_q, max_logits, lse,
            ng, s_kv, topk, q_row_stride, kv_row_stride, indices_row_stride, nullptr, nullptr, 1};
  return run_fp8(a, outs, n_outs, stream);
}

// Synchronous read (and optional reset) of the device status block of the FP8 attention
// kernels on the current device: out[0] = first wait site that expired since the last reset
// (0 = none), out[1] = block, out[2] = iteration, out[3] = launches completed since the reset.
extern "C" int litedsa_attn_status(int* out4_host, int reset) {
  using namespace lt;
  if (out4_host &&
      cudaMemcpyFromSymbol(out4_host, g_attn_status, sizeof(int) * 4) != cudaSuccess)
    return LITEDSA_ERR_CUDA;
  if (reset) {
    const int z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (cudaMemcpyToSymbol(g_attn_status, z, sizeof(z)) != cudaSuccess) return LITEDSA_ERR_CUDA;
  }
  return (out4_host && out4_host[0] != 0) ? LITEDSA_ERR_TIMEOUT : LITEDSA_OK;
}

// Self-test of the bounded wait, for test suites: a one-warp kernel waits with the given
// limit on an mbarrier that nobody arrives on.  The wait must give up, record its site
// (kSiteSelfTest) in the same status block the attention kernels use, and the kernel must
// return normally.  Synchronous.  Returns LITEDSA_ERR_TIMEOUT when the wait expired as it
// should, LITEDSA_OK if it (wrongly) succeeded.  Nothing hangs or faults.
namespace lt {
__global__ void wait_selftest_kernel(int epoch, unsigned long long limit_ns, int* returned) {
  __shared__ uint64_t bar;
  const Waiter wt{g_attn_status, epoch, limit_ns};
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  __syncwarp();
  const bool ok = mbar_wait(&bar, 0, wt, kSiteSelfTest, 7);
  if (threadIdx.x == 0) *returned = ok ? 1 : 2;
}
}  // namespace lt
extern "C" int litedsa_selftest_wait_timeout(uint64_t limit_ns, int* returned_device) {
  using namespace lt;
  if (!returned_device || limit_ns == 0 || limit_ns > 1000000000ull) return LITEDSA_ERR_ARG;
  wait_selftest_kernel<<<1, 32>>>(next_launch_epoch(), limit_ns, returned_device);
  if (cudaGetLastError() != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) return LITEDSA_ERR_CUDA;
  int st[4] = {0, 0, 0, 0};
  if (cudaMemcpyFromSymbol(st, g_attn_status, sizeof(st)) != cudaSuccess) return LITEDSA_ERR_CUDA;
  return st[0] != 0 ? LITEDSA_ERR_TIMEOUT : LITEDSA_OK;
}

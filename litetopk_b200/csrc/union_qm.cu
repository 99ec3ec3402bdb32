// Per-tile union of the top-k index lists of the G tokens that share one 128-row
// attention tile, plus the query-major membership bitmask.
//
// Contract (what every LIVE output word must equal), stated by the reference at
// kernels/b200/dsa/litedsa_union.cuh:4-25 and implemented there at :34-184:
//   counts[g]        number of distinct positions p, 0 <= p < seq_space, in the tile
//   u_phys[g, r]     physical slot of the r-th smallest such position (r < count)
//   memb_qm[g,q,w]   bit b set  <=>  rank 32*w+b is in token q's own list
// Only the algorithmic idea "a position bitmap makes sort + dedup a scan" is shared
// with the reference; this kernel is laid out for B200 differently:
//   * 256-thread CTAs (several resident per SM, so one tile's barrier phases overlap
//     another tile's loads) instead of one 1024-thread CTA per SM slot;
//   * the tile's indices are read from HBM ONCE with 16-byte loads and stay in
//     registers for the second (rank) pass;
//   * a per-word exclusive rank table makes the rank lookup one popcount;
//   * the sorted list is staged in shared memory and leaves the SM as 16-byte
//     coalesced stores.
// Integer-only, HBM-bound work: no tensor cores, no TMA.
#include "common.cuh"

namespace lt {


struct UnionParams {
  const int32_t* idx;       // [T, k]
  int32_t* u_phys;          // [ng, cap]
  int32_t* counts;          // [ng]
  uint32_t* memb;           // [ng, G, cap/32]
  const int32_t* req_pg;    // [ng] or null (identity table)
  const int32_t* btab;      // [nreq, bt_stride] or null
  int bt_stride, bt_blocks, bsz;
  uint32_t bsz_mul;         // ceil(2^32 / bsz), or 0: divide
  int kq;                   // k / 4: 16-byte loads per token row
  uint32_t kq_mul;          // ceil(2^32 / kq), or 0: divide
  int k, G, cap, s_words;   // s_words = seq_space / 32
  int rank_shift;           // rank table holds one entry per (1 << rank_shift) bitmap words
  int stage_list;           // 1: sorted list staged in smem
  int fill_tail;            // 1: also write -1 / 0 beyond the live prefixes
};

// Shared-memory carve-up (bytes): bitmap | rank table (u16) | qm accumulator | list stage
__host__ __device__ inline size_t union_smem_bytes(int s_words, int rank_shift, int G, int cap,
                                                   int stage_list) {
  size_t b = (size_t)s_words * 4;
  b += (((size_t)(s_words >> rank_shift) * 2) + 15) & ~(size_t)15;
  b += (size_t)G * (cap / 32) * 4;
  if (stage_list) b += (size_t)cap * 4;
  return b;
}

// n / d through a multiply-high when the host proved it exact (n * d < 2^32, d > 1)
__device__ __forceinline__ int fast_div(int n, int d, uint32_t mul) {
  return mul ? (int)__umulhi((uint32_t)n, mul) : n / d;
}
inline uint32_t fast_div_mul(int64_t n_max, int d) {
  if (d <= 1 || n_max * d >= (int64_t(1) << 32)) return 0;
  return (uint32_t)(((int64_t(1) << 32) + d - 1) / d);
}

// NT threads per tile; VPT int4 loads cached per thread (0: nothing cached, the second
// pass re-reads the tile).  PLAIN: no block table and one rank-table entry per bitmap word
// (the common case), so the candidate pass carries neither the translation nor the
// partial-rank loop.  (Forcing 32 registers per thread so that every warp slot of the SM is
// filled was measured 3-8 % slower: the kernel is bound by shared-memory transactions, not
// by occupancy.)
template <int NT, int VPT, bool PLAIN>
__global__ void __launch_bounds__(NT)
union_qm_kernel(const UnionParams p) {
  constexpr int kUnionThreads = NT;
  extern __shared__ __align__(16) uint32_t smem[];
  __shared__ int warp_tot[kUnionThreads / 32];

  const int g = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int s_words = p.s_words, cap = p.cap, capw = cap >> 5, total = p.G * p.k;
  const int S = s_words << 5;
  uint32_t* bm = smem;
  uint16_t* rtab = reinterpret_cast<uint16_t*>(bm + s_words);
  const int rt_entries = s_words >> p.rank_shift;
  uint32_t* qm_s = reinterpret_cast<uint32_t*>(
      reinterpret_cast<char*>(rtab) + ((((size_t)rt_entries * 2) + 15) & ~(size_t)15));
  int32_t* list_s = reinterpret_cast<int32_t*>(qm_s + (size_t)p.G * capw);

  // phase 0: clear bitmap
  {
    uint4* b4 = reinterpret_cast<uint4*>(bm);
    for (int i = tid; i < (s_words >> 2); i += kUnionThreads) b4[i] = make_uint4(0, 0, 0, 0);
  }
  // issue the tile's loads while the clear drains
  const int4* src = reinterpret_cast<const int4*>(p.idx + (size_t)g * total);
  const int nquad = total >> 2;
  int4 v[VPT > 0 ? VPT : 1];
  if (VPT > 0) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int qd = i * kUnionThreads + tid;
      v[i] = qd < nquad ? __ldg(src + qd) : make_int4(-1, -1, -1, -1);
    }
  }
  __syncthreads();

  // phase 1: insert
  auto insert = [&](int pos) {
    if ((unsigned)pos < (unsigned)S) atomicOr(&bm[pos >> 5], 1u << (pos & 31));
  };
  if (VPT > 0) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) { insert(v[i].x); insert(v[i].y); insert(v[i].z); insert(v[i].w); }
  } else {
    for (int qd = tid; qd < nquad; qd += kUnionThreads) {
      const int4 t = __ldg(src + qd);
      insert(t.x); insert(t.y); insert(t.z); insert(t.w);
    }
  }
  __syncthreads();

  // phase 2: per-thread popcount of a contiguous run of words; warp scan, then every
  // thread adds the totals of the warps before its own
  const int wpt = (s_words + kUnionThreads - 1) / kUnionThreads;   // words per thread
  const int w0 = min(tid * wpt, s_words), w1 = min(w0 + wpt, s_words);
  int mine = 0;
  for (int w = w0; w < w1; ++w) mine += __popc(bm[w]);
  int incl = mine;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += t;
  }
  if (lane == 31) warp_tot[wid] = incl;
  __syncthreads();
  int before = 0, count = 0;
#pragma unroll
  for (int i = 0; i < kUnionThreads / 32; ++i) {
    const int t = warp_tot[i];
    before += i < wid ? t : 0;
    count += t;
  }
  const int live = min(count, cap);
  if (tid == 0) p.counts[g] = count;

  // phase 3: exclusive rank of every bitmap word (or every 2^rank_shift-th word)
  {
    int r = before + incl - mine;
    const int rank_shift = PLAIN ? 0 : p.rank_shift;
    const int rmask = (1 << rank_shift) - 1;
    for (int w = w0; w < w1; ++w) {
      if ((w & rmask) == 0) rtab[w >> rank_shift] = (uint16_t)r;
      r += __popc(bm[w]);
    }
  }
  // live mask words per query row: max(4, roundup4(ceil(live / 32)))
  const int active = max(4, (((live + 31) >> 5) + 3) & ~3);
  for (int i = tid; i < p.G * active; i += kUnionThreads) qm_s[i] = 0u;
  __syncthreads();

  // phase 4: every candidate looks up its rank, sets its token's membership bit and
  // writes its own slot of the sorted list (duplicates write the same value)
  const int32_t* bt_row = (!PLAIN && p.btab) ? p.btab + (size_t)p.req_pg[g] * p.bt_stride : nullptr;
  int32_t* out_row = p.u_phys + (size_t)g * cap;
  int32_t* list_dst = p.stage_list ? list_s : out_row;
  auto mark = [&](int pos, int qrow) {
    if ((unsigned)pos >= (unsigned)S) return;
    const int w = pos >> 5;
    int r;
    if (PLAIN) {
      r = rtab[w];
    } else {
      r = rtab[w >> p.rank_shift];
      if (p.rank_shift)
        for (int x = (w >> p.rank_shift) << p.rank_shift; x < w; ++x) r += __popc(bm[x]);
    }
    r += __popc(bm[w] & ((1u << (pos & 31)) - 1u));
    if (r >= cap) return;
    atomicOr(&qm_s[qrow + (r >> 5)], 1u << (r & 31));
    int phys = pos;
    if (!PLAIN && bt_row) {
      const int blk = fast_div(pos, p.bsz, p.bsz_mul);
      phys = blk < p.bt_blocks ? bt_row[blk] * p.bsz + (pos - blk * p.bsz) : -1;
    }
    list_dst[r] = phys;
  };
  if (VPT > 0) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      // k % 4 == 0: the four candidates of one 16-byte load belong to one token
      const int qrow = fast_div(i * kUnionThreads + tid, p.kq, p.kq_mul) * active;
      mark(v[i].x, qrow); mark(v[i].y, qrow); mark(v[i].z, qrow); mark(v[i].w, qrow);
    }
  } else {
    for (int qd = tid; qd < nquad; qd += kUnionThreads) {
      const int4 t = __ldg(src + qd);
      const int qrow = fast_div(qd, p.kq, p.kq_mul) * active;
      mark(t.x, qrow); mark(t.y, qrow); mark(t.z, qrow); mark(t.w, qrow);
    }
  }
  __syncthreads();

  // sorted list -> global, 16-byte stores (the last quad is padded with -1)
  if (p.stage_list) {
    const int q_live = (live + 3) >> 2;
    const int q_end = p.fill_tail ? (cap >> 2) : q_live;
    int4* dst = reinterpret_cast<int4*>(out_row);
    for (int i = tid; i < q_end; i += kUnionThreads) {
      int4 o;
      const int b = i << 2;
      o.x = b + 0 < live ? list_s[b + 0] : -1;
      o.y = b + 1 < live ? list_s[b + 1] : -1;
      o.z = b + 2 < live ? list_s[b + 2] : -1;
      o.w = b + 3 < live ? list_s[b + 3] : -1;
      dst[i] = o;
    }
  } else if (p.fill_tail) {
    for (int i = live + tid; i < cap; i += kUnionThreads) out_row[i] = -1;
  }

  // phase 5: dump the live mask words (whole rows when fill_tail)
  {
    const int a4 = active >> 2, c4 = capw >> 2;
    const int per_row = p.fill_tail ? c4 : a4;
    uint4* dst = reinterpret_cast<uint4*>(p.memb + (size_t)g * p.G * capw);
    const uint4* s4 = reinterpret_cast<const uint4*>(qm_s);
    for (int i = tid; i < p.G * per_row; i += kUnionThreads) {
      const int q = i / per_row, j = i - q * per_row;
      dst[q * c4 + j] = j < a4 ? s4[q * a4 + j] : make_uint4(0, 0, 0, 0);
    }
  }
}

template <int NT, int VPT>
static int launch_union(const UnionParams& p, int ng, size_t smem, cudaStream_t stream) {
  constexpr int kUnionThreads = NT;
  const bool plain = p.btab == nullptr && p.rank_shift == 0;
  auto kern = plain ? union_qm_kernel<NT, VPT, true> : union_qm_kernel<NT, VPT, false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return LITEDSA_ERR_CUDA;
  kern<<<ng, kUnionThreads, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? LITEDSA_OK : LITEDSA_ERR_CUDA;
}

}  // namespace lt

// C-ABI entry point; argument order and meaning follow the reference operator
// union_qm(topk_indices, u_phys, counts, memb_qm, req_pg, block_table, block_size, seq_space)
// (kernels/b200/dsa/litedsa.cu:31-75), with tensor shapes passed as integers.
extern "C" int litedsa_union_qm(const int32_t* topk_indices, int32_t* u_phys, int32_t* counts,
                                uint32_t* memb_qm, const int32_t* req_pg,
                                const int32_t* block_table, int T, int k, int ng, int cap, int G,
                                int bt_rows, int bt_blocks, int block_size, int64_t seq_space,
                                int fill_tail, void* stream) {
  using namespace lt;
  // same argument checks as the reference launcher (litedsa.cu:43-59)
  if (!topk_indices || !u_phys || !counts || !memb_qm) return LITEDSA_ERR_ARG;
  if (ng <= 0 || G <= 0 || k <= 0 || T != ng * G) return LITEDSA_ERR_SHAPE;
  if (cap != G * k || cap % 128 != 0) return LITEDSA_ERR_SHAPE;
  if (G > 16 || (int64_t)G * (cap / 32) > 16 * 1024) return LITEDSA_ERR_SHAPE;
  if (seq_space <= 0 || seq_space > (1 << 20)) return LITEDSA_ERR_SHAPE;
  const int s_words = (int)((seq_space + 31) / 32);
  if (s_words % 32 != 0) return LITEDSA_ERR_SHAPE;   // 1024-position aligned
  if ((block_table != nullptr) != (req_pg != nullptr)) return LITEDSA_ERR_ARG;
  if (block_table && (block_size <= 0 || bt_blocks <= 0 || bt_rows <= 0)) return LITEDSA_ERR_SHAPE;
  if (k % 4 != 0) return LITEDSA_ERR_UNSUPPORTED;    // 16-byte row loads
  if (cap > 65536) return LITEDSA_ERR_UNSUPPORTED;   // 16-bit rank table

  UnionParams p;
  p.idx = topk_indices; p.u_phys = u_phys; p.counts = counts; p.memb = memb_qm;
  p.req_pg = req_pg; p.btab = block_table;
  p.bt_stride = bt_blocks; p.bt_blocks = bt_blocks; p.bsz = block_table ? block_size : 1;
  p.bsz_mul = fast_div_mul(int64_t(s_words) * 32, p.bsz);
  p.kq = k / 4; p.kq_mul = fast_div_mul(int64_t(G) * (k / 4), k / 4);
  p.k = k; p.G = G; p.cap = cap; p.s_words = s_words; p.fill_tail = fill_tail ? 1 : 0;
  // pick the richest shared-memory plan that fits (227 KB per CTA on sm_100)
  const size_t limit = 220 * 1024;
  p.rank_shift = 0; p.stage_list = 1;
  if (union_smem_bytes(s_words, 0, G, cap, 1) > limit) p.stage_list = 0;
  if (union_smem_bytes(s_words, 0, G, cap, p.stage_list) > limit) p.rank_shift = 2;
  const size_t smem = union_smem_bytes(s_words, p.rank_shift, G, cap, p.stage_list);
  if (smem > limit) return LITEDSA_ERR_UNSUPPORTED;

  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int quads = G * k / 4;
  // small tiles: 256-thread CTAs, several per SM; tiles whose shared memory leaves room for
  // only a few CTAs per SM get 1024 threads each to keep the SM's warp slots filled
  if (smem <= 48 * 1024) {
    const int qpt = (quads + 255) / 256;
    if (qpt <= 1) return launch_union<256, 1>(p, ng, smem, st);
    if (qpt <= 4) return launch_union<256, 4>(p, ng, smem, st);
    if (qpt <= 16) return launch_union<256, 16>(p, ng, smem, st);
    return launch_union<256, 0>(p, ng, smem, st);
  }
  const int qpt = (quads + 1023) / 1024;
  if (qpt <= 2) return launch_union<1024, 2>(p, ng, smem, st);
  if (qpt <= 4) return launch_union<1024, 4>(p, ng, smem, st);
  if (qpt <= 8) return launch_union<1024, 8>(p, ng, smem, st);
  return launch_union<1024, 0>(p, ng, smem, st);
}

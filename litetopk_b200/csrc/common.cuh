// Small hand-written PTX wrappers for sm_100a (mbarrier, TMA, tcgen05, clusters) and
// the error codes shared by every translation unit of the library.  No CUTLASS / CuTe.
//
// These replace the pieces of the reference's vendored helper layer that its kernels
// actually use (kernels/b200/dsa/litedsa_attention_sm100.cuh:405-423 gather4 TMA,
// :645-665 tcgen05 commit/fences, :670-702 and :770-800 TMEM ld/st, :1533-1631 the
// FP8 2-CTA MMA issue) with direct inline PTX.
#pragma once
#include <cuda.h>          // CUtensorMap (type only; the encoder is fetched at run time)
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "../../include/litedsa_b200.h"

namespace lt {

// ---------------------------------------------------------------- host-side helpers (abi.cu)
// A fresh epoch for one kernel launch (never 0; process-wide counter) and the current limit
// of a single device-side wait (default kWaitLimitNs; litedsa_set_wait_limit_ns changes it).
int next_launch_epoch();
unsigned long long wait_limit_ns();

// Arguments of the FP8 attention operator as every entry point of the library passes them
// to the shared checker / launcher (attn_fp8.cu).
struct Fp8Args {
  const void* q8;
  const void* kv8;
  const int32_t* indices;
  float sm_scale, out_scale;
  const int32_t* topk_length;
  const uint32_t* memb_qm;
  int h_per_q;
  float* max_logits;
  float* lse;
  int ng, s_kv, topk;
  int64_t q_row_stride, kv_row_stride, indices_row_stride;
  const float* attn_sink;
  const int32_t* topk_length_per_q;
  int q_group_div;
  // in-place ("zero-copy") addressing of q and out inside [T, H_padded, d] tensors that hold
  // h_per_q real heads per token: strides in ELEMENTS, 0 = the dense packed layout
  int64_t q_token_stride, q_head_stride, out_token_stride, out_head_stride;
};
int check_fp8_args(const Fp8Args& a);                                   // no CUDA call
// attn_dsv4.cu: classify the tiles' index lists and enqueue the range kernel in rank mode, gated on
// "every list is two contiguous runs" (workspace: 16 + 16 * ng bytes; word 0 is the gate)
int dsv4_rank_enqueue(const void* q, const void* kv, const int32_t* indices, const int32_t* pref,
                      const int32_t* win_lo, const int32_t* win_hi, const int32_t* counts,
                      float sm_scale, int h_per_q, void* out, float* lse, const float* attn_sink,
                      int ng, int s_kv, int topk, int d, int64_t q_row_stride, int64_t kv_row_stride,
                      int64_t indices_row_stride, int64_t q_token_stride, int64_t q_head_stride,
                      int64_t out_token_stride, int64_t out_head_stride, void* workspace,
                      cudaStream_t stream);
int run_fp8(const Fp8Args& a, void* const* outs, int n_outs, void* stream);

// ---------------------------------------------------------------- addresses / cluster
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `smem_addr` (a shared::cta address) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;"
               ::: "memory");
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// arrive on a barrier that may live in the peer CTA (shared::cluster address)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// non-blocking probe (try_wait may suspend the thread for a hardware-defined time)
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Every wait in the library goes through here: it gives up after the
// launch's time limit, or as soon as any other wait of the SAME launch gave up (the abort
// word carries that launch's epoch), records where, and returns false.  Callers then fall
// through to their normal tear-down, so a lost arrival costs a wrong result and an error
// status, never a hung GPU.
//
// Status block of a kernel family (ints): [0] first wait site that ever expired since the
// last reset (sticky; 0 = none), [1] its block, [2] its loop iteration, [3] launches
// completed, [4] epoch of the launch that is aborting.  Later launches carry another
// epoch, so one expired wait does not make them give up too.
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // default limit: 2 s
struct Waiter {
  int* status;                  // the family's status block (device global)
  int epoch;                    // this launch's epoch (never 0)
  unsigned long long limit_ns;  // how long one wait may take
  __device__ __forceinline__ bool aborting() const {
    return reinterpret_cast<volatile int*>(status)[4] == epoch;
  }
  // record the first failure (sticky) and make every other wait of this launch give up
  __device__ __forceinline__ void fail(int site, int iter) const {
    if (atomicCAS(status, 0, site) == 0) {
      status[1] = (int)blockIdx.x;
      status[2] = iter;
    }
    atomicExch(status + 4, epoch);
  }
};
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
static __device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, const Waiter w,
                                                   int site, int iter) {
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (w.aborting()) return false;
    if (globaltimer_ns() - t0 > w.limit_ns) {
      w.fail(site, iter);
      return false;
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const Waiter& w, int site,
                                          int iter = 0) {
  for (int i = 0; i < 64; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, w, site, iter);
}

// release at cluster scope: orders this thread's earlier (distributed) shared-memory stores
__device__ __forceinline__ void mbar_arrive_cluster_release(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------- TMA (no multicast anywhere)
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
// tiled 2-D load into this CTA's smem; completion bytes go to `mbar_cluster_addr`, which
// may be the pair leader's barrier (.cta_group::2 form)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst_smem, const CUtensorMap* map, int x,
                                                 int y, uint32_t mbar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes.cta_group::2"
      " [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst_smem), "l"(map), "r"(x), "r"(y), "r"(mbar_cluster_addr)
      : "memory");
}

// tiled 3-D load (x, y, z) into this CTA's smem, completion bytes to a barrier that may be the
// pair leader's (.cta_group::2 form).  Used for Q tiles addressed as (dim, head, token).
__device__ __forceinline__ void tma_load_3d_pair_hint(uint32_t dst_smem, const CUtensorMap* map,
                                                      int x, int y, int z, uint32_t mbar_cluster_addr,
                                                      uint64_t pol) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes.cta_group::2"
      ".L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;"
      ::"r"(dst_smem), "l"(map), "r"(x), "r"(y), "r"(z), "r"(mbar_cluster_addr), "l"(pol)
      : "memory");
}
// tiled 3-D load into this CTA's smem, completion bytes on this CTA's own barrier
__device__ __forceinline__ void tma_load_3d_hint(uint32_t dst_smem, const CUtensorMap* map, int x, int y,
                                                 int z, uint64_t* mbar, uint64_t pol) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;"
      ::"r"(dst_smem), "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(mbar)), "l"(pol)
      : "memory");
}
// tiled 2-D load into this CTA's smem, completion bytes on this CTA's own barrier
__device__ __forceinline__ void tma_load_2d_hint(uint32_t dst_smem, const CUtensorMap* map, int x, int y,
                                                 uint64_t* mbar, uint64_t pol) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
      ::"r"(dst_smem), "l"(map), "r"(x), "r"(y), "r"(smem_u32(mbar)), "l"(pol)
      : "memory");
}
// untiled bulk copy global -> this CTA's shared memory (both addresses 16-byte aligned, size a
// multiple of 16), completion bytes on this CTA's own barrier
__device__ __forceinline__ void bulk_load_1d(uint32_t dst_smem, const void* src, uint32_t bytes,
                                             uint64_t* mbar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(smem_u32(mbar))
      : "memory");
}
// TMA 3-D tile store shared -> global (bulk async-group completion)
__device__ __forceinline__ void tma_store_3d_hint(const void* map, uint32_t src_smem, int x, int y,
                                                  int z, uint64_t pol) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group.L2::cache_hint"
               " [%0, {%2, %3, %4}], [%1], %5;"
               :: "l"(map), "r"(src_smem), "r"(x), "r"(y), "r"(z), "l"(pol) : "memory");
}
__device__ __forceinline__ void tma_store_3d(const void* map, uint32_t src_smem, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               :: "l"(map), "r"(src_smem), "r"(x), "r"(y), "r"(z) : "memory");
}

// TMA tile store shared -> global (bulk async-group completion)
__device__ __forceinline__ void tma_store_2d(const void* map, uint32_t src_smem, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               :: "l"(map), "r"(src_smem), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// all committed bulk groups of this thread have finished READING their shared-memory source
__device__ __forceinline__ void bulk_wait_read_all() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// ... all but the most recent one
__device__ __forceinline__ void bulk_wait_read_1() {
  asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
}
// all committed bulk groups of this thread are complete (writes performed)
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// L2 eviction-priority policies for streaming (read or written once) and resident data
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}

// 16-byte asynchronous global -> shared copy (LSU path, any shared destination), and below the
// asynchronous arrival that fires when all earlier cp.async of the thread have landed (.noinc:
// the arrival counts against the barrier's expected count).  No L2 cache-policy operand on
// purpose: with `.L2::cache_hint` the copy raised "illegal instruction" at its first execution
// in several builds of the attention kernels that differed from a working build only in the
// surrounding code of the gather warps (located with a per-warp progress log in pinned host
// memory); without the operand the same builds run, bit-identical and at the same speed.
__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void tma_store_2d_hint(const void* map, uint32_t src_smem, int x, int y,
                                                  uint64_t pol) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint"
               " [%0, {%2, %3}], [%1], %4;"
               :: "l"(map), "r"(src_smem), "r"(x), "r"(y), "l"(pol) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair_hint(uint32_t dst_smem, const CUtensorMap* map,
                                                      int x, int y, uint32_t mbar_cluster_addr,
                                                      uint64_t pol) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes.cta_group::2"
      ".L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
      ::"r"(dst_smem), "l"(map), "r"(x), "r"(y), "r"(mbar_cluster_addr), "l"(pol)
      : "memory");
}
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---------------------------------------------------------------- TMEM / tcgen05
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(dst_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
// single-CTA (cta_group::1) forms: TMEM allocation, one FP8 MMA with shared-memory operands,
// commit to a barrier of this CTA.  Issued by ONE thread (mma / commit) or one warp (alloc).
__device__ __forceinline__ void tmem_alloc_cta(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(dst_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_cta() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_cta(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void mma_f8_cta(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                           uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit_cta(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(smem_u32(bar))
               : "memory");
}
// A whole K-loop of MMAs in one instruction stream, executed by a fully converged warp whose
// elected lane issues (warp-uniform code lets the descriptors live in uniform registers).
// The fewest possible issue slots: the
// issuing thread shares its scheduler with busy warps, and every extra integer instruction per
// MMA costs tensor-pipe time.  Descriptors differ only in their low word (start address >> 4),
// so each step is two 32-bit adds, two register-pair moves and the MMA.
//   QK^T of one 128-key block: 18 steps.  The 512 latent dims of Q sit in TENSOR MEMORY (A
//   operand read from TMEM: lane = row, four e4m3 values per 32-bit column, 8 columns per
//   32-dim step; with 64 rows per CTA the rows are duplicated in lanes 64-127), because with
//   only 64 rows per CTA the shared-memory operand reads of an N = 128 step (A 2 KB + this
//   CTA's half of B for both CTAs 4 KB per ~35 tensor cycles) exceed what shared memory
//   delivers.  K comes from shared memory: four 128-byte-swizzled chunks of 128 dims (step
//   (j,kk): +512*j + 2*kk in 16-byte units) and the compact 64-byte-swizzled rope chunk (two
//   steps at +2048, +2050), whose 64 Q dims also stay in shared memory (a_rope_lo, hi64).
#define LT_QK_TS_STEP(AINC, BINC, PRED)                                        \
  "add.u32 qa, %2, " #AINC ";\n\tadd.u32 blo, %3, " #BINC ";\n\tmov.b64 bd, {blo, %4};\n\t" \
  "@pe tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], [qa], bd, %1, " #PRED ";\n\t"
#define LT_QK_SS_STEP(INC, PRED)                                               \
  "add.u32 alo, %6, " #INC ";\n\tadd.u32 blo, %3, 2048 + " #INC ";\n\t"           \
  "mov.b64 ad, {alo, %5};\n\tmov.b64 bd, {blo, %5};\n\t"                       \
  "@pe tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], ad, bd, %1, " #PRED ";\n\t"
__device__ __forceinline__ void mma_f8_pair_qk18(uint32_t d_tmem, uint32_t idesc, uint32_t q_tmem,
                                                 uint32_t b_lo, uint32_t hi128, uint32_t hi64,
                                                 uint32_t a_rope_lo) {
  asm volatile(
      "{\n\t.reg .pred pz, po, pe;\n\t.reg .b32 qa, alo, blo;\n\t.reg .b64 ad, bd;\n\t"
      "setp.ne.b32 pz, 0, 0;\n\tsetp.eq.b32 po, 0, 0;\n\telect.sync _|pe, 0xffffffff;\n\t"
      LT_QK_TS_STEP(0, 0, pz) LT_QK_TS_STEP(8, 2, po) LT_QK_TS_STEP(16, 4, po) LT_QK_TS_STEP(24, 6, po)
      LT_QK_TS_STEP(32, 512, po) LT_QK_TS_STEP(40, 514, po) LT_QK_TS_STEP(48, 516, po) LT_QK_TS_STEP(56, 518, po)
      LT_QK_TS_STEP(64, 1024, po) LT_QK_TS_STEP(72, 1026, po) LT_QK_TS_STEP(80, 1028, po) LT_QK_TS_STEP(88, 1030, po)
      LT_QK_TS_STEP(96, 1536, po) LT_QK_TS_STEP(104, 1538, po) LT_QK_TS_STEP(112, 1540, po) LT_QK_TS_STEP(120, 1542, po)
      LT_QK_SS_STEP(0, po) LT_QK_SS_STEP(2, po)
      "}"
      ::"r"(d_tmem), "r"(idesc), "r"(q_tmem), "r"(b_lo), "r"(hi128), "r"(hi64), "r"(a_rope_lo)
      : "memory");
}
//   P V of one 128-key block: two N = 256 halves (D column offset 128, V chunk +1024) x four
//   32-key steps (P +128, V +256 per step); `first` = 0 zeroes the accumulator in step 0
#define LT_PV_STEP(DOFF, AINC, BINC, PRED)                              \
  "add.u32 dd, %0, " #DOFF ";\n\tadd.u32 alo, %2, " #AINC ";\n\tadd.u32 blo, %3, " #BINC ";\n\t" \
  "mov.b64 ad, {alo, %4};\n\tmov.b64 bd, {blo, %5};\n\t"                  \
  "@pe tcgen05.mma.cta_group::2.kind::f8f6f4 [dd], ad, bd, %1, " #PRED ";\n\t"
__device__ __forceinline__ void mma_f8_pair_pv8(uint32_t d_tmem, uint32_t idesc, uint32_t a_lo,
                                                uint32_t b_lo, uint32_t a_hi, uint32_t b_hi,
                                                uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred pf, po, pe;\n\t.reg .b32 alo, blo, dd;\n\t.reg .b64 ad, bd;\n\t"
      "setp.ne.b32 pf, %6, 0;\n\tsetp.eq.b32 po, 0, 0;\n\telect.sync _|pe, 0xffffffff;\n\t"
      LT_PV_STEP(0, 0, 0, pf) LT_PV_STEP(0, 128, 256, po) LT_PV_STEP(0, 256, 512, po)
      LT_PV_STEP(0, 384, 768, po)
      LT_PV_STEP(128, 0, 1024, pf) LT_PV_STEP(128, 128, 1280, po) LT_PV_STEP(128, 256, 1536, po)
      LT_PV_STEP(128, 384, 1792, po)
      "}"
      ::"r"(d_tmem), "r"(idesc), "r"(a_lo), "r"(b_lo), "r"(a_hi), "r"(b_hi), "r"(accumulate_first)
      : "memory");
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp gets lane (base_lane + i)
// the same, issued by one elected lane of a fully converged warp (keeps the caller warp-uniform)
__device__ __forceinline__ void mma_commit_pair_elect(uint32_t cluster_addr) {
  asm volatile(
      "{\n\t.reg .pred pe;\n\telect.sync _|pe, 0xffffffff;\n\t"
      "@pe tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
      ::"r"(cluster_addr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* v) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
        "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]),
        "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- UMMA descriptors
// Shared-memory matrix descriptor (sm_100 format, version field = 1):
//   [0,14) start address >> 4, [16,30) leading byte offset >> 4, [32,46) stride byte offset >> 4,
//   [46,48) = 1, [61,64) swizzle: 0 none, 2 = 128 B, 4 = 64 B, 6 = 32 B.
enum : uint32_t { kSwzNone = 0, kSwz128 = 2, kSwz64 = 4, kSwz32 = 6 };
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                              uint32_t sbo_bytes, uint32_t swizzle) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)swizzle << 61;
  return d;
}
// Instruction descriptor for kind::f8f6f4 / kind::f16 with fp32 accumulation:
//   [4,6) D format (1 = f32), [7,10) A format, [10,13) B format, [15] A MN-major, [16] B MN-major,
//   [17,23) N >> 3, [24,29) M >> 4.   Formats: f8f6f4: 0 = e4m3;  f16: 0 = f16, 1 = bf16.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t a_fmt, uint32_t b_fmt, bool a_mn,
                                                  bool b_mn, uint32_t M, uint32_t N) {
  return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | ((a_mn ? 1u : 0u) << 15) |
         ((b_mn ? 1u : 0u) << 16) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

}  // namespace lt

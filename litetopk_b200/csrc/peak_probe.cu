// Measurement aid: the dense tcgen05 tensor-core rate of this GPU for the MMA kinds and tile
// shapes the attention kernels use, measured with a kernel that does nothing but issue MMAs
// from shared memory.  The roofline denominators of the benchmark come from here where no
// measured figure exists otherwise (FP8 dense).  No counterpart in the reference.
//
// One cluster of 2 CTAs per SM pair; one elected lane of the leader CTA issues `iters`
// back-to-back tcgen05.mma.cta_group::2 instructions (N = 256, K = 32 bytes of e4m3 or 16 bf16
// per step) whose operands sit in shared memory (random non-NaN bytes), alternating between two
// TMEM accumulators, then commits and waits (bounded) for completion.  M is 256 per pair (128
// rows per CTA: the shape that reaches the pipe's peak) or 128 per pair (64 rows per CTA: the
// attention kernels' shape, forced by d_v = 512 columns of O per row in 512 TMEM columns).
#include "common.cuh"

namespace lt {
namespace probe {

constexpr int kThreads = 128;
constexpr uint32_t kABytes = 128 * 128;      // up to 128 rows x 128 bytes (one SW128 chunk)
constexpr uint32_t kBBytes = 128 * 128;      // this CTA's half of N = 256: 128 rows x 128 bytes
constexpr uint32_t kSmem = kABytes + kBBytes + 1024;

__device__ int g_status[8];

template <bool kF8>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
mma_rate_kernel(int iters, int m_pair, int epoch, unsigned long long limit_ns) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint32_t* sm = reinterpret_cast<uint32_t*>(smem_raw + (sbase - raw));
  const Waiter wt{g_status, epoch, limit_ns};
  // operand bytes: pseudo-random, exponent never all ones (no NaN / inf in e4m3 or bf16)
  for (uint32_t i = threadIdx.x; i < (kABytes + kBBytes) / 4; i += kThreads)
    sm[i] = ((i + 977u * blockIdx.x) * 2654435761u) & (kF8 ? 0x37373737u : 0x3f7f3f7fu);
  const uint32_t cta = cluster_ctarank();
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_mbar_init();
  }
  fence_proxy_async_smem();
  __syncthreads();
  cluster_sync_all();
  if (warp == 0) {
    tmem_alloc_pair(&tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  cluster_sync_all();
  if (cta == 0 && warp == 0) {
    const uint32_t idesc = umma_idesc(kF8 ? 0 : 1, kF8 ? 0 : 1, false, false, (uint32_t)m_pair, 256);
    const uint64_t ad = umma_desc(sbase, 16, 1024, kSwz128);
    const uint64_t bd = umma_desc(sbase + kABytes, 16, 1024, kSwz128);
    for (int it = 0; it < iters; ++it) {
      // four K-steps inside the 128-byte chunk, two accumulators of 256 columns
      const uint64_t step = (uint64_t)((it & 3) * 2);
      const uint32_t d = tmem + ((it >> 2) & 1) * 256;
      if (kF8) {
        asm volatile(
            "{\n\t.reg .pred p, pe;\n\tsetp.ne.b32 p, %4, 0;\n\telect.sync _|pe, 0xffffffff;\n\t"
            "@pe tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d), "l"(ad + step), "l"(bd + step), "r"(idesc), "r"(it >= 8 ? 1u : 0u) : "memory");
      } else {
        asm volatile(
            "{\n\t.reg .pred p, pe;\n\tsetp.ne.b32 p, %4, 0;\n\telect.sync _|pe, 0xffffffff;\n\t"
            "@pe tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d), "l"(ad + step), "l"(bd + step), "r"(idesc), "r"(it >= 8 ? 1u : 0u) : "memory");
      }
    }
    mma_commit_pair_elect(smem_u32(&bar));
    mbar_wait(&bar, 0, wt, 301, iters);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 0) tmem_dealloc_pair(tmem, 512);
}

}  // namespace probe
}  // namespace lt

// Dense MMA rate of the current device in TFLOP/s (synchronous; a few milliseconds).
//   kind: 0 = FP8 e4m3 (kind::f8f6f4, K = 32 per instruction), 1 = bf16 (kind::f16, K = 16)
//   m_pair: 256 (128 rows per CTA of the pair) or 128 (64 rows per CTA)
//   iters: MMAs issued per CTA pair (multiple of 8, >= 64)
// *tflops_out (host) = clusters x iters x 2 x m_pair x 256 x K / time.  Every SM pair runs one
// cluster, so this is a whole-GPU figure under the power and clock conditions of the moment.
extern "C" int litedsa_probe_mma_tflops(int kind, int m_pair, int iters, double* tflops_out) {
  using namespace lt;
  using namespace lt::probe;
  if (!tflops_out) return LITEDSA_ERR_ARG;
  if ((kind != 0 && kind != 1) || (m_pair != 128 && m_pair != 256) || iters < 64 || iters % 8)
    return LITEDSA_ERR_SHAPE;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) != cudaSuccess) return LITEDSA_ERR_CUDA;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int clusters = sms / 2;
  auto kern = kind == 0 ? mma_rate_kernel<true> : mma_rate_kernel<false>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem) != cudaSuccess)
    return LITEDSA_ERR_CUDA;
  cudaEvent_t e0, e1;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return LITEDSA_ERR_CUDA;
  float best = 1e30f;
  for (int rep = 0; rep < 4; ++rep) {     // first repetition warms up; best of the rest
    cudaEventRecord(e0, 0);
    kern<<<2 * clusters, kThreads, kSmem, 0>>>(iters, m_pair, next_launch_epoch(), wait_limit_ns());
    cudaEventRecord(e1, 0);
    if (cudaEventSynchronize(e1) != cudaSuccess) { best = -1.f; break; }
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    if (rep > 0 && ms < best) best = ms;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (cudaGetLastError() != cudaSuccess || best <= 0.f) return LITEDSA_ERR_CUDA;
  int st[4] = {0, 0, 0, 0};
  cudaMemcpyFromSymbol(st, g_status, sizeof(st));
  if (st[0] != 0) return LITEDSA_ERR_TIMEOUT;
  const double flop = (double)clusters * iters * 2.0 * m_pair * 256.0 * (kind == 0 ? 32.0 : 16.0);
  *tflops_out = flop / (best * 1e-3) / 1e12;
  return LITEDSA_OK;
}

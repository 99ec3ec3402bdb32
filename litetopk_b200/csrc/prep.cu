// Operand preparation for the FP8 attention path (HBM-bound element-wise kernels).
//
// The reference module consumes q as e4m3 [ng,128,576] and a 576-byte all-e4m3 KV row
// with ONE scalar scale (kernels/b200/dsa/litedsa.cu:82-92,
// kernels/b200/dsa/litedsa_attention_sm100.cuh:2125-2133).  Callers that hold bf16
// queries, or a DeepSeek-V3.2 style packed cache row (512 e4m3 codes | 4 fp32 scales |
// 64 bf16 rope = 656 bytes), convert with the two kernels below.
#include "common.cuh"

namespace lt {

// out[i] = e4m3_satfinite(in[i] * inv_scale), 8 elements per thread (16-byte loads)
__global__ void __launch_bounds__(256) quantize_e4m3_kernel(const uint4* __restrict__ in,
                                                             uint2* __restrict__ out, size_t n8,
                                                             float inv_scale) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
    const uint4 v = __ldg(in + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&w[2 * j]);
      const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&w[2 * j + 1]);
      float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
      fa.x *= inv_scale; fa.y *= inv_scale; fb.x *= inv_scale; fb.y *= inv_scale;
      const uint32_t lo = __nv_cvt_float2_to_fp8x2(fa, __NV_SATFINITE, __NV_E4M3);
      const uint32_t hi = __nv_cvt_float2_to_fp8x2(fb, __NV_SATFINITE, __NV_E4M3);
      o[j] = lo | (hi << 16);
    }
    out[i] = make_uint2(o[0], o[1]);
  }
}

// One warp per cache row: copy the 512 latent codes, re-encode the bf16 rope part as
// e4m3(rope / scale), and flag rows whose four per-128 scales are not all == scale
// (such a cache cannot be expressed with one scalar scale without requantising).
__global__ void __launch_bounds__(256) repack_kv656_kernel(const uint8_t* __restrict__ in,
                                                            uint8_t* __restrict__ out, int s_kv,
                                                            long long out_pitch, float scale,
                                                            int* __restrict__ mismatch) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const float inv = 1.0f / scale;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < s_kv;
       row += gridDim.x * warps_per_block) {
    const uint8_t* src = in + (size_t)row * 656;
    uint8_t* dst = out + (size_t)row * out_pitch;
    // 656 = 41 x 16 bytes: lanes 0..31 move the 512 code bytes
    reinterpret_cast<uint4*>(dst)[lane] = __ldg(reinterpret_cast<const uint4*>(src) + lane);
    if (lane < 4) {
      const float sc = __ldg(reinterpret_cast<const float*>(src + 512) + lane);
      if (sc != scale) atomicOr(mismatch, 1);
    }
    // rope: 64 bf16 -> 64 e4m3, 2 per lane
    const __nv_bfloat162 r2 = __ldg(reinterpret_cast<const __nv_bfloat162*>(src + 528) + lane);
    float2 f = __bfloat1622float2(r2);
    f.x *= inv; f.y *= inv;
    const uint16_t q = __nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3);
    reinterpret_cast<uint16_t*>(dst + 512)[lane] = q;
  }
}

// KV-split merge: the outputs of q_group_div consecutive tiles that share one Q tile (slices of
// one long union list) are combined with their lse into the attention over the whole list.
// One warp per merged row; lane j holds part j's lse, lane i the dims [8i, 8i + 8) and
// [256 + 8i, 256 + 8i + 8) of the row (two fully coalesced 512-byte requests per part).
// Part j of row (t, r) weighs (e^lse_j + e^sink_r) / (sum_k e^lse_k + e^sink_r): the kernels
// normalise a part by its own row sum plus the sink, while lse never contains the sink.
__global__ void __launch_bounds__(256) merge_kv_splits_kernel(
    const uint4* __restrict__ out_parts, const float* __restrict__ lse_parts,
    const float* __restrict__ max_parts, const float* __restrict__ sink, uint4* __restrict__ out,
    float* __restrict__ lse, float* __restrict__ max_logits, int n_rows, int div) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < n_rows; row += warps) {
    const int t = row >> 7, r = row & 127;
    const size_t prow0 = ((size_t)t * div) * 128 + r;          // part j: prow0 + 128 j
    float lj = -INFINITY, mj = -INFINITY;
    if (lane < div) {
      const float v = __ldcs(lse_parts + prow0 + (size_t)lane * 128);
      lj = (v == INFINITY || v != v) ? -INFINITY : v;          // +inf marks a part without keys
      if (max_parts) mj = __ldcs(max_parts + prow0 + (size_t)lane * 128);
    }
    float m = lj;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
      mj = fmaxf(mj, __shfl_xor_sync(0xffffffffu, mj, off));
    }
    const float e = lj == -INFINITY ? 0.f : __expf(lj - m);
    float sum = e;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    const float es = (sink && m != -INFINITY) ? __expf(__ldg(sink + r) - m) : 0.f;
    const float w = e > 0.f ? __fdividef(e + es, sum + es) : 0.f;
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    for (int j = 0; j < div; ++j) {
      const float wj = __shfl_sync(0xffffffffu, w, j);
      if (wj == 0.f) continue;                                  // warp-uniform
      const uint4* src = out_parts + (prow0 + (size_t)j * 128) * 64;
      const uint4 a = __ldcs(src + lane), b = __ldcs(src + 32 + lane);
      const uint32_t u[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u[i]));
        acc[2 * i] = fmaf(wj, f.x, acc[2 * i]);
        acc[2 * i + 1] = fmaf(wj, f.y, acc[2 * i + 1]);
      }
    }
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const __nv_bfloat162 v = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      o[i] = *reinterpret_cast<const uint32_t*>(&v);
    }
    uint4* dst = out + (size_t)row * 64;
    __stcs(dst + lane, make_uint4(o[0], o[1], o[2], o[3]));
    __stcs(dst + 32 + lane, make_uint4(o[4], o[5], o[6], o[7]));
    if (lane == 0) {
      lse[row] = m == -INFINITY ? INFINITY : m + __logf(sum);
      if (max_logits) max_logits[row] = mj;
    }
  }
}

}  // namespace lt

// bf16 -> e4m3 with a scalar scale: out = e4m3(in / scale).  n must be a multiple of 8 and
// both pointers 16-byte aligned.  No counterpart in the reference (its callers hand it e4m3 q).
extern "C" int litedsa_quantize_e4m3(const void* in_bf16, void* out_e4m3, int64_t n, float scale,
                                     void* stream) {
  using namespace lt;
  if (!in_bf16 || !out_e4m3) return LITEDSA_ERR_ARG;
  if (n <= 0 || n % 8 || !(scale > 0.f)) return LITEDSA_ERR_SHAPE;
  if (((uintptr_t)in_bf16 | (uintptr_t)out_e4m3) & 15) return LITEDSA_ERR_UNSUPPORTED;
  const size_t n8 = (size_t)n / 8;
  const int blocks = (int)min((size_t)148 * 8, (n8 + 255) / 256);
  quantize_e4m3_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(in_bf16), reinterpret_cast<uint2*>(out_e4m3), n8, 1.0f / scale);
  return cudaGetLastError() == cudaSuccess ? LITEDSA_OK : LITEDSA_ERR_CUDA;
}

// Packed 656-byte cache rows -> 576-byte all-e4m3 rows sharing the scalar `scale`.
// *mismatch_flag (device int, caller zeroes it) becomes non-zero if any per-128 scale of
// the source differs from `scale`.  out_pitch = bytes between output rows (>= 576, % 16 == 0).
extern "C" int litedsa_repack_kv656(const void* kv656, void* kv576, int s_kv, int64_t out_pitch,
                                    float scale, int* mismatch_flag, void* stream) {
  using namespace lt;
  if (!kv656 || !kv576 || !mismatch_flag) return LITEDSA_ERR_ARG;
  if (s_kv <= 0 || out_pitch < 576 || out_pitch % 16 || !(scale > 0.f)) return LITEDSA_ERR_SHAPE;
  if (((uintptr_t)kv656 | (uintptr_t)kv576) & 15) return LITEDSA_ERR_UNSUPPORTED;
  const int blocks = min(148 * 8, (s_kv + 7) / 8);
  repack_kv656_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint8_t*>(kv656), reinterpret_cast<uint8_t*>(kv576), s_kv, out_pitch,
      scale, mismatch_flag);
  return cudaGetLastError() == cudaSuccess ? LITEDSA_OK : LITEDSA_ERR_CUDA;
}

// Merge of KV-split outputs (see merge_kv_splits_kernel).  out_parts [ng, 128, 512] bf16 and
// lse_parts [ng, 128] are what litedsa_masked_mla_fp8_ex wrote with q_group_div > 1; out
// [ng / q_group_div, 128, 512] bf16, lse [ng / q_group_div, 128].  max_parts / max_logits and
// attn_sink ([128], natural-log units, the same array the attention call got) are optional.
// The reference leaves this step to its callers (litedsa_attention_sm100.cuh:1383-1385).
extern "C" int litedsa_merge_kv_splits(const void* out_parts, const float* lse_parts,
                                       const float* max_parts, const float* attn_sink, void* out,
                                       float* lse, float* max_logits, int ng, int q_group_div,
                                       void* stream) {
  using namespace lt;
  if (!out_parts || !lse_parts || !out || !lse) return LITEDSA_ERR_ARG;
  if ((max_parts == nullptr) != (max_logits == nullptr)) return LITEDSA_ERR_ARG;
  if (ng <= 0 || q_group_div < 1 || ng % q_group_div) return LITEDSA_ERR_SHAPE;
  if (q_group_div > 32) return LITEDSA_ERR_UNSUPPORTED;
  if (((uintptr_t)out_parts | (uintptr_t)out) & 15) return LITEDSA_ERR_UNSUPPORTED;
  const int n_rows = ng / q_group_div * 128;
  const int blocks = min(148 * 8, (n_rows + 7) / 8);
  merge_kv_splits_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const uint4*>(out_parts), lse_parts, max_parts, attn_sink,
      reinterpret_cast<uint4*>(out), lse, max_logits, n_rows, q_group_div);
  return cudaGetLastError() == cudaSuccess ? LITEDSA_OK : LITEDSA_ERR_CUDA;
}

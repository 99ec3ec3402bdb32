// Allocation-free entry point: masked FP8 MLA prefill straight from DeepSeek-V3.2 style
// packed cache rows (656 bytes), using a scratch buffer that lives inside the library.
//
// Who needs this: hosts that may not call cudaMalloc on the path where attention runs.
// Typical cases are a serving runtime that has handed its whole device memory to its own
// pool (a late cudaMalloc there fails or fragments the pool), a plugin boundary whose
// contract forbids the callee to allocate, and code that runs under a memory budget
// fixed at start-up.  The regular route from packed rows (litedsa_repack_kv656 into a
// caller-allocated 576-byte-row buffer, then litedsa_masked_mla_fp8) needs that temporary
// buffer from somebody; here the library brings its own.
//
// The scratch is a file-scope device array of fixed size: every GPU that loads the
// library holds kScratchBytes (about 36 MiB) until the process exits, and caches longer
// than kNoAllocMaxRows rows are refused.  All calls share it and it keeps the previous
// call's rows, so two calls whose GPU work overlaps (different streams, or different host
// threads) race on it: serialise them.
#include "common.cuh"

#include <mutex>

extern "C" int litedsa_repack_kv656(const void* kv656, void* kv576, int s_kv, int64_t out_pitch,
                                    float scale, int* mismatch_flag, void* stream);

namespace {

constexpr int kNoAllocMaxRows = 65536;            // longest cache this entry point serves
constexpr size_t kFlagBytes = 256;                // slot 0: the scale-mismatch word
constexpr size_t kScratchBytes = kFlagBytes + (size_t)kNoAllocMaxRows * 576;

// In host code this name is only a handle for the runtime, not a device address: kernels
// must be given the pointer cudaGetSymbolAddress returns for the CURRENT device.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
void* g_scratch_ptr[kMaxDevices] = {};

// Device address of the scratch on the current device, looked up once per device.
int scratch_for_current_device(unsigned char** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return LITEDSA_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr)
      return LITEDSA_ERR_CUDA;
    g_scratch_ptr[dev] = p;
  }
  *out = static_cast<unsigned char*>(g_scratch_ptr[dev]);
  return LITEDSA_OK;
}

}  // namespace

// See include/litedsa_b200.h.  Calls no cudaMalloc / cudaFree and no allocating library
// routine: one cudaMemsetAsync (the mismatch word must start at zero), the repack kernel
// into the built-in scratch, then the attention kernel reading the scratch.  Every argument
// rule is checked before the scratch is touched or anything is enqueued.
extern "C" int litedsa_masked_mla_fp8_kv656_noalloc(
    const void* q8, const void* kv656, const int32_t* indices, float sm_scale, float kv_scale,
    const int32_t* topk_length, const uint32_t* memb_qm, int h_per_q, void* out, float* max_logits,
    float* lse, int ng, int s_kv, int topk, int64_t q_row_stride, int64_t indices_row_stride,
    int* mismatch_flag, void* stream) {
  if (!kv656 || !memb_qm || !out) return LITEDSA_ERR_ARG;
  if (((uintptr_t)kv656 | (uintptr_t)out) & 15) return LITEDSA_ERR_UNSUPPORTED;
  if (!(kv_scale > 0.f)) return LITEDSA_ERR_SHAPE;
  // the operator's own rules, with the scratch rows standing in for kv8 (576-byte pitch)
  lt::Fp8Args a{q8, kv656, indices, sm_scale, kv_scale, topk_length, memb_qm, h_per_q, max_logits,
                lse, ng, s_kv, topk, q_row_stride, 576, indices_row_stride, nullptr, nullptr, 1};
  int rc = lt::check_fp8_args(a);
  if (rc != LITEDSA_OK) return rc;
  if (s_kv > kNoAllocMaxRows) return LITEDSA_ERR_UNSUPPORTED;   // beyond the built-in scratch
  unsigned char* scratch = nullptr;
  rc = scratch_for_current_device(&scratch);
  if (rc != LITEDSA_OK) return rc;
  int* flag = mismatch_flag ? mismatch_flag : reinterpret_cast<int*>(scratch);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(flag, 0, sizeof(int), st) != cudaSuccess) return LITEDSA_ERR_CUDA;
  unsigned char* rows = scratch + kFlagBytes;
  rc = litedsa_repack_kv656(kv656, rows, s_kv, 576, kv_scale, flag, stream);
  if (rc != LITEDSA_OK) return rc;
  a.kv8 = rows;
  void* outs[1] = {out};
  return lt::run_fp8(a, outs, 1, stream);
}

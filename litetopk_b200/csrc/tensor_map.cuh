// Host-side construction of TMA tensor maps without linking libcuda: the encoder is
// looked up through the runtime (cudaGetDriverEntryPoint).  The reference builds the
// same kind of 2-D byte-typed maps over its KV cache with cuTensorMapEncodeTiled
// (kernels/b200/dsa/litedsa_attention_sm100.cuh:2538-2573).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lt {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) !=
            cudaSuccess || qr != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// 2-D row-major tensor [rows, cols] of `elem_bytes`-wide elements, row pitch in bytes,
// box = box_cols x box_rows, 128-byte swizzle unless told otherwise, out-of-bounds elements
// read as zero (and are not written by stores).
inline bool make_map_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype,
                        uint64_t cols, uint64_t rows, uint64_t pitch_bytes, uint32_t box_cols,
                        uint32_t box_rows,
                        CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t size[2] = {cols, rows};
  cuuint64_t stride[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, dtype, 2, const_cast<void*>(base), size, stride, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 3-D tensor [tokens, heads, cols] (cols innermost, unit stride) of `elem_bytes`-wide elements:
// heads `head_pitch_bytes` apart, tokens `token_pitch_bytes` apart; box = box_cols x box_heads x
// box_tokens.  This is how a 128-row attention tile is addressed in place: its row r is
// (token r / h, head r % h) of a [T, H_padded, d] tensor that holds only h real heads per
// token -- the layout a tensor-parallel model hands over
// (kernels/b200/dsa/DSV4_ZEROCOPY_PLAN.md:12-22) -- and equally of the dense packed layout.
inline bool make_map_3d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype,
                        uint64_t cols, uint64_t heads, uint64_t tokens, uint64_t head_pitch_bytes,
                        uint64_t token_pitch_bytes, uint32_t box_cols, uint32_t box_heads,
                        uint32_t box_tokens,
                        CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t size[3] = {cols, heads, tokens};
  cuuint64_t stride[2] = {head_pitch_bytes, token_pitch_bytes};
  cuuint32_t box[3] = {box_cols, box_heads, box_tokens};
  cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, dtype, 3, const_cast<void*>(base), size, stride, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace lt

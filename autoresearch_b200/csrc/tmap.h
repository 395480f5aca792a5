// Host-side construction of TMA tensor maps for [B, T, H, D] bf16 tensors.
// cuTensorMapEncodeTiled is fetched through the runtime's driver-entry-point query so
// the library does not link libcuda directly (it must load on a machine without a driver).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ar {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Map over a [B, T, H, D] bf16 tensor with dimensions ordered (d, h, t, b): heads of one token
// adjacent, token t at t * pitch_t rows of D elements, batch b at b * pitch_b rows (contiguous:
// pitch_t = H, pitch_b = T * H; 0 selects that).  One box is 64 elements of d (128 bytes, the
// swizzle span) by `box_rows` consecutive t of one head of one batch.  Rows past T read as zero.
inline bool make_tmap_bthd(CUtensorMap* map, const void* base, int64_t B, int64_t T, int64_t H,
                           int64_t D, int box_rows, int64_t pitch_t = 0, int64_t pitch_b = 0) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  if (pitch_t == 0) pitch_t = H;
  if (pitch_b == 0) pitch_b = T * pitch_t;
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)T, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)(D * 2), (cuuint64_t)(pitch_t * D * 2),
                           (cuuint64_t)(pitch_b * D * 2)};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace ar

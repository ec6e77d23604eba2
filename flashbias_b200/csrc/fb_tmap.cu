// TMA tensor-map construction.  cuTensorMapEncodeTiled is looked up through the runtime so the
// library links against cudart only.
#include <mutex>

#include "fb_common.cuh"
#include "fb_internal.h"

namespace fb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
  });
  return fn;
}

bool tma_compatible(const void* ptr, int64_t stride_row, int64_t stride_head, int64_t stride_batch, int64_t heads,
                    int64_t batch) {
  // 16-bit elements: base 16-byte aligned, every stride a multiple of 8 elements (16 bytes)
  if (reinterpret_cast<uintptr_t>(ptr) & 15) return false;
  if (stride_row <= 0 || (stride_row & 7)) return false;
  if (heads > 1 && (stride_head <= 0 || (stride_head & 7))) return false;
  if (batch > 1 && (stride_batch <= 0 || (stride_batch & 7))) return false;
  return true;
}

int make_tmap_4d(CUtensorMap* out, const void* ptr, int cols, int64_t rows, int64_t heads, int64_t batch,
                 int64_t stride_row, int64_t stride_head, int64_t stride_batch, int box_cols, int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return FB_ENOTBUILT;
  // A dimension of extent 1 never advances; give it any legal stride.
  if (heads <= 1) stride_head = stride_row * rows;
  if (batch <= 1) stride_batch = stride_head * (heads > 1 ? heads : 1);
  cuuint64_t dims[4] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)(heads > 0 ? heads : 1),
                        (cuuint64_t)(batch > 0 ? batch : 1)};
  cuuint64_t strides[3] = {(cuuint64_t)stride_row * 2, (cuuint64_t)stride_head * 2, (cuuint64_t)stride_batch * 2};
  cuuint32_t box[4] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  const int swb = swizzle_bytes(box_cols);
  CUtensorMapSwizzle sw = swb == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                          : swb == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                          : swb == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                      : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : FB_EINVAL_STRIDE;
}

}  // namespace fb

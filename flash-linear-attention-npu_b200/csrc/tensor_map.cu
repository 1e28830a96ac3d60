#include "tensor_map.h"

#include <mutex>

namespace fla {

namespace {
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;
std::once_flag g_once;

void resolve() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult st;
  if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000, cudaEnableDefault, &st) == cudaSuccess &&
      st == cudaDriverEntryPointSuccess)
    g_encode = reinterpret_cast<EncodeFn>(fn);
}
}  // namespace

static int encode(CUtensorMap* map, CUtensorMapDataType dt, uint64_t esz, uint32_t box_cols, const void* base, uint64_t cols,
                  uint64_t heads, uint64_t rows, uint64_t head_stride, uint64_t row_stride) {
  std::call_once(g_once, resolve);
  if (!g_encode) return 6;
  const cuuint64_t dims[3] = {cols, heads, rows};
  const cuuint64_t strides[2] = {head_stride * esz, row_stride * esz};   // bytes, dims 1 and 2
  const cuuint32_t box[3] = {box_cols, 1, 64};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = g_encode(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 6;
}

int make_bhtd_tile_map(CUtensorMap* map, const void* base, int elem_bytes, uint64_t D, uint64_t T, uint64_t H, uint64_t B,
                       uint64_t st, uint64_t sh, uint64_t sb, uint32_t box_cols, uint32_t box_rows) {
  std::call_once(g_once, resolve);
  if (!g_encode) return 6;
  const uint64_t esz = uint64_t(elem_bytes);
  // a dimension of extent 1 is only ever addressed at coordinate 0: give it a stride the encoder accepts
  if (T == 1) st = D;
  if (H == 1) sh = st * T;
  if (B == 1) sb = sh * H;
  const cuuint64_t dims[4] = {D, T, H, B};
  const cuuint64_t strides[3] = {st * esz, sh * esz, sb * esz};
  const cuuint32_t box[4] = {box_cols, box_rows, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const CUresult r = g_encode(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 6;
}

int make_row_tile_map(CUtensorMap* map, const void* base, uint64_t cols, uint64_t heads, uint64_t rows,
                      uint64_t head_stride, uint64_t row_stride) {
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 64, base, cols, heads, rows, head_stride, row_stride);
}

int make_row_tile_map_f32(CUtensorMap* map, const void* base, uint64_t cols, uint64_t heads, uint64_t rows,
                          uint64_t head_stride, uint64_t row_stride) {
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, 32, base, cols, heads, rows, head_stride, row_stride);
}

}  // namespace fla

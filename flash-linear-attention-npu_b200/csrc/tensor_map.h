// Host-side construction of TMA tensor maps (cuTensorMapEncodeTiled through the runtime's driver entry point, so the
// library does not link against libcuda) and the device-side tiled bulk load that consumes them.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace fla {

// bf16 tensor viewed as [rows][heads][cols] (cols contiguous; strides in elements): boxes of 64 rows x 1 head x 64
// columns, written to shared memory in the 128-byte-swizzled panel layout the MMA descriptors expect.
// Returns 0, or 6 (FLA_ERR_CUDA) when the driver refuses the map.
int make_row_tile_map(CUtensorMap* map, const void* base, uint64_t cols, uint64_t heads, uint64_t rows,
                      uint64_t head_stride, uint64_t row_stride);

// fp32 tensor viewed as [rows][heads][cols]: boxes of 64 rows x 1 head x 32 columns (128 bytes), same swizzle.
int make_row_tile_map_f32(CUtensorMap* map, const void* base, uint64_t cols, uint64_t heads, uint64_t rows,
                          uint64_t head_stride, uint64_t row_stride);

// Tensor addressed as [B, H, T, D] through element strides (D contiguous): boxes of box_rows tokens x box_cols columns
// (box_cols * elem_bytes == 128) of one (b, h), same swizzle.  Tokens past T read as zero.
int make_bhtd_tile_map(CUtensorMap* map, const void* base, int elem_bytes, uint64_t D, uint64_t T, uint64_t H, uint64_t B,
                       uint64_t st, uint64_t sh, uint64_t sb, uint32_t box_cols, uint32_t box_rows);

#ifdef __CUDACC__
// One box of a make_bhtd_tile_map tensor at (col0, t0, h, b); col0 * elem_bytes must be a multiple of 16.
__device__ __forceinline__ void tma_load_tile4(uint32_t smem_dst, const CUtensorMap* map, int col0, int t0, int h, int b,
                                               uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_dst), "l"(map), "r"(static_cast<uint32_t>(__cvta_generic_to_shared(bar))), "r"(col0), "r"(t0), "r"(h), "r"(b)
      : "memory");
}
// One 64 x 64 bf16 box (8 KB) at (col0, head, row0) -> shared memory; completes `bytes` on the mbarrier.
// col0 must be a multiple of 8 elements (16 bytes); rows past the tensor's end read as zero.  No multicast.
__device__ __forceinline__ void tma_load_tile(uint32_t smem_dst, const CUtensorMap* map, int col0, int head, int row0,
                                              uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_dst), "l"(map), "r"(static_cast<uint32_t>(__cvta_generic_to_shared(bar))), "r"(col0), "r"(head), "r"(row0)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
#endif

}  // namespace fla

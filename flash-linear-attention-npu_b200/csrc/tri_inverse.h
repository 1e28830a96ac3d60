// Launcher of the shared 64x64 unit-lower-triangular inverse kernel (tri_inverse.cu).
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace fla {

struct TriInverseParams {
  const float* at;              // [chunks * HV][64][64]: A^T row-major (at[j][i] = A[i][j], j < i), fp32
  __nv_bfloat16* x_rows;        // optional out: [tokens, HV, 64] row i of the chunk's inverse at its token
  __nv_bfloat16* x_strips;      // optional out: per (chunk, head) [value | residual] x [8 strips of 8 rows][64 columns][8 row entries =
                                // 16 bytes] (un-swizzled strip layout, 16 KB), rows past the end of the sequence as zeros
  __nv_bfloat16* x_img;         // optional out: swizzled 64 x 64 operand panel per (chunk, head), `img_stride` elements apart
  __nv_bfloat16* x_img_lo;      // optional out: bf16 residual of x_img (same stride)
  const int32_t* cu_seqlens;    // sequence geometry, as in the chunk kernels
  const int32_t* chunk_offsets;
  int T, HV;
  int img_stride;               // elements between the panels of consecutive (chunk, head) pairs; 0 means 64 * 64
};

// Returns 0 or FLA_ERR_CUDA (6).
int launch_tri_inverse(const TriInverseParams& p, int nt_max, int N, cudaStream_t stream);

}  // namespace fla

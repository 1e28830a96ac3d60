// Inverse of 64x64 unit lower-triangular matrices  X = (I + A)^-1,  A strictly lower triangular, fp32.
// Shared by the GDN and KDA chunk kernels (the reference's solve_tri operator,
// fla/ops/ascendc/gdn/chunk_gdn_fwd/solve_tri/README.md:9-13, which inverts in bf16 on the matrix unit;
// here the inverse is built in fp32 and rounded to bf16 once at the end).
// One CTA handles two matrices (64 threads each; small CTAs under a register bound of 96 keep ten solves in flight per SM: 0.198 -> 0.184 ms against four per CTA at two CTAs per SM).  Thread c solves column c by right-looking forward
// substitution:  r = e_c;  for j: x_j = r_j;  r_i -= A[i][j] x_j (i > j).  The updates of one step are
// independent, so the FMA pipeline stays full, and a warp skips the steps before its first column
// because the entries above a column's diagonal are zero.
#include "gdn_common.cuh"
#include "tri_inverse.h"
#include <atomic>

namespace fla {

constexpr int kTriTiles = 2;     // matrices per CTA (64 threads each)
constexpr int kTriStride = 68;   // fp32 row stride of A^T in shared memory (16-byte aligned rows, spread banks)

__global__ void __launch_bounds__(64 * kTriTiles, 5) tri_inverse_kernel(TriInverseParams p) {
  extern __shared__ float tri_smem[];
  const int tid = threadIdx.x, grp = tid / 64, c = tid % 64;
  const int n = blockIdx.z;
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  const int chunk = blockIdx.x;
  if (chunk >= sq.nt) return;
  const int hv = blockIdx.y * kTriTiles + grp;
  const bool active = hv < p.HV;
  const int rows = min(kC, sq.len - chunk * kC);
  const int64_t tok0 = int64_t(sq.bos) + chunk * kC;
  const int64_t cidx = (int64_t(sq.cbase) + chunk) * p.HV + hv;
  float* AT = tri_smem + grp * kC * kTriStride;
  if (active) {
    // A^T row-major: src[j * 64 + i] = A[i][j].  16-byte pieces, all of a thread's sixteen requested before the first is
    // stored (one round trip to memory instead of eight), and only the pieces that hold an entry below the diagonal
    // (i > j): the others are neither written by the producer nor read by the solve.
    const float4* src = reinterpret_cast<const float4*>(p.at + cidx * (kC * kC));
    float4 v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int idx = c + i * 64, j = idx >> 4, q4 = idx & 15;
      if (4 * q4 + 3 > j) v[i] = src[idx];
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int idx = c + i * 64, j = idx >> 4, q4 = idx & 15;
      if (4 * q4 + 3 > j) *reinterpret_cast<float4*>(AT + j * kTriStride + 4 * q4) = v[i];
    }
  }
  __syncthreads();
  if (!active) return;
  float x[kC];
#pragma unroll
  for (int i = 0; i < kC; ++i) x[i] = (i == c) ? 1.f : 0.f;
  const int jmin = c & ~31;  // warp-uniform
#pragma unroll
  for (int j = 0; j < kC - 1; ++j) {
    if (j >= jmin) {
      const float xj = x[j];
      const float* col = AT + j * kTriStride;
#pragma unroll
      for (int i4 = (j + 1) & ~3; i4 < kC; i4 += 4) {
        const float4 a4 = *reinterpret_cast<const float4*>(col + i4);
        if (i4 > j) x[i4] -= a4.x * xj;
        if (i4 + 1 > j) x[i4 + 1] -= a4.y * xj;
        if (i4 + 2 > j) x[i4 + 2] -= a4.z * xj;
        if (i4 + 3 > j) x[i4 + 3] -= a4.w * xj;
      }
    }
  }
  if (p.x_rows) {            // token-major rows: X[(tok0 + i), hv, c]
    bf16* xg = p.x_rows + ((tok0 * p.HV + hv) * kC) + c;
#pragma unroll
    for (int i = 0; i < kC; ++i)
      if (i < rows) xg[int64_t(i) * p.HV * kC] = __float2bfloat16_rn(x[i]);
  }
  if (p.x_strips) {          // strips of 8 rows: column c stores its 8 entries of every strip as 16 bytes next to its neighbours'
    uint8_t* img = reinterpret_cast<uint8_t*>(p.x_strips + cidx * 8192) + c * 16;
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      float xs[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) xs[i] = (g * 8 + i < rows) ? x[g * 8 + i] : 0.f;
      uint4 hi, lo;
      split8(xs, hi, lo);
      *reinterpret_cast<uint4*>(img + g * 1024) = hi;
      *reinterpret_cast<uint4*>(img + 8192 + g * 1024) = lo;
    }
  }
  if (p.x_img) {             // swizzled 64x64 operand panel per (chunk, head); rows past the sequence end are zero
    const int64_t stride = p.img_stride ? p.img_stride : kC * kC;
    uint8_t* img = reinterpret_cast<uint8_t*>(p.x_img + cidx * stride);
    uint8_t* img_lo = p.x_img_lo ? reinterpret_cast<uint8_t*>(p.x_img_lo + cidx * stride) : nullptr;
#pragma unroll
    for (int i = 0; i < kC; ++i) {
      const float xv = i < rows ? x[i] : 0.f;
      const bf16 hi = __float2bfloat16_rn(xv);
      *reinterpret_cast<bf16*>(img + panel_off(i, c)) = hi;
      if (img_lo) *reinterpret_cast<bf16*>(img_lo + panel_off(i, c)) = __float2bfloat16_rn(xv - __bfloat162float(hi));
    }
  }
}

int launch_tri_inverse(const TriInverseParams& p, int nt_max, int N, cudaStream_t stream) {
  const int smem = kTriTiles * kC * kTriStride * 4;
  static std::atomic<bool> attr_done_dev[64] = {};   // per device ordinal; setting the attributes twice is harmless
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 6;
  if (!attr_done_dev[dev]) {
    if (cudaFuncSetAttribute(tri_inverse_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return 6;
    attr_done_dev[dev] = true;
  }
  tri_inverse_kernel<<<dim3(nt_max, (p.HV + kTriTiles - 1) / kTriTiles, N), 64 * kTriTiles, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 6;
}

}  // namespace fla

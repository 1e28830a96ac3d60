// Hardware self-test of the tensor-core building blocks in common/sm100.cuh: one CTA stages two
// bf16 tiles in the swizzled panel layout, issues tcgen05.mma over them in the requested
// operand-major combination, and dumps the whole 128-lane TMEM accumulator so the host can check
// both the arithmetic and the accumulator's lane mapping (M = 128: row r -> lane r;
// M = 64: row r -> lane (r % 16) + 32 * (r / 16) + lane offset).
#include "common/sm100.cuh"
#include "fla_b200_internal.h"

namespace fla {

struct SelftestParams {
  const __nv_bfloat16* a;  // a_mn == 0: [M][K] row-major, else [K][M]
  const __nv_bfloat16* b;  // b_mn == 0: [N][K] row-major, else [K][N]
  float* d;                // [128][N] TMEM dump
  int M, N, K, a_mn, b_mn, d_lane_off, prefill;
  int* err;
};

// Copy a row-major [rows][cols] bf16 matrix (cols % 64 == 0) into panels at `dst`.
__device__ void stage_panels(uint8_t* dst, const __nv_bfloat16* src, int rows, int cols) {
  const int chunks_per_row = cols / 8;
  const int total = rows * chunks_per_row;
  for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
    const int r = idx / chunks_per_row, ch = idx % chunks_per_row;
    const uint4 val = *reinterpret_cast<const uint4*>(src + size_t(r) * cols + ch * 8);
    const int panel = ch / 8, c = ch % 8;
    *reinterpret_cast<uint4*>(dst + size_t(panel) * rows * 128 + panel_chunk_off(r, c)) = val;
  }
}

__global__ void __launch_bounds__(128) selftest_mma_kernel(SelftestParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t bar;

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int a_rows = p.a_mn ? p.K : p.M, a_cols = p.a_mn ? p.M : p.K;
  const int b_rows = p.b_mn ? p.K : p.N, b_cols = p.b_mn ? p.N : p.K;
  uint8_t* sa = smem;
  uint8_t* sb = smem + 32768;

  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 256);
    tmem_relinquish();
  }
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_init_fence();
  }
  stage_panels(sa, p.a, a_rows, a_cols);
  stage_panels(sb, p.b, b_rows, b_cols);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = tmem_base_s;

  if (p.prefill) {  // D starts as lane*4 + col/64 pattern written with tcgen05.st, MMA accumulates on top
    for (int c0 = 0; c0 < p.N; c0 += 16) {
      float v[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = float(warp * 32 + lane) + float(c0 + i) * 0.001f;
      tmem_st16(tmem_addr(tbase, warp * 32, c0), v);
    }
    tmem_st_wait();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }

  if (threadIdx.x == 0) {
    Operand A{smem_u32(sa), uint32_t(a_rows) * 128u, p.a_mn};
    Operand B{smem_u32(sb), uint32_t(b_rows) * 128u, p.b_mn};
    mma_tile(tmem_addr(tbase, p.d_lane_off, 0), A, B, p.M, p.N, p.K / 16, p.prefill != 0);
    mma_commit(&bar);
  }
  const bool ok = mbar_wait(&bar, 0, p.err, 1);
  tc_fence_after();
  if (ok) {
    for (int c0 = 0; c0 < p.N; c0 += 16) {
      float v[16];
      tmem_ld16(tmem_addr(tbase, warp * 32, c0), v);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; ++i) p.d[size_t(warp * 32 + lane) * p.N + c0 + i] = v[i];
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 256);
}

// The same product with the A operand read from tensor memory: thread r packs row r of A (bf16 pairs, element 2c in the low
// half of column c) and writes it with tcgen05.st; B is staged in panels as above.  Pins the packing and the column stride
// of a K = 16 step (8 columns) that the transposed scan kernels rely on.
__global__ void __launch_bounds__(128) selftest_mma_ts_kernel(SelftestParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t bar;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int b_rows = p.b_mn ? p.K : p.N, b_cols = p.b_mn ? p.N : p.K;
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_init_fence();
  }
  stage_panels(smem, p.b, b_rows, b_cols);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = tmem_base_s;
  const uint32_t a_col = 256 + uint32_t(p.d_lane_off);   // d_lane_off doubles as a column offset of the A operand here
  {
    const __nv_bfloat16* arow = p.a + size_t(threadIdx.x) * p.K;
    for (int c0 = 0; c0 < p.K / 2; c0 += 16) {
      float v[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint32_t lo = __bfloat16_as_ushort(arow[2 * (c0 + i)]), hi = __bfloat16_as_ushort(arow[2 * (c0 + i) + 1]);
        v[i] = __uint_as_float(lo | (hi << 16));
      }
      tmem_st16(tmem_addr(tbase, warp * 32, a_col + c0), v);
    }
    tmem_st_wait();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x == 0) {
    Operand B{smem_u32(smem), uint32_t(b_rows) * 128u, p.b_mn};
    mma_tile_ts(tbase, tbase + a_col, B, p.N, p.K / 16, false);
    mma_commit(&bar);
  }
  const bool ok = mbar_wait(&bar, 0, p.err, 1);
  tc_fence_after();
  if (ok) {
    for (int c0 = 0; c0 < p.N; c0 += 16) {
      float v[16];
      tmem_ld16(tmem_addr(tbase, warp * 32, c0), v);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; ++i) p.d[size_t(warp * 32 + lane) * p.N + c0 + i] = v[i];
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 512);
}

// B operand in the UN-swizzled "interleaved" layout [N / 8][K rows][8 elements = 16 bytes] (reduction dim along rows, 8 x 16-byte
// core matrices of 128 contiguous bytes), A from tensor memory.  `variant` chooses which descriptor field carries which stride.
__global__ void __launch_bounds__(128) selftest_mma_nosw_kernel(SelftestParams p, int variant) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t bar;
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_init_fence();
  }
  // p.b is [K][N] row-major (b_mn layout of the other self-tests): element (k, n) -> group n / 8, row k
  // (variant 2: p.b is [N][K] row-major and element (n, k) -> group k / 8, row n)
  {
    const int R = variant == 2 ? p.N : p.K, C = variant == 2 ? p.K : p.N;
    for (int idx = threadIdx.x; idx < R * C / 8; idx += blockDim.x) {
      const int r = idx / (C / 8), j = idx % (C / 8);
      *reinterpret_cast<uint4*>(smem + size_t(j) * R * 16 + r * 16) = *reinterpret_cast<const uint4*>(p.b + size_t(r) * C + j * 8);
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = tmem_base_s;
  const uint32_t a_col = 256;
  {
    const __nv_bfloat16* arow = p.a + size_t(threadIdx.x) * p.K;
    for (int c0 = 0; c0 < p.K / 2; c0 += 16) {
      float v[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const uint32_t lo = __bfloat16_as_ushort(arow[2 * (c0 + i)]), hi = __bfloat16_as_ushort(arow[2 * (c0 + i) + 1]);
        v[i] = __uint_as_float(lo | (hi << 16));
      }
      tmem_st16(tmem_addr(tbase, warp * 32, a_col + c0), v);
    }
    tmem_st_wait();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (variant == 1) {   // A in strips as well: element (m, k) of the row-major [128][K] input -> strip m / 8, row k
    for (int idx = threadIdx.x; idx < 128 * p.K; idx += blockDim.x) {
      const int m = idx / p.K, k = idx % p.K;
      *reinterpret_cast<__nv_bfloat16*>(smem + 32768 + size_t(m / 8) * p.K * 16 + k * 16 + (m % 8) * 2) = p.a[idx];
    }
    fence_async_smem();
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    tc_fence_after();
    // variant 2: the strips hold B^T, i.e. [K / 8][N rows][16 bytes] (strips along the reduction dim): the host passes b as
    // [N][K] row-major for it, staged by the same loop with the roles of the two dims swapped
    const Operand B = variant == 2 ? Operand{smem_u32(smem), uint32_t(p.N) * 16u, 3} : Operand{smem_u32(smem), uint32_t(p.K) * 16u, 2};
    if (variant == 1) {
      const Operand A{smem_u32(smem) + 32768, uint32_t(p.K) * 16u, 2};
      mma_tile(tbase, A, B, 128, p.N, p.K / 16, false);
    } else {
      mma_tile_ts(tbase, tbase + a_col, B, p.N, p.K / 16, false);
    }
    mma_commit(&bar);
  }
  const bool ok = mbar_wait(&bar, 0, p.err, 1);
  tc_fence_after();
  if (ok) {
    for (int c0 = 0; c0 < p.N; c0 += 16) {
      float v[16];
      tmem_ld16(tmem_addr(tbase, warp * 32, c0), v);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; ++i) p.d[size_t(warp * 32 + lane) * p.N + c0 + i] = v[i];
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 512);
}

// A CTA that holds TMEM and waits on an mbarrier nobody arrives at: the wait gives up after `spin_limit` polls, records
// FLA_ERR_TIMEOUT in the status word, releases the TMEM and returns - the way every kernel of the library leaves a wait
// that runs out.  Nothing traps and nothing spins without a bound.
__global__ void __launch_bounds__(128) selftest_wait_timeout_kernel(uint32_t spin_limit, int* status) {
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t bar;
  const int warp = threadIdx.x / 32;
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 32);
    tmem_relinquish();
  }
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_init_fence();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = tmem_base_s;
  mbar_wait_limit(&bar, 0, spin_limit, status, FLA_ERR_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 32);
}

}  // namespace fla

extern "C" FLA_API int fla_b200_selftest_wait_timeout(uint32_t spin_limit, void* status_word, void* stream) {
  if (!status_word) return FLA_ERR_NULL;
  if (spin_limit == 0 || spin_limit > (1u << 20)) return FLA_ERR_VALUE;   // a test hook: keep the wait short
  fla::selftest_wait_timeout_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(spin_limit, static_cast<int*>(status_word));
  return cudaGetLastError() == cudaSuccess ? FLA_OK : FLA_ERR_CUDA;
}

extern "C" FLA_API int fla_b200_selftest_mma_ts(const void* a, const void* b, float* d, int N, int K, int b_mn, int a_col_off,
                                                int* err_flag, void* stream) {
  using namespace fla;
  if (!a || !b || !d || !err_flag) return FLA_ERR_NULL;
  if (N % 16 || N < 16 || N > 256 || K % 32 || K < 32 || K > 128) return FLA_ERR_SHAPE;
  if ((b_mn ? N : K) % 64 || N * K * 2 > 65536) return FLA_ERR_SHAPE;
  if (a_col_off < 0 || a_col_off % 8 || a_col_off + K / 2 > 256) return FLA_ERR_VALUE;
  SelftestParams p{static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), d, 128, N, K,
                   0, b_mn, a_col_off, 0, err_flag};
  const int smem = 65536 + 1024;
  if (cudaFuncSetAttribute(selftest_mma_ts_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return FLA_ERR_CUDA;
  selftest_mma_ts_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? FLA_OK : FLA_ERR_CUDA;
}

extern "C" FLA_API int fla_b200_selftest_mma_nosw(const void* a, const void* b, float* d, int N, int K, int variant, int* err_flag,
                                                  void* stream) {
  using namespace fla;
  if (!a || !b || !d || !err_flag) return FLA_ERR_NULL;
  if (N % 16 || N < 16 || N > 256 || K % 32 || K < 32 || K > 128 || N * K * 2 > 32768) return FLA_ERR_SHAPE;
  SelftestParams p{static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), d, 128, N, K, 0, 1, 0, 0, err_flag};
  const int smem = 65536 + 1024;
  if (cudaFuncSetAttribute(selftest_mma_nosw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return FLA_ERR_CUDA;
  selftest_mma_nosw_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(p, variant);
  return cudaGetLastError() == cudaSuccess ? FLA_OK : FLA_ERR_CUDA;
}

extern "C" FLA_API int fla_b200_selftest_mma(const void* a, const void* b, float* d, int M, int N, int K, int a_mn, int b_mn,
                                     int d_lane_off, int prefill, int* err_flag, void* stream) {
  using namespace fla;
  if (!a || !b || !d || !err_flag) return FLA_ERR_NULL;
  if (!(M == 64 || M == 128) || N % 16 || N < 16 || N > 256 || K % 16 || K < 16 || K > 128) return FLA_ERR_SHAPE;
  if ((a_mn ? M : K) % 64 || (b_mn ? N : K) % 64) return FLA_ERR_SHAPE;
  if (M * K * 2 > 32768 || N * K * 2 > 32768) return FLA_ERR_SHAPE;
  SelftestParams p{static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), d, M, N, K,
                   a_mn, b_mn, d_lane_off, prefill, err_flag};
  const int smem = 65536 + 1024;
  cudaError_t e = cudaFuncSetAttribute(selftest_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return FLA_ERR_CUDA;
  selftest_mma_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? FLA_OK : FLA_ERR_CUDA;
}

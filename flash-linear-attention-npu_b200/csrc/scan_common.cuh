// Pieces shared by the two scan kernels of the chunked gated delta rule (forward state scan, reverse state-gradient scan)
// that keep their state TRANSPOSED in tensor memory: TMEM lane v holds the state column of value channel v, so every
// operand an epilogue produces is a LEFT operand whose rows are TMEM lanes.  It is written with tcgen05.st as packed
// bf16 pairs and consumed by tcgen05.mma straight from tensor memory; only the inputs (which arrive by TMA in the panel
// layout the descriptors want) are read from shared memory.
//
// Thread roles: the first warps are epilogue warps (TMEM lane quadrant = warp % 4, warp / 4 selects the part of a tile's
// columns they own: eight warps with a half each in the reverse scan, sixteen with a quarter each in the forward scan); thread 0 issues every product right after the CTA barrier that publishes its operands (measured:
// 0.64 ms against 0.75 ms with the products issued by a separate warp, which has to win an issue slot first); the last warp is
// a helper that issues the TMA loads a chunk ahead and the bulk copy of the chunk's per-token factor record two chunks
// ahead, so that neither latency is ever waited for.  Epilogues walk their tokens in groups of 16 with a
// compiler fence between groups: without it the loads of all groups are hoisted and the 168 registers a thread gets at
// 288 threads per CTA spill.
#pragma once
#include "gdn_common.cuh"
#include "tensor_map.h"

namespace fla {

constexpr int kScanEpiThreads = 256;
constexpr int kScanThreads = 288;

// The prep kernel leaves, behind the P tile of every (chunk, value head), the chunk's per-token factors as one ScanFactors
// record: both scans fetch it with a single bulk copy straight into shared memory (global loads issued by the helper warp
// took it thousands of cycles per chunk, with the whole CTA waiting at its next barrier).
// [dO^T | dZ^T | residual of dZ^T] strips of one 64-channel half of a (chunk, head): bf16 elements
constexpr int64_t kDzHalf = 12288;
constexpr int64_t kPTileBytes = 16384;                 // P: value + residual, 64 x 64 bf16 each
constexpr int64_t kPImgBytes = kPTileBytes + 1152;     // + the factor record (1040 bytes used), 128-byte aligned stride
constexpr int64_t kPImg = kPImgBytes / 2;              // in bf16 elements: the per-(chunk, head) stride of p_img
struct __align__(16) ScanFactors {     // per-token factors of one chunk, made by the prep kernel
  float b[kC];           // beta_j
  float bg[kC];          // beta_j e^{gam_j}
  float dk[kC];          // e^{gam_L - gam_j}
  float se[kC];          // scale e^{gam_j}
  float dl;              // e^{gam_L}
  float pad[3];
};

__device__ __forceinline__ void tmem_st16u(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st8u(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]),
               "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_ld16u(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
// keeps the compiler from hoisting the loads of a later group of tokens above the work of an earlier one (registers)
__device__ __forceinline__ void group_fence() { asm volatile("" ::: "memory"); }
// 16 fp32 values -> 8 packed bf16 pairs of the value and 8 of the residual
__device__ __forceinline__ void split16(const float* x, uint32_t* hi, uint32_t* lo) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    hi[i] = pack_bf16(x[2 * i], x[2 * i + 1]);
    const float h0 = __uint_as_float(hi[i] << 16), h1 = __uint_as_float(hi[i] & 0xffff0000u);
    lo[i] = pack_bf16(x[2 * i] - h0, x[2 * i + 1] - h1);
  }
}
__device__ __forceinline__ void pack16(const float* x, uint32_t* w) {
#pragma unroll
  for (int i = 0; i < 8; ++i) w[i] = pack_bf16(x[2 * i], x[2 * i + 1]);
}
// A wait for threads that are in no hurry (the helper warp waiting for a product to release a buffer): sleeps between polls
// so that it does not compete for issue slots with the epilogue warps of its scheduler.
__device__ __forceinline__ void lazy_wait_or_mark(uint64_t* bar, uint32_t& phase, bool& dead, int* status) {
  if (!dead) {
    bool ok = false;
    for (uint32_t it = 0; it < (kSpinLimit >> 4) && !ok; ++it) {
      ok = mbar_try_wait(bar, phase);
      if (!ok) __nanosleep(64);
    }
    if (!ok) {
      if (status) atomicExch(status, 8 /* FLA_ERR_TIMEOUT */);
      dead = true;
    }
  }
  phase ^= 1;
}
// every warp of the CTA (epilogue warps + the helper warp)
__device__ __forceinline__ void scan_sync() { __syncthreads(); }
// the 8 epilogue warps of the reverse scan only
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// 64 x 64 identity panel: the B operand that copies a 64-token tile of rows into tensor memory TRANSPOSED
// (D[v][j] = sum_t tile[t][v] I[j][t]: exact, every product is with one or zero).
__device__ __forceinline__ void write_identity_panel(uint8_t* pan, int tid, int nthreads) {
  for (int idx = tid; idx < 512; idx += nthreads) {   // 16-byte pieces: row r has a one in column r
    const int r = idx >> 3, ch = idx & 7;
    uint4 val = make_uint4(0, 0, 0, 0);
    if ((r >> 3) == ch) {
      const uint32_t one = 0x3f80u << (16 * (r & 1));
      const int w = (r & 7) >> 1;
      val = make_uint4(w == 0 ? one : 0, w == 1 ? one : 0, w == 2 ? one : 0, w == 3 ? one : 0);
    }
    *reinterpret_cast<uint4*>(pan + panel_chunk_off(r, ch)) = val;
  }
}

// A [kRows tokens][128 channels] tile staged in shared memory (kRowBytes per token) leaves for global memory as 16-byte
// pieces of rows; the first `rows` tokens are valid.  Two-byte stores scattered over tokens, which is what each
// thread's own data would need, cost several thousand cycles per chunk.
template <int kRowBytes, int kRows>
__device__ __forceinline__ void copy_out_tile(const uint8_t* tile, uint8_t* gbase, int64_t g_row_bytes, int rows, int tid) {
  constexpr int kPerRow = kRowBytes / 16, kIters = kRows * kPerRow / kScanEpiThreads;
#pragma unroll
  for (int i = 0; i < kIters; ++i) {
    const int id = tid + i * kScanEpiThreads, r = id / kPerRow, c16 = id % kPerRow;
    if (r < rows) *reinterpret_cast<uint4*>(gbase + r * g_row_bytes + c16 * 16) = *reinterpret_cast<const uint4*>(tile + r * kRowBytes + c16 * 16);
  }
}

// Each epilogue thread holds one channel (`vrow`) of 32 tokens (t_lo .. t_lo + 31) of a [64 tokens][128 channels] result.
// The tile is transposed through a 16 KB shared-memory buffer: bf16 results in one pass, fp32 results in two (the 32
// tokens of each half of the warps).  `g` points at the chunk's first token, channel 0 of this block.
__device__ __forceinline__ void store_rows_transposed(uint8_t* tile, const float* ov, void* g, int64_t g_row_elems, bool f32, int rows,
                                                      int half, int vrow, int tid) {
  if (f32) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (half == h) {
#pragma unroll
        for (int i = 0; i < 32; ++i) *reinterpret_cast<float*>(tile + i * 512 + vrow * 4) = ov[i];
      }
      epi_sync();
      copy_out_tile<512, 32>(tile, reinterpret_cast<uint8_t*>(static_cast<float*>(g) + h * 32 * g_row_elems), g_row_elems * 4, rows - h * 32, tid);
      epi_sync();
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) *reinterpret_cast<bf16*>(tile + (half * 32 + i) * 256 + vrow * 2) = __float2bfloat16_rn(ov[i]);
    epi_sync();
    copy_out_tile<256, 64>(tile, static_cast<uint8_t*>(g), g_row_elems * 2, rows, tid);
  }
}

}  // namespace fla

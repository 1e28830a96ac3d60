// Forward scan of the chunked gated delta rule (recompute_w_u + chunk_gated_delta_rule_fwd_h + chunk_fwd_o of the
// reference, examples/flash_gated_delta_rule.py:840-880, with the WY factors folded away).
//
// One CTA per (sequence, value head, 128-column block of V); the state lives transposed in tensor memory for the whole
// sequence (scan_common.cuh).  Per chunk, with S the state at chunk start, gam the chunk-local cumulative log decay,
// X = (I + A)^-1 (bf16 value + residual) and P = tril(Q K^T e^{gam_i-gam_j}) from the prep kernels:
//     [QS^T | KS^T] = S^T [Q; K]^T          N = 128 tokens of the [q; k] panel, reduction over the 128 key dims
//     Z^T     = beta (V^T - e^gam KS^T)     epilogue; V^T arrives through an identity product
//     v_new^T = Z^T X^T                     N = 64; X is a value + a residual (a single bf16 X is what dominated the error)
//     S^T    <- e^{gam_L} S^T + vhat^T K    N = 128 key dims, reduction over the 64 tokens, vhat = e^{gam_L-gam} v_new
//     o^T     = scale (e^gam QS^T + v_new^T P^T)
// Operands the result is sensitive to (state copy, Z, v_new, vhat, P) are a bf16 value plus a bf16 residual and enter
// two or three products; q, k, v enter as the exact bf16 inputs; accumulation is fp32.
// For the backward the kernel saves, per (chunk, head, block), the state and v_new as ready-made operands in the
// un-swizzled strip layout (sm100.cuh), rows = value channels: a thread owns one channel, so the 16 bytes it stores for a
// strip lie next to its neighbours' (512 contiguous bytes per warp store).  Swizzled panels, whose rows are 128 bytes
// apart, had to be staged in shared memory and written by bulk copies: 0.83 ms per launch against 0.7x ms.
//     s_img   [64-channel half][value | residual][16 strips of 8 key dims][64 rows x 16 bytes]   = 64 KB
//     vn_img  [64-channel half][value | residual][8 strips of 8 tokens][64 rows x 16 bytes]      = 32 KB
#pragma once
#include "scan_common.cuh"

namespace fla {

// tensor-memory columns (512 allocated)
constexpr uint32_t tST = 0;        // S^T fp32 accumulator (128 columns = key dims)
constexpr uint32_t tSAh = 128;     // bf16 copy of S^T as A operand: 128 key dims packed in 64 columns
constexpr uint32_t tSAl = 192;     // its residual
constexpr uint32_t tKQ = 256;      // [QS^T (64 tokens) | KS^T (64 tokens)] accumulator
constexpr uint32_t tVN = 320;      // v_new^T accumulator, later the (v_new^T P^T) accumulator: reuses the KS^T columns
constexpr uint32_t tZAh = 384;     // Z^T, then v_new^T, as A operand: 64 tokens packed in 32 columns
constexpr uint32_t tZAl = 416;
constexpr uint32_t tVAh = 448;     // V^T (fp32, 64 columns) until Z is built, then the decayed v_new^T as A operand
constexpr uint32_t tVAl = 480;

// shared memory (offsets from a 1024-byte aligned base); the load buffers exist twice (chunk parity)
constexpr uint32_t sQK = 0;                  // 2 x 32 KB: [q; k] rows, two 64-column panels of 128 rows
constexpr uint32_t sX = 65536;               // 2 x 16 KB: the chunk's inverse as value + residual strips
constexpr uint32_t sP = 98304;               // 2 x 16 KB (value, residual)
constexpr uint32_t sV = 131072;              // 2 x 16 KB: v rows of the chunk, two 64-column panels of 64 rows
constexpr uint32_t sO = 163840;              // 16 KB: the chunk's output rows on their way out
constexpr uint32_t sI = 180224;              // 8 KB: identity panel
constexpr uint32_t kScanFwdSmem = 188416;

// Epilogue warps of the forward scan: TMEM lane quadrant = warp % 4, warp / 4 selects which of the kFwdSplit column
// ranges of a tile the warp owns (64 / kFwdSplit tokens, 128 / kFwdSplit key dims); the helper warp comes after them.
// Sixteen warps with a quarter of the columns each against eight with a half: 0.577 -> 0.564 ms (training) and
// 0.498 -> 0.485 ms (inference); the per-chunk chain is mostly hand-off latency, not epilogue issue.
constexpr int kFwdSplit = 4;
constexpr int kFwdEpiWarps = 4 * kFwdSplit, kFwdEpiThreads = 32 * kFwdEpiWarps, kFwdThreads = kFwdEpiThreads + 32;
constexpr int kFwdTT = 64 / kFwdSplit, kFwdKT = 128 / kFwdSplit;     // tokens / key dims per thread
__device__ __forceinline__ void fwd_epi_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kFwdEpiThreads) : "memory"); }
template <int kRowBytes, int kRows>
__device__ __forceinline__ void fwd_copy_out_tile(const uint8_t* tile, uint8_t* gbase, int64_t g_row_bytes, int rows, int tid) {
  constexpr int kPerRow = kRowBytes / 16, kIters = kRows * kPerRow / kFwdEpiThreads;
#pragma unroll
  for (int i = 0; i < kIters; ++i) {
    const int id = tid + i * kFwdEpiThreads, r = id / kPerRow, c16 = id % kPerRow;
    if (r < rows) *reinterpret_cast<uint4*>(gbase + r * g_row_bytes + c16 * 16) = *reinterpret_cast<const uint4*>(tile + r * kRowBytes + c16 * 16);
  }
}
// Each epilogue thread holds one channel (`vrow`) of kFwdTT tokens (cs * kFwdTT ..) of a [64 tokens][128 channels] result.
// The tile is transposed through a 16 KB shared-memory buffer: bf16 results in one pass, fp32 results in two (32 tokens each).
__device__ __forceinline__ void fwd_store_rows_transposed(uint8_t* tile, const float* ov, void* g, int64_t g_row_elems, bool f32, int rows,
                                                          int cs, int vrow, int tid) {
  if (f32) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if ((cs * kFwdTT) / 32 == h) {
#pragma unroll
        for (int i = 0; i < kFwdTT; ++i) *reinterpret_cast<float*>(tile + ((cs * kFwdTT) % 32 + i) * 512 + vrow * 4) = ov[i];
      }
      fwd_epi_sync();
      fwd_copy_out_tile<512, 32>(tile, reinterpret_cast<uint8_t*>(static_cast<float*>(g) + h * 32 * g_row_elems), g_row_elems * 4, rows - h * 32, tid);
      fwd_epi_sync();
    }
  } else {
#pragma unroll
    for (int i = 0; i < kFwdTT; ++i) *reinterpret_cast<bf16*>(tile + (cs * kFwdTT + i) * 256 + vrow * 2) = __float2bfloat16_rn(ov[i]);
    fwd_epi_sync();
    fwd_copy_out_tile<256, 64>(tile, static_cast<uint8_t*>(g), g_row_elems * 2, rows, tid);
  }
}

struct ScanBars {
  uint64_t *mma_bar, *o_bar, *qk_bar, *x_bar, *p_bar, *v_bar;   // two barriers each (index = chunk parity) but the first two
};
// The three batches of products of one chunk.  All of warp 0 runs them and the lane `lead` marks issues: built from
// warp-uniform values in converged code a product costs a handful of instructions; out of line, or in a branch that one
// thread takes, it cost some thirty and the tensor pipe waited for its issuer (0.65 -> 0.53 ms for the inference forward).
__device__ __forceinline__ bool scan_fwd_mma1(uint32_t tbase, uint32_t sb, int c, ScanBars bars, int* status, bool dead, uint32_t lead) {
  const int b = c & 1;
  const uint32_t ph = (c >> 1) & 1;
  tc_fence_after();
  if (!dead && !mbar_wait(&bars.qk_bar[b], ph, status, FLA_ERR_TIMEOUT)) dead = true;
  const Operand opKQ{sb + sQK + b * 32768, 16384, 0};
  mma_tile_ts(tbase + tKQ, tbase + tSAh, opKQ, 128, 8, false, lead);
  mma_tile_ts(tbase + tKQ, tbase + tSAl, opKQ, 128, 8, true, lead);
  // V^T into the columns the decayed v_new of this chunk will occupy later
  if (!dead && !mbar_wait(&bars.v_bar[b], ph, status, FLA_ERR_TIMEOUT)) dead = true;
  const Operand opVt{sb + sV + b * 16384, 8192, 1}, opI{sb + sI, 8192, 0};
  mma_tile(tbase + tVAh, opVt, opI, 128, 64, 4, false, lead);
  mma_commit(bars.mma_bar, lead);
  return dead;
}
__device__ __forceinline__ bool scan_fwd_mma2(uint32_t tbase, uint32_t sb, int c, ScanBars bars, int* status, bool dead, uint32_t lead) {
  const int b = c & 1;
  tc_fence_after();
  if (!dead && !mbar_wait(&bars.x_bar[b], (c >> 1) & 1, status, FLA_ERR_TIMEOUT)) dead = true;
  // X in strips of 8 rows: rows of X are N here, its columns the reduction dim
  const Operand opXh{sb + sX + b * 16384, 1024, 2}, opXl{sb + sX + b * 16384 + 8192, 1024, 2};
  mma_tile_ts(tbase + tVN, tbase + tZAh, opXh, 64, 4, false, lead);
  mma_tile_ts(tbase + tVN, tbase + tZAl, opXh, 64, 4, true, lead);
  mma_tile_ts(tbase + tVN, tbase + tZAh, opXl, 64, 4, true, lead);
  mma_commit(bars.mma_bar, lead);
  return dead;
}
__device__ __forceinline__ bool scan_fwd_mma3(uint32_t tbase, uint32_t sb, int c, ScanBars bars, int* status, bool dead, uint32_t lead) {
  const int b = c & 1;
  tc_fence_after();
  const Operand opK{sb + sQK + b * 32768 + 8192, 16384, 1};   // k rows: reduction over tokens, N = 128 key dims over two panels
  mma_tile_ts(tbase + tST, tbase + tVAh, opK, 128, 4, true, lead);
  mma_tile_ts(tbase + tST, tbase + tVAl, opK, 128, 4, true, lead);
  mma_commit(bars.mma_bar, lead);                                   // the state update: what the next chunk waits for
  if (!dead && !mbar_wait(&bars.p_bar[b], (c >> 1) & 1, status, FLA_ERR_TIMEOUT)) dead = true;
  const uint32_t pp = sb + sP + b * 16384;
  const Operand opPh{pp, 1024, 3}, opPl{pp + 8192, 1024, 3};   // P in strips of 8 columns: N = rows i, reduction along j
  mma_tile_ts(tbase + tVN, tbase + tZAh, opPh, 64, 4, false, lead);
  mma_tile_ts(tbase + tVN, tbase + tZAl, opPh, 64, 4, true, lead);
  mma_tile_ts(tbase + tVN, tbase + tZAh, opPl, 64, 4, true, lead);
  mma_commit(bars.o_bar, lead);                                     // the output product: read when the next chunk's state is out
  return dead;
}

template <bool kSave>
__global__ void __launch_bounds__(kFwdThreads, 1) gdn_scan_fwd_kernel(GdnFwdParams p, const __grid_constant__ CUtensorMap tm_q,
                                                                        const __grid_constant__ CUtensorMap tm_k,
                                                                        const __grid_constant__ CUtensorMap tm_v) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ ScanFactors fac[3];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t mma_bar, o_bar, qk_bar[2], x_bar[2], p_bar[2], v_bar[2], f_bar[3];

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int vb = blockIdx.x, hv = blockIdx.y, n = blockIdx.z;
  const int hk = hv / (p.HV / p.HK);
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  const uint32_t sb = smem_u32(smem);
  const int nt = sq.nt;

  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(&mma_bar, 1);
    mbar_init(&o_bar, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qk_bar[i], 1);
      mbar_init(&x_bar[i], 1);
      mbar_init(&p_bar[i], 1);
      mbar_init(&v_bar[i], 1);
    }
    for (int i = 0; i < 3; ++i) mbar_init(&f_bar[i], 1);
    mbar_init_fence();
  }
  write_identity_panel(smem + sI, tid, kFwdThreads);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = tmem_base_s;
  bool dead = false;

  if (warp == kFwdEpiWarps) {
    // ============================================================ helper warp: TMA loads and per-token factors
    auto load_qk = [&](int c) {
      const int b = c & 1, row0 = sq.bos + c * kC;
      const uint32_t qk = sb + sQK + b * 32768;
      mbar_arrive_expect_tx(&qk_bar[b], 32768);
      tma_load_tile(qk, &tm_q, 0, hk, row0, &qk_bar[b]);
      tma_load_tile(qk + 16384, &tm_q, 64, hk, row0, &qk_bar[b]);
      tma_load_tile(qk + 8192, &tm_k, 0, hk, row0, &qk_bar[b]);
      tma_load_tile(qk + 16384 + 8192, &tm_k, 64, hk, row0, &qk_bar[b]);
    };
    auto load_rest = [&](int c) {
      const int b = c & 1, row0 = sq.bos + c * kC;
      mbar_arrive_expect_tx(&v_bar[b], 16384);
      tma_load_tile(sb + sV + b * 16384, &tm_v, vb * 128, hv, row0, &v_bar[b]);
      tma_load_tile(sb + sV + b * 16384 + 8192, &tm_v, vb * 128 + 64, hv, row0, &v_bar[b]);
      mbar_arrive_expect_tx(&x_bar[b], 16384);
      bulk_load(sb + sX + b * 16384, p.X + ((int64_t(sq.cbase) + c) * p.HV + hv) * 8192, 16384, &x_bar[b]);
      mbar_arrive_expect_tx(&p_bar[b], 16384);
      bulk_load(sb + sP + b * 16384, p.p_img + ((int64_t(sq.cbase) + c) * p.HV + hv) * kPImg, 16384, &p_bar[b]);
    };
    // the per-token factors of chunk c (made by the prep kernel, behind the chunk's P tile) into buffer c % 3
    auto load_factors = [&](int c) {
      if (c < nt) {
        mbar_arrive_expect_tx(&f_bar[c % 3], uint32_t(sizeof(ScanFactors)));
        bulk_load(smem_u32(&fac[c % 3]), reinterpret_cast<const uint8_t*>(p.p_img + ((int64_t(sq.cbase) + c) * p.HV + hv) * kPImg) + kPTileBytes,
                  uint32_t(sizeof(ScanFactors)), &f_bar[c % 3]);
      }
    };
    if (lane == 0) {
      tma_prefetch_descriptor(&tm_q);
      tma_prefetch_descriptor(&tm_k);
      tma_prefetch_descriptor(&tm_v);
      if (nt > 0) {
        load_qk(0);
        load_rest(0);
      }
      load_factors(0);
      load_factors(1);
    }
    __syncwarp();
    scan_sync();   // (pairs with the epilogue warps' barrier after they have loaded the initial state)
    for (int c = 0; c < nt; ++c) {
      scan_sync();                                          // sync 1: chunk c - 1 no longer reads the other buffers
      if (lane == 0) {
        if (c + 1 < nt) {
          load_qk(c + 1);
          load_rest(c + 1);
        }
        load_factors(c + 2);                                // buffer (c + 2) % 3 was last read for chunk c - 1's output rows
      }
      __syncwarp();
      scan_sync();                                          // sync 2
      scan_sync();                                          // sync 3
    }
    scan_sync();   // matches the epilogue warps' barrier before the TMEM is released
    return;
  }

  // ================================================================ epilogue warps
  const ScanBars bars{&mma_bar, &o_bar, qk_bar, x_bar, p_bar, v_bar};
  // The products are issued by one elected lane of warp 0 inside code that the whole warp runs: descriptors built from
  // warp-uniform values stay in uniform registers, which is what the instruction takes; built in a branch that a single
  // thread takes they cost some thirty instructions per product to move there.
  const int warp_u = __shfl_sync(0xffffffffu, warp, 0);
  const uint32_t tbase_u = __shfl_sync(0xffffffffu, tbase, 0), sb_u = __shfl_sync(0xffffffffu, sb, 0);
  const int quad = warp & 3, cs = warp >> 2;
  const int vrow = quad * 32 + lane;                       // my value channel inside the block = my TMEM lane
  const uint32_t tlane = tmem_addr(tbase, quad * 32, 0);
  const int t_lo = cs * kFwdTT;                            // my tokens of a token-indexed tile
  const int k_lo = cs * kFwdKT;                            // my key dims of the state row
  uint32_t mphase = 0, ophase = 0;

  // the initial state goes straight into the accumulator columns: every chunk starts by reading its state from there
  {
    const float* src = p.h0 ? p.h0 + ((int64_t(n) * p.HV + hv) * kK + k_lo) * p.V + vb * 128 + vrow : nullptr;
#pragma unroll
    for (int part = 0; part < kFwdKT / 16; ++part) {
      float s16[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) s16[i] = src ? src[int64_t(part * 16 + i) * p.V] : 0.f;
      tmem_st16(tlane + tST + k_lo + part * 16, s16);
    }
    tmem_st_wait();
  }
  scan_sync();   // factors of chunk 0 are visible

  // Output rows of chunk c: the values are formed before sync 1 of chunk c + 1 (the accumulators they come from are
  // overwritten by that chunk's first product) and leave for global memory while that product runs.
  float ov[kFwdTT];
  auto form_o = [&](int c) {
    const ScanFactors& f = fac[c % 3];
#pragma unroll
    for (int g = 0; g < kFwdTT / 16; ++g) {
      float qs[16], pv[16];
      tmem_ld16(tlane + tKQ + t_lo + g * 16, qs);
      tmem_ld16(tlane + tVN + t_lo + g * 16, pv);
      tmem_ld_wait();
#pragma unroll
      for (int i4 = 0; i4 < 16; i4 += 4) {
        const float4 se = *reinterpret_cast<const float4*>(&f.se[t_lo + g * 16 + i4]);
        ov[g * 16 + i4] = se.x * qs[i4] + p.scale * pv[i4];
        ov[g * 16 + i4 + 1] = se.y * qs[i4 + 1] + p.scale * pv[i4 + 1];
        ov[g * 16 + i4 + 2] = se.z * qs[i4 + 2] + p.scale * pv[i4 + 2];
        ov[g * 16 + i4 + 3] = se.w * qs[i4 + 3] + p.scale * pv[i4 + 3];
      }
      group_fence();
    }
  };
  auto store_o = [&](int c) {
    const int rows = min(kC, sq.len - c * kC);
    const int64_t off = (int64_t(sq.bos) + c * kC) * p.o_st + hv * p.o_sh + vb * 128;
    void* g = p.o_is_f32 ? static_cast<void*>(static_cast<float*>(p.o) + off) : static_cast<void*>(static_cast<bf16*>(p.o) + off);
    fwd_store_rows_transposed(smem + sO, ov, g, p.o_st, p.o_is_f32 != 0, rows, cs, vrow, tid);
  };

  for (int c = 0; c < nt; ++c) {
    const ScanFactors& f = fac[c % 3];
    if (!dead && !mbar_wait(&f_bar[c % 3], (c / 3) & 1, p.status, FLA_ERR_TIMEOUT)) dead = true;   // requested two chunks ago
    const int rows = min(kC, sq.len - c * kC);
    const int64_t cidx = ((int64_t(sq.cbase) + c) * p.HV + hv) * (p.V / 128) + vb;

    // ---- A: publish the state at chunk start: bf16 value + residual as A operand (and as the saved image), decayed
    //         fp32 copy as accumulator
    {
      const float dl = f.dl;
      uint8_t* s_row = kSave ? reinterpret_cast<uint8_t*>(p.s_img + cidx * 32768) + (vrow >> 6) * 32768 + (vrow & 63) * 16 : nullptr;
#pragma unroll 1
      for (int g4 = 0; g4 < kFwdKT / 16; ++g4) {         // 16 key dims at a time: 8 packed columns per operand store
        float s16[16];
        tmem_ld16(tlane + tST + k_lo + g4 * 16, s16);
        tmem_ld_wait();
        uint32_t hi[8], lo[8];
        split16(s16, hi, lo);
        tmem_st8u(tlane + tSAh + cs * (kFwdKT / 2) + g4 * 8, hi);
        tmem_st8u(tlane + tSAl + cs * (kFwdKT / 2) + g4 * 8, lo);
        if (kSave) {   // strips k_lo / 8 + g4 * 2 and the next one of my channel's row
          uint8_t* dst = s_row + (cs * (kFwdKT / 8) + g4 * 2) * 1024;
          *reinterpret_cast<uint4*>(dst) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
          *reinterpret_cast<uint4*>(dst + 1024) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
          *reinterpret_cast<uint4*>(dst + 16384) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
          *reinterpret_cast<uint4*>(dst + 16384 + 1024) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) s16[i] *= dl;
        tmem_st16(tlane + tST + k_lo + g4 * 16, s16);
        group_fence();
      }
      tmem_st_wait();
    }
    if (c > 0) {   // the output accumulators of chunk c - 1: into registers before the next product overwrites them
      wait_or_mark(&o_bar, ophase, dead, p.status);
      tc_fence_after();
      form_o(c - 1);
    }
    tc_fence_before();
    scan_sync();                                   // sync 1
    tc_fence_after();
    if (warp_u == 0) dead = scan_fwd_mma1(tbase_u, sb_u, c, bars, p.status, dead, elect_one());
    // ---- while [QS^T | KS^T] runs: output rows of chunk c - 1
    if (c > 0) store_o(c - 1);
    wait_or_mark(&mma_bar, mphase, dead, p.status);
    tc_fence_after();

    // ---- C: Z^T = beta (V^T - e^gam KS^T) for my 32 tokens
    {
#pragma unroll 1
      for (int g = 0; g < kFwdTT / 16; ++g) {
        float ks[16], vt[16];
        tmem_ld16(tlane + tKQ + 64 + t_lo + g * 16, ks);
        tmem_ld16(tlane + tVAh + t_lo + g * 16, vt);
        tmem_ld_wait();
#pragma unroll
        for (int i4 = 0; i4 < 16; i4 += 4) {
          const float4 b4 = *reinterpret_cast<const float4*>(&f.b[t_lo + g * 16 + i4]);
          const float4 g4 = *reinterpret_cast<const float4*>(&f.bg[t_lo + g * 16 + i4]);
          ks[i4] = b4.x * vt[i4] - g4.x * ks[i4];
          ks[i4 + 1] = b4.y * vt[i4 + 1] - g4.y * ks[i4 + 1];
          ks[i4 + 2] = b4.z * vt[i4 + 2] - g4.z * ks[i4 + 2];
          ks[i4 + 3] = b4.w * vt[i4 + 3] - g4.w * ks[i4 + 3];
        }
        uint32_t hi[8], lo[8];
        split16(ks, hi, lo);
        tmem_st8u(tlane + tZAh + cs * (kFwdTT / 2) + g * 8, hi);
        tmem_st8u(tlane + tZAl + cs * (kFwdTT / 2) + g * 8, lo);
        group_fence();
      }
      tmem_st_wait();
    }
    tc_fence_before();
    scan_sync();                                   // sync 2
    tc_fence_after();
    if (warp_u == 0) dead = scan_fwd_mma2(tbase_u, sb_u, c, bars, p.status, dead, elect_one());
    wait_or_mark(&mma_bar, mphase, dead, p.status);
    tc_fence_after();

    // ---- E: v_new^T (rows past the end of the sequence are zero) and its decayed copy
    {
#pragma unroll 1
      for (int g = 0; g < kFwdTT / 16; ++g) {
        float vn[16];
        tmem_ld16(tlane + tVN + t_lo + g * 16, vn);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) vn[i] = (t_lo + g * 16 + i < rows) ? vn[i] : 0.f;
        uint32_t hi[8], lo[8];
        split16(vn, hi, lo);
        tmem_st8u(tlane + tZAh + cs * (kFwdTT / 2) + g * 8, hi);
        tmem_st8u(tlane + tZAl + cs * (kFwdTT / 2) + g * 8, lo);
        if (kSave) {                                 // v_new image: strips t_lo / 8 + g * 2 and the next one
          uint8_t* dst = reinterpret_cast<uint8_t*>(p.vn_img + cidx * 16384) + (vrow >> 6) * 16384 + (cs * (kFwdTT / 8) + g * 2) * 1024 + (vrow & 63) * 16;
          *reinterpret_cast<uint4*>(dst) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
          *reinterpret_cast<uint4*>(dst + 1024) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
          *reinterpret_cast<uint4*>(dst + 8192) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
          *reinterpret_cast<uint4*>(dst + 8192 + 1024) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
        }
#pragma unroll
        for (int i4 = 0; i4 < 16; i4 += 4) {
          const float4 d4 = *reinterpret_cast<const float4*>(&f.dk[t_lo + g * 16 + i4]);
          vn[i4] *= d4.x; vn[i4 + 1] *= d4.y; vn[i4 + 2] *= d4.z; vn[i4 + 3] *= d4.w;
        }
        split16(vn, hi, lo);
        tmem_st8u(tlane + tVAh + cs * (kFwdTT / 2) + g * 8, hi);
        tmem_st8u(tlane + tVAl + cs * (kFwdTT / 2) + g * 8, lo);
        group_fence();
      }
      tmem_st_wait();
    }
    tc_fence_before();
    scan_sync();                                   // sync 3
    tc_fence_after();
    if (warp_u == 0) dead = scan_fwd_mma3(tbase_u, sb_u, c, bars, p.status, dead, elect_one());
    wait_or_mark(&mma_bar, mphase, dead, p.status);    // the state update has completed (the output product may still run)
    tc_fence_after();
  }

  if (nt > 0) {
    wait_or_mark(&o_bar, ophase, dead, p.status);
    tc_fence_after();
    form_o(nt - 1);
    store_o(nt - 1);
  }
  if (!dead && p.ht) {
    float* dst = p.ht + ((int64_t(n) * p.HV + hv) * kK + k_lo) * p.V + vb * 128 + vrow;
#pragma unroll
    for (int part = 0; part < kFwdKT / 16; ++part) {
      float s16[16];
      tmem_ld16(tlane + tST + k_lo + part * 16, s16);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; ++i) dst[int64_t(part * 16 + i) * p.V] = s16[i];
    }
  }
  tc_fence_before();
  scan_sync();
  if (warp == 0) tmem_dealloc(tbase, 512);
}

}  // namespace fla

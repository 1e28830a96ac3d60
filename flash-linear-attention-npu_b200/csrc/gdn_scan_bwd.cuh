// Reverse scan of the chunked gated-delta-rule backward (chunk_bwd_dv_local + chunk_gated_delta_rule_bwd_dhu of the
// reference, examples/flash_gated_delta_rule.py:930-960, and the dv / du parts of prepare_wy_repr_bwd_*).
//
// One CTA per (sequence, value head, 128-column block of V); the state gradient lives transposed in tensor memory
// (scan_common.cuh: TMEM lane v = value channel v).  Per chunk, in reverse order, with dS' the gradient entering the
// chunk from the right:
//     W1^T   = dS'^T K^T                           N = 64 tokens, reduction over the 128 key dims
//     U1^T   = dO^T P                              (= (P^T dO)^T; both operands from shared memory)
//     dVn^T  = scale U1^T + e^{gam_L-gam} W1^T     epilogue, zero for tokens past the end of the sequence
//     dZ^T   = dVn^T X                             (= (X^T dVn)^T)
//     dV     = beta dZ;   bz = sum_v dZ V  (partial sums per 32 value channels);   dR = -beta e^gam dZ
//     dS^T   = e^{gam_L} dS'^T + [scale e^gam dO^T | dR^T] [Q; K]     N = 128 key dims, reduction over 128 rows
// dO^T and V^T reach tensor memory through identity products.  For the chunk-parallel kernel the scan saves, per
// (chunk, head, block), operands in the un-swizzled strip layout (sm100.cuh) whose rows are value channels, stored by
// the thread that owns the channel (coalesced):
//     ds_img  dS' as [64-channel half][value | residual][16 strips of 8 key dims][64 rows x 16 bytes]   = 64 KB
//     dz_img  [64-channel half][dO^T | dZ^T | residual of dZ^T][8 strips of 8 tokens][64 rows x 16 bytes] = 48 KB
#pragma once
#include "scan_common.cuh"

namespace fla {

// tensor-memory columns (512 allocated)
constexpr uint32_t uDS = 0;        // dS^T fp32 accumulator (128 key dims)
constexpr uint32_t uAh = 128;      // dS'^T as A operand (128 key dims in 64 columns); later [scale e^gam dO^T | dR^T] (128 rows of [q; k])
constexpr uint32_t uAl = 192;      // residuals of the same
constexpr uint32_t uW = 256;       // W1^T accumulator, later the dZ^T accumulator
constexpr uint32_t uU = 320;       // U1^T accumulator, later dO^T (fp32)
constexpr uint32_t uDVh = 384;     // dVn^T as A operand: 64 tokens in 32 columns
constexpr uint32_t uDVl = 416;
constexpr uint32_t uVT = 448;      // V^T (fp32, 64 tokens)

// shared memory: load buffers twice (step parity)
constexpr uint32_t bQK = 0;                  // 2 x 32 KB
constexpr uint32_t bX = 65536;               // 2 x 16 KB: the chunk's inverse as value + residual strips
constexpr uint32_t bP = 98304;               // 2 x 16 KB (value, residual)
constexpr uint32_t bV = 131072;              // 2 x 16 KB: v rows, two 64-column panels of 64 rows
constexpr uint32_t bD = 163840;              // 2 x 16 KB: dO rows, same layout
constexpr uint32_t bO = 196608;              // 16 KB: dV rows on their way out
constexpr uint32_t bI = 212992;              // 8 KB: identity panel
constexpr uint32_t kScanBwdSmem = 221184;

struct ScanBwdBars {
  uint64_t *mma_bar, *qk_bar, *x_bar, *p_bar, *v_bar, *d_bar;
};
__device__ __forceinline__ bool scan_bwd_mma1(uint32_t tbase, uint32_t sb, int s, ScanBwdBars bars, int* status, bool dead, uint32_t lead) {
  const int b = s & 1;
  const uint32_t ph = (s >> 1) & 1;
  tc_fence_after();
  if (!dead && !mbar_wait(&bars.qk_bar[b], ph, status, FLA_ERR_TIMEOUT)) dead = true;
  const Operand opK{sb + bQK + b * 32768 + 8192, 16384, 0};          // k rows as B: N = 64 tokens, reduction over key dims
  mma_tile_ts(tbase + uW, tbase + uAh, opK, 64, 8, false, lead);
  mma_tile_ts(tbase + uW, tbase + uAl, opK, 64, 8, true, lead);
  if (!dead && !mbar_wait(&bars.d_bar[b], ph, status, FLA_ERR_TIMEOUT)) dead = true;
  if (!dead && !mbar_wait(&bars.p_bar[b], ph, status, FLA_ERR_TIMEOUT)) dead = true;
  const Operand opDt{sb + bD + b * 16384, 8192, 1};                  // dO^T: M = 128 channels over two panels, reduction over tokens
  const Operand opPh{sb + bP + b * 16384, 1024, 2}, opPl{sb + bP + b * 16384 + 8192, 1024, 2};   // P (strips of 8 columns j = N) with its rows as the reduction
  mma_tile(tbase + uU, opDt, opPh, 128, 64, 4, false, lead);
  mma_tile(tbase + uU, opDt, opPl, 128, 64, 4, true, lead);
  mma_commit(bars.mma_bar, lead);
  return dead;
}
__device__ __forceinline__ bool scan_bwd_mma2(uint32_t tbase, uint32_t sb, int s, ScanBwdBars bars, int* status, bool dead, uint32_t lead) {
  const int b = s & 1;
  const uint32_t ph = (s >> 1) & 1;
  tc_fence_after();
  if (!dead && !mbar_wait(&bars.x_bar[b], ph, status, FLA_ERR_TIMEOUT)) dead = true;
  // X in strips of 8 rows, read with its rows as the reduction dim: X^T dVn
  const Operand opXh{sb + bX + b * 16384, 1024, 3}, opXl{sb + bX + b * 16384 + 8192, 1024, 3};
  mma_tile_ts(tbase + uW, tbase + uDVh, opXh, 64, 4, false, lead);
  mma_tile_ts(tbase + uW, tbase + uDVl, opXh, 64, 4, true, lead);
  mma_tile_ts(tbase + uW, tbase + uDVh, opXl, 64, 4, true, lead);
  if (!dead && !mbar_wait(&bars.v_bar[b], ph, status, FLA_ERR_TIMEOUT)) dead = true;
  const Operand opI{sb + bI, 8192, 0};
  const Operand opDt{sb + bD + b * 16384, 8192, 1}, opVt{sb + bV + b * 16384, 8192, 1};
  mma_tile(tbase + uU, opDt, opI, 128, 64, 4, false, lead);                // dO^T, exact
  mma_tile(tbase + uVT, opVt, opI, 128, 64, 4, false, lead);               // V^T, exact
  mma_commit(bars.mma_bar, lead);
  return dead;
}
__device__ __forceinline__ bool scan_bwd_mma3(uint32_t tbase, uint32_t sb, int s, ScanBwdBars bars, bool dead, uint32_t lead) {
  const int b = s & 1;
  tc_fence_after();
  const Operand opQK{sb + bQK + b * 32768, 16384, 1};                // [q; k] rows as the reduction, N = 128 key dims
  mma_tile_ts(tbase + uDS, tbase + uAh, opQK, 128, 8, true, lead);
  mma_tile_ts(tbase + uDS, tbase + uAl, opQK, 128, 8, true, lead);
  mma_commit(bars.mma_bar, lead);
  return dead;
}

// 32 values per lane -> lane l keeps the sum over the warp of value l (recursive halving: 31 shuffles)
__device__ __forceinline__ float warp_transpose_reduce32(float* x, int lane) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    const bool up = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < off; ++i) {
      const float send = up ? x[i] : x[i + off];
      const float keep = up ? x[i + off] : x[i];
      x[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
  return x[0];
}

__global__ void __launch_bounds__(kScanThreads, 1) gdn_scan_bwd_kernel(GdnBwdParams p, const __grid_constant__ CUtensorMap tm_q,
                                                                        const __grid_constant__ CUtensorMap tm_k,
                                                                        const __grid_constant__ CUtensorMap tm_v,
                                                                        const __grid_constant__ CUtensorMap tm_d) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ ScanFactors fac[3];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t mma_bar, qk_bar[2], x_bar[2], p_bar[2], v_bar[2], d_bar[2], f_bar[3];

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int vb = blockIdx.x, hv = blockIdx.y, n = blockIdx.z + p.n0;
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
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qk_bar[i], 1);
      mbar_init(&x_bar[i], 1);
      mbar_init(&p_bar[i], 1);
      mbar_init(&v_bar[i], 1);
      mbar_init(&d_bar[i], 1);
    }
    for (int i = 0; i < 3; ++i) mbar_init(&f_bar[i], 1);
    mbar_init_fence();
  }
  write_identity_panel(smem + bI, tid, kScanThreads);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = tmem_base_s;
  bool dead = false;
  // chunks are visited last to first; step s = 0, 1, ... handles chunk nt - 1 - s and uses the buffers of parity s & 1

  if (warp == 8) {
    // ============================================================ helper warp: TMA loads and per-token factors
    auto issue_loads = [&](int s) {
      const int c = nt - 1 - s, b = s & 1, row0 = sq.bos + c * kC;
      const uint32_t qk = sb + bQK + b * 32768;
      mbar_arrive_expect_tx(&qk_bar[b], 32768);
      tma_load_tile(qk, &tm_q, 0, hk, row0, &qk_bar[b]);
      tma_load_tile(qk + 16384, &tm_q, 64, hk, row0, &qk_bar[b]);
      tma_load_tile(qk + 8192, &tm_k, 0, hk, row0, &qk_bar[b]);
      tma_load_tile(qk + 16384 + 8192, &tm_k, 64, hk, row0, &qk_bar[b]);
      mbar_arrive_expect_tx(&d_bar[b], 16384);
      tma_load_tile(sb + bD + b * 16384, &tm_d, vb * 128, hv, row0, &d_bar[b]);
      tma_load_tile(sb + bD + b * 16384 + 8192, &tm_d, vb * 128 + 64, hv, row0, &d_bar[b]);
      mbar_arrive_expect_tx(&p_bar[b], 16384);
      bulk_load(sb + bP + b * 16384, p.p_img + ((int64_t(sq.cbase) + c) * p.HV + hv) * kPImg, 16384, &p_bar[b]);
      mbar_arrive_expect_tx(&x_bar[b], 16384);
      bulk_load(sb + bX + b * 16384, p.X + ((int64_t(sq.cbase) + c) * p.HV + hv) * 8192, 16384, &x_bar[b]);
      mbar_arrive_expect_tx(&v_bar[b], 16384);
      tma_load_tile(sb + bV + b * 16384, &tm_v, vb * 128, hv, row0, &v_bar[b]);
      tma_load_tile(sb + bV + b * 16384 + 8192, &tm_v, vb * 128 + 64, hv, row0, &v_bar[b]);
    };
    // the per-token factors of step s (chunk nt - 1 - s; made by the prep kernel, behind the chunk's P tile) into buffer s % 3
    auto load_factors = [&](int s) {
      if (s < nt) {
        const int c = nt - 1 - s;
        mbar_arrive_expect_tx(&f_bar[s % 3], uint32_t(sizeof(ScanFactors)));
        bulk_load(smem_u32(&fac[s % 3]), reinterpret_cast<const uint8_t*>(p.p_img + ((int64_t(sq.cbase) + c) * p.HV + hv) * kPImg) + kPTileBytes,
                  uint32_t(sizeof(ScanFactors)), &f_bar[s % 3]);
      }
    };
    if (lane == 0) {
      tma_prefetch_descriptor(&tm_q);
      tma_prefetch_descriptor(&tm_k);
      tma_prefetch_descriptor(&tm_v);
      tma_prefetch_descriptor(&tm_d);
      if (nt > 0) issue_loads(0);
      load_factors(0);
      load_factors(1);
    }
    __syncwarp();
    scan_sync();   // (pairs with the epilogue warps' barrier after they have loaded the final-state gradient)
    for (int s = 0; s < nt; ++s) {
      scan_sync();                                          // sync 1: step s - 1 no longer reads the other buffers
      if (lane == 0) {
        if (s + 1 < nt) issue_loads(s + 1);
        load_factors(s + 2);                                // buffer (s + 2) % 3 was last read by step s - 1
      }
      __syncwarp();
      scan_sync();                                          // sync 2
      scan_sync();                                          // sync 3
    }
    scan_sync();
    return;
  }

  // ================================================================ epilogue warps
  const ScanBwdBars bars{&mma_bar, qk_bar, x_bar, p_bar, v_bar, d_bar};
  // products: one elected lane of warp 0 in code the whole warp runs, so that the descriptors are warp-uniform values
  const int warp_u = __shfl_sync(0xffffffffu, warp, 0);
  const uint32_t tbase_u = __shfl_sync(0xffffffffu, tbase, 0), sb_u = __shfl_sync(0xffffffffu, sb, 0);
  const int quad = warp & 3, half = warp >> 2;
  const int vrow = quad * 32 + lane;
  const uint32_t tlane = tmem_addr(tbase, quad * 32, 0);
  const int t_lo = half * 32;
  const int k_lo = half * 64;
  uint32_t mphase = 0;

  {   // dht (or zero) into the accumulator columns
    const float* src = p.dht ? p.dht + ((int64_t(n) * p.HV + hv) * kK + k_lo) * p.V + vb * 128 + vrow : nullptr;
#pragma unroll
    for (int part = 0; part < 4; ++part) {
      float s16[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) s16[i] = src ? src[int64_t(part * 16 + i) * p.V] : 0.f;
      tmem_st16(tlane + uDS + k_lo + part * 16, s16);
    }
    tmem_st_wait();
  }
  // The dO rows of a ragged last chunk that lie past the end of the sequence belong to whatever follows in memory: they
  // are zeroed in shared memory (every other operand meets a zero row of beta or of dVn there).
  if (nt > 0 && sq.len - (nt - 1) * kC < kC) {
    const int rows = sq.len - (nt - 1) * kC;
    if (!mbar_wait(&d_bar[0], 0, p.status, FLA_ERR_TIMEOUT)) dead = true;
    for (int idx = tid; idx < (kC - rows) * 16; idx += kScanEpiThreads) {
      const int r = rows + idx / 16, pc = idx % 16;
      *reinterpret_cast<uint4*>(smem + bD + (pc >> 3) * 8192 + panel_chunk_off(r, pc & 7)) = make_uint4(0, 0, 0, 0);
    }
    fence_async_smem();
  }
  scan_sync();   // factors of the first step are visible

  // dV rows of the chunk handled in step s: formed in the second epilogue, stored while the state update runs
  float ov[32];
  auto store_dv = [&](int c) {
    const int rows = min(kC, sq.len - c * kC);
    const int64_t off = (int64_t(sq.bos) + c * kC) * p.dv_st + hv * p.dv_sh + vb * 128;
    void* g = p.grads_f32 ? static_cast<void*>(static_cast<float*>(p.dv) + off) : static_cast<void*>(static_cast<bf16*>(p.dv) + off);
    store_rows_transposed(smem + bO, ov, g, p.dv_st, p.grads_f32 != 0, rows, half, vrow, tid);
  };

  for (int s = 0; s < nt; ++s) {
    const int c = nt - 1 - s;
    const ScanFactors& f = fac[s % 3];
    if (!dead && !mbar_wait(&f_bar[s % 3], (s / 3) & 1, p.status, FLA_ERR_TIMEOUT)) dead = true;   // requested two steps ago
    const int rows = min(kC, sq.len - c * kC);
    const int64_t cidx = ((int64_t(sq.cbase) + c) * p.HV + hv) * (p.V / 128) + vb;

    // ---- A: publish dS' (the gradient entering this chunk): bf16 value + residual as A operand, decayed copy as accumulator
    {
      const float dl = f.dl;
      uint8_t* s_row = reinterpret_cast<uint8_t*>(p.ds_img + cidx * 32768) + (vrow >> 6) * 32768 + (vrow & 63) * 16;
#pragma unroll 1
      for (int g4 = 0; g4 < 4; ++g4) {
        float s16[16];
        tmem_ld16(tlane + uDS + k_lo + g4 * 16, s16);
        tmem_ld_wait();
        uint32_t hi[8], lo[8];
        split16(s16, hi, lo);
        tmem_st8u(tlane + uAh + half * 32 + g4 * 8, hi);
        tmem_st8u(tlane + uAl + half * 32 + g4 * 8, lo);
        {   // the dS' image for the chunk-parallel kernel: strips half * 8 + g4 * 2 and the next one of my channel's row
          uint8_t* dst = s_row + (half * 8 + g4 * 2) * 1024;
          *reinterpret_cast<uint4*>(dst) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
          *reinterpret_cast<uint4*>(dst + 1024) = make_uint4(hi[4], hi[5], hi[6], hi[7]);
          *reinterpret_cast<uint4*>(dst + 16384) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
          *reinterpret_cast<uint4*>(dst + 16384 + 1024) = make_uint4(lo[4], lo[5], lo[6], lo[7]);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) s16[i] *= dl;
        tmem_st16(tlane + uDS + k_lo + g4 * 16, s16);
        group_fence();
      }
      tmem_st_wait();
    }
    tc_fence_before();
    scan_sync();                                   // sync 1
    tc_fence_after();
    if (warp_u == 0) dead = scan_bwd_mma1(tbase_u, sb_u, s, bars, p.status, dead, elect_one());
    wait_or_mark(&mma_bar, mphase, dead, p.status);
    tc_fence_after();

    // ---- B: dVn^T = scale U1^T + e^{gam_L-gam} W1^T (zero past the end of the sequence) for my 32 tokens
    {
#pragma unroll 1
      for (int g = 0; g < 2; ++g) {
        float w1[16], u1[16];
        tmem_ld16(tlane + uW + t_lo + g * 16, w1);
        tmem_ld16(tlane + uU + t_lo + g * 16, u1);
        tmem_ld_wait();
#pragma unroll
        for (int i4 = 0; i4 < 16; i4 += 4) {
          const float4 d4 = *reinterpret_cast<const float4*>(&f.dk[t_lo + g * 16 + i4]);
          const float dv4[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int i = i4 + j;
            u1[i] = (t_lo + g * 16 + i < rows) ? p.scale * u1[i] + dv4[j] * w1[i] : 0.f;
          }
        }
        uint32_t hi[8], lo[8];
        split16(u1, hi, lo);
        tmem_st8u(tlane + uDVh + half * 16 + g * 8, hi);
        tmem_st8u(tlane + uDVl + half * 16 + g * 8, lo);
        group_fence();
      }
      tmem_st_wait();
    }
    tc_fence_before();
    scan_sync();                                   // sync 2
    tc_fence_after();
    if (warp_u == 0) dead = scan_bwd_mma2(tbase_u, sb_u, s, bars, p.status, dead, elect_one());
    wait_or_mark(&mma_bar, mphase, dead, p.status);
    tc_fence_after();

    // ---- C: dZ^T -> dV rows, partial sums of dZ V, the [dO^T | dZ^T] image, the operand [scale e^gam dO^T | -beta e^gam dZ^T]
    {
      // the [dO^T | dZ^T] image: my channel's row of strips half * 4 + g * 2 and the next one
      uint8_t* img = reinterpret_cast<uint8_t*>(p.dz_img + cidx * (2 * kDzHalf)) + (vrow >> 6) * (2 * kDzHalf) + (vrow & 63) * 16;
      float pr[32];
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        float dz[16], t16[16];
        tmem_ld16(tlane + uW + t_lo + g * 16, dz);
        tmem_ld16(tlane + uVT + t_lo + g * 16, t16);     // V^T
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) pr[g * 16 + i] = dz[i] * t16[i];
        uint32_t w8[8];
        {
          uint32_t zl[8];
          split16(dz, w8, zl);     // dZ as value + residual: dA = -tril(dZ Vn^T) feeds dk, dg, dbeta through cancelling sums
          *reinterpret_cast<uint4*>(img + 8192 + (half * 4 + g * 2) * 1024) = make_uint4(w8[0], w8[1], w8[2], w8[3]);
          *reinterpret_cast<uint4*>(img + 8192 + (half * 4 + g * 2 + 1) * 1024) = make_uint4(w8[4], w8[5], w8[6], w8[7]);
          *reinterpret_cast<uint4*>(img + 16384 + (half * 4 + g * 2) * 1024) = make_uint4(zl[0], zl[1], zl[2], zl[3]);
          *reinterpret_cast<uint4*>(img + 16384 + (half * 4 + g * 2 + 1) * 1024) = make_uint4(zl[4], zl[5], zl[6], zl[7]);
        }
#pragma unroll
        for (int i4 = 0; i4 < 16; i4 += 4) {
          const float4 b4 = *reinterpret_cast<const float4*>(&f.b[t_lo + g * 16 + i4]);
          const float4 g4 = *reinterpret_cast<const float4*>(&f.bg[t_lo + g * 16 + i4]);
          ov[g * 16 + i4] = b4.x * dz[i4];         dz[i4] *= -g4.x;
          ov[g * 16 + i4 + 1] = b4.y * dz[i4 + 1]; dz[i4 + 1] *= -g4.y;
          ov[g * 16 + i4 + 2] = b4.z * dz[i4 + 2]; dz[i4 + 2] *= -g4.z;
          ov[g * 16 + i4 + 3] = b4.w * dz[i4 + 3]; dz[i4 + 3] *= -g4.w;
        }
        uint32_t hi[8], lo[8];
        split16(dz, hi, lo);                              // dR^T: rows 64..127 of the [q; k] reduction = columns 32..63 of the operand
        tmem_st8u(tlane + uAh + 32 + half * 16 + g * 8, hi);
        tmem_st8u(tlane + uAl + 32 + half * 16 + g * 8, lo);
        tmem_ld16(tlane + uU + t_lo + g * 16, t16);       // dO^T
        tmem_ld_wait();
        pack16(t16, w8);                                  // exact: these are the bf16 inputs
        *reinterpret_cast<uint4*>(img + (half * 4 + g * 2) * 1024) = make_uint4(w8[0], w8[1], w8[2], w8[3]);
        *reinterpret_cast<uint4*>(img + (half * 4 + g * 2 + 1) * 1024) = make_uint4(w8[4], w8[5], w8[6], w8[7]);
#pragma unroll
        for (int i4 = 0; i4 < 16; i4 += 4) {
          const float4 s4 = *reinterpret_cast<const float4*>(&f.se[t_lo + g * 16 + i4]);
          t16[i4] *= s4.x; t16[i4 + 1] *= s4.y; t16[i4 + 2] *= s4.z; t16[i4 + 3] *= s4.w;
        }
        split16(t16, hi, lo);                             // scale e^gam dO^T: rows 0..63 of the reduction
        tmem_st8u(tlane + uAh + half * 16 + g * 8, hi);
        tmem_st8u(tlane + uAl + half * 16 + g * 8, lo);
        group_fence();
      }
      tmem_st_wait();
      // sum over my warp's 32 channels of dZ V for each of my 32 tokens; lane l ends up with token t_lo + l
      const float bzsum = warp_transpose_reduce32(pr, lane);
      if (t_lo + lane < rows)
        p.bz[(int64_t(vb * 4 + quad) * p.total_tokens + int64_t(sq.bos) + c * kC + t_lo + lane) * p.HV + hv] = bzsum;
    }
    tc_fence_before();
    scan_sync();                                   // sync 3
    tc_fence_after();
    if (warp_u == 0) dead = scan_bwd_mma3(tbase_u, sb_u, s, bars, dead, elect_one());
    store_dv(c);                                   // while the state-gradient update runs
    wait_or_mark(&mma_bar, mphase, dead, p.status);
    tc_fence_after();
  }

  if (!dead && p.dh0) {
    float* dst = p.dh0 + ((int64_t(n) * p.HV + hv) * kK + k_lo) * p.V + vb * 128 + vrow;
#pragma unroll
    for (int part = 0; part < 4; ++part) {
      float s16[16];
      tmem_ld16(tlane + uDS + k_lo + part * 16, s16);
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

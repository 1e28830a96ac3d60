// Forward scan of the chunked gated delta rule (recompute_w_u + chunk_gated_delta_rule_fwd_h + chunk_fwd_o of the
// reference, examples/flash_gated_delta_rule.py:840-880, with the WY factors folded away).
//
// One CTA per (sequence, value head, 128-column block of V); the state lives transposed in tensor memory for the whole
// sequence (scan_common.cuh).  Per chunk, with S the state at chunk start, gam the chunk-local cumulative log decay,
// X = (I + A)^-1 and P = tril(Q K^T e^{gam_i-gam_j}) from the prep kernels:
//     [QS^T | KS^T] = S^T [Q; K]^T          N = 128 tokens of the [q; k] panel, reduction over the 128 key dims
//     Z^T     = beta (V^T - e^gam KS^T)     epilogue; V^T arrives through an identity product
//     v_new^T = Z^T X^T                     N = 64
//     S^T    <- e^{gam_L} S^T + vhat^T K    N = 128 key dims, reduction over the 64 tokens, vhat = e^{gam_L-gam} v_new
//     o^T     = scale (e^gam QS^T + v_new^T P^T)
// Operands the result is sensitive to (state copy, Z, v_new, vhat, P) are a bf16 value plus a bf16 residual and enter
// two or three products; q, k, v enter as the exact bf16 inputs; accumulation is fp32.
// For the backward the kernel saves, per (chunk, head, block), the state and v_new as ready-made operand panels
// whose rows are value channels:
//     s_img   [value | residual] x [key dims 0-63 | 64-127] x 128 rows (v) x 64 columns   = 64 KB
//     vn_img  [value | residual] x 128 rows (v) x 64 columns (tokens)                      = 32 KB
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

// shared memory (offsets from a 1024-byte aligned base).  The [q; k] panels exist twice (chunk parity): k is read by the
// last product of a chunk and q, k of the next chunk by the first one right after.  X, P and the v rows have one buffer
// each: they are reloaded as soon as the product that reads them has completed, most of a chunk before their next use.
constexpr uint32_t sQK = 0;                  // 2 x 32 KB: [q; k] rows, two 64-column panels of 128 rows
constexpr uint32_t sX = 65536;               // 8 KB
constexpr uint32_t sP = 73728;               // 16 KB (value, residual)
constexpr uint32_t sV = 90112;               // 16 KB: v rows of the chunk, two 64-column panels of 64 rows
constexpr uint32_t sO = 106496;              // 16 KB: the chunk's output rows on their way out
constexpr uint32_t sI = 122880;              // 8 KB: identity panel
constexpr uint32_t sG = 131072;              // 64 KB: the saved panels of a chunk on their way out (state image, then v_new image)
constexpr uint32_t kScanFwdSmem = 196608;
constexpr uint32_t sX2 = sG, sP2 = sG + 8192, sV2 = sG + 24576;   // second buffers (forward without saving only)

struct ScanBars {
  uint64_t *mma_bar, *o_bar, *qk_bar, *x_bar, *p_bar, *v_bar;   // x / p / v: two barriers each (index = buffer)
};
// Where chunk c finds its X, P and v rows.  While saving for the backward the staging panels take the space of the
// second buffers: there is one buffer, used by every chunk (barrier parity = chunk parity).  Otherwise there are two
// (the second set lies in the staging area) and chunk c uses buffer c & 1 (parity (c >> 1) & 1).
template <bool kSave>
struct ScanBuf {
  __device__ static int buf(int c) { return kSave ? 0 : (c & 1); }
  __device__ static uint32_t par(int c) { return kSave ? uint32_t(c & 1) : uint32_t((c >> 1) & 1); }
};
// The three batches of products of one chunk, each issued by one thread.  Kept out of line: inlined into the epilogue
// code their unrolled descriptor arithmetic costs registers the accumulator rows need.
template <bool kSave>
__device__ __noinline__ bool scan_fwd_mma1(uint32_t tbase, uint32_t sb, int c, ScanBars bars, int* status, bool dead) {
  const int b = c & 1, xb = ScanBuf<kSave>::buf(c);
  const uint32_t ph = (c >> 1) & 1, xph = ScanBuf<kSave>::par(c);
  tc_fence_after();
  if (!dead && !mbar_wait(&bars.qk_bar[b], ph, status, FLA_ERR_TIMEOUT)) dead = true;
  const Operand opKQ{sb + sQK + b * 32768, 16384, 0};
  mma_tile_ts(tbase + tKQ, tbase + tSAh, opKQ, 128, 8, false);
  mma_tile_ts(tbase + tKQ, tbase + tSAl, opKQ, 128, 8, true);
  // V^T into the columns the decayed v_new of this chunk will occupy later
  if (!dead && !mbar_wait(&bars.v_bar[xb], xph, status, FLA_ERR_TIMEOUT)) dead = true;
  const Operand opVt{sb + (xb ? sV2 : sV), 8192, 1}, opI{sb + sI, 8192, 0};
  mma_tile(tbase + tVAh, opVt, opI, 128, 64, 4, false);
  mma_commit(bars.mma_bar);
  return dead;
}
template <bool kSave>
__device__ __noinline__ bool scan_fwd_mma2(uint32_t tbase, uint32_t sb, int c, ScanBars bars, int* status, bool dead) {
  const int xb = ScanBuf<kSave>::buf(c);
  tc_fence_after();
  if (!dead && !mbar_wait(&bars.x_bar[xb], ScanBuf<kSave>::par(c), status, FLA_ERR_TIMEOUT)) dead = true;
  const Operand opX{sb + (xb ? sX2 : sX), 8192, 0};
  mma_tile_ts(tbase + tVN, tbase + tZAh, opX, 64, 4, false);
  mma_tile_ts(tbase + tVN, tbase + tZAl, opX, 64, 4, true);
  mma_commit(bars.mma_bar);
  return dead;
}
template <bool kSave>
__device__ __noinline__ bool scan_fwd_mma3(uint32_t tbase, uint32_t sb, int c, ScanBars bars, int* status, bool dead) {
  const int b = c & 1, xb = ScanBuf<kSave>::buf(c);
  tc_fence_after();
  const Operand opK{sb + sQK + b * 32768 + 8192, 16384, 1};   // k rows: reduction over tokens, N = 128 key dims over two panels
  mma_tile_ts(tbase + tST, tbase + tVAh, opK, 128, 4, true);
  mma_tile_ts(tbase + tST, tbase + tVAl, opK, 128, 4, true);
  mma_commit(bars.mma_bar);                                   // the state update: what the next chunk waits for
  if (!dead && !mbar_wait(&bars.p_bar[xb], ScanBuf<kSave>::par(c), status, FLA_ERR_TIMEOUT)) dead = true;
  const uint32_t pp = sb + (xb ? sP2 : sP);
  const Operand opPh{pp, 8192, 0}, opPl{pp + 8192, 8192, 0};
  mma_tile_ts(tbase + tVN, tbase + tZAh, opPh, 64, 4, false);
  mma_tile_ts(tbase + tVN, tbase + tZAl, opPh, 64, 4, true);
  mma_tile_ts(tbase + tVN, tbase + tZAh, opPl, 64, 4, true);
  mma_commit(bars.o_bar);                                     // the output product: read when the next chunk's state is out
  return dead;
}

template <bool kSave>
__global__ void __launch_bounds__(kScanThreads, 1) gdn_scan_fwd_kernel(GdnFwdParams p, const __grid_constant__ CUtensorMap tm_q,
                                                                        const __grid_constant__ CUtensorMap tm_k,
                                                                        const __grid_constant__ CUtensorMap tm_x,
                                                                        const __grid_constant__ CUtensorMap tm_v) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ ScanFactors fac[3];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t mma_bar, o_bar, qk_bar[2], x_bar[2], p_bar[2], v_bar[2];

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
    mbar_init_fence();
  }
  write_identity_panel(smem + sI, tid, kScanThreads);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = tmem_base_s;
  bool dead = false;

  if (warp == 8) {
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
    auto load_v = [&](int c) {
      const int row0 = sq.bos + c * kC, xb = ScanBuf<kSave>::buf(c);
      const uint32_t dst = sb + (xb ? sV2 : sV);
      mbar_arrive_expect_tx(&v_bar[xb], 16384);
      tma_load_tile(dst, &tm_v, vb * 128, hv, row0, &v_bar[xb]);
      tma_load_tile(dst + 8192, &tm_v, vb * 128 + 64, hv, row0, &v_bar[xb]);
    };
    auto load_x = [&](int c) {
      const int xb = ScanBuf<kSave>::buf(c);
      mbar_arrive_expect_tx(&x_bar[xb], 8192);
      tma_load_tile(sb + (xb ? sX2 : sX), &tm_x, 0, hv, sq.bos + c * kC, &x_bar[xb]);
    };
    auto load_p = [&](int c) {
      const int xb = ScanBuf<kSave>::buf(c);
      mbar_arrive_expect_tx(&p_bar[xb], 16384);
      bulk_load(sb + (xb ? sP2 : sP), p.p_img + ((int64_t(sq.cbase) + c) * p.HV + hv) * 8192, 16384, &p_bar[xb]);
    };
    // lane l handles tokens l and l + 32; the raw values of a chunk are requested two chunks ahead and wait in registers
    float pf_g[2] = {0.f, 0.f}, pf_b[2] = {0.f, 0.f}, pf_gl = 0.f;
    auto load_scalars = [&](int c) {
      if (c < nt) {
        const int rows = min(kC, sq.len - c * kC);
        const int64_t tok0 = int64_t(sq.bos) + c * kC;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int t = lane + 32 * j;
          // rows past the end of the sequence carry the last valid cumulative decay so every exponent stays finite
          pf_g[j] = p.gam[(tok0 + min(t, rows - 1)) * p.HV + hv];
          pf_b[j] = t < rows ? ld_scalar(p.beta, (tok0 + t) * p.beta_st + hv, p.beta_is_f32) : 0.f;
        }
        pf_gl = p.gam[(tok0 + rows - 1) * p.HV + hv];
      }
    };
    auto make_factors = [&](int c) {
      if (c < nt) {
        ScanFactors& f = fac[c % 3];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int t = lane + 32 * j;
          const float eg = __expf(pf_g[j]);
          f.b[t] = pf_b[j];
          f.bg[t] = pf_b[j] * eg;
          f.se[t] = p.scale * eg;
          f.dk[t] = __expf(pf_gl - pf_g[j]);
        }
        if (lane == 0) f.dl = __expf(pf_gl);
      }
    };
    if (lane == 0) {
      tma_prefetch_descriptor(&tm_q);
      tma_prefetch_descriptor(&tm_k);
      tma_prefetch_descriptor(&tm_x);
      tma_prefetch_descriptor(&tm_v);
      if (nt > 0) {
        load_qk(0);
        load_v(0);
        load_x(0);
        load_p(0);
      }
    }
    __syncwarp();
    load_scalars(0);
    make_factors(0);
    load_scalars(1);
    scan_sync();   // factors of chunk 0 are visible
    uint32_t mphase = 0, ophase = 0;
    for (int c = 0; c < nt; ++c) {
      const bool more = c + 1 < nt;
      scan_sync();                                          // sync 1: chunk c - 1 no longer reads the other [q; k] buffer
      if (lane == 0) {
        if (more) load_qk(c + 1);
        if (!kSave && more) {                               // two buffers: chunk c - 1, their last reader, has completed
          load_v(c + 1);
          load_x(c + 1);
          load_p(c + 1);
        }
        if (kSave) {
          lazy_wait_or_mark(&mma_bar, mphase, dead, p.status);   // the first batch of products has read the v rows
          if (more) load_v(c + 1);
        }
      }
      __syncwarp();
      make_factors(c + 1);                                  // read from sync 3 of this chunk on
      load_scalars(c + 2);
      scan_sync();                                          // sync 2
      if (lane == 0) {
        if (kSave) {
          lazy_wait_or_mark(&mma_bar, mphase, dead, p.status);   // X has been read
          if (more) load_x(c + 1);
        }
      }
      __syncwarp();
      scan_sync();                                          // sync 3
      if (lane == 0) {
        if (kSave) {
          lazy_wait_or_mark(&mma_bar, mphase, dead, p.status);
          lazy_wait_or_mark(&o_bar, ophase, dead, p.status);     // the output product has read P
          if (more) load_p(c + 1);
        }
      }
      __syncwarp();
    }
    scan_sync();   // matches the epilogue warps' barrier before the TMEM is released
    return;
  }

  // ================================================================ epilogue warps
  const ScanBars bars{&mma_bar, &o_bar, qk_bar, x_bar, p_bar, v_bar};
  const int quad = warp & 3, half = warp >> 2;
  const int vrow = quad * 32 + lane;                       // my value channel inside the block = my TMEM lane
  const uint32_t tlane = tmem_addr(tbase, quad * 32, 0);
  const int t_lo = half * 32;                              // my 32 tokens of a token-indexed tile
  const int k_lo = half * 64;                              // my 64 key dims of the state row
  uint32_t mphase = 0, ophase = 0;

  // the initial state goes straight into the accumulator columns: every chunk starts by reading its state from there
  {
    const float* src = p.h0 ? p.h0 + ((int64_t(n) * p.HV + hv) * kK + k_lo) * p.V + vb * 128 + vrow : nullptr;
#pragma unroll
    for (int part = 0; part < 4; ++part) {
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
  float ov[32];
  auto form_o = [&](int c) {
    const ScanFactors& f = fac[c % 3];
#pragma unroll
    for (int g = 0; g < 2; ++g) {
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
    store_rows_transposed(smem + sO, ov, g, p.o_st, p.o_is_f32 != 0, rows, half, vrow, tid);
  };

  for (int c = 0; c < nt; ++c) {
    const ScanFactors& f = fac[c % 3];
    const int rows = min(kC, sq.len - c * kC);
    const int64_t cidx = ((int64_t(sq.cbase) + c) * p.HV + hv) * (p.V / 128) + vb;

    // ---- A: publish the state at chunk start: bf16 value + residual as A operand, decayed fp32 copy as accumulator
    {
      const float dl = f.dl;
#pragma unroll
      for (int g4 = 0; g4 < 4; ++g4) {                   // 16 key dims at a time: 8 packed columns per operand store
        float s16[16];
        tmem_ld16(tlane + tST + k_lo + g4 * 16, s16);
        tmem_ld_wait();
        uint32_t hi[8], lo[8];
        split16(s16, hi, lo);
        tmem_st8u(tlane + tSAh + half * 32 + g4 * 8, hi);
        tmem_st8u(tlane + tSAl + half * 32 + g4 * 8, lo);
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
    if (tid == 0) {
      dead = scan_fwd_mma1<kSave>(tbase, sb, c, bars, p.status, dead);
      if (kSave) bulk_wait_read();                 // the v_new image of chunk c - 1 has left the staging panels
    }
    // ---- while [QS^T | KS^T] runs: output rows of chunk c - 1, saved state image
    if (c > 0) store_o(c - 1);
    if (kSave) {
      epi_sync();                                  // ... and every thread knows it
      // The state image: every thread copies its row of the operand just published (value, residual: 2 x 128 bytes)
      // from tensor memory into the staging panels; one bulk copy then moves the 64 KB to global memory.  Stores made
      // by the threads themselves would be 16-byte pieces 128 bytes apart: measured 0.4 ms per launch.
      uint8_t* stg = smem + sG;
      uint32_t w[16];
#pragma unroll
      for (int part = 0; part < 4; ++part) {             // my 64 key dims = one panel row = 8 pieces of 16 bytes; 16 columns per load
        tmem_ld16u(tlane + ((part < 2) ? tSAh : tSAl) + half * 32 + (part & 1) * 16, w);
        tmem_ld_wait();
        uint8_t* dst = stg + (part < 2 ? 0 : 32768) + half * 16384;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch)
          *reinterpret_cast<uint4*>(dst + panel_chunk_off(vrow, (part & 1) * 4 + ch)) = make_uint4(w[4 * ch], w[4 * ch + 1], w[4 * ch + 2], w[4 * ch + 3]);
      }
      fence_async_smem();
      epi_sync();
      if (tid == 0) {
        bulk_store(p.s_img + cidx * 32768, sb + sG, 32768);
        bulk_store(p.s_img + cidx * 32768 + 16384, sb + sG + 32768, 32768);
        bulk_commit();
      }
    }
    wait_or_mark(&mma_bar, mphase, dead, p.status);
    tc_fence_after();

    // ---- C: Z^T = beta (V^T - e^gam KS^T) for my 32 tokens
    {
#pragma unroll
      for (int g = 0; g < 2; ++g) {
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
        tmem_st8u(tlane + tZAh + half * 16 + g * 8, hi);
        tmem_st8u(tlane + tZAl + half * 16 + g * 8, lo);
        group_fence();
      }
      tmem_st_wait();
    }
    tc_fence_before();
    scan_sync();                                   // sync 2
    tc_fence_after();
    if (tid == 0) {
      dead = scan_fwd_mma2<kSave>(tbase, sb, c, bars, p.status, dead);
      if (kSave) bulk_wait_read();                 // the state image has left the staging panels
    }
    wait_or_mark(&mma_bar, mphase, dead, p.status);
    tc_fence_after();
    if (kSave) epi_sync();

    // ---- E: v_new^T (rows past the end of the sequence are zero) and its decayed copy
    {
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        float vn[16];
        tmem_ld16(tlane + tVN + t_lo + g * 16, vn);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) vn[i] = (t_lo + g * 16 + i < rows) ? vn[i] : 0.f;
        uint32_t hi[8], lo[8];
        split16(vn, hi, lo);
        tmem_st8u(tlane + tZAh + half * 16 + g * 8, hi);
        tmem_st8u(tlane + tZAl + half * 16 + g * 8, lo);
        if (kSave) {                                 // v_new image (value panel, residual panel) into the staging panels
          uint8_t* stg = smem + sG;
#pragma unroll
          for (int ch = 0; ch < 2; ++ch) {
            *reinterpret_cast<uint4*>(stg + panel_chunk_off(vrow, half * 4 + g * 2 + ch)) = make_uint4(hi[4 * ch], hi[4 * ch + 1], hi[4 * ch + 2], hi[4 * ch + 3]);
            *reinterpret_cast<uint4*>(stg + 16384 + panel_chunk_off(vrow, half * 4 + g * 2 + ch)) = make_uint4(lo[4 * ch], lo[4 * ch + 1], lo[4 * ch + 2], lo[4 * ch + 3]);
          }
        }
#pragma unroll
        for (int i4 = 0; i4 < 16; i4 += 4) {
          const float4 d4 = *reinterpret_cast<const float4*>(&f.dk[t_lo + g * 16 + i4]);
          vn[i4] *= d4.x; vn[i4 + 1] *= d4.y; vn[i4 + 2] *= d4.z; vn[i4 + 3] *= d4.w;
        }
        split16(vn, hi, lo);
        tmem_st8u(tlane + tVAh + half * 16 + g * 8, hi);
        tmem_st8u(tlane + tVAl + half * 16 + g * 8, lo);
        group_fence();
      }
      tmem_st_wait();
    }
    if (kSave) fence_async_smem();
    tc_fence_before();
    scan_sync();                                   // sync 3
    tc_fence_after();
    if (tid == 0) {
      dead = scan_fwd_mma3<kSave>(tbase, sb, c, bars, p.status, dead);
      if (kSave) {
        bulk_store(p.vn_img + cidx * 16384, sb + sG, 32768);
        bulk_commit();
      }
    }
    wait_or_mark(&mma_bar, mphase, dead, p.status);    // the state update has completed (the output product may still run)
    tc_fence_after();
  }

  if (nt > 0) {
    wait_or_mark(&o_bar, ophase, dead, p.status);
    tc_fence_after();
    form_o(nt - 1);
    store_o(nt - 1);
  }
  if (kSave && tid == 0) bulk_wait_all();            // every saved panel is in global memory before the CTA ends
  if (!dead && p.ht) {
    float* dst = p.ht + ((int64_t(n) * p.HV + hv) * kK + k_lo) * p.V + vb * 128 + vrow;
#pragma unroll
    for (int part = 0; part < 4; ++part) {
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

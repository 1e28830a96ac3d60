// Chunked gated-delta-rule forward (chunk = 64 tokens, K = V = 128) as two kernels:
//
//  gdn_prep_kernel   (parallel over chunks): gam = chunk-local cumsum(g);
//                    A[i,j] = beta_i exp(gam_i - gam_j) k_i.k_j (j < i);  X = (I + A)^-1
//                    KK^T on tcgen05 (shared by the value heads of a GVA group); the unit-lower
//                    triangular inverse runs in tri_inverse_kernel (fp32 forward substitution on CUDA cores).
//                    Replaces chunk_local_cumsum + chunk_scaled_dot_kkt + solve_tri of the reference
//                    (examples/flash_gated_delta_rule.py:811-838).
//  gdn_fwd_kernel    (sequential over chunks, one CTA per (sequence, value head, 64-column block of V)):
//                    v_new = X (beta * (V - exp(gam) * (K S)))
//                    o     = scale (exp(gam) * (Q S) + tril(Q K^T * exp(gam_i - gam_j)) v_new)
//                    S    <- exp(gam_L) S + K^T (exp(gam_L - gam) * v_new)
//                    which is recompute_w_u + chunk_gated_delta_rule_fwd_h + chunk_fwd_o of the reference
//                    (examples/flash_gated_delta_rule.py:840-880) with the WY factors w, u folded away so
//                    that no per-chunk intermediate (A, w, u, h, v_new) round-trips through HBM.
//
// The fp32 state lives in TMEM for the whole sequence.  Tensor-core operands that the result is
// sensitive to (the state copy, beta*(V - ...), v_new, the decayed score tile) are split into a bf16
// "hi" part and a bf16 residual and multiplied in two or three passes; q, k, v enter as the exact
// bf16 inputs.  All matrix products run as tcgen05.mma with M = 128 (unused accumulator rows are
// ignored) so that TMEM lane == accumulator row for every tile.
#include "gdn_common.cuh"
#include "fla_b200_internal.h"
#include "kernel_timer.h"
#include "tri_inverse.h"
#include "tensor_map.h"

namespace fla {

struct GdnFwdParams {
  const bf16* q; const bf16* k; const bf16* v;
  const void* g; const void* beta;
  float* gam;          // [tokens, HV]      chunk-local cumulative log decay (saved for backward)
  bf16* X;             // [tokens, HV, 64]  row i of the chunk's (I + A)^-1 (saved for backward)
  float* at;           // [chunks, HV, 64, 64] scratch: A^T handed to the triangular-inverse kernel
  bf16* p_img;         // [chunks, HV, 2, 64x64] tril(Q K^T * decay) as hi / lo operand panels (scratch, reused by backward)
  const float* h0;     // [N, HV, K, V] or null
  float* ht;           // [N, HV, K, V] or null
  void* o;             // [tokens, HV, V]
  bf16* s_img;         // [chunks, HV, V/64, 2, 128x64] panel images of the state at chunk start (hi, lo), optional
  bf16* vn_img;        // [chunks, HV, V/64, 2, 64x64]  panel images of v_new (hi, lo), optional
  const int32_t* cu_seqlens; const int32_t* chunk_offsets;
  int64_t q_st, q_sh, k_st, k_sh, v_st, v_sh, o_st, o_sh, g_st, beta_st;
  int N, T, HK, HV, g_is_f32, beta_is_f32, o_is_f32;
  int V, nvb;          // value head dim (128 or 256) and its number of 64-column blocks
  float scale;
  int* status;
};

// --------------------------------------------------------------------------------------------- prep
// One CTA per (chunk, q/k head).  One M = 128 product [q; k] k^T leaves Q K^T in TMEM lanes 0..63 and K K^T in
// lanes 64..127; each thread keeps its row in registers and, per value head of the GVA group, the q-side
// threads emit P = tril(Q K^T * e^{gam_i - gam_j}) as split operand panels and the k-side threads emit A^T.
__global__ void __launch_bounds__(128) gdn_prep_kernel(GdnFwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* qk_pan = smem;                        // 2 panels x 128 rows: rows 0..63 q, rows 64..127 k
  __shared__ float gam_s[kC];
  __shared__ float wsum_s[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t bar;

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int hk = blockIdx.y, n = blockIdx.z;
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  const int t0 = blockIdx.x * kC;
  if (t0 >= sq.len) return;
  const int rows = min(kC, sq.len - t0);
  const int64_t tok0 = int64_t(sq.bos) + t0;
  {
    uint4 val[16];   // all loads in flight before the first one is consumed
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int idx = tid + i * 128, r = (idx / 16) & 63, ch = idx % 16;
      const bool isk = idx >= 1024;
      val[i] = make_uint4(0, 0, 0, 0);
      if (r < rows) {
        const bf16* src = isk ? p.k + (tok0 + r) * p.k_st + hk * p.k_sh : p.q + (tok0 + r) * p.q_st + hk * p.q_sh;
        val[i] = *reinterpret_cast<const uint4*>(src + ch * 8);
      }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int idx = tid + i * 128, r = ((idx / 16) & 63) + (idx >= 1024 ? 64 : 0), ch = idx % 16;
      *reinterpret_cast<uint4*>(qk_pan + (ch / 8) * 16384 + panel_chunk_off(r, ch % 8)) = val[i];
    }
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 64);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(&bar, 1);
    mbar_init_fence();
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = tmem_base_s;
  if (tid == 0) {
    const Operand a{smem_u32(qk_pan), 16384u, 0};
    const Operand b{smem_u32(qk_pan) + 8192u, 16384u, 0};   // k rows as B (N = 64 tokens)
    mma_tile(tbase, a, b, 128, 64, 8, false);
    mma_commit(&bar);
  }
  const int G = p.HV / p.HK;
  const bool kside = tid >= 64;
  const int tok = tid & 63;
  const bool ok = mbar_wait(&bar, 0, p.status, FLA_ERR_TIMEOUT);
  tc_fence_after();
  float sc[kC];   // my row of Q K^T (q side) or K K^T (k side)
  if (ok) tmem_ld_row64(tmem_addr(tbase, warp * 32, 0), sc);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 64);
  if (!ok) return;

  for (int h = 0; h < G; ++h) {
    const int hv = hk * G + h;
    const int64_t cidx = (int64_t(sq.cbase) + blockIdx.x) * p.HV + hv;
    // chunk-local cumulative sum of g (threads 0..63, two warps)
    float gv = 0.f;
    if (!kside) {
      gv = tok < rows ? ld_scalar(p.g, (tok0 + tok) * p.g_st + hv, p.g_is_f32) : 0.f;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, gv, o);
        if (lane >= o) gv += up;
      }
      if (lane == 31) wsum_s[warp] = gv;
    }
    const float bi = (kside && tok < rows) ? ld_scalar(p.beta, (tok0 + tok) * p.beta_st + hv, p.beta_is_f32) : 0.f;
    __syncthreads();
    if (!kside) {
      if (warp == 1) gv += wsum_s[0];
      gam_s[tok] = gv;
      if (tok < rows) p.gam[(tok0 + tok) * p.HV + hv] = gv;
    }
    __syncthreads();
    const float gam_i = gam_s[tok];
    if (!kside) {
      // P row as split bf16, written straight into the (swizzled) panel images
      uint8_t* img = reinterpret_cast<uint8_t*>(p.p_img + cidx * 8192);
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        float t[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const int j = ch * 8 + jj;
          const float e = __expf(fminf(gam_i - gam_s[j], 0.f));
          t[jj] = sc[j] * ((j <= tok) ? e : 0.f);
        }
        uint4 hi, lo;
        split8(t, hi, lo);
        const uint32_t off = panel_chunk_off(tok, ch);
        *reinterpret_cast<uint4*>(img + off) = hi;
        *reinterpret_cast<uint4*>(img + 8192 + off) = lo;
      }
    } else {
      // A^T[j][i] = beta_i exp(gam_i - gam_j) (k_i . k_j) for j < i, written coalesced along i
      float* at = p.at + cidx * (kC * kC);
#pragma unroll
      for (int j = 0; j < kC - 1; ++j)
        if (j < tok) at[j * kC + tok] = bi * __expf(gam_i - gam_s[j]) * sc[j];
    }
    __syncthreads();
  }
}

// --------------------------------------------------------------------------------------------- forward
// Shared-memory map of gdn_fwd_kernel (offsets from a 1024-byte aligned base).
constexpr uint32_t kOffQK = 0;                    // 2 panels x 128 rows: rows 0-63 q, rows 64-127 k
constexpr uint32_t kQKPanel = 16384;
constexpr uint32_t kOffSH = 32768, kOffSL = 49152;            // state copy hi / lo: 128 rows x 64 cols
constexpr uint32_t kOffZH = 65536, kOffZL = 73728;            // beta*(V - ..) hi / lo, then v_new hi / lo
constexpr uint32_t kOffVH = 81920, kOffVL = 90112;            // decayed v_new hi / lo
constexpr uint32_t kOffX = 98304;                             // X panel (64 rows); the 64 rows before it are VL
constexpr uint32_t kFwdSmem = 106496;
constexpr uint32_t kColS = 0, kColRQ = 64, kColQK = 128, kColVN = 192;  // TMEM column map (256 columns)
constexpr int kFwdThreads = 256;

struct FwdPrefetch {
  uint4 v[4];
  float gb;
};


// q and k rows reach their operand panels as four 64 x 64 TMA tiles per chunk (the 128-byte swizzle of the tensor map
// is the panel layout); rows past the end of a sequence then hold whatever follows in memory (zero past the end of
// the tensor): harmless, because every product with them is multiplied by a zero row of X, P or beta.
__global__ void __launch_bounds__(kFwdThreads, 2) gdn_fwd_kernel(GdnFwdParams p, const __grid_constant__ CUtensorMap tm_q,
                                                                  const __grid_constant__ CUtensorMap tm_k,
                                                                  const __grid_constant__ CUtensorMap tm_x) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ float gam_s[2][kC], beta_s[2][kC];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t bar, pbar, qk_bar, x_bar;

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int vb = blockIdx.x, hv = blockIdx.y, n = blockIdx.z;
  const int hk = hv / (p.HV / p.HK);
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  const int quad = warp & 3, half = warp >> 2;   // TMEM lane quadrant; which 32 of the tile's 64 columns
  const bool kside = quad >= 2;                  // rows 64..127 hold the k-side results
  const int row = quad * 32 + lane;              // TMEM lane == accumulator row
  const int tok = row & 63;                      // token row inside the chunk
  const int c0 = half * 32;

  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 256);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(&bar, 1);
    mbar_init(&pbar, 1);
    mbar_init(&qk_bar, 1);
    mbar_init(&x_bar, 1);
    mbar_init_fence();
    tma_prefetch_descriptor(&tm_q);
    tma_prefetch_descriptor(&tm_k);
    tma_prefetch_descriptor(&tm_x);
  }
  __syncthreads();
  const uint32_t tbase = tmem_base_s;
  const uint32_t trow = tmem_addr(tbase, quad * 32, c0);
  uint32_t phase = 0, pphase = 0, qkphase = 0, xphase = 0;
  bool dead = false;
  const uint32_t sb = smem_u32(smem);

  FwdPrefetch pf;
  auto prefetch_load = [&](int c) {
    const int t0 = c * kC;
    const int rows = min(kC, sq.len - t0);
    const int64_t tok0 = int64_t(sq.bos) + t0;
    if (kside) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        pf.v[i] = make_uint4(0, 0, 0, 0);
        if (tok < rows) pf.v[i] = *reinterpret_cast<const uint4*>(p.v + (tok0 + tok) * p.v_st + hv * p.v_sh + vb * kBV + c0 + i * 8);
      }
    }
  };
  // The per-token scalars travel separately and early: they are published to shared memory well before the
  // barriers that precede their first use in the next iteration.
  auto prefetch_scalars = [&](int c) {
    const int t0 = c * kC;
    const int rows = min(kC, sq.len - t0);
    const int64_t tok0 = int64_t(sq.bos) + t0;
    if (kside) {
      pf.gb = tok < rows ? ld_scalar(p.beta, (tok0 + tok) * p.beta_st + hv, p.beta_is_f32) : 0.f;
    } else {
      // rows past the end of the sequence carry the last valid cumulative decay so every exponent stays finite
      pf.gb = p.gam[(tok0 + min(tok, rows - 1)) * p.HV + hv];
    }
  };
  // Touch the next chunk's rows early so that the register loads issued late in the iteration hit L2.
  auto prefetch_l2 = [&](int c) {
    const int t0 = c * kC;
    const int rows = min(kC, sq.len - t0);
    const int64_t tok0 = int64_t(sq.bos) + t0;
    if (tid < 128) {
      const int r = tid & 63;
      if (r < rows) {
        const bf16* src = tid >= 64 ? p.k + (tok0 + r) * p.k_st + hk * p.k_sh : p.q + (tok0 + r) * p.q_st + hk * p.q_sh;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(src));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(src + 64));
      }
    } else if (tid < 192) {
      const int r = tid - 128;
      if (r < rows) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p.X + ((tok0 + r) * p.HV + hv) * kC));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p.v + (tok0 + r) * p.v_st + hv * p.v_sh + vb * kBV));
      }
    }
  };
  uint4 vcur[4];
  auto store_scalars = [&](int c) {   // double-buffered by chunk parity: may be written while chunk c-1 is in flight
    if (half == 0) {
      if (kside) beta_s[c & 1][tok] = pf.gb;
      else gam_s[c & 1][tok] = pf.gb;
    }
  };
  auto store_panels = [&]() {
#pragma unroll
    for (int i = 0; i < 4; ++i) vcur[i] = pf.v[i];
  };

  auto issue_qk_load = [&](int c) {   // one thread: the chunk's q rows (panel rows 0-63) and k rows (rows 64-127)
    const int row0 = sq.bos + c * kC;
    mbar_arrive_expect_tx(&qk_bar, 4 * 8192);
    tma_load_tile(sb + kOffQK, &tm_q, 0, hk, row0, &qk_bar);
    tma_load_tile(sb + kOffQK + kQKPanel, &tm_q, 64, hk, row0, &qk_bar);
    tma_load_tile(sb + kOffQK + 8192, &tm_k, 0, hk, row0, &qk_bar);
    tma_load_tile(sb + kOffQK + kQKPanel + 8192, &tm_k, 64, hk, row0, &qk_bar);
  };

  auto issue_x_load = [&](int c) {    // one thread: the chunk's 64 x 64 inverse
    mbar_arrive_expect_tx(&x_bar, 8192);
    tma_load_tile(sb + kOffX, &tm_x, 0, hv, sq.bos + c * kC, &x_bar);
  };

  // operands (shared addresses)
  const Operand opQK{sb + kOffQK, kQKPanel, 0};                 // [q; k]  M = 128, reduction over K
  const Operand opKT{sb + kOffQK + 8192, kQKPanel, 1};          // k^T     M = 128 (K dims), reduction over tokens
  const Operand opSH{sb + kOffSH, 16384, 1}, opSL{sb + kOffSL, 16384, 1};
  const Operand opZH{sb + kOffZH, 8192, 1}, opZL{sb + kOffZL, 8192, 1};
  const Operand opVH{sb + kOffVH, 8192, 1}, opVL{sb + kOffVL, 8192, 1};
  const Operand opX{sb + kOffX - 8192, 16384, 0};               // rows 64..127 of this tile are X
  const Operand opPH{sb + kOffQK, kQKPanel, 0}, opPL{sb + kOffQK + kQKPanel, kQKPanel, 0};  // alias the q rows

  float srow[32];   // this thread's 32 columns of the fp32 state row

  // ---- prologue: chunk 0 operands and the initial state.  A sequence without tokens (packed batches may hold some)
  // requests nothing: its chunk loop does not run and the final state below is the initial state.
  if (sq.nt > 0) {
    if (tid == 0) {
      issue_qk_load(0);
      issue_x_load(0);
    }
    prefetch_load(0);
    prefetch_scalars(0);
    store_scalars(0);
    store_panels();
  }
  if (p.h0) {
    const float* src = p.h0 + ((int64_t(n) * p.HV + hv) * kK + row) * p.V + vb * kBV + c0;
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      const float4 t = *reinterpret_cast<const float4*>(src + i);
      srow[i] = t.x; srow[i + 1] = t.y; srow[i + 2] = t.z; srow[i + 3] = t.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) srow[i] = 0.f;
  }
  __syncthreads();  // gam_s[0] visible

  for (int c = 0; c < sq.nt; ++c) {
    const int cur = c & 1;
    const int t0 = c * kC;
    const int rows = min(kC, sq.len - t0);
    const int64_t tok0 = int64_t(sq.bos) + t0;
    const float gam_last = gam_s[cur][rows - 1];
    const float gam_i = gam_s[cur][tok];

    // ---- stage 0: publish the state at chunk start (split copy for the MMAs, pre-decayed master in TMEM)
    row32_to_hilo(smem + kOffSH, smem + kOffSL, row, half, srow);
    {
      const float dl = __expf(gam_last);
#pragma unroll
      for (int i = 0; i < 32; ++i) srow[i] *= dl;
      tmem_st_row32(trow + kColS, srow);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    // ---- stage 1: [Q;K] S  (split state: two passes)
    if (tid == 0) {
      if (!mbar_wait(&qk_bar, qkphase, p.status, FLA_ERR_TIMEOUT)) dead = true;   // q, k tiles have landed
      mma_tile(tbase + kColRQ, opQK, opSH, 128, 64, 8, false);
      mma_tile(tbase + kColRQ, opQK, opSL, 128, 64, 8, true);
      mma_commit(&bar);
    }
    qkphase ^= 1;
    if (p.s_img) {  // the split state copy in shared memory is already in the saved panel-image format: plain 16-byte
                    // copies by all threads while the MMAs run (bulk stores would queue ahead of the chunk's TMA loads)
      uint4* dst = reinterpret_cast<uint4*>(p.s_img + (((int64_t(sq.cbase) + c) * p.HV + hv) * p.nvb + vb) * (2 * 8192));
      const uint4* src = reinterpret_cast<const uint4*>(smem + kOffSH);
#pragma unroll
      for (int i = 0; i < 8; ++i) dst[tid + i * kFwdThreads] = src[tid + i * kFwdThreads];
    }
    if (c + 1 < sq.nt) {
      prefetch_l2(c + 1);
      prefetch_scalars(c + 1);
      store_scalars(c + 1);
    }
    wait_or_mark(&bar, phase, dead, p.status);
    tc_fence_after();
    if (tid == 0) {  // the q rows are consumed: the chunk's P panels (from the prep kernel) take their place
      const bf16* src = p.p_img + ((int64_t(sq.cbase) + c) * p.HV + hv) * 8192;
      mbar_arrive_expect_tx(&pbar, 16384);
      bulk_load(sb + kOffQK, src, 8192, &pbar);
      bulk_load(sb + kOffQK + kQKPanel, src + 4096, 8192, &pbar);
    }

    // ---- stage 2: k-side rows build Z = beta (V - exp(gam) K S)
    float acc[32];
    if (kside) {
      tmem_ld_row32(trow + kColRQ, acc);
      const float eg = __expf(gam_i), bi = beta_s[cur][tok];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float vv[8];
        unpack_bf16x8(vcur[i], vv);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i * 8 + j] = bi * (vv[j] - eg * acc[i * 8 + j]);
      }
      row32_to_hilo(smem + kOffZH, smem + kOffZL, tok, half, acc);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    // ---- stage 3: v_new = X Z  (rows 64..127 of the accumulator)
    if (tid == 0) {
      if (!mbar_wait(&x_bar, xphase, p.status, FLA_ERR_TIMEOUT)) dead = true;   // the X tile has landed
      mma_tile(tbase + kColVN, opX, opZH, 128, 64, 4, false);
      mma_tile(tbase + kColVN, opX, opZL, 128, 64, 4, true);
      mma_commit(&bar);
    }
    xphase ^= 1;
    wait_or_mark(&bar, phase, dead, p.status);
    tc_fence_after();
    if (tid == 0 && c + 1 < sq.nt) issue_x_load(c + 1);

    // ---- stage 4: k-side rows publish v_new and its decayed copy
    if (kside) {
      tmem_ld_row32(trow + kColVN, acc);
      if (tok >= rows) {   // rows of the X tile past the end of the sequence belong to whatever follows in memory
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = 0.f;
      }
      row32_to_hilo(smem + kOffZH, smem + kOffZL, tok, half, acc);
      const float dk = __expf(gam_last - gam_i);
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] *= dk;
      row32_to_hilo(smem + kOffVH, smem + kOffVL, tok, half, acc);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    // ---- stage 5: P v_new (three passes) and the state update S += K^T vhat
    if (tid == 0) {
      mma_tile(tbase + kColS, opKT, opVH, 128, 64, 4, true);
      mma_tile(tbase + kColS, opKT, opVL, 128, 64, 4, true);
      if (!mbar_wait(&pbar, pphase, p.status, FLA_ERR_TIMEOUT)) dead = true;   // P panels have landed
      mma_tile(tbase + kColQK, opPH, opZH, 128, 64, 4, false);
      mma_tile(tbase + kColQK, opPH, opZL, 128, 64, 4, true);
      mma_tile(tbase + kColQK, opPL, opZH, 128, 64, 4, true);
      mma_commit(&bar);
    }
    pphase ^= 1;
    if (p.vn_img) {
      uint4* dst = reinterpret_cast<uint4*>(p.vn_img + (((int64_t(sq.cbase) + c) * p.HV + hv) * p.nvb + vb) * (2 * 4096));
      const uint4* src = reinterpret_cast<const uint4*>(smem + kOffZH);     // Z_hi and Z_lo panels are adjacent
#pragma unroll
      for (int i = 0; i < 4; ++i) dst[tid + i * kFwdThreads] = src[tid + i * kFwdThreads];
    }
    if (c + 1 < sq.nt) prefetch_load(c + 1);   // the next chunk's rows (L2-resident by now) travel while the MMAs run
    wait_or_mark(&bar, phase, dead, p.status);
    tc_fence_after();
    if (tid == 0 && c + 1 < sq.nt) issue_qk_load(c + 1);   // every reader of the q / k / P panels has completed

    // ---- stage 6: output rows, next state, next chunk's operand panels
    if (!kside) {
      float qs[32];
      tmem_ld32(trow + kColRQ, qs);
      tmem_ld32(trow + kColQK, acc);
      tmem_ld_wait();
      const float eg = __expf(gam_i) * p.scale;
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = eg * qs[i] + p.scale * acc[i];
      if (tok < rows) {
        const int64_t off = (tok0 + tok) * p.o_st + hv * p.o_sh + vb * kBV + c0;
        if (p.o_is_f32) {
          float* dst = static_cast<float*>(p.o) + off;
#pragma unroll
          for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
        } else {
          bf16* dst = static_cast<bf16*>(p.o) + off;
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) *reinterpret_cast<uint4*>(dst + ch * 8) = pack8(acc + ch * 8);
        }
      }
    }
    tmem_ld_row32(trow + kColS, srow);
    // The only readers of the q/k/X panels were this chunk's MMAs, which have completed; no barrier is needed
    // before the next iteration (its first barrier orders everything else).
    if (c + 1 < sq.nt) store_panels();
  }

  if (!dead && p.ht) {
    float* dst = p.ht + ((int64_t(n) * p.HV + hv) * kK + row) * p.V + vb * kBV + c0;
#pragma unroll
    for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(srow[i], srow[i + 1], srow[i + 2], srow[i + 3]);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 256);
}

}  // namespace fla

using namespace fla;

static int check_token_tensor(const fla_tensor_t& t, int64_t heads, int64_t dim, int dtype_a, int dtype_b) {
  // [B, T, H, D] with D contiguous, rows 16-byte aligned, and batch rows laid out back to back
  if (!t.data) return FLA_ERR_NULL;
  if (t.ndim != 4 || t.shape[2] != heads || t.shape[3] != dim) return FLA_ERR_SHAPE;
  if (t.dtype != dtype_a && t.dtype != dtype_b) return FLA_ERR_DTYPE;
  const int64_t esz = t.dtype == FLA_F32 ? 4 : 2;
  if (t.stride[3] != 1 || (t.stride[2] * esz) % 16 || (t.stride[1] * esz) % 16 || !aligned16(t.data)) return FLA_ERR_LAYOUT;
  if (t.shape[0] > 1 && t.stride[0] != t.shape[1] * t.stride[1]) return FLA_ERR_LAYOUT;
  return FLA_OK;
}
static int check_gate_tensor(const fla_tensor_t& t, int64_t B, int64_t T, int64_t heads) {
  if (!t.data) return FLA_ERR_NULL;
  if (t.ndim != 3 || t.shape[0] != B || t.shape[1] != T || t.shape[2] != heads) return FLA_ERR_SHAPE;
  if (t.dtype != FLA_F32 && t.dtype != FLA_BF16) return FLA_ERR_DTYPE;
  if (t.stride[2] != 1 || (B > 1 && t.stride[0] != T * t.stride[1])) return FLA_ERR_LAYOUT;
  return FLA_OK;
}

extern "C" FLA_API int fla_b200_gdn_chunk_fwd_workspace_size(const fla_gdn_chunk_fwd_args* a, uint64_t* bytes) {
  if (!a || !bytes) return FLA_ERR_NULL;
  if (!a->q.data || a->q.ndim != 4 || !a->v.data || a->v.ndim != 4) return FLA_ERR_SHAPE;
  int64_t chunks = a->q.shape[0] * ((a->q.shape[1] + kC - 1) / kC);
  if (a->cu_seqlens.data) chunks = a->total_chunks;
  if (chunks <= 0) return FLA_ERR_VALUE;
  // status block + A^T scratch for the inverse + P panels (unless the caller keeps them for the backward)
  *bytes = 256 + uint64_t(chunks) * a->v.shape[2] * (kC * kC * 4 + (a->p_img.data ? 0 : 8192 * 2));
  return FLA_OK;
}

extern "C" FLA_API int fla_b200_gdn_chunk_fwd(const fla_gdn_chunk_fwd_args* a, void* workspace, uint64_t workspace_bytes,
                                              void* stream) {
  if (!a) return FLA_ERR_NULL;
  if (!workspace || workspace_bytes < 256 || !aligned16(workspace)) return FLA_ERR_WORKSPACE;
  const fla_tensor_t &q = a->q, &k = a->k, &v = a->v, &o = a->o;
  if (!q.data || !k.data || !v.data || !o.data) return FLA_ERR_NULL;
  if (q.ndim != 4 || v.ndim != 4) return FLA_ERR_SHAPE;
  const int64_t B = q.shape[0], T = q.shape[1], HK = q.shape[2], HV = v.shape[2];
  if (B <= 0 || T <= 0 || HK <= 0 || HV <= 0 || HV % HK || v.shape[0] != B || v.shape[1] != T) return FLA_ERR_SHAPE;
  int st;
  if ((st = check_token_tensor(q, HK, kK, FLA_BF16, FLA_BF16))) return st;
  if ((st = check_token_tensor(k, HK, kK, FLA_BF16, FLA_BF16))) return st;
  const int64_t V = v.shape[3];
  if (V != kV && V != 2 * kV) return FLA_ERR_SHAPE;
  if ((st = check_token_tensor(v, HV, V, FLA_BF16, FLA_BF16))) return st;
  if ((st = check_token_tensor(o, HV, V, FLA_BF16, FLA_F32))) return st;
  if (k.shape[0] != B || k.shape[1] != T || o.shape[0] != B || o.shape[1] != T) return FLA_ERR_SHAPE;
  if ((st = check_gate_tensor(a->g, B, T, HV))) return st;
  if ((st = check_gate_tensor(a->beta, B, T, HV))) return st;
  if (a->chunk_size != kC) return FLA_ERR_VALUE;
  if (!(a->scale == a->scale)) return FLA_ERR_VALUE;

  int N = int(B);
  int64_t total_chunks = B * ((T + kC - 1) / kC);
  int max_len = int(T);
  if (a->cu_seqlens.data) {
    if (B != 1 || a->cu_seqlens.dtype != FLA_I32 || a->cu_seqlens.ndim != 1 || a->cu_seqlens.shape[0] < 2) return FLA_ERR_SHAPE;
    N = int(a->cu_seqlens.shape[0] - 1);
    if (!a->chunk_offsets.data || a->chunk_offsets.dtype != FLA_I32 || a->chunk_offsets.shape[0] != N + 1) return FLA_ERR_SHAPE;
    if (a->max_seqlen <= 0 || a->max_seqlen > T || a->total_chunks <= 0) return FLA_ERR_VALUE;
    max_len = a->max_seqlen;
    total_chunks = a->total_chunks;
  }
  const fla_tensor_t &gam = a->gam, &X = a->x_inv;
  if (!gam.data || !X.data) return FLA_ERR_NULL;
  if (gam.dtype != FLA_F32 || gam.ndim != 3 || gam.shape[0] != B || gam.shape[1] != T || gam.shape[2] != HV ||
      gam.stride[2] != 1 || gam.stride[1] != HV || (B > 1 && gam.stride[0] != T * HV))
    return FLA_ERR_SHAPE;
  if (X.dtype != FLA_BF16 || X.ndim != 4 || X.shape[0] != B || X.shape[1] != T || X.shape[2] != HV || X.shape[3] != kC ||
      X.stride[3] != 1 || X.stride[2] != kC || X.stride[1] != HV * kC || !aligned16(X.data))
    return FLA_ERR_SHAPE;
  for (const fla_tensor_t* s : {&a->initial_state, &a->final_state}) {
    if (!s->data) continue;
    if (s->dtype != FLA_F32) return FLA_ERR_DTYPE;
    if (s->ndim != 4 || s->shape[0] != N || s->shape[1] != HV || s->shape[2] != kK || s->shape[3] != V) return FLA_ERR_SHAPE;
    if (s->stride[3] != 1 || s->stride[2] != V || s->stride[1] != kK * V || s->stride[0] != HV * kK * V || !aligned16(s->data))
      return FLA_ERR_LAYOUT;
  }
  GdnFwdParams p{};
  p.q = static_cast<const bf16*>(q.data); p.k = static_cast<const bf16*>(k.data); p.v = static_cast<const bf16*>(v.data);
  p.g = a->g.data; p.beta = a->beta.data;
  p.gam = static_cast<float*>(gam.data); p.X = static_cast<bf16*>(X.data);
  p.h0 = static_cast<const float*>(a->initial_state.data); p.ht = static_cast<float*>(a->final_state.data);
  p.o = o.data;
  if (a->s_img.data || a->vn_img.data) {
    const fla_tensor_t &si = a->s_img, &vi = a->vn_img;
    if (!si.data || !vi.data) return FLA_ERR_NULL;
    if (si.dtype != FLA_BF16 || si.ndim != 1 || si.shape[0] != total_chunks * HV * (V / kBV) * 16384 || !aligned16(si.data)) return FLA_ERR_SHAPE;
    if (vi.dtype != FLA_BF16 || vi.ndim != 1 || vi.shape[0] != total_chunks * HV * (V / kBV) * 8192 || !aligned16(vi.data)) return FLA_ERR_SHAPE;
    p.s_img = static_cast<bf16*>(si.data);
    p.vn_img = static_cast<bf16*>(vi.data);
  }
  p.cu_seqlens = static_cast<const int32_t*>(a->cu_seqlens.data);
  p.chunk_offsets = static_cast<const int32_t*>(a->chunk_offsets.data);
  p.q_st = q.stride[1]; p.q_sh = q.stride[2]; p.k_st = k.stride[1]; p.k_sh = k.stride[2];
  p.v_st = v.stride[1]; p.v_sh = v.stride[2]; p.o_st = o.stride[1]; p.o_sh = o.stride[2];
  p.g_st = a->g.stride[1]; p.beta_st = a->beta.stride[1];
  p.N = N; p.T = int(T); p.HK = int(HK); p.HV = int(HV); p.V = int(V); p.nvb = int(V / kBV);
  p.g_is_f32 = a->g.dtype == FLA_F32; p.beta_is_f32 = a->beta.dtype == FLA_F32; p.o_is_f32 = o.dtype == FLA_F32;
  p.scale = a->scale;
  p.status = static_cast<int*>(workspace);
  {
    const uint64_t per = uint64_t(total_chunks) * HV;
    if (workspace_bytes < 256 + per * (kC * kC * 4 + (a->p_img.data ? 0 : 8192 * 2))) return FLA_ERR_WORKSPACE;
    p.at = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + 256);
    if (a->p_img.data) {
      const fla_tensor_t& pi = a->p_img;
      if (pi.dtype != FLA_BF16 || pi.ndim != 1 || pi.shape[0] != int64_t(per) * 8192 || !aligned16(pi.data)) return FLA_ERR_SHAPE;
      p.p_img = static_cast<bf16*>(pi.data);
    } else {
      p.p_img = reinterpret_cast<bf16*>(static_cast<uint8_t*>(workspace) + 256 + per * kC * kC * 4);
    }
  }

  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(workspace, 0, 256, cs) != cudaSuccess) return FLA_ERR_CUDA;
  const int prep_smem = 32768 + 1024;
  static std::atomic<bool> attr_done_dev[64] = {};   // per device ordinal; setting the attributes twice is harmless
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FLA_ERR_CUDA;
  std::atomic<bool>& attr_done = attr_done_dev[dev];
  if (!attr_done) {
    if (cudaFuncSetAttribute(gdn_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, prep_smem) != cudaSuccess) return FLA_ERR_CUDA;
    if (cudaFuncSetAttribute(gdn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kFwdSmem) + 1024) != cudaSuccess) return FLA_ERR_CUDA;
    attr_done = true;
  }
  const int nt_max = (max_len + kC - 1) / kC;
  {
    KernelTimer kt("gdn_prep", cs);
    gdn_prep_kernel<<<dim3(nt_max, unsigned(HK), N), 128, prep_smem, cs>>>(p);
  }
  if (cudaGetLastError() != cudaSuccess) return FLA_ERR_CUDA;
  {
    KernelTimer kt("tri_inverse", cs);
    TriInverseParams tp{p.at, p.X, nullptr, nullptr, p.cu_seqlens, p.chunk_offsets, p.T, p.HV, 0};
    if (launch_tri_inverse(tp, nt_max, N, cs)) return FLA_ERR_CUDA;
  }
  CUtensorMap tm_q, tm_k, tm_x;
  if (make_row_tile_map(&tm_q, p.q, kK, uint64_t(HK), uint64_t(B * T), uint64_t(p.q_sh), uint64_t(p.q_st)) ||
      make_row_tile_map(&tm_k, p.k, kK, uint64_t(HK), uint64_t(B * T), uint64_t(p.k_sh), uint64_t(p.k_st)) ||
      make_row_tile_map(&tm_x, p.X, kC, uint64_t(HV), uint64_t(B * T), uint64_t(kC), uint64_t(HV) * kC))
    return FLA_ERR_CUDA;
  {
    KernelTimer kt("gdn_fwd", cs);
    gdn_fwd_kernel<<<dim3(unsigned(p.nvb), unsigned(HV), N), kFwdThreads, kFwdSmem + 1024, cs>>>(p, tm_q, tm_k, tm_x);
  }
  return cuda_status(cudaGetLastError());
}


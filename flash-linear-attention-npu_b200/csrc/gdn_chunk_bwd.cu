// Chunked gated-delta-rule backward (chunk = 64, K = V = 128) as two kernels.
//
// With per chunk  gam = cumsum(g),  P = tril(Q K^T * e^{gam_i-gam_j}),  X = (I + strict_tril(beta_i e^{gam_i-gam_j} k_i.k_j))^-1,
// S = state at chunk start, Vn = v_new (both saved by the forward as bf16 value + residual strip images) and dS' the state
// gradient entering the chunk from the right:
//
//  gdn_scan_bwd_kernel  (gdn_scan_bwd.cuh; reverse-sequential over chunks, one CTA per (sequence, value head, 128 channels of V)):
//      dVn = scale P^T dO + e^{gam_L-gam} * (K dS')          dZ = X^T dVn          dV = beta * dZ
//      dS  = e^{gam_L} dS' + (scale e^{gam} * Q)^T dO - K^T (beta e^{gam} * dZ)     dh0 = dS after the first chunk
//      saves dS' and [dO; dZ] as strip images and the partial row sums  sum_v dZ*V  for the second kernel.
//      Replaces chunk_bwd_dv_local + chunk_gated_delta_rule_bwd_dhu of the reference
//      (examples/flash_gated_delta_rule.py:930-960) and the dv / du parts of prepare_wy_repr_bwd_*.
//  gdn_bwd_par_kernel  (parallel over chunks, one CTA per (chunk, q/k head), looping over the value heads of the group):
//      dP  = scale tril(dO Vn^T * e^{gam_i-gam_j})            dA = -strict_tril(dZ Vn^T)       dAt = dA * beta_i e^{gam_i-gam_j}
//      dq  = scale e^{gam} * (dO S^T) + dP K
//      dk  = dP^T Q + dAt^T K + dAt K + e^{gam_L-gam} * (Vn dS'^T) - beta e^{gam} * (dZ S^T)
//      dbeta = sum_v dZ*V - e^{gam} k.(dZ S^T) + sum_j dA_ij e^{gam_i-gam_j} k_i.k_j
//      dgam  = q.dq - k.dk + 2 beta (sum_j dA_ij e^{..} k_i.k_j) - 2 beta e^{gam} k.(dZ S^T);
//      dgam_L += e^{gam_L} <S, dS'> + sum_i e^{gam_L-gam_i} k_i.(Vn dS'^T)_i;   dg = reverse chunk-local cumsum(dgam)
//      with dq, dk summed over the value heads of a GVA group in registers (deterministic, no atomics).
//      Replaces chunk_bwd_dqkwg + prepare_wy_repr_bwd_da + prepare_wy_repr_bwd_full + the reverse cumsum
//      (examples/flash_gated_delta_rule.py:962-1021).
//
// Operands the gradients are sensitive to travel as bf16 hi + bf16 residual and are multiplied in two or three
// tcgen05.mma passes; q, k, dO enter as the exact bf16 inputs; accumulation is fp32 in TMEM.
#include "gdn_common.cuh"
#include "fla_b200_internal.h"
#include "kernel_timer.h"
#include "aux_stream.h"
#include "tensor_map.h"

namespace fla {

struct GdnBwdParams {
  const bf16* q; const bf16* k; const bf16* v; const bf16* dO;
  const void* beta;
  const float* gam; const bf16* X;
  const bf16* s_img; const bf16* vn_img; const bf16* p_img;
  bf16* ds_img;        // [chunks, HV, V/64, 2, 128x64]  state gradient entering each chunk (hi, lo)
  bf16* dz_img;        // [chunks, HV, V/64, 192x64: rows 0-63 dO, rows 64-127 dZ rounded to bf16, rows 128-191 the residual of dZ]
  float* bz;           // [V/32, tokens, HV] partial sums of dZ * V over the 32-column slices of V
  const float* dht; float* dh0;
  void* dq; void* dk; void* dv; void* dg; void* dbeta;
  const int32_t* cu_seqlens; const int32_t* chunk_offsets;
  int64_t q_st, q_sh, k_st, k_sh, v_st, v_sh, do_st, do_sh, beta_st;
  int64_t dq_st, dq_sh, dk_st, dk_sh, dv_st, dv_sh;
  int64_t total_tokens;
  int N, T, HK, HV, beta_is_f32, grads_f32;
  int V, nvb;          // value head dim (128 or 256) and its number of 64-column blocks
  int n0;              // first sequence of this launch (the backward may be launched as two halves of the batch)
  float scale;
  int* status;
};

}  // namespace fla
#include "gdn_scan_bwd.cuh"
namespace fla {

constexpr int64_t kSImg = 16384;   // bf16 elements of the state images per (chunk, head, 64-column block of V): (hi, lo) x 128x64
constexpr int64_t kVnImg = 8192;   // v_new images per (chunk, head, block): (hi, lo) x 64x64
constexpr int64_t kDzImg = kDzHalf;   // per (chunk, head, block): 64x64 dO, 64x64 dZ and the residual of dZ

// ============================================================================================= par
constexpr uint32_t rOffQK = 0, rQKPanel = 16384;
constexpr uint32_t rOffAH = 49152;             // [dO^T | dZ^T] strips of one 64-channel step (16 KB)
constexpr uint32_t rOffAL = 32768;             // [0 | residual of dZ^T]: 8 KB of zeros written once, then the step's 8 KB of strips
// v_new^T and S strips, value / residual, interleaved so that [Vn_lo | S_hi] and [Vn_hi | S_lo] are each one contiguous B operand
// of 24 strips.  As an A operand with valid rows 64..127 the view of v_new^T starts 8 KB earlier, inside the dZ^T strips or the
// S strips (any finite contents do).
constexpr uint32_t rOffVNL = 65536, rOffSH = 73728, rOffVNH = 90112, rOffSL = 98304, rOffDSH = 114688, rOffDSL = 131072;
constexpr uint32_t rOffPAH = 147456, rOffPAL = 163840;   // [dP ; dAt] hi / lo (128 rows x 64)
constexpr uint32_t kParSmem = 180224;
constexpr uint32_t rColQK = 0, rColDV = 64, rColTA = 128, rColTB = 256;
constexpr uint32_t rColAcc = 384;   // running dq (q-side rows) / dk (k-side rows) over the value heads of the group: 128 columns
constexpr uint32_t kStepBytes = 16384 + 8192 + 16384 + 32768 + 32768;

__device__ __forceinline__ void row_dot64(const uint8_t* pan0, uint32_t panel_stride, int row, int col0, const float* x,
                                          float& acc) {
  // acc += sum_c bf16_panel[row][col0 + c] * x[c], c in [0, 64); col0 is 0 or 64 (one panel)
  const uint8_t* pan = pan0 + (col0 / 64) * panel_stride;
#pragma unroll
  for (int ch = 0; ch < 8; ++ch) {
    float f[8];
    unpack_bf16x8(*reinterpret_cast<const uint4*>(pan + panel_chunk_off(row, ch)), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += f[j] * x[ch * 8 + j];
  }
}


template <int NVB>   // 64-column blocks of V per head (2 or 4): a compile-time trip count keeps the block loop unrolled
__global__ void __launch_bounds__(256, 1) gdn_bwd_par_kernel(GdnBwdParams p, const __grid_constant__ CUtensorMap tm_q,
                                                                const __grid_constant__ CUtensorMap tm_k) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // per-head row scalars and row reductions, double-buffered by head parity: the dg / dbeta rows of a head are
  // finished while the tensor cores work on the next head
  __shared__ float gam_s2[2][kC], beta_s2[2][kC];
  __shared__ float red2[2][5][2][kC];  // qdq, kdk, rkG, rkB, ma : [half][row]
  __shared__ float sds_s2[2][8];
  __shared__ float fin_s[2][2];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t mma_bar, load_bar, qk_bar;

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int hk = blockIdx.y, n = blockIdx.z + p.n0;
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  const int c = blockIdx.x;
  if (c >= sq.nt) return;
  const int t0 = c * kC;
  const int rows = min(kC, sq.len - t0);
  const int64_t tok0 = int64_t(sq.bos) + t0;
  const int G = p.HV / p.HK;
  const int quad = warp & 3, half = warp >> 2;
  const int row = quad * 32 + lane;           // accumulator row == TMEM lane
  const bool kside = quad >= 2;
  const int tok = row & 63;

  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  const uint32_t sb = smem_u32(smem);
  // One thread: operands of one (value head, 64-channel half of a block of V) step.  The scans store every saved operand
  // per half, so a step is four contiguous pieces.
  auto issue_loads = [&](int hv, int vb) {
    const int64_t blk = ((int64_t(sq.cbase) + c) * p.HV + hv) * (NVB / 2) + (vb >> 1);
    const int64_t hf = vb & 1;
    mbar_arrive_expect_tx(&load_bar, kStepBytes);
    bulk_load(sb + rOffAH, p.dz_img + blk * (2 * kDzHalf) + hf * kDzHalf, 16384, &load_bar);      // [dO^T | dZ^T] strips
    bulk_load(sb + rOffAL + 8192, p.dz_img + blk * (2 * kDzHalf) + hf * kDzHalf + 8192, 8192, &load_bar);   // residual of dZ^T
    bulk_load(sb + rOffVNH, p.vn_img + blk * 16384 + hf * 8192, 8192, &load_bar);           // value
    bulk_load(sb + rOffVNL, p.vn_img + blk * 16384 + hf * 8192 + 4096, 8192, &load_bar);    // residual
    bulk_load(sb + rOffSH, p.s_img + blk * 32768 + hf * 16384, 16384, &load_bar);           // value, 16 strips
    bulk_load(sb + rOffSL, p.s_img + blk * 32768 + hf * 16384 + 8192, 16384, &load_bar);    // residual
    bulk_load(sb + rOffDSH, p.ds_img + blk * 32768 + hf * 16384, 32768, &load_bar);
  };
  // the same four pieces asked into L2 one step ahead: the buffer they will land in is still being read, so the load itself
  // cannot be issued yet, but the DRAM part of its latency can be spent meanwhile
  auto prefetch_loads = [&](int hv, int vb) {
    const int64_t blk = ((int64_t(sq.cbase) + c) * p.HV + hv) * (NVB / 2) + (vb >> 1);
    const int64_t hf = vb & 1;
    bulk_prefetch_l2(p.dz_img + blk * (2 * kDzHalf) + hf * kDzHalf, 24576);
    bulk_prefetch_l2(p.vn_img + blk * 16384 + hf * 8192, 16384);
    bulk_prefetch_l2(p.s_img + blk * 32768 + hf * 16384, 32768);
    bulk_prefetch_l2(p.ds_img + blk * 32768 + hf * 16384, 32768);
  };
  if (tid == 0) {
    mbar_init(&mma_bar, 1);
    mbar_init(&load_bar, 1);
    mbar_init(&qk_bar, 1);
    mbar_init_fence();
    // q, k rows of the chunk (shared by the value heads of the group): four 64 x 64 tiles into the [q; k] panels.
    // Rows past the end of the sequence hold whatever follows in memory; every product with them meets a zero
    // row or column of dO, dZ, v_new or the masked score gradients, and those rows are never stored.
    mbar_arrive_expect_tx(&qk_bar, 32768);
    tma_load_tile(sb + rOffQK, &tm_q, 0, hk, int(tok0), &qk_bar);
    tma_load_tile(sb + rOffQK + 8192, &tm_k, 0, hk, int(tok0), &qk_bar);
    tma_load_tile(sb + rOffQK + rQKPanel, &tm_q, 64, hk, int(tok0), &qk_bar);
    tma_load_tile(sb + rOffQK + rQKPanel + 8192, &tm_k, 64, hk, int(tok0), &qk_bar);
    issue_loads(hk * G, 0);
  }
  // per-row scalars of the first value head (later heads: fetched one head ahead)
  float pf_gam = 0.f, pf_beta = 0.f;
  auto prefetch_scalars = [&](int hv) {
    if (tid < kC) {
      pf_gam = p.gam[(tok0 + min(tid, rows - 1)) * p.HV + hv];
      pf_beta = tid < rows ? ld_scalar(p.beta, (tok0 + tid) * p.beta_st + hv, p.beta_is_f32) : 0.f;
    }
  };
  prefetch_scalars(hk * G);
  reinterpret_cast<uint4*>(smem + rOffAL)[tid] = make_uint4(0, 0, 0, 0);          // the zero rows of [0 | residual of dZ^T]
  reinterpret_cast<uint4*>(smem + rOffAL)[tid + 256] = make_uint4(0, 0, 0, 0);
  fence_async_smem();
  __syncthreads();
  const uint32_t tbase = tmem_base_s;
  const uint32_t trow = tmem_addr(tbase, quad * 32, 0);
  uint32_t mphase = 0, lphase = 0;
  bool ok = true;

  const Operand opQK{sb + rOffQK, rQKPanel, 0};                      // [q; k], reduction over key dims
  const Operand opKb{sb + rOffQK + 8192, rQKPanel, 0};               // k as B, N = 64 tokens
  const Operand opKn{sb + rOffQK + 8192, rQKPanel, 1};               // k as B, N = 128 key dims, reduction over tokens
  const Operand opQKn{sb + rOffQK, rQKPanel, 1};                     // [q; k] as B, N = 128 key dims, reduction over 128 rows
  // operands of a step: un-swizzled strips (sm100.cuh) whose 64 rows are value channels, the reduction dim of these products
  const Operand opAH{sb + rOffAH, 1024, 2};                                               // [dO; dZ]: M = 128 tokens = 16 strips
  const Operand opAL{sb + rOffAL, 1024, 2};                                               // [0; residual of dZ]: enters dA = -tril(dZ Vn^T) only
  const Operand opVNbH{sb + rOffVNH, 1024, 2}, opVNbL{sb + rOffVNL, 1024, 2};            // Vn as B (N = 64 tokens = 8 strips)
  const Operand opVNaH{sb + rOffVNH - 8192, 1024, 2}, opVNaL{sb + rOffVNL - 8192, 1024, 2};  // Vn as A: accumulator rows 64..127 are valid
  // (the S block, N = 128 key dims = 16 strips, follows each Vn image: the B operands of the N = 192 products start at Vn)
  const Operand opDSH{sb + rOffDSH, 1024, 2}, opDSL{sb + rOffDSL, 1024, 2};
  const Operand opPAH{sb + rOffPAH, 16384, 0}, opPAL{sb + rOffPAL, 16384, 0};            // [dP; dAt], reduction over j
  const Operand opPATh{sb + rOffPAH - 8192, 8192, 1}, opPATl{sb + rOffPAL - 8192, 8192, 1};  // its transpose, valid rows 64..127

  // The running dq (q-side rows) / dk (k-side rows) of the group lives in the last 128 tensor-memory columns, this thread's
  // 64 key-dim columns at rColAcc + half * 64: in registers it would leave none for the issuing code of warp 0.

  // dg / dbeta rows of one value head from its row reductions (threads 0..63 = the two warps that own the 64 rows).
  // dg = reverse chunk-local cumulative sum of dgam; the last row additionally carries
  // e^{gam_L} <S, dS'> + sum_i e^{gam_L - gam_i} k_i.(Vn dS'^T)_i, which therefore reaches every row.
  auto finish_head = [&](int hvf, int fb, float bz) {
    const int i = tid;
    const float (*rd)[2][kC] = red2[fb];
    const float qdq = rd[0][0][i] + rd[0][1][i], kdk = rd[1][0][i] + rd[1][1][i];
    const float g_ = rd[2][0][i] + rd[2][1][i], b_ = rd[3][0][i] + rd[3][1][i], ma = rd[4][0][i] + rd[4][1][i];
    const float gi = gam_s2[fb][i], bi = beta_s2[fb][i], egi = __expf(gi), gl = gam_s2[fb][rows - 1], el = __expf(gl - gi);
    const bool live = i < rows;
    float suf = live ? qdq - kdk + 2.f * bi * ma - 2.f * bi * egi * g_ : 0.f;
    float tot3 = live ? el * b_ : 0.f;
    const int64_t gidx = (tok0 + i) * p.HV + hvf;
    if (live) {
      const float db = bz - egi * g_ + ma;
      if (p.grads_f32) static_cast<float*>(p.dbeta)[gidx] = db;
      else static_cast<bf16*>(p.dbeta)[gidx] = __float2bfloat16_rn(db);
    }
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float dn = __shfl_down_sync(0xffffffffu, suf, o);
      if (lane + o < 32) suf += dn;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tot3 += __shfl_xor_sync(0xffffffffu, tot3, o);
    if (lane == 0) {
      fin_s[0][warp] = suf;      // total of this warp's 32 rows (suffix sum at its first row)
      fin_s[1][warp] = tot3;
    }
    asm volatile("bar.sync 2, 64;" ::: "memory");
    if (warp == 0) suf += fin_s[0][1];
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += sds_s2[fb][w];
    const float dgv = suf + __expf(gl) * tot + fin_s[1][0] + fin_s[1][1];
    if (live) {
      if (p.grads_f32) static_cast<float*>(p.dg)[gidx] = dgv;
      else static_cast<bf16*>(p.dg)[gidx] = __float2bfloat16_rn(dgv);
    }
    asm volatile("bar.sync 2, 64;" ::: "memory");   // fin_s is free again
  };
  auto load_bz = [&](int hvf) -> float {   // sum of the reverse scan's partial row sums of dZ . V (one per 32 columns of V)
    if (tid >= rows) return 0.f;
    const int64_t gidx = (tok0 + tid) * p.HV + hvf;
    const int64_t bzs = p.total_tokens * p.HV;
    float acc = 0.f;
    for (int i = 0; i < NVB; ++i) acc += p.bz[(2 * i) * bzs + gidx] + p.bz[(2 * i + 1) * bzs + gidx];
    return acc;
  };

  float bz_prev = 0.f;
  for (int h = 0; h < G && ok; ++h) {
    const int hv = hk * G + h;
    const int hb = h & 1;
    float* gam_s = gam_s2[hb];
    float* beta_s = beta_s2[hb];
    float (*red)[2][kC] = red2[hb];
    if (tid < kC) {
      gam_s[tid] = pf_gam;
      beta_s[tid] = pf_beta;
    }
    if (h + 1 < G) prefetch_scalars(hv + 1);
    const float bz_cur = load_bz(hv);     // lands while the step's operands are awaited
    float sds = 0.f;
    for (int vb = 0; vb < NVB; ++vb) {
      ok = mbar_wait(&load_bar, lphase, p.status, FLA_ERR_TIMEOUT);
      lphase ^= 1;
      if (h == 0 && vb == 0) ok = mbar_wait(&qk_bar, 0, p.status, FLA_ERR_TIMEOUT) && ok;
      if (!__syncthreads_and(ok)) { ok = false; break; }
      if (tid == 0) {
        tc_fence_after();
        if (h == 0 && vb == 0) mma_tile(tbase + rColQK, opQK, opKb, 128, 64, 8, false);
        const bool accf = vb > 0;
        // [dO; dZ] . [Vn_lo | S_hi]^T and [dO; dZ] . [Vn_hi | S_lo]^T as N = 192 products (the images are neighbours in shared memory, their
        // accumulators neighbours in tensor memory): the A operand is read once for both
        static_assert(rOffVNL + 8192 == rOffSH && rOffVNH + 8192 == rOffSL && rColDV + 64 == rColTA, "the N = 192 products need these adjacent");
        mma_tile(tbase + rColDV, opAH, opVNbL, 128, 192, 4, accf);
        mma_tile(tbase + rColDV, opAH, opVNbH, 128, 192, 4, true);     // [Vn_hi | S_lo]
        mma_tile(tbase + rColDV, opAL, opVNbH, 128, 64, 4, true);
        mma_tile(tbase + rColTB, opVNaH, opDSH, 128, 128, 4, accf);
        mma_tile(tbase + rColTB, opVNaH, opDSL, 128, 128, 4, true);
        mma_tile(tbase + rColTB, opVNaL, opDSH, 128, 128, 4, true);
        mma_commit(&mma_bar);
        if (vb + 1 < NVB) prefetch_loads(hv, vb + 1);
        else if (h + 1 < G) prefetch_loads(hv + 1, 0);
      }
      if (h > 0 && vb == 0 && tid < kC) finish_head(hv - 1, hb ^ 1, bz_prev);   // while the MMAs run
      // <S, dS'> over this V block while the MMAs run (elementwise on the raw images).  Values and residuals: the terms
      // have either sign, so the sum is no larger than its rounding noise would be with the values alone (ragged chunks,
      // where this term dominates dg, then miss the bar by 10x).
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t off = (tid + i * 256) * 16;
        float s1[8], s2[8], d1[8], d2[8];
        unpack_bf16x8(*reinterpret_cast<const uint4*>(smem + rOffSH + off), s1);
        unpack_bf16x8(*reinterpret_cast<const uint4*>(smem + rOffSL + off), s2);
        unpack_bf16x8(*reinterpret_cast<const uint4*>(smem + rOffDSH + off), d1);
        unpack_bf16x8(*reinterpret_cast<const uint4*>(smem + rOffDSL + off), d2);
#pragma unroll
        for (int j = 0; j < 8; ++j) sds += (s1[j] + s2[j]) * (d1[j] + d2[j]);
      }
      ok = mbar_wait(&mma_bar, mphase, p.status, FLA_ERR_TIMEOUT);
      mphase ^= 1;
      if (!__syncthreads_and(ok)) { ok = false; break; }   // also: every thread is done reading the step's buffers
      tc_fence_after();
      if (tid == 0) {
        if (vb + 1 < NVB) issue_loads(hv, vb + 1);
        else if (h + 1 < G) issue_loads(hv + 1, 0);
      }
    }
    if (!ok) break;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sds += __shfl_xor_sync(0xffffffffu, sds, o);
    if (lane == 0) sds_s2[hb][warp] = sds;

    // ---- epilogue 1: score-tile gradients -> [dP; dAt] operand, first parts of this head's dq / dk rows
    const float gam_i = gam_s[tok], beta_i = beta_s[tok], gam_last = gam_s[rows - 1];
    const float eg = __expf(gam_i);
    float ma_part = 0.f;
    {
      float sc[32], dvv[32];
      tmem_ld32(trow + rColQK + half * 32, sc);
      tmem_ld32(trow + rColDV + half * 32, dvv);
      tmem_ld_wait();
      if (!kside) {
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) {
          const int j = half * 32 + jj;
          const float e = p.scale * __expf(fminf(gam_i - gam_s[j], 0.f));
          dvv[jj] *= (j <= tok) ? e : 0.f;
        }
      } else {
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) {
          const int j = half * 32 + jj;
          const float e = __expf(fminf(gam_i - gam_s[j], 0.f));
          const float dec = (j < tok) ? e : 0.f;
          const float dA = -dvv[jj] * dec;
          ma_part += dA * sc[jj];
          dvv[jj] = dA * beta_i;
        }
      }
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint4 hi, lo;
        split8(dvv + ch * 8, hi, lo);
        const uint32_t off = panel_chunk_off(row, half * 4 + ch);
        *reinterpret_cast<uint4*>(smem + rOffPAH + off) = hi;
        *reinterpret_cast<uint4*>(smem + rOffPAL + off) = lo;
      }
    }
    float part[64];   // this head's contribution to my dq / dk row (64 key-dim columns)
    float rkG = 0.f, rkB = 0.f;
    tmem_ld_row64(trow + rColTA + half * 64, part);
    if (!kside) {
      const float f = p.scale * eg;
#pragma unroll
      for (int i = 0; i < 64; ++i) part[i] *= f;
    } else {
      row_dot64(smem + rOffQK, rQKPanel, 64 + tok, half * 64, part, rkG);
      float bk[64];
      tmem_ld_row64(trow + rColTB + half * 64, bk);
      row_dot64(smem + rOffQK, rQKPanel, 64 + tok, half * 64, bk, rkB);
      const float f1 = -beta_i * eg, f2 = __expf(gam_last - gam_i);
#pragma unroll
      for (int i = 0; i < 64; ++i) part[i] = f1 * part[i] + f2 * bk[i];
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();

    // ---- [dP; dAt] K  and  [dP^T | dAt^T] [Q; K]
    if (tid == 0) {
      tc_fence_after();
      mma_tile(tbase + rColTA, opPAH, opKn, 128, 128, 4, false);
      mma_tile(tbase + rColTA, opPAL, opKn, 128, 128, 4, true);
      mma_tile(tbase + rColTB, opPATh, opQKn, 128, 128, 8, false);
      mma_tile(tbase + rColTB, opPATl, opQKn, 128, 128, 8, true);
      mma_commit(&mma_bar);
    }
    ok = mbar_wait(&mma_bar, mphase, p.status, FLA_ERR_TIMEOUT);
    mphase ^= 1;
    if (!__syncthreads_and(ok)) { ok = false; break; }
    tc_fence_after();

    // ---- epilogue 2: finish the rows, row dots for dg / dbeta
    {
      float t[64];
      tmem_ld_row64(trow + rColTA + half * 64, t);
#pragma unroll
      for (int i = 0; i < 64; ++i) part[i] += t[i];
      if (kside) {
        tmem_ld_row64(trow + rColTB + half * 64, t);
#pragma unroll
        for (int i = 0; i < 64; ++i) part[i] += t[i];
      }
    }
    float xdx = 0.f;  // q.dq (q-side) or k.dk (k-side) over my columns
    row_dot64(smem + rOffQK, rQKPanel, row, half * 64, part, xdx);
    if (h > 0) {
      float t[64];
      tmem_ld_row64(trow + rColAcc + half * 64, t);
#pragma unroll
      for (int i = 0; i < 64; ++i) part[i] += t[i];
    }
    if (h + 1 < G) tmem_st_row64(trow + rColAcc + half * 64, part);
    else if (tok < rows) {   // the last head: the rows are complete
      void* base = kside ? p.dk : p.dq;
      const int64_t off = kside ? (tok0 + tok) * p.dk_st + hk * p.dk_sh + half * 64 : (tok0 + tok) * p.dq_st + hk * p.dq_sh + half * 64;
      if (p.grads_f32) {
        float* dst = static_cast<float*>(base) + off;
#pragma unroll
        for (int i = 0; i < 64; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(part[i], part[i + 1], part[i + 2], part[i + 3]);
      } else {
        bf16* dst = static_cast<bf16*>(base) + off;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(dst + ch * 8) = pack8(part + ch * 8);
      }
    }
    if (!kside) {
      red[0][half][tok] = xdx;
    } else {
      red[1][half][tok] = xdx;
      red[2][half][tok] = rkG;
      red[3][half][tok] = rkB;
      red[4][half][tok] = ma_part;
    }
    tc_fence_before();
    __syncthreads();
    bz_prev = bz_cur;
  }
  if (__syncthreads_and(ok) && tid < kC) finish_head(hk * G + G - 1, (G - 1) & 1, bz_prev);

  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 512);
}

}  // namespace fla

using namespace fla;

static uint64_t bwd_ws_layout(int64_t total_chunks, int64_t HV, int64_t nvb, int64_t tokens, uint64_t* off_ds, uint64_t* off_dz,
                              uint64_t* off_bz) {
  uint64_t o = 256;  // status block
  *off_ds = o; o += align_up(uint64_t(total_chunks) * HV * nvb * kSImg * 2, 256);
  *off_dz = o; o += align_up(uint64_t(total_chunks) * HV * nvb * kDzImg * 2, 256);
  *off_bz = o; o += align_up(uint64_t(2 * nvb) * tokens * HV * 4, 256);
  return o;
}

static int bwd_geometry(const fla_gdn_chunk_bwd_args* a, int64_t* total_chunks, int* N, int* max_len) {
  const fla_tensor_t& q = a->q;
  if (!q.data || q.ndim != 4 || !a->v.data || a->v.ndim != 4) return FLA_ERR_SHAPE;
  const int64_t B = q.shape[0], T = q.shape[1];
  *N = int(B);
  *total_chunks = B * ((T + kC - 1) / kC);
  *max_len = int(T);
  if (a->cu_seqlens.data) {
    if (B != 1 || a->cu_seqlens.dtype != FLA_I32 || a->cu_seqlens.ndim != 1 || a->cu_seqlens.shape[0] < 2) return FLA_ERR_SHAPE;
    *N = int(a->cu_seqlens.shape[0] - 1);
    if (!a->chunk_offsets.data || a->chunk_offsets.dtype != FLA_I32 || a->chunk_offsets.shape[0] != *N + 1) return FLA_ERR_SHAPE;
    if (a->max_seqlen <= 0 || a->max_seqlen > T || a->total_chunks <= 0) return FLA_ERR_VALUE;
    *max_len = a->max_seqlen;
    *total_chunks = a->total_chunks;
  }
  return FLA_OK;
}

extern "C" FLA_API int fla_b200_gdn_chunk_bwd_workspace_size(const fla_gdn_chunk_bwd_args* a, uint64_t* bytes) {
  if (!a || !bytes) return FLA_ERR_NULL;
  int64_t total_chunks; int N, max_len;
  int st = bwd_geometry(a, &total_chunks, &N, &max_len);
  if (st) return st;
  uint64_t o1, o2, o3;
  const int64_t V = a->v.shape[3];
  if (V != kV && V != 2 * kV) return FLA_ERR_SHAPE;
  *bytes = bwd_ws_layout(total_chunks, a->v.shape[2], V / kBV, a->q.shape[0] * a->q.shape[1], &o1, &o2, &o3);
  return FLA_OK;
}

static int check_tok4(const fla_tensor_t& t, int64_t B, int64_t T, int64_t heads, int64_t dim, bool allow_f32) {
  if (!t.data) return FLA_ERR_NULL;
  if (t.ndim != 4 || t.shape[0] != B || t.shape[1] != T || t.shape[2] != heads || t.shape[3] != dim) return FLA_ERR_SHAPE;
  if (t.dtype != FLA_BF16 && !(allow_f32 && t.dtype == FLA_F32)) return FLA_ERR_DTYPE;
  const int64_t esz = t.dtype == FLA_F32 ? 4 : 2;
  if (t.stride[3] != 1 || (t.stride[2] * esz) % 16 || (t.stride[1] * esz) % 16 || !aligned16(t.data)) return FLA_ERR_LAYOUT;
  if (B > 1 && t.stride[0] != T * t.stride[1]) return FLA_ERR_LAYOUT;
  return FLA_OK;
}
static int check_tok3(const fla_tensor_t& t, int64_t B, int64_t T, int64_t heads, bool dense) {
  if (!t.data) return FLA_ERR_NULL;
  if (t.ndim != 3 || t.shape[0] != B || t.shape[1] != T || t.shape[2] != heads) return FLA_ERR_SHAPE;
  if (t.dtype != FLA_BF16 && t.dtype != FLA_F32) return FLA_ERR_DTYPE;
  if (t.stride[2] != 1 || (B > 1 && t.stride[0] != T * t.stride[1])) return FLA_ERR_LAYOUT;
  if (dense && t.stride[1] != heads) return FLA_ERR_LAYOUT;
  return FLA_OK;
}


static int gdn_chunk_bwd_impl(const fla_gdn_chunk_bwd_args* a, void* workspace, uint64_t workspace_bytes, void* stream,
                              bool allow_split) {
  if (!a) return FLA_ERR_NULL;
  int64_t total_chunks; int N, max_len;
  int st = bwd_geometry(a, &total_chunks, &N, &max_len);
  if (st) return st;
  const int64_t B = a->q.shape[0], T = a->q.shape[1], HK = a->q.shape[2], HV = a->v.shape[2];
  if (HK <= 0 || HV <= 0 || HV % HK) return FLA_ERR_SHAPE;
  const int64_t V = a->v.shape[3], nvb = V / kBV;
  if (V != kV && V != 2 * kV) return FLA_ERR_SHAPE;
  if ((st = check_tok4(a->q, B, T, HK, kK, false))) return st;
  if ((st = check_tok4(a->k, B, T, HK, kK, false))) return st;
  if ((st = check_tok4(a->v, B, T, HV, V, false))) return st;
  if ((st = check_tok4(a->d_o, B, T, HV, V, false))) return st;
  if ((st = check_tok4(a->dq, B, T, HK, kK, true))) return st;
  if ((st = check_tok4(a->dk, B, T, HK, kK, true))) return st;
  if ((st = check_tok4(a->dv, B, T, HV, V, true))) return st;
  if ((st = check_tok3(a->beta, B, T, HV, false))) return st;
  if ((st = check_tok3(a->dg, B, T, HV, true))) return st;
  if ((st = check_tok3(a->dbeta, B, T, HV, true))) return st;
  const int gdt = a->dq.dtype;
  if (a->dk.dtype != gdt || a->dv.dtype != gdt || a->dg.dtype != gdt || a->dbeta.dtype != gdt) return FLA_ERR_DTYPE;
  const fla_tensor_t &gam = a->gam, &X = a->x_inv;
  if (!gam.data || !X.data || !a->s_img.data || !a->vn_img.data || !a->p_img.data) return FLA_ERR_NULL;
  if (gam.dtype != FLA_F32 || gam.ndim != 3 || gam.shape[0] != B || gam.shape[1] != T || gam.shape[2] != HV ||
      gam.stride[2] != 1 || gam.stride[1] != HV || (B > 1 && gam.stride[0] != T * HV))
    return FLA_ERR_SHAPE;
  if (X.dtype != FLA_BF16 || X.ndim != 1 || X.shape[0] != total_chunks * HV * 8192 || !aligned16(X.data))
    return FLA_ERR_SHAPE;
  if (a->p_img.dtype != FLA_BF16 || a->p_img.ndim != 1 || a->p_img.shape[0] != total_chunks * HV * kPImg || !aligned16(a->p_img.data))
    return FLA_ERR_SHAPE;
  if (a->s_img.dtype != FLA_BF16 || a->s_img.ndim != 1 || a->s_img.shape[0] != total_chunks * HV * nvb * kSImg || !aligned16(a->s_img.data))
    return FLA_ERR_SHAPE;
  if (a->vn_img.dtype != FLA_BF16 || a->vn_img.ndim != 1 || a->vn_img.shape[0] != total_chunks * HV * nvb * kVnImg || !aligned16(a->vn_img.data))
    return FLA_ERR_SHAPE;
  for (const fla_tensor_t* s : {&a->dht, &a->dh0}) {
    if (!s->data) continue;
    if (s->dtype != FLA_F32) return FLA_ERR_DTYPE;
    if (s->ndim != 4 || s->shape[0] != N || s->shape[1] != HV || s->shape[2] != kK || s->shape[3] != V) return FLA_ERR_SHAPE;
    if (s->stride[3] != 1 || s->stride[2] != V || s->stride[1] != kK * V || s->stride[0] != HV * kK * V || !aligned16(s->data))
      return FLA_ERR_LAYOUT;
  }
  if (a->chunk_size != kC) return FLA_ERR_VALUE;
  uint64_t off_ds, off_dz, off_bz;
  const uint64_t need = bwd_ws_layout(total_chunks, HV, nvb, B * T, &off_ds, &off_dz, &off_bz);
  if (!workspace || workspace_bytes < need || !aligned16(workspace)) return FLA_ERR_WORKSPACE;

  GdnBwdParams p{};
  p.q = static_cast<const bf16*>(a->q.data); p.k = static_cast<const bf16*>(a->k.data);
  p.v = static_cast<const bf16*>(a->v.data); p.dO = static_cast<const bf16*>(a->d_o.data);
  p.beta = a->beta.data; p.gam = static_cast<const float*>(gam.data); p.X = static_cast<const bf16*>(X.data);
  p.s_img = static_cast<const bf16*>(a->s_img.data); p.vn_img = static_cast<const bf16*>(a->vn_img.data);
  p.p_img = static_cast<const bf16*>(a->p_img.data);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  p.status = reinterpret_cast<int*>(ws);
  p.ds_img = reinterpret_cast<bf16*>(ws + off_ds);
  p.dz_img = reinterpret_cast<bf16*>(ws + off_dz);
  p.bz = reinterpret_cast<float*>(ws + off_bz);
  p.dht = static_cast<const float*>(a->dht.data); p.dh0 = static_cast<float*>(a->dh0.data);
  p.dq = a->dq.data; p.dk = a->dk.data; p.dv = a->dv.data; p.dg = a->dg.data; p.dbeta = a->dbeta.data;
  p.cu_seqlens = static_cast<const int32_t*>(a->cu_seqlens.data);
  p.chunk_offsets = static_cast<const int32_t*>(a->chunk_offsets.data);
  p.q_st = a->q.stride[1]; p.q_sh = a->q.stride[2]; p.k_st = a->k.stride[1]; p.k_sh = a->k.stride[2];
  p.v_st = a->v.stride[1]; p.v_sh = a->v.stride[2]; p.do_st = a->d_o.stride[1]; p.do_sh = a->d_o.stride[2];
  p.beta_st = a->beta.stride[1];
  p.dq_st = a->dq.stride[1]; p.dq_sh = a->dq.stride[2]; p.dk_st = a->dk.stride[1]; p.dk_sh = a->dk.stride[2];
  p.dv_st = a->dv.stride[1]; p.dv_sh = a->dv.stride[2];
  p.total_tokens = B * T;
  p.N = N; p.T = int(T); p.HK = int(HK); p.HV = int(HV); p.V = int(V); p.nvb = int(nvb);
  p.beta_is_f32 = a->beta.dtype == FLA_F32; p.grads_f32 = gdt == FLA_F32;
  p.scale = a->scale;

  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(workspace, 0, 256, cs) != cudaSuccess) return FLA_ERR_CUDA;
  static std::atomic<bool> attr_done_dev[64] = {};   // per device ordinal; setting the attributes twice is harmless
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FLA_ERR_CUDA;
  if (!attr_done_dev[dev]) {
    if (cudaFuncSetAttribute(gdn_scan_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kScanBwdSmem) + 1024) != cudaSuccess) return FLA_ERR_CUDA;
    if (cudaFuncSetAttribute(gdn_bwd_par_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kParSmem) + 1024) != cudaSuccess) return FLA_ERR_CUDA;
    if (cudaFuncSetAttribute(gdn_bwd_par_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kParSmem) + 1024) != cudaSuccess) return FLA_ERR_CUDA;
    attr_done_dev[dev] = true;
  }
  CUtensorMap tm_q, tm_k, tm_v, tm_d;
  if (make_row_tile_map(&tm_q, p.q, kK, uint64_t(HK), uint64_t(B * T), uint64_t(p.q_sh), uint64_t(p.q_st)) ||
      make_row_tile_map(&tm_k, p.k, kK, uint64_t(HK), uint64_t(B * T), uint64_t(p.k_sh), uint64_t(p.k_st)) ||
      make_row_tile_map(&tm_v, p.v, uint64_t(V), uint64_t(HV), uint64_t(B * T), uint64_t(p.v_sh), uint64_t(p.v_st)) ||
      make_row_tile_map(&tm_d, p.dO, uint64_t(V), uint64_t(HV), uint64_t(B * T), uint64_t(p.do_sh), uint64_t(p.do_st)))
    return FLA_ERR_CUDA;
  const int nt_max = (max_len + kC - 1) / kC;
  auto launch_scan = [&](const GdnBwdParams& pp, int nseq, cudaStream_t st) {
    gdn_scan_bwd_kernel<<<dim3(unsigned(V / 128), unsigned(HV), nseq), kScanThreads, kScanBwdSmem + 1024, st>>>(pp, tm_q, tm_k, tm_v, tm_d);
  };
  auto launch_par = [&](const GdnBwdParams& pp, int nseq, cudaStream_t st) {
    if (nvb == 2) gdn_bwd_par_kernel<2><<<dim3(nt_max, unsigned(HK), nseq), 256, kParSmem + 1024, st>>>(pp, tm_q, tm_k);
    else gdn_bwd_par_kernel<4><<<dim3(nt_max, unsigned(HK), nseq), 256, kParSmem + 1024, st>>>(pp, tm_q, tm_k);
  };
  // The reverse scan launches one CTA per (sequence, value head, 128 channels) and each needs a whole SM: when there are
  // more chains than SMs the last round leaves SMs idle for the length of a chain.  The batch is then launched as two
  // halves on two streams, so that the chunk-parallel kernel of the first half fills the SMs the second half's scan
  // leaves free.  Not while per-kernel timing is on (its events bracket single launches), not during stream capture, not
  // for the allocation-free entry (creating the second stream may allocate).
  AuxStream* aux = nullptr;
  if (allow_split && N >= 2 && int64_t(V / 128) * HV * N > sm_count(dev) && !kernel_timing_enabled()) aux = aux_stream_for(dev, cs);
  if (aux) {
    std::lock_guard<std::mutex> lk(aux->mu);   // the fork / join events are shared by the callers of this stream
    const int n1 = N / 2;
    GdnBwdParams p2 = p;
    p2.n0 = n1;
    bool okc = cudaEventRecord(aux->fork, cs) == cudaSuccess && cudaStreamWaitEvent(aux->s, aux->fork, 0) == cudaSuccess;
    if (!okc) return FLA_ERR_CUDA;
    launch_scan(p, n1, cs);
    launch_scan(p2, N - n1, aux->s);
    launch_par(p, n1, cs);
    launch_par(p2, N - n1, aux->s);
    okc = cudaEventRecord(aux->join, aux->s) == cudaSuccess && cudaStreamWaitEvent(cs, aux->join, 0) == cudaSuccess;
    if (!okc) return FLA_ERR_CUDA;
    return cuda_status(cudaGetLastError());
  }
  {
    KernelTimer kt("gdn_bwd_dhu", cs);
    launch_scan(p, N, cs);
  }
  if (cudaGetLastError() != cudaSuccess) return FLA_ERR_CUDA;
  {
    KernelTimer kt("gdn_bwd_par", cs);
    launch_par(p, N, cs);
  }
  return cuda_status(cudaGetLastError());
}

extern "C" FLA_API int fla_b200_gdn_chunk_bwd(const fla_gdn_chunk_bwd_args* a, void* workspace, uint64_t workspace_bytes,
                                              void* stream) {
  return gdn_chunk_bwd_impl(a, workspace, workspace_bytes, stream, true);
}

// ----------------------------------------------------------------------------- allocation-free variant
// Some hosts of this library may not allocate device memory at the point where they call the backward:
// an inference / training runtime that sized one device arena at start-up and forbids any later
// cudaMalloc (an allocation can synchronise the whole device and stall the other streams of a serving
// process), a plugin running inside another framework's callback that owns the allocator, or a
// real-time loop with a fixed memory budget.  For them the scratch that fla_b200_gdn_chunk_bwd normally
// receives from the caller lives here instead, in one fixed array that is part of the library image:
// every GPU whose context loads libfla_b200.so carries these 32 MiB until the process exits.
constexpr uint64_t kStaticScratchBytes = 32ull << 20;
static __device__ __align__(256) unsigned char g_bwd_static_scratch[kStaticScratchBytes];

#include <mutex>
namespace {
std::mutex g_static_mu;
void* g_static_ptr[64] = {};   // device address of the array, per device ordinal
}  // namespace

extern "C" FLA_API int fla_b200_gdn_chunk_bwd_static_scratch_bytes(uint64_t* bytes) {
  if (!bytes) return FLA_ERR_NULL;
  *bytes = kStaticScratchBytes;
  return FLA_OK;
}

extern "C" FLA_API int fla_b200_gdn_chunk_bwd_noalloc(const fla_gdn_chunk_bwd_args* a, void* stream) {
  if (!a) return FLA_ERR_NULL;
  uint64_t need = 0;
  const int st = fla_b200_gdn_chunk_bwd_workspace_size(a, &need);
  if (st != FLA_OK) return st;
  if (need > kStaticScratchBytes) return FLA_ERR_TOO_LARGE;   // the problem does not fit the built-in scratch
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FLA_ERR_CUDA;
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (!g_static_ptr[dev]) {
      // In host code the array's name is only a handle; the address the kernels can use has to be asked for,
      // once per device, while that device is current.
      void* ptr = nullptr;
      if (cudaGetSymbolAddress(&ptr, g_bwd_static_scratch) != cudaSuccess || !ptr) return FLA_ERR_CUDA;
      g_static_ptr[dev] = ptr;
    }
    scratch = g_static_ptr[dev];
  }
  // The regular entry point clears the status block at the head of the scratch on `stream` and overwrites
  // every other byte it later reads, so nothing else of the previous call's contents matters.
  return gdn_chunk_bwd_impl(a, scratch, kStaticScratchBytes, stream, false);   // one stream: creating a second one may allocate
}

// The status word of the allocation-free entry lives at the head of the built-in array, which the caller cannot
// address; this copies it out after waiting for `stream` (the stream of the call being checked).
extern "C" FLA_API int fla_b200_gdn_chunk_bwd_noalloc_status(void* stream, int32_t* status_out) {
  if (!status_out) return FLA_ERR_NULL;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FLA_ERR_CUDA;
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_static_mu);
    scratch = g_static_ptr[dev];
  }
  if (!scratch) {   // no call on this device yet: nothing has run, nothing can have timed out
    *status_out = FLA_OK;
    return FLA_OK;
  }
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  int32_t word = 0;
  if (cudaMemcpyAsync(&word, scratch, sizeof(word), cudaMemcpyDeviceToHost, cs) != cudaSuccess) return FLA_ERR_CUDA;
  if (cudaStreamSynchronize(cs) != cudaSuccess) return FLA_ERR_CUDA;
  *status_out = word;
  return FLA_OK;
}


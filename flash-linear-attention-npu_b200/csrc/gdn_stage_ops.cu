// Stand-alone stages of the chunked gated-delta-rule forward, one entry point per reference operator
// (torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py): chunk_local_cumsum (:875-904),
// chunk_scaled_dot_kkt (:907-936), solve_tri (:1786-1800), recompute_w_u_fwd (:618-651),
// chunk_gated_delta_rule_fwd_h (:552-615) and chunk_fwd_o (:517-549).
//
// The fused kernels (gdn_chunk_fwd.cu) never materialise A, w, u or the per-chunk states; these operators exist for
// call sites that drive the reference's stage-by-stage chain and therefore read and write those tensors in HBM.
// Operands that arrive as bf16 tensors enter the MMAs as they are; operands computed on the way (k beta e^g, v beta, the
// state copy, the decayed v_new, the decayed score tile) are split into a bf16 value and a bf16 residual and multiplied in
// two passes, so each stage is accurate to fp32 round-off for the inputs it is given (the reference rounds them to one
// bf16).  The running state of fwd_h stays in fp32 (in tensor memory) for the whole sequence.
//
// Every tensor is addressed as [B, H, T, D] (or [B, H, T]) through its strides, so the reference's head-first
// tensors and sequence-first views of the same memory are both accepted; D must be contiguous.
// Tensor-core tiles are M = 128 tcgen05 MMAs whose rows 0..63 hold the chunk's 64 tokens (rows 64..127 are
// never read back), except for kkt, which packs two consecutive chunks into one 128-row tile.
#include <algorithm>
#include "gdn_common.cuh"
#include "fla_b200_internal.h"
#include "kernel_timer.h"
#include "tensor_map.h"

namespace fla {

struct StageView {     // [B, H, T, D] view, D contiguous
  const void* p;
  int64_t sb, sh, st;
  int dtype;           // fla_dtype
};

struct StageParams {
  StageView q, k, v, w, u, g, beta, a, h, h0;
  StageView o0, o1, o2, o3;
  float* ws_dq;   // dqkwg with GVA: per-value-head fp32 rows [B*H*T, 128] of dq and dk, reduced over the group afterwards
  float* ws_dk;
  const int32_t* cu_seqlens;
  const int32_t* chunk_offsets;
  int T, H, HK, D;
  int reverse, want_final;
  int wy_mode;              // prepare_wy_repr_bwd: 0 fused, 1 dA only, 2 dk / dv / dbeta / dg from a given dA
  int gate_mode;            // cumsum of per-channel gates: 0 raw, 1 -e^{A_log} softplus(g + dt_bias), 2 lower_bound sigmoid(e^{A_log} (g + dt_bias))
  const float* a_log;       // [H]
  const float* dt_bias;     // [H, D] or null
  float lower_bound;
  float scale;
  int* status;
};

__device__ __forceinline__ float ld_any(const void* p, int64_t idx, int dtype) {
  if (dtype == FLA_F32) return static_cast<const float*>(p)[idx];
  if (dtype == FLA_BF16) return __bfloat162float(static_cast<const bf16*>(p)[idx]);
  return __half2float(static_cast<const __half*>(p)[idx]);
}
__device__ __forceinline__ void st_any(void* p, int64_t idx, int dtype, float v) {
  if (dtype == FLA_F32) static_cast<float*>(p)[idx] = v;
  else if (dtype == FLA_BF16) static_cast<bf16*>(p)[idx] = __float2bfloat16_rn(v);
  else static_cast<__half*>(p)[idx] = __float2half_rn(v);
}
// first element of row (b, h, t)
__device__ __forceinline__ int64_t row_off(const StageView& v, int64_t b, int64_t h, int64_t t) {
  return b * v.sb + h * v.sh + t * v.st;
}

// ----------------------------------------------------------------------------- chunk_local_cumsum
// out[t] = scale * sum of g over the tokens of t's chunk up to t (reverse: from t on).  D == 1: one thread per token,
// two warps per chunk, shuffle scan.  D > 1 (per-channel gates): one thread per channel, serial over the chunk.
__global__ void __launch_bounds__(128) stage_cumsum_kernel(StageParams p) {
  const int n = blockIdx.z, hh = blockIdx.y, c = blockIdx.x;
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  if (c >= sq.nt) return;
  const int rows = min(kC, sq.len - c * kC);
  const int64_t b = p.cu_seqlens ? 0 : n;
  const int64_t t0 = (p.cu_seqlens ? sq.bos : 0) + c * kC;
  const int tid = threadIdx.x;
  if (p.D == 1) {
    __shared__ float wsum[2];
    const int lane = tid & 31, warp = tid >> 5;
    const int t = p.reverse ? kC - 1 - tid : tid;    // scan position tid <-> token t
    float x = (tid < kC && t < rows) ? ld_any(p.g.p, row_off(p.g, b, hh, t0 + t), p.g.dtype) : 0.f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float up = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += up;
    }
    if (lane == 31 && warp < 2) wsum[warp] = x;
    __syncthreads();
    if (warp == 1) x += wsum[0];
    if (tid < kC && t < rows) st_any(const_cast<void*>(p.o0.p), row_off(p.o0, b, hh, t0 + t), p.o0.dtype, x * p.scale);
  } else {
    for (int d = tid; d < p.D; d += blockDim.x) {
      float run = 0.f;
      const float eig = p.gate_mode ? __expf(p.a_log[hh]) : 0.f;
      const float bias = (p.gate_mode && p.dt_bias) ? p.dt_bias[hh * p.D + d] : 0.f;
      for (int i = 0; i < rows; ++i) {
        const int t = p.reverse ? rows - 1 - i : i;
        float x = ld_any(p.g.p, row_off(p.g, b, hh, t0 + t) + d, p.g.dtype);
        if (p.gate_mode == 1) {
          const float r = x + bias;
          x = -eig * (r > 20.f ? r : log1pf(__expf(r)));
        } else if (p.gate_mode == 2) {
          x = p.lower_bound / (1.f + __expf(-eig * (x + bias)));
        }
        run += x;
        st_any(const_cast<void*>(p.o0.p), row_off(p.o0, b, hh, t0 + t) + d, p.o0.dtype, run * p.scale);
      }
    }
  }
}

__device__ __forceinline__ uint8_t* align1024(uint8_t* raw) {
  return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
}

// ----------------------------------------------------------------------------- chunk_scaled_dot_kkt
// A[i, j] = beta_i exp(clamp(g_i - g_j, -50, 50)) k_i . k_j for j < i, else 0.  One CTA per (chunk pair, q/k head):
// one 128 x 128 product [k_c; k_c+1] [k_c; k_c+1]^T serves both chunks (diagonal blocks) and all value heads of the group.
constexpr uint32_t kKktSmem = 32768;
__global__ void __launch_bounds__(128) stage_kkt_kernel(StageParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  __shared__ float gam_s[2][kC];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t mma_bar;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int n = blockIdx.z, hk = blockIdx.y, c0 = blockIdx.x * 2;
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  if (c0 >= sq.nt) return;
  const int64_t b = p.cu_seqlens ? 0 : n;
  const int64_t tbeg = p.cu_seqlens ? sq.bos : 0;
  const int G = p.H / p.HK;
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 128);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(&mma_bar, 1);
    mbar_init_fence();
  }
  {   // k rows of both chunks: all sixteen 16-byte loads of a thread are issued before the first shared-memory store (a store
      // through a generic pointer between two loads would keep the compiler from overlapping them)
    uint4 val[16];
#pragma unroll
    for (int it = 0; it < 16; ++it) {
      const int which = it >> 3, idx = tid + (it & 7) * 128, r = idx >> 4, ch = idx & 15;
      const int c = c0 + which;
      const int rows = c < sq.nt ? min(kC, sq.len - c * kC) : 0;
      val[it] = make_uint4(0, 0, 0, 0);
      if (r < rows) {
        const bf16* src = static_cast<const bf16*>(p.k.p) + row_off(p.k, b, hk, tbeg + c * kC);
        val[it] = *reinterpret_cast<const uint4*>(src + r * p.k.st + ch * 8);
      }
    }
#pragma unroll
    for (int it = 0; it < 16; ++it) {
      const int which = it >> 3, idx = tid + (it & 7) * 128, r = idx >> 4, ch = idx & 15;
      *reinterpret_cast<uint4*>(smem + which * 8192 + (ch >> 3) * 16384 + panel_chunk_off(r, ch & 7)) = val[it];
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  const uint32_t tbase = tmem_base_s;
  const uint32_t sb = smem_u32(smem);
  if (tid == 0) {
    tc_fence_after();
    const Operand opK{sb, 16384, 0};
    mma_tile(tbase, opK, opK, 128, 128, 8, false);
    mma_commit(&mma_bar);
  }
  const bool ok = mbar_wait(&mma_bar, 0, p.status, FLA_ERR_TIMEOUT);
  tc_fence_after();
  const int which = tid >> 6, i = tid & 63;
  const int c = c0 + which;
  const int rows = c < sq.nt ? min(kC, sq.len - c * kC) : 0;
  float s[64];
  tmem_ld_row64(tmem_addr(tbase, warp * 32, which * 64), s);
  // gate and beta of my row: fetched one value head ahead of their use
  auto load_gb = [&](int hv, float& gv, float& bv) {
    gv = i < rows ? ld_any(p.g.p, row_off(p.g, b, hv, tbeg + c * kC + i), p.g.dtype) : 0.f;
    bv = i < rows ? ld_any(p.beta.p, row_off(p.beta, b, hv, tbeg + c * kC + i), p.beta.dtype) : 0.f;
  };
  float g_next, b_next;
  load_gb(hk * G, g_next, b_next);
  for (int h = 0; h < G; ++h) {
    const int hv = hk * G + h;
    const float bi = b_next;
    __syncthreads();
    gam_s[which][i] = g_next;
    if (h + 1 < G) load_gb(hv + 1, g_next, b_next);
    __syncthreads();
    if (ok && i < rows) {
      const float gi = gam_s[which][i];
      float* dst = static_cast<float*>(const_cast<void*>(p.o0.p)) + row_off(p.o0, b, hv, tbeg + c * kC + i);
#pragma unroll
      for (int j4 = 0; j4 < kC; j4 += 4) {
        float r[4];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          const int j = j4 + jj;
          const float e = __expf(fminf(fmaxf(gi - gam_s[which][j], -50.f), 50.f));
          r[jj] = (j < i) ? bi * e * s[j] : 0.f;
        }
        *reinterpret_cast<float4*>(dst + j4) = make_float4(r[0], r[1], r[2], r[3]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 128);
}

// ----------------------------------------------------------------------------- solve_tri
// X = (I + A)^-1 per chunk, A strictly lower triangular (entries on and above the diagonal are ignored), fp32
// forward substitution, one thread per column (the scheme of tri_inverse.cu), two matrices per CTA.
constexpr int kSolveStride = 68;
constexpr int kSolveTiles = 2;   // matrices per CTA; small CTAs under a register bound keep ten solves in flight per SM
__global__ void __launch_bounds__(64 * kSolveTiles, 5) stage_solve_tri_kernel(StageParams p) {
  extern __shared__ float tri_sm[];
  const int tid = threadIdx.x, grp = tid / 64, c = tid % 64;
  const int n = blockIdx.z, chunk = blockIdx.x;
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  if (chunk >= sq.nt) return;
  const int hh = blockIdx.y * kSolveTiles + grp;
  const bool active = hh < p.H;
  const int rows = min(kC, sq.len - chunk * kC);
  const int64_t b = p.cu_seqlens ? 0 : n;
  const int64_t t0 = (p.cu_seqlens ? sq.bos : 0) + chunk * kC;
  float* AT = tri_sm + grp * kC * kSolveStride;
  // The matrices of the CTA are staged together as AT[j][i] = A[i][j] (j < i).  A warp covers 8 rows x 16 columns:
  // each thread reads four consecutive elements of a row (64 contiguous bytes per row and warp for fp32) and the
  // transposed stores of a warp fall on at most two addresses per bank.
  const bool vec4 = p.a.dtype == FLA_F32 && (reinterpret_cast<uintptr_t>(p.a.p) & 15) == 0 && ((p.a.sb | p.a.sh | p.a.st) & 3) == 0;
#pragma unroll 4
  for (int idx = tid; idx < kSolveTiles * kC * 16; idx += 64 * kSolveTiles) {
    const int m = idx >> 10, i = ((idx >> 5) & 7) * 8 + (idx & 7), jc = ((idx >> 8) & 3) * 4 + ((idx >> 3) & 3);
    const int hm = blockIdx.y * kSolveTiles + m;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (hm < p.H && i < rows && jc * 4 < i) {
      const int64_t off = row_off(p.a, b, hm, t0 + i) + jc * 4;
      if (vec4) {
        const float4 t = *reinterpret_cast<const float4*>(static_cast<const float*>(p.a.p) + off);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) v[q] = ld_any(p.a.p, off + q, p.a.dtype);
      }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) tri_sm[m * kC * kSolveStride + (jc * 4 + q) * kSolveStride + i] = (jc * 4 + q < i) ? v[q] : 0.f;
  }
  __syncthreads();
  if (!active) return;
  float x[kC];
#pragma unroll
  for (int i = 0; i < kC; ++i) x[i] = (i == c) ? 1.f : 0.f;
  const int jmin = c & ~31;
#pragma unroll
  for (int j = 0; j < kC - 1; ++j) {
    if (j >= jmin) {
      const float xj = x[j];
      const float* col = AT + j * kSolveStride;
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
#pragma unroll
  for (int i = 0; i < kC; ++i)
    if (i < rows) st_any(const_cast<void*>(p.o0.p), row_off(p.o0, b, hh, t0 + i) + c, p.o0.dtype, c < rows ? x[i] : 0.f);
}

// ----------------------------------------------------------------------------- recompute_w_u_fwd
// u = X (v beta),  w = X (k beta e^g) per chunk and value head; X is the chunk's 64 x 64 block of (I + A)^-1.
// X, k and v rows arrive as TMA tiles; the scaled rows replace the raw k / v tiles in place (bf16 value) next to a
// residual panel.
constexpr uint32_t wuOffX = 0, wuOffKh = 8192, wuOffKl = 24576, wuOffVh = 40960, wuOffVl = 57344;
constexpr uint32_t kWuSmem = 73728;
__global__ void __launch_bounds__(256) stage_wu_kernel(StageParams p, const __grid_constant__ CUtensorMap tm_k,
                                                       const __grid_constant__ CUtensorMap tm_v,
                                                       const __grid_constant__ CUtensorMap tm_x) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  __shared__ float rs_k[kC], rs_v[kC];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t mma_bar, load_bar;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int n = blockIdx.z, hv = blockIdx.y, c = blockIdx.x;
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  if (c >= sq.nt) return;
  const int rows = min(kC, sq.len - c * kC);
  const int b = p.cu_seqlens ? 0 : n;
  const int t0 = (p.cu_seqlens ? sq.bos : 0) + c * kC;
  const int hk = hv / (p.H / p.HK);
  const uint32_t sb = smem_u32(smem);
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 256);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(&mma_bar, 1);
    mbar_init(&load_bar, 1);
    mbar_init_fence();
    mbar_arrive_expect_tx(&load_bar, 8192 + 16384 + 16384);
    tma_load_tile4(sb + wuOffX, &tm_x, 0, t0, hv, b, &load_bar);
    tma_load_tile4(sb + wuOffKh, &tm_k, 0, t0, hk, b, &load_bar);
    tma_load_tile4(sb + wuOffKh + 8192, &tm_k, 64, t0, hk, b, &load_bar);
    tma_load_tile4(sb + wuOffVh, &tm_v, 0, t0, hv, b, &load_bar);
    tma_load_tile4(sb + wuOffVh + 8192, &tm_v, 64, t0, hv, b, &load_bar);
  }
  if (tid < kC) {
    const float bt = tid < rows ? ld_any(p.beta.p, row_off(p.beta, b, hv, t0 + tid), p.beta.dtype) : 0.f;
    const float gm = tid < rows ? ld_any(p.g.p, row_off(p.g, b, hv, t0 + tid), p.g.dtype) : 0.f;
    rs_v[tid] = bt;             // rows past the end of the sequence are scaled to zero
    rs_k[tid] = bt * __expf(gm);
  }
  __syncthreads();
  bool ok = mbar_wait(&load_bar, 0, p.status, FLA_ERR_TIMEOUT);
  // scale the raw rows in place and write the residual panels
  for (int idx = tid; idx < 2 * kC * 16; idx += 256) {
    const int isv = idx >> 10, r = (idx >> 4) & 63, ch = idx & 15;
    const uint32_t off = (ch >> 3) * 8192 + panel_chunk_off(r, ch & 7);
    uint8_t* hi = smem + (isv ? wuOffVh : wuOffKh) + off;
    uint8_t* lo = smem + (isv ? wuOffVl : wuOffKl) + off;
    float f[8];
    unpack_bf16x8(*reinterpret_cast<const uint4*>(hi), f);
    const float sc = isv ? rs_v[r] : rs_k[r];
    uint4 h4 = make_uint4(0, 0, 0, 0), l4 = make_uint4(0, 0, 0, 0);
    if (r < rows) {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] *= sc;
      split8(f, h4, l4);
    }
    *reinterpret_cast<uint4*>(hi) = h4;
    *reinterpret_cast<uint4*>(lo) = l4;
  }
  if (rows < kC) {   // a short chunk: columns of X past its end may hold anything
    for (int idx = tid; idx < kC * kC; idx += 256) {
      const int r = idx >> 6, cc = idx & 63;
      if (cc >= rows) *reinterpret_cast<uint16_t*>(smem + wuOffX + panel_off(r, cc)) = 0;
    }
  }
  fence_async_smem();
  tc_fence_before();
  ok = __syncthreads_and(ok);
  const uint32_t tbase = tmem_base_s;
  if (ok) {
    if (tid == 0) {
      tc_fence_after();
      // X as A: rows 64..127 of the M = 128 tile read the k panels behind it and are never used
      const Operand opX{sb + wuOffX, 8192, 0}, opKh{sb + wuOffKh, 8192, 1}, opKl{sb + wuOffKl, 8192, 1}, opVh{sb + wuOffVh, 8192, 1},
          opVl{sb + wuOffVl, 8192, 1};
      mma_tile(tbase, opX, opKh, 128, 128, 4, false);
      mma_tile(tbase, opX, opKl, 128, 128, 4, true);
      mma_tile(tbase + 128, opX, opVh, 128, 128, 4, false);
      mma_tile(tbase + 128, opX, opVl, 128, 128, 4, true);
      mma_commit(&mma_bar);
    }
    ok = mbar_wait(&mma_bar, 0, p.status, FLA_ERR_TIMEOUT);
    tc_fence_after();
    if ((warp & 3) < 2) {   // warps 0, 1 / 4, 5 read the 64 accumulator rows: 64 of the 128 columns of w and of u each
      const int i = tid & 63, half = warp >> 2;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const StageView& ov = which ? p.o1 : p.o0;
        bf16* dst = static_cast<bf16*>(const_cast<void*>(ov.p)) + row_off(ov, b, hv, t0 + i);
        {
          float r[64];
          tmem_ld_row64(tmem_addr(tbase, (warp & 3) * 32, which * 128 + half * 64), r);
          if (ok && i < rows) {
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(dst + half * 64 + ch * 8) = pack8(r + ch * 8);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 256);
}

// ----------------------------------------------------------------------------- chunk_gated_delta_rule_fwd_h
// Sequential over the chunks of one (sequence, value head, block of 64 value columns):
//   h_c = S;  v_new = u - w S;  S <- e^{g_last} S + k^T (e^{g_last - g} v_new).
// S lives in tensor memory in fp32 (lane = key dim, 64 columns); its bf16 value is the stored h_c and, with a bf16
// residual, the MMA operand.  w, k and u tiles of the next chunk are fetched by TMA as soon as their buffer is free.
constexpr uint32_t hsOffW = 0, hsOffK = 16384, hsOffS = 32768, hsOffSl = 49152, hsOffVd = 65536, hsOffVdl = 73728, hsOffU = 81920;
constexpr uint32_t kFwdHSmem = 90112;
__global__ void __launch_bounds__(128) stage_fwd_h_kernel(StageParams p, const __grid_constant__ CUtensorMap tm_w,
                                                          const __grid_constant__ CUtensorMap tm_k,
                                                          const __grid_constant__ CUtensorMap tm_u) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  __shared__ float gam_s[kC];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t mma_bar, w_bar, k_bar, u_bar;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int n = blockIdx.z, hv = blockIdx.y, vb = blockIdx.x;
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  const int b = p.cu_seqlens ? 0 : n;
  const int tbeg = p.cu_seqlens ? sq.bos : 0;
  const int hk = hv / (p.H / p.HK);
  const uint32_t sb = smem_u32(smem);
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 128);
    tmem_relinquish();
  }
  auto load_w = [&](int c) {
    mbar_arrive_expect_tx(&w_bar, 16384);
    tma_load_tile4(sb + hsOffW, &tm_w, 0, tbeg + c * kC, hv, b, &w_bar);
    tma_load_tile4(sb + hsOffW + 8192, &tm_w, 64, tbeg + c * kC, hv, b, &w_bar);
  };
  auto load_k = [&](int c) {
    mbar_arrive_expect_tx(&k_bar, 16384);
    tma_load_tile4(sb + hsOffK, &tm_k, 0, tbeg + c * kC, hk, b, &k_bar);
    tma_load_tile4(sb + hsOffK + 8192, &tm_k, 64, tbeg + c * kC, hk, b, &k_bar);
  };
  auto load_u = [&](int c) {
    mbar_arrive_expect_tx(&u_bar, 8192);
    tma_load_tile4(sb + hsOffU, &tm_u, vb * 64, tbeg + c * kC, hv, b, &u_bar);
  };
  if (tid == 0) {
    mbar_init(&mma_bar, 1);
    mbar_init(&w_bar, 1);
    mbar_init(&k_bar, 1);
    mbar_init(&u_bar, 1);
    mbar_init_fence();
    if (sq.nt > 0) {
      load_w(0);
      load_k(0);
      load_u(0);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = tmem_base_s;
  const uint32_t trow = tmem_addr(tbase, warp * 32, 0);
  // w as A: rows 64..127 of the M = 128 tile read the memory behind each 64-row panel and are never used
  const Operand opW{sb + hsOffW, 8192, 0}, opS{sb + hsOffS, 16384, 1}, opSl{sb + hsOffSl, 16384, 1}, opKt{sb + hsOffK, 8192, 1},
      opVd{sb + hsOffVd, 8192, 1}, opVdl{sb + hsOffVdl, 8192, 1};
  // my state row (key dim tid, value columns vb*64 ..)
  {
    float s[64];
    if (p.h0.p) {
      const float* src = static_cast<const float*>(p.h0.p) + (int64_t(n) * p.H + hv) * kK * kV + tid * kV + vb * 64;
#pragma unroll
      for (int i = 0; i < 64; i += 4) {
        const float4 t = *reinterpret_cast<const float4*>(src + i);
        s[i] = t.x; s[i + 1] = t.y; s[i + 2] = t.z; s[i + 3] = t.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 64; ++i) s[i] = 0.f;
    }
    tmem_st_row64(trow, s);
  }
  auto load_gate = [&](int c) -> float {
    if (tid >= kC || c >= sq.nt) return 0.f;
    const int rows_c = min(kC, sq.len - c * kC);
    return ld_any(p.g.p, row_off(p.g, b, hv, tbeg + c * kC + min(tid, rows_c - 1)), p.g.dtype);
  };
  float pf_g = load_gate(0);
  uint32_t mphase = 0, lphase = 0;
  bool ok = true;
  for (int c = 0; c < sq.nt; ++c) {
    const int rows = min(kC, sq.len - c * kC);
    const int t0 = tbeg + c * kC;
    if (tid < kC) gam_s[tid] = pf_g;
    pf_g = load_gate(c + 1);
    __syncthreads();
    const float g_last = gam_s[rows - 1];
    {
      float s[64];
      tmem_ld_row64(trow, s);
      row64_to_hilo(smem + hsOffS, smem + hsOffSl, tid, s);
      bf16* hd = static_cast<bf16*>(const_cast<void*>(p.o0.p)) +
                 ((int64_t(b) * p.H + hv) * p.o0.sh + (p.cu_seqlens ? sq.cbase : 0) + c) * int64_t(kK * kV) + tid * kV + vb * 64;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(hd + ch * 8) = pack8(s + ch * 8);
      const float el = __expf(g_last);
#pragma unroll
      for (int i = 0; i < 64; ++i) s[i] *= el;
      tmem_st_row64(trow, s);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      ok = mbar_wait(&w_bar, lphase, p.status, FLA_ERR_TIMEOUT);
      tc_fence_after();
      mma_tile(tbase + 64, opW, opS, 128, 64, 8, false);
      mma_tile(tbase + 64, opW, opSl, 128, 64, 8, true);
      mma_commit(&mma_bar);
    }
    float uval[64];
    if (warp < 2) {
      ok = mbar_wait(&u_bar, lphase, p.status, FLA_ERR_TIMEOUT) && ok;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) unpack_bf16x8(*reinterpret_cast<const uint4*>(smem + hsOffU + panel_chunk_off(tid, ch)), uval + ch * 8);
    }
    ok = mbar_wait(&mma_bar, mphase, p.status, FLA_ERR_TIMEOUT) && ok;
    mphase ^= 1;
    tc_fence_after();
    if (warp < 2) {
      float d1[64];
      tmem_ld_row64(trow + 64, d1);
      const bool live = tid < rows;     // rows past the end of the sequence (foreign or zero tile rows) carry nothing
#pragma unroll
      for (int i = 0; i < 64; ++i) d1[i] = live ? uval[i] - d1[i] : 0.f;
      if (live && ok) {
        bf16* vd = static_cast<bf16*>(const_cast<void*>(p.o1.p)) + row_off(p.o1, b, hv, t0 + tid) + vb * 64;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(vd + ch * 8) = pack8(d1 + ch * 8);
      }
      const float dec = __expf(g_last - gam_s[tid]);
#pragma unroll
      for (int i = 0; i < 64; ++i) d1[i] *= dec;
      row64_to_hilo(smem + hsOffVd, smem + hsOffVdl, tid, d1);
    }
    fence_async_smem();
    tc_fence_before();
    if (!__syncthreads_and(ok)) { ok = false; break; }
    if (tid == 0) {
      if (c + 1 < sq.nt) {   // w and u of this chunk are consumed
        load_w(c + 1);
        load_u(c + 1);
      }
      ok = mbar_wait(&k_bar, lphase, p.status, FLA_ERR_TIMEOUT);
      tc_fence_after();
      mma_tile(tbase, opKt, opVd, 128, 64, 4, true);
      mma_tile(tbase, opKt, opVdl, 128, 64, 4, true);
      mma_commit(&mma_bar);
    }
    ok = mbar_wait(&mma_bar, mphase, p.status, FLA_ERR_TIMEOUT) && ok;
    mphase ^= 1;
    lphase ^= 1;
    tc_fence_after();
    if (!__syncthreads_and(ok)) { ok = false; break; }
    if (tid == 0 && c + 1 < sq.nt) load_k(c + 1);
  }
  if (ok && p.want_final) {
    float s[64];
    tmem_ld_row64(trow, s);
    float* dst = static_cast<float*>(const_cast<void*>(p.o2.p)) + (int64_t(n) * p.H + hv) * kK * kV + tid * kV + vb * 64;
#pragma unroll
    for (int i = 0; i < 64; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(s[i], s[i + 1], s[i + 2], s[i + 3]);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 128);
}

// ----------------------------------------------------------------------------- chunk_fwd_o
// o = scale [ e^{g_i} (q h_c) + tril(q k^T e^{g_i - g_j}) v_new ] per chunk and value head.  All operands arrive as TMA
// tiles issued up front; the decayed score tile is split into a bf16 value and a residual (which reuses the k panels).
constexpr uint32_t foOffP = 0, foOffQ = 8192, foOffK = 24576, foOffH = 40960, foOffVn = 73728;
constexpr uint32_t kFwdOSmem = 90112;
__global__ void __launch_bounds__(256) stage_fwd_o_kernel(StageParams p, const __grid_constant__ CUtensorMap tm_q,
                                                          const __grid_constant__ CUtensorMap tm_k,
                                                          const __grid_constant__ CUtensorMap tm_v,
                                                          const __grid_constant__ CUtensorMap tm_h) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  __shared__ float gam_s[kC];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t mma_bar, load_bar;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int n = blockIdx.z, hv = blockIdx.y, c = blockIdx.x;
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  if (c >= sq.nt) return;
  const int rows = min(kC, sq.len - c * kC);
  const int b = p.cu_seqlens ? 0 : n;
  const int t0 = (p.cu_seqlens ? sq.bos : 0) + c * kC;
  const int hk = hv / (p.H / p.HK);
  const uint32_t sb = smem_u32(smem);
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 256);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(&mma_bar, 1);
    mbar_init(&load_bar, 1);
    mbar_init_fence();
    mbar_arrive_expect_tx(&load_bar, 16384 + 16384 + 32768 + 16384);
    tma_load_tile4(sb + foOffQ, &tm_q, 0, t0, hk, b, &load_bar);
    tma_load_tile4(sb + foOffQ + 8192, &tm_q, 64, t0, hk, b, &load_bar);
    tma_load_tile4(sb + foOffK, &tm_k, 0, t0, hk, b, &load_bar);
    tma_load_tile4(sb + foOffK + 8192, &tm_k, 64, t0, hk, b, &load_bar);
    // h_c: 128 key rows x 128 value columns of the dense [chunks * 128, 128] state tensor
    const int hrow = int((((int64_t(b) * p.H + hv) * p.h.sh + (p.cu_seqlens ? sq.cbase : 0) + c)) * kK);
    tma_load_tile4(sb + foOffH, &tm_h, 0, hrow, 0, 0, &load_bar);
    tma_load_tile4(sb + foOffH + 16384, &tm_h, 64, hrow, 0, 0, &load_bar);
    tma_load_tile4(sb + foOffVn, &tm_v, 0, t0, hv, b, &load_bar);
    tma_load_tile4(sb + foOffVn + 8192, &tm_v, 64, t0, hv, b, &load_bar);
  }
  if (tid < kC) gam_s[tid] = ld_any(p.g.p, row_off(p.g, b, hv, t0 + min(tid, rows - 1)), p.g.dtype);
  tc_fence_before();
  __syncthreads();
  const uint32_t tbase = tmem_base_s;
  const int half = warp >> 2;                       // warps 0, 1 / 4, 5 read the 64 accumulator rows: one column half each
  const bool rowwarp = (warp & 3) < 2;
  const uint32_t trow = tmem_addr(tbase, (warp & 3) * 32, 0);
  // q and the score tile as A: rows 64..127 of the M = 128 tiles read the panels behind them and are never used
  const Operand opQ{sb + foOffQ, 8192, 0}, opK{sb + foOffK, 8192, 0}, opH{sb + foOffH, 16384, 1}, opVn{sb + foOffVn, 8192, 1},
      opP{sb + foOffP, 8192, 0}, opPl{sb + foOffK, 8192, 0};
  bool ok = true;
  if (tid == 0) {
    ok = mbar_wait(&load_bar, 0, p.status, FLA_ERR_TIMEOUT);
    tc_fence_after();
    mma_tile(tbase, opQ, opK, 128, 64, 8, false);          // columns 0..63: q k^T
    mma_tile(tbase + 64, opQ, opH, 128, 128, 8, false);    // columns 64..191: q h_c
    mma_commit(&mma_bar);
  }
  ok = mbar_wait(&mma_bar, 0, p.status, FLA_ERR_TIMEOUT) && ok;
  tc_fence_after();
  if (rowwarp) {
    const int i = tid & 63;
    const float gi = gam_s[i];
    {
      float s[32];
      tmem_ld32(trow + half * 32, s);
      tmem_ld_wait();
      // rows and columns past the end of the sequence (foreign or zero tile rows) are masked here
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int jj = half * 32 + j;
        s[j] = (jj <= i && jj < rows && i < rows) ? s[j] * __expf(gi - gam_s[jj]) : 0.f;
      }
      row32_to_hilo(smem + foOffP, smem + foOffK, i, half, s);
    }
    const float eg = __expf(gi);
    {
      float r[64];
      tmem_ld_row64(trow + 64 + half * 64, r);
#pragma unroll
      for (int j = 0; j < 64; ++j) r[j] *= eg;
      tmem_st_row64(trow + 64 + half * 64, r);
    }
  }
  fence_async_smem();
  tc_fence_before();
  ok = __syncthreads_and(ok);
  if (ok) {
    if (tid == 0) {
      tc_fence_after();
      mma_tile(tbase + 64, opP, opVn, 128, 128, 4, true);
      mma_tile(tbase + 64, opPl, opVn, 128, 128, 4, true);
      mma_commit(&mma_bar);
    }
    ok = mbar_wait(&mma_bar, 1, p.status, FLA_ERR_TIMEOUT);
    tc_fence_after();
    if (rowwarp) {
      const int i = tid & 63;
      bf16* dst = static_cast<bf16*>(const_cast<void*>(p.o0.p)) + row_off(p.o0, b, hv, t0 + i);
      {
        float r[64];
        tmem_ld_row64(trow + 64 + half * 64, r);
        if (ok && i < rows) {
#pragma unroll
          for (int j = 0; j < 64; ++j) r[j] *= p.scale;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(dst + half * 64 + ch * 8) = pack8(r + ch * 8);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 256);
}

// ----------------------------------------------------------------------------- chunk_bwd_dv_local
// dv_j = sum_{i >= j} scale (k_j . q_i) e^{g_i - g_j} dO_i inside a chunk, per value head.
constexpr uint32_t dvOffP = 0, dvOffPl = 8192, dvOffK = 16384, dvOffQ = 32768, dvOffDo = 49152;
constexpr uint32_t kDvLocalSmem = 65536;
__global__ void __launch_bounds__(256) stage_dv_local_kernel(StageParams p, const __grid_constant__ CUtensorMap tm_q,
                                                             const __grid_constant__ CUtensorMap tm_k,
                                                             const __grid_constant__ CUtensorMap tm_do) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  __shared__ float gam_s[kC];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t mma_bar, load_bar;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int n = blockIdx.z, hv = blockIdx.y, c = blockIdx.x;
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  if (c >= sq.nt) return;
  const int rows = min(kC, sq.len - c * kC);
  const int b = p.cu_seqlens ? 0 : n;
  const int t0 = (p.cu_seqlens ? sq.bos : 0) + c * kC;
  const int hk = hv / (p.H / p.HK);
  const uint32_t sb = smem_u32(smem);
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 256);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(&mma_bar, 1);
    mbar_init(&load_bar, 1);
    mbar_init_fence();
    mbar_arrive_expect_tx(&load_bar, 3 * 16384);
    tma_load_tile4(sb + dvOffK, &tm_k, 0, t0, hk, b, &load_bar);
    tma_load_tile4(sb + dvOffK + 8192, &tm_k, 64, t0, hk, b, &load_bar);
    tma_load_tile4(sb + dvOffQ, &tm_q, 0, t0, hk, b, &load_bar);
    tma_load_tile4(sb + dvOffQ + 8192, &tm_q, 64, t0, hk, b, &load_bar);
    tma_load_tile4(sb + dvOffDo, &tm_do, 0, t0, hv, b, &load_bar);
    tma_load_tile4(sb + dvOffDo + 8192, &tm_do, 64, t0, hv, b, &load_bar);
  }
  if (tid < kC) gam_s[tid] = ld_any(p.g.p, row_off(p.g, b, hv, t0 + min(tid, rows - 1)), p.g.dtype);
  tc_fence_before();
  __syncthreads();
  const uint32_t tbase = tmem_base_s;
  const int half = warp >> 2;                       // warps 0, 1 / 4, 5 read the 64 accumulator rows: one column half each
  const bool rowwarp = (warp & 3) < 2;
  const uint32_t trow = tmem_addr(tbase, (warp & 3) * 32, 0);
  // k and the score tile as A: rows 64..127 of the M = 128 tiles read the panels behind them and are never used
  const Operand opK{sb + dvOffK, 8192, 0}, opQ{sb + dvOffQ, 8192, 0}, opDo{sb + dvOffDo, 8192, 1}, opP{sb + dvOffP, 8192, 0},
      opPl{sb + dvOffPl, 8192, 0};
  bool ok = true;
  if (tid == 0) {
    ok = mbar_wait(&load_bar, 0, p.status, FLA_ERR_TIMEOUT);
    tc_fence_after();
    mma_tile(tbase, opK, opQ, 128, 64, 8, false);   // rows j (keys), columns i (queries)
    mma_commit(&mma_bar);
  }
  ok = mbar_wait(&mma_bar, 0, p.status, FLA_ERR_TIMEOUT) && ok;
  tc_fence_after();
  if (rowwarp) {
    const int j = tid & 63;
    const float gj = gam_s[j];
    float s[32];
    tmem_ld32(trow + half * 32, s);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int ii = half * 32 + i;
      s[i] = (ii >= j && ii < rows && j < rows) ? p.scale * s[i] * __expf(gam_s[ii] - gj) : 0.f;
    }
    row32_to_hilo(smem + dvOffP, smem + dvOffPl, j, half, s);
  }
  fence_async_smem();
  tc_fence_before();
  ok = __syncthreads_and(ok);
  if (ok) {
    if (tid == 0) {
      tc_fence_after();
      mma_tile(tbase + 64, opP, opDo, 128, 128, 4, false);
      mma_tile(tbase + 64, opPl, opDo, 128, 128, 4, true);
      mma_commit(&mma_bar);
    }
    ok = mbar_wait(&mma_bar, 1, p.status, FLA_ERR_TIMEOUT);
    tc_fence_after();
    if (rowwarp) {
      const int j = tid & 63;
      bf16* dst = static_cast<bf16*>(const_cast<void*>(p.o0.p)) + row_off(p.o0, b, hv, t0 + j);
      {
        float r[64];
        tmem_ld_row64(trow + 64 + half * 64, r);
        if (ok && j < rows) {
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(dst + half * 64 + ch * 8) = pack8(r + ch * 8);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 256);
}

// ----------------------------------------------------------------------------- chunk_gated_delta_rule_bwd_dhu
// Reverse scan over the chunks of one (sequence, value head, block of 64 value columns):
//   dh_c = dS;  dv2 = dv + e^{g_last - g} (k dS);  dS <- e^{g_last} dS + q^T (scale e^{g} dO) - w^T dv2.
// dS lives in tensor memory in fp32 (lane = key dim); its bf16 value is the stored dh_c and, with a residual, the MMA
// operand.  k and w share one buffer (k is consumed by the first product of a chunk, w by the last).
constexpr uint32_t bhOffKW = 0, bhOffQ = 16384, bhOffS = 32768, bhOffSl = 49152, bhOffDo = 65536, bhOffDol = 73728, bhOffDv = 81920,
                   bhOffDvl = 90112;
constexpr uint32_t kBwdDhuSmem = 98304;
__global__ void __launch_bounds__(128) stage_bwd_dhu_kernel(StageParams p, const __grid_constant__ CUtensorMap tm_q,
                                                            const __grid_constant__ CUtensorMap tm_k,
                                                            const __grid_constant__ CUtensorMap tm_w,
                                                            const __grid_constant__ CUtensorMap tm_do,
                                                            const __grid_constant__ CUtensorMap tm_dv) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  __shared__ float gam_s[kC];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t mma_bar, kw_bar, q_bar, d_bar;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int n = blockIdx.z, hv = blockIdx.y, vb = blockIdx.x;
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  const int b = p.cu_seqlens ? 0 : n;
  const int tbeg = p.cu_seqlens ? sq.bos : 0;
  const int hk = hv / (p.H / p.HK);
  const uint32_t sb = smem_u32(smem);
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 128);
    tmem_relinquish();
  }
  auto load_k = [&](int c) {
    mbar_arrive_expect_tx(&kw_bar, 16384);
    tma_load_tile4(sb + bhOffKW, &tm_k, 0, tbeg + c * kC, hk, b, &kw_bar);
    tma_load_tile4(sb + bhOffKW + 8192, &tm_k, 64, tbeg + c * kC, hk, b, &kw_bar);
  };
  auto load_w = [&](int c) {
    mbar_arrive_expect_tx(&kw_bar, 16384);
    tma_load_tile4(sb + bhOffKW, &tm_w, 0, tbeg + c * kC, hv, b, &kw_bar);
    tma_load_tile4(sb + bhOffKW + 8192, &tm_w, 64, tbeg + c * kC, hv, b, &kw_bar);
  };
  auto load_q = [&](int c) {
    mbar_arrive_expect_tx(&q_bar, 16384);
    tma_load_tile4(sb + bhOffQ, &tm_q, 0, tbeg + c * kC, hk, b, &q_bar);
    tma_load_tile4(sb + bhOffQ + 8192, &tm_q, 64, tbeg + c * kC, hk, b, &q_bar);
  };
  auto load_d = [&](int c) {   // the dO and dv blocks of this CTA's value columns
    mbar_arrive_expect_tx(&d_bar, 16384);
    tma_load_tile4(sb + bhOffDo, &tm_do, vb * 64, tbeg + c * kC, hv, b, &d_bar);
    tma_load_tile4(sb + bhOffDv, &tm_dv, vb * 64, tbeg + c * kC, hv, b, &d_bar);
  };
  if (tid == 0) {
    mbar_init(&mma_bar, 1);
    mbar_init(&kw_bar, 1);
    mbar_init(&q_bar, 1);
    mbar_init(&d_bar, 1);
    mbar_init_fence();
    if (sq.nt > 0) {
      load_k(sq.nt - 1);
      load_q(sq.nt - 1);
      load_d(sq.nt - 1);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = tmem_base_s;
  const uint32_t trow = tmem_addr(tbase, warp * 32, 0);
  // k as A (rows = tokens): rows 64..127 of the M = 128 tile read the memory behind each panel and are never used
  const Operand opK{sb + bhOffKW, 8192, 0}, opWt{sb + bhOffKW, 8192, 1}, opQt{sb + bhOffQ, 8192, 1}, opS{sb + bhOffS, 16384, 1},
      opSl{sb + bhOffSl, 16384, 1}, opDo{sb + bhOffDo, 8192, 1}, opDol{sb + bhOffDol, 8192, 1}, opDv{sb + bhOffDv, 8192, 1},
      opDvl{sb + bhOffDvl, 8192, 1};
  {
    float s[64];
    if (p.h0.p) {   // the cotangent of the final state
      const float* src = static_cast<const float*>(p.h0.p) + (int64_t(n) * p.H + hv) * kK * kV + tid * kV + vb * 64;
#pragma unroll
      for (int i = 0; i < 64; i += 4) {
        const float4 t = *reinterpret_cast<const float4*>(src + i);
        s[i] = t.x; s[i + 1] = t.y; s[i + 2] = t.z; s[i + 3] = t.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 64; ++i) s[i] = 0.f;
    }
    tmem_st_row64(trow, s);
  }
  auto load_gate = [&](int c) -> float {
    if (tid >= kC || c < 0) return 0.f;
    const int rows_c = min(kC, sq.len - c * kC);
    return ld_any(p.g.p, row_off(p.g, b, hv, tbeg + c * kC + min(tid, rows_c - 1)), p.g.dtype);
  };
  float pf_g = load_gate(sq.nt - 1);
  uint32_t mphase = 0, kwphase = 0, lphase = 0;
  bool ok = true;
  for (int c = sq.nt - 1; c >= 0; --c) {
    const int rows = min(kC, sq.len - c * kC);
    const int t0 = tbeg + c * kC;
    if (tid < kC) gam_s[tid] = pf_g;
    pf_g = load_gate(c - 1);
    __syncthreads();
    const float g_last = gam_s[rows - 1];
    {
      float s[64];
      tmem_ld_row64(trow, s);
      row64_to_hilo(smem + bhOffS, smem + bhOffSl, tid, s);
      bf16* hd = static_cast<bf16*>(const_cast<void*>(p.o0.p)) +
                 ((int64_t(b) * p.H + hv) * p.o0.sh + (p.cu_seqlens ? sq.cbase : 0) + c) * int64_t(kK * kV) + tid * kV + vb * 64;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(hd + ch * 8) = pack8(s + ch * 8);
      const float el = __expf(g_last);
#pragma unroll
      for (int i = 0; i < 64; ++i) s[i] *= el;
      tmem_st_row64(trow, s);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      ok = mbar_wait(&kw_bar, kwphase, p.status, FLA_ERR_TIMEOUT);
      tc_fence_after();
      mma_tile(tbase + 64, opK, opS, 128, 64, 8, false);
      mma_tile(tbase + 64, opK, opSl, 128, 64, 8, true);
      mma_commit(&mma_bar);
    }
    kwphase ^= 1;
    float dov[64], dvv[64];
    if (warp < 2) {
      ok = mbar_wait(&d_bar, lphase, p.status, FLA_ERR_TIMEOUT) && ok;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        unpack_bf16x8(*reinterpret_cast<const uint4*>(smem + bhOffDo + panel_chunk_off(tid, ch)), dov + ch * 8);
        unpack_bf16x8(*reinterpret_cast<const uint4*>(smem + bhOffDv + panel_chunk_off(tid, ch)), dvv + ch * 8);
      }
    }
    ok = mbar_wait(&mma_bar, mphase, p.status, FLA_ERR_TIMEOUT) && ok;
    mphase ^= 1;
    tc_fence_after();
    if (!__syncthreads_and(ok)) { ok = false; break; }
    if (tid == 0) load_w(c);   // k is consumed: its buffer takes this chunk's w
    if (warp < 2) {
      float d1[64];
      tmem_ld_row64(trow + 64, d1);
      const bool live = tid < rows;     // rows past the end of the sequence (foreign or zero tile rows) carry nothing
      const float gi = gam_s[tid];
      const float dec = __expf(g_last - gi), qs = live ? p.scale * __expf(gi) : 0.f;
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        d1[i] = live ? dvv[i] + dec * d1[i] : 0.f;
        dov[i] *= qs;
      }
      if (live) {
        bf16* vd = static_cast<bf16*>(const_cast<void*>(p.o1.p)) + row_off(p.o1, b, hv, t0 + tid) + vb * 64;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(vd + ch * 8) = pack8(d1 + ch * 8);
      }
#pragma unroll
      for (int i = 0; i < 64; ++i) d1[i] = -d1[i];
      row64_to_hilo(smem + bhOffDo, smem + bhOffDol, tid, dov);   // in place over the raw tiles
      row64_to_hilo(smem + bhOffDv, smem + bhOffDvl, tid, d1);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      ok = mbar_wait(&q_bar, lphase, p.status, FLA_ERR_TIMEOUT);
      ok = mbar_wait(&kw_bar, kwphase, p.status, FLA_ERR_TIMEOUT) && ok;
      tc_fence_after();
      mma_tile(tbase, opQt, opDo, 128, 64, 4, true);
      mma_tile(tbase, opQt, opDol, 128, 64, 4, true);
      mma_tile(tbase, opWt, opDv, 128, 64, 4, true);
      mma_tile(tbase, opWt, opDvl, 128, 64, 4, true);
      mma_commit(&mma_bar);
    }
    kwphase ^= 1;
    ok = mbar_wait(&mma_bar, mphase, p.status, FLA_ERR_TIMEOUT) && ok;
    mphase ^= 1;
    lphase ^= 1;
    tc_fence_after();
    if (!__syncthreads_and(ok)) { ok = false; break; }
    if (tid == 0 && c > 0) {
      load_k(c - 1);
      load_q(c - 1);
      load_d(c - 1);
    }
  }
  if (ok && p.want_final) {
    float s[64];
    tmem_ld_row64(trow, s);
    float* dst = static_cast<float*>(const_cast<void*>(p.o2.p)) + (int64_t(n) * p.H + hv) * kK * kV + tid * kV + vb * 64;
#pragma unroll
    for (int i = 0; i < 64; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(s[i], s[i + 1], s[i + 2], s[i + 3]);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 128);
}

// ----------------------------------------------------------------------------- chunk_bwd_dqkwg
// Per chunk and value head (v = v_new, dv = dv2 of the reverse state pass, h / dh = state and its gradient at the chunk):
//   dq = scale e^{g_i} (dO h^T) + ds k,   dk = e^{g_last - g_i} (v dh^T) + ds^T q,   dw = -(dv h^T),
//   ds = scale tril(dO v^T e^{g_i - g_j}),
//   dg_i = q_i.dq_state_i - k_i.dk_state_i + sum_j ds2_ij - sum_j ds2_ji  (ds2 = ds * q k^T),
//   dg_last += e^{g_last} <h, dh> + sum_i k_i.dk_state_i.
// [dO; dv] are stacked into one 128-row operand so that dO h^T and dv h^T are one product.  dq / dk of a value head
// go to fp32 scratch rows when several value heads share a q/k head (summed by stage_group_sum_kernel).
constexpr uint32_t dqOffA = 0, dqOffV = 32768, dqOffQ = 49152, dqOffK = 65536, dqOffH = 81920, dqOffDH = 114688, dqOffDS = 147456,
                   dqOffDSl = 155648;
constexpr uint32_t kDqkwgSmem = 172032;   // 8 KB behind the residual panel: rows 64..127 of the M = 128 views of it
constexpr int kColTile = 65;              // fp32 row stride of the ds2 tile (reuses the h panels)
__global__ void __launch_bounds__(256) stage_dqkwg_kernel(StageParams p, const __grid_constant__ CUtensorMap tm_q,
                                                          const __grid_constant__ CUtensorMap tm_k,
                                                          const __grid_constant__ CUtensorMap tm_v,
                                                          const __grid_constant__ CUtensorMap tm_do,
                                                          const __grid_constant__ CUtensorMap tm_dv,
                                                          const __grid_constant__ CUtensorMap tm_h,
                                                          const __grid_constant__ CUtensorMap tm_dh) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  __shared__ float gam_s[kC];
  __shared__ float red_s[10];        // <h, dh> per warp (8), k.dk_state per row warp (2)
  __shared__ float part_s[3][kC];    // second column half's partial row sums dgA, dgB, dgC
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t mma_bar, load_bar;
  // 8 warps: warp w reads TMEM lanes 32 (w % 4) ..; `half` = w / 4 selects which half of a tile's columns it handles
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int half = warp >> 2, quad = warp & 3;
  const int n = blockIdx.z, hv = blockIdx.y, c = blockIdx.x;
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  if (c >= sq.nt) return;
  const int rows = min(kC, sq.len - c * kC);
  const int b = p.cu_seqlens ? 0 : n;
  const int t0 = (p.cu_seqlens ? sq.bos : 0) + c * kC;
  const int G = p.H / p.HK, hk = hv / G;
  const uint32_t sb = smem_u32(smem);
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(&mma_bar, 1);
    mbar_init(&load_bar, 1);
    mbar_init_fence();
    mbar_arrive_expect_tx(&load_bar, 147456);
    const int hrow = int((((int64_t(b) * p.H + hv) * p.h.sh + (p.cu_seqlens ? sq.cbase : 0) + c)) * kK);
    tma_load_tile4(sb + dqOffH, &tm_h, 0, hrow, 0, 0, &load_bar);
    tma_load_tile4(sb + dqOffH + 16384, &tm_h, 64, hrow, 0, 0, &load_bar);
    tma_load_tile4(sb + dqOffDH, &tm_dh, 0, hrow, 0, 0, &load_bar);
    tma_load_tile4(sb + dqOffDH + 16384, &tm_dh, 64, hrow, 0, 0, &load_bar);
    tma_load_tile4(sb + dqOffA, &tm_do, 0, t0, hv, b, &load_bar);             // panel 0: dO rows | dv rows
    tma_load_tile4(sb + dqOffA + 8192, &tm_dv, 0, t0, hv, b, &load_bar);
    tma_load_tile4(sb + dqOffA + 16384, &tm_do, 64, t0, hv, b, &load_bar);    // panel 1
    tma_load_tile4(sb + dqOffA + 24576, &tm_dv, 64, t0, hv, b, &load_bar);
    tma_load_tile4(sb + dqOffV, &tm_v, 0, t0, hv, b, &load_bar);
    tma_load_tile4(sb + dqOffV + 8192, &tm_v, 64, t0, hv, b, &load_bar);
    tma_load_tile4(sb + dqOffQ, &tm_q, 0, t0, hk, b, &load_bar);
    tma_load_tile4(sb + dqOffQ + 8192, &tm_q, 64, t0, hk, b, &load_bar);
    tma_load_tile4(sb + dqOffK, &tm_k, 0, t0, hk, b, &load_bar);
    tma_load_tile4(sb + dqOffK + 8192, &tm_k, 64, t0, hk, b, &load_bar);
  }
  if (tid < kC) gam_s[tid] = ld_any(p.g.p, row_off(p.g, b, hv, t0 + min(tid, rows - 1)), p.g.dtype);
  tc_fence_before();
  __syncthreads();
  const uint32_t tbase = tmem_base_s;
  const uint32_t trow = tmem_addr(tbase, quad * 32, 0);
  constexpr uint32_t cT0 = 0, cT1 = 128, cDs = 256, cQk = 320;
  const Operand opA{sb + dqOffA, 16384, 0}, opH{sb + dqOffH, 16384, 0}, opDH{sb + dqOffDH, 16384, 0}, opVa{sb + dqOffV, 8192, 0},
      opQa{sb + dqOffQ, 8192, 0}, opKb{sb + dqOffK, 8192, 0}, opKn{sb + dqOffK, 8192, 1}, opQn{sb + dqOffQ, 8192, 1},
      opDS{sb + dqOffDS, 8192, 0}, opDSl{sb + dqOffDSl, 8192, 0}, opDSt{sb + dqOffDS, 8192, 1}, opDSlt{sb + dqOffDSl, 8192, 1};
  bool ok = mbar_wait(&load_bar, 0, p.status, FLA_ERR_TIMEOUT);
  if (tid == 0) {
    tc_fence_after();
    mma_tile(tbase + cT0, opA, opH, 128, 128, 8, false);     // rows 0..63: dO h^T, rows 64..127: dv h^T
    mma_tile(tbase + cT1, opVa, opDH, 128, 128, 8, false);   // v dh^T
    mma_tile(tbase + cDs, opA, opVa, 128, 64, 8, false);     // dO v^T
    mma_tile(tbase + cQk, opQa, opKb, 128, 64, 8, false);    // q k^T
    mma_commit(&mma_bar);
  }
  // <h, dh> while the MMAs run: thread t owns one panel (64 value columns) of key row t % 128 of both tiles
  float hd = 0.f;
#pragma unroll
  for (int ch = 0; ch < 8; ++ch) {
    const uint32_t off = (tid >> 7) * 16384 + panel_chunk_off(tid & 127, ch);
    float a[8], d[8];
    unpack_bf16x8(*reinterpret_cast<const uint4*>(smem + dqOffH + off), a);
    unpack_bf16x8(*reinterpret_cast<const uint4*>(smem + dqOffDH + off), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) hd += a[j] * d[j];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) hd += __shfl_xor_sync(0xffffffffu, hd, o);
  if (lane == 0) red_s[warp] = hd;
  ok = mbar_wait(&mma_bar, 0, p.status, FLA_ERR_TIMEOUT) && ok;
  tc_fence_after();
  ok = __syncthreads_and(ok);   // also: every thread is done with the h / dh panels (the ds2 tile reuses them)
  if (ok) {
    float* tile = reinterpret_cast<float*>(smem + dqOffH);
    float dgA = 0.f, dgB = 0.f, dgC = 0.f;
    const int i = tid & 63;
    const bool live = i < rows;
    const float gi = gam_s[i], gl = gam_s[rows - 1];
    if (quad >= 2) {
      // dw rows: -(dv h^T), my 64 of the 128 key columns
      if (p.o2.p) {
        bf16* dst = static_cast<bf16*>(const_cast<void*>(p.o2.p)) + row_off(p.o2, b, hv, t0 + i);
        {
          float r[64];
          tmem_ld_row64(trow + cT0 + half * 64, r);
          if (live) {
#pragma unroll
            for (int j = 0; j < 64; ++j) r[j] = -r[j];
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(dst + half * 64 + ch * 8) = pack8(r + ch * 8);
          }
        }
      }
    } else {
      {   // my 32 of the 64 score columns
        float ds[32], qk[32];
        tmem_ld32(trow + cDs + half * 32, ds);
        tmem_ld32(trow + cQk + half * 32, qk);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int jj = half * 32 + j;
          ds[j] = (live && jj <= i) ? p.scale * ds[j] * __expf(gi - gam_s[jj]) : 0.f;
          const float d2 = ds[j] * qk[j];
          dgC += d2;
          tile[i * kColTile + jj] = d2;
        }
        row32_to_hilo(smem + dqOffDS, smem + dqOffDSl, i, half, ds);
      }
      const float fq = live ? p.scale * __expf(gi) : 0.f, fk = live ? __expf(gl - gi) : 0.f;
      {   // my 64 of the 128 key columns
        float r[64];
        tmem_ld_row64(trow + cT0 + half * 64, r);
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          float qv[8];
          unpack_bf16x8(*reinterpret_cast<const uint4*>(smem + dqOffQ + half * 8192 + panel_chunk_off(i, ch)), qv);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            r[ch * 8 + j] *= fq;
            dgA += r[ch * 8 + j] * qv[j];
          }
        }
        tmem_st_row64(trow + cT0 + half * 64, r);
        tmem_ld_row64(trow + cT1 + half * 64, r);
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          float kv[8];
          unpack_bf16x8(*reinterpret_cast<const uint4*>(smem + dqOffK + half * 8192 + panel_chunk_off(i, ch)), kv);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            r[ch * 8 + j] *= fk;
            dgB += r[ch * 8 + j] * kv[j];
          }
        }
        tmem_st_row64(trow + cT1 + half * 64, r);
      }
      if (half == 1) { part_s[0][i] = dgA; part_s[1][i] = dgB; part_s[2][i] = dgC; }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      mma_tile(tbase + cT0, opDS, opKn, 128, 128, 4, true);      // += ds k
      mma_tile(tbase + cT0, opDSl, opKn, 128, 128, 4, true);
      mma_tile(tbase + cT1, opDSt, opQn, 128, 128, 4, true);     // += ds^T q
      mma_tile(tbase + cT1, opDSlt, opQn, 128, 128, 4, true);
      mma_commit(&mma_bar);
    }
    if (warp < 2) {
      // dg while the MMAs run (first column half's threads, which add the other half's row sums): column sums of ds2,
      // the last-row term
      dgA += part_s[0][i]; dgB += part_s[1][i]; dgC += part_s[2][i];
      float col = 0.f;
#pragma unroll 8
      for (int r = 0; r < kC; ++r) col += tile[r * kColTile + i];
      float sB = dgB;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sB += __shfl_xor_sync(0xffffffffu, sB, o);
      if (lane == 0) red_s[8 + warp] = sB;
      asm volatile("bar.sync 3, 64;" ::: "memory");
      float dg = dgA - dgB + dgC - col;
      if (i == rows - 1)
        dg += __expf(gl) * (((red_s[0] + red_s[1]) + (red_s[2] + red_s[3])) + ((red_s[4] + red_s[5]) + (red_s[6] + red_s[7]))) + red_s[8] + red_s[9];
      if (live) st_any(const_cast<void*>(p.o3.p), row_off(p.o3, b, hv, t0 + i), p.o3.dtype, dg);
    }
    ok = mbar_wait(&mma_bar, 1, p.status, FLA_ERR_TIMEOUT);
    tc_fence_after();
    if (quad < 2) {
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const StageView& ov = which ? p.o1 : p.o0;
        float* wrow = (which ? p.ws_dk : p.ws_dq);
        {   // my 64 of the 128 key columns
          float r[64];
          tmem_ld_row64(trow + (which ? cT1 : cT0) + half * 64, r);
          if (ok && live) {
            if (wrow) {   // per-value-head fp32 rows, summed over the group afterwards
              float* dst = wrow + ((int64_t(b) * p.H + hv) * p.T + (t0 + i)) * kK + half * 64;
#pragma unroll
              for (int j = 0; j < 64; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(r[j], r[j + 1], r[j + 2], r[j + 3]);
            } else {
              bf16* dst = static_cast<bf16*>(const_cast<void*>(ov.p)) + row_off(ov, b, hk, t0 + i) + half * 64;
#pragma unroll
              for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(dst + ch * 8) = pack8(r + ch * 8);
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 512);
}

// dq / dk of a q/k head = sum over the value heads of its group of the fp32 scratch rows
__global__ void __launch_bounds__(256) stage_group_sum_kernel(StageParams p, int B, int n_out) {
  const int G = p.H / p.HK;
  const int64_t total = int64_t(B) * p.HK * p.T * (kK / 4);
  for (int64_t idx = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; idx < total; idx += int64_t(gridDim.x) * blockDim.x) {
    const int c4 = int(idx % (kK / 4));
    const int64_t t = (idx / (kK / 4)) % p.T;
    const int64_t hk = (idx / (kK / 4) / p.T) % p.HK, b = idx / (kK / 4) / p.T / p.HK;
    for (int which = 0; which < n_out; ++which) {
      const float* src = which ? p.ws_dk : p.ws_dq;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int g = 0; g < G; ++g) {
        const float4 v = *reinterpret_cast<const float4*>(src + ((b * p.H + hk * G + g) * p.T + t) * kK + c4 * 4);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      const StageView& ov = which ? p.o1 : p.o0;
      bf16* dst = static_cast<bf16*>(const_cast<void*>(ov.p)) + row_off(ov, b, hk, t) + c4 * 4;
      *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
    }
  }
}

// ----------------------------------------------------------------------------- prepare_wy_repr_bwd (+ _da, _full)
// Backward of  w = X (k beta e^g),  u = X (v beta),  X = (I + A)^-1,  A_ij = beta_i e^{g_i - g_j} k_i.k_j (j < i),
// per chunk and value head, from dw and du:
//   P   = strict_lower(dw (k beta e^g)^T + du (v beta)^T)
//   dA  = strict_lower(-(X^T P X^T) * e^{g_i - g_j})          (stored transposed, like the reference operator)
//   dkbg = X^T dw,  dvb = X^T du,  dv = beta dvb
//   dk  = dA^T (k beta) + beta (dA k) + beta e^g dkbg          (summed over the value heads of a group)
//   dbeta = (dA k).k + e^g dkbg.k + dvb.v
//   dg  = beta e^g dkbg.k + rowsum(W) - colsum(W),  W = dA * (beta_i k_i.k_j)
// wy_mode 0 runs everything, 1 stops after dA, 2 reads dA (transposed) instead of computing it.
constexpr uint32_t wyOffX = 0, wyOffK = 8192, wyOffV = 24576, wyOffDW = 40960, wyOffDU = 57344, wyOffR = 73728;
// region R (80 KB): first (k beta e^g) hi, lo and (v beta) hi, lo (16 KB each); once the first products are done it is
// reused for P (hi, lo), X^T-side P5 (hi, lo), dA (hi, lo), beta dA (hi, lo) (8 KB each) and the fp32 W tile
constexpr uint32_t wyOffKbg = wyOffR, wyOffKbgl = wyOffR + 16384, wyOffVb = wyOffR + 32768, wyOffVbl = wyOffR + 49152;
constexpr uint32_t wyOffP = wyOffR, wyOffPl = wyOffR + 8192, wyOffP5 = wyOffR + 16384, wyOffP5l = wyOffR + 24576,
                   wyOffM = wyOffR + 32768, wyOffMl = wyOffR + 40960, wyOffMb = wyOffR + 49152, wyOffMbl = wyOffR + 57344,
                   wyOffW = wyOffR + 65536;
constexpr uint32_t kWySmem = wyOffR + 65536 + 16896;
__global__ void __launch_bounds__(256) stage_wy_bwd_kernel(StageParams p, const __grid_constant__ CUtensorMap tm_x,
                                                           const __grid_constant__ CUtensorMap tm_k,
                                                           const __grid_constant__ CUtensorMap tm_v,
                                                           const __grid_constant__ CUtensorMap tm_dw,
                                                           const __grid_constant__ CUtensorMap tm_du) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align1024(smem_raw);
  __shared__ float gam_s[kC], beta_s[kC];
  __shared__ float part_s[5][kC];    // second column half's partial row sums: row_w, dbeta, col_w, kdk, kdkbg
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t mma_bar, load_bar;
  // 8 warps: the accumulator rows 0..63 live in TMEM lanes 0..63, which only warps 0, 1, 4, 5 can read; warps 0, 1 take
  // the first half of a tile's columns and warps 4, 5 the second (`half`), the other four warps help with the
  // cooperative shared-memory passes only.
  const int tid = threadIdx.x, warp = tid >> 5;
  const int half = warp >> 2;
  const bool rowwarp = (warp & 3) < 2;
  const int n = blockIdx.z, hv = blockIdx.y, c = blockIdx.x;
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  if (c >= sq.nt) return;
  const int rows = min(kC, sq.len - c * kC);
  const int b = p.cu_seqlens ? 0 : n;
  const int t0 = (p.cu_seqlens ? sq.bos : 0) + c * kC;
  const int G = p.H / p.HK, hk = hv / G;
  const uint32_t sb = smem_u32(smem);
  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(&mma_bar, 1);
    mbar_init(&load_bar, 1);
    mbar_init_fence();
    mbar_arrive_expect_tx(&load_bar, 8192 + 4 * 16384);
    tma_load_tile4(sb + wyOffX, &tm_x, 0, t0, hv, b, &load_bar);
    tma_load_tile4(sb + wyOffK, &tm_k, 0, t0, hk, b, &load_bar);
    tma_load_tile4(sb + wyOffK + 8192, &tm_k, 64, t0, hk, b, &load_bar);
    tma_load_tile4(sb + wyOffV, &tm_v, 0, t0, hv, b, &load_bar);
    tma_load_tile4(sb + wyOffV + 8192, &tm_v, 64, t0, hv, b, &load_bar);
    tma_load_tile4(sb + wyOffDW, &tm_dw, 0, t0, hv, b, &load_bar);
    tma_load_tile4(sb + wyOffDW + 8192, &tm_dw, 64, t0, hv, b, &load_bar);
    tma_load_tile4(sb + wyOffDU, &tm_du, 0, t0, hv, b, &load_bar);
    tma_load_tile4(sb + wyOffDU + 8192, &tm_du, 64, t0, hv, b, &load_bar);
  }
  if (tid < kC) {
    gam_s[tid] = ld_any(p.g.p, row_off(p.g, b, hv, t0 + min(tid, rows - 1)), p.g.dtype);
    beta_s[tid] = tid < rows ? ld_any(p.beta.p, row_off(p.beta, b, hv, t0 + tid), p.beta.dtype) : 0.f;
  }
  tc_fence_before();
  __syncthreads();
  const uint32_t tbase = tmem_base_s;
  const uint32_t trow = tmem_addr(tbase, (warp & 3) * 32, 0);
  constexpr uint32_t cP = 0, cS = 64, cKbg = 128, cVb = 256, cT2 = 384;   // cVb is reused for dA k
  bool ok = mbar_wait(&load_bar, 0, p.status, FLA_ERR_TIMEOUT);
  // rows >= rows of every tile are zeroed in place (they hold the next sequence's rows or zeros), X also in its columns
  for (int idx = tid; idx < kC * 72; idx += 256) {
    const int r = idx / 72, ch = idx % 72;
    if (r < rows && (ch >= 8 || ch * 8 + 8 <= rows)) continue;
    uint8_t* base = ch < 8 ? smem + wyOffX + panel_chunk_off(r, ch)
                           : smem + wyOffK + ((ch - 8) >> 4) * 16384 + (((ch - 8) >> 3) & 1) * 8192 + panel_chunk_off(r, (ch - 8) & 7);
    if (r >= rows) {
      *reinterpret_cast<uint4*>(base) = make_uint4(0, 0, 0, 0);
    } else {   // a chunk of X that straddles the end of a short chunk
      uint16_t* e = reinterpret_cast<uint16_t*>(base);
      for (int j = 0; j < 8; ++j)
        if (ch * 8 + j >= rows) e[j] = 0;
    }
  }
  __syncthreads();
  // (k beta e^g) and (v beta) as value + residual
  for (int idx = tid; idx < 2 * kC * 16; idx += 256) {
    const int isv = idx >> 10, r = (idx >> 4) & 63, ch = idx & 15;
    const uint32_t off = (ch >> 3) * 8192 + panel_chunk_off(r, ch & 7);
    float f[8];
    unpack_bf16x8(*reinterpret_cast<const uint4*>(smem + (isv ? wyOffV : wyOffK) + off), f);
    const float sc = isv ? beta_s[r] : beta_s[r] * __expf(gam_s[r]);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] *= sc;
    uint4 h4, l4;
    split8(f, h4, l4);
    *reinterpret_cast<uint4*>(smem + (isv ? wyOffVb : wyOffKbg) + off) = h4;
    *reinterpret_cast<uint4*>(smem + (isv ? wyOffVbl : wyOffKbgl) + off) = l4;
  }
  fence_async_smem();
  tc_fence_before();
  ok = __syncthreads_and(ok);
  // operands; rows 64..127 of every M = 128 A view read the memory behind the panel and are never used
  const Operand opXb{sb + wyOffX, 8192, 0}, opXt{sb + wyOffX, 8192, 1}, opKa{sb + wyOffK, 8192, 0}, opKn{sb + wyOffK, 8192, 1},
      opDWa{sb + wyOffDW, 8192, 0}, opDWn{sb + wyOffDW, 8192, 1}, opDUa{sb + wyOffDU, 8192, 0}, opDUn{sb + wyOffDU, 8192, 1},
      opKbg{sb + wyOffKbg, 8192, 0}, opKbgl{sb + wyOffKbgl, 8192, 0}, opVb{sb + wyOffVb, 8192, 0}, opVbl{sb + wyOffVbl, 8192, 0},
      opP{sb + wyOffP, 8192, 0}, opPl{sb + wyOffPl, 8192, 0}, opP5{sb + wyOffP5, 8192, 1}, opP5l{sb + wyOffP5l, 8192, 1},
      opM{sb + wyOffM, 8192, 0}, opMl{sb + wyOffMl, 8192, 0}, opMbt{sb + wyOffMb, 8192, 1}, opMblt{sb + wyOffMbl, 8192, 1};
  uint32_t mphase = 0;
  const int i = tid & 63;
  const bool live = i < rows;
  float m_row[32];   // my 32 columns (32 * half ..) of row i of dA (row = later token)
  if (ok) {
    if (tid == 0) {
      tc_fence_after();
      if (p.wy_mode != 2) {
        mma_tile(tbase + cP, opDWa, opKbg, 128, 64, 8, false);
        mma_tile(tbase + cP, opDWa, opKbgl, 128, 64, 8, true);
        mma_tile(tbase + cP, opDUa, opVb, 128, 64, 8, true);
        mma_tile(tbase + cP, opDUa, opVbl, 128, 64, 8, true);
      }
      if (p.wy_mode != 1) {
        mma_tile(tbase + cS, opKa, opKa, 128, 64, 8, false);        // k k^T
        mma_tile(tbase + cKbg, opXt, opDWn, 128, 128, 4, false);    // X^T dw
        mma_tile(tbase + cVb, opXt, opDUn, 128, 128, 4, false);     // X^T du
      }
      mma_commit(&mma_bar);
    }
    ok = mbar_wait(&mma_bar, mphase, p.status, FLA_ERR_TIMEOUT);
    mphase ^= 1;
    tc_fence_after();
    ok = __syncthreads_and(ok);
  }
  if (ok && p.wy_mode != 2) {
    if (rowwarp) {
      float r[32];
      tmem_ld32(trow + cP + half * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] = (live && half * 32 + j < i) ? r[j] : 0.f;
      row32_to_hilo(smem + wyOffP, smem + wyOffPl, i, half, r);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      mma_tile(tbase + cP, opP, opXb, 128, 64, 4, false);    // P X^T
      mma_tile(tbase + cP, opPl, opXb, 128, 64, 4, true);
      mma_commit(&mma_bar);
    }
    ok = mbar_wait(&mma_bar, mphase, p.status, FLA_ERR_TIMEOUT);
    mphase ^= 1;
    tc_fence_after();
    if (rowwarp) {
      float r[32];
      tmem_ld32(trow + cP + half * 32, r);
      tmem_ld_wait();
      row32_to_hilo(smem + wyOffP5, smem + wyOffP5l, i, half, r);
    }
    fence_async_smem();
    tc_fence_before();
    ok = __syncthreads_and(ok);
    if (ok) {
      if (tid == 0) {
        tc_fence_after();
        mma_tile(tbase + cP, opXt, opP5, 128, 64, 4, false);   // X^T (P X^T)
        mma_tile(tbase + cP, opXt, opP5l, 128, 64, 4, true);
        mma_commit(&mma_bar);
      }
      ok = mbar_wait(&mma_bar, mphase, p.status, FLA_ERR_TIMEOUT);
      mphase ^= 1;
      tc_fence_after();
      if (rowwarp) {
        tmem_ld32(trow + cP + half * 32, m_row);
        tmem_ld_wait();
        const float gi = gam_s[i];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int jj = half * 32 + j;
          m_row[j] = (live && jj < i) ? -m_row[j] * __expf(gi - gam_s[jj]) : 0.f;
        }
        if (p.wy_mode == 1) {   // dA is stored transposed: element (j, i) of the chunk's block (zero on and above the diagonal)
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (half * 32 + j < rows)
              st_any(const_cast<void*>(p.o0.p), row_off(p.o0, b, hv, t0 + half * 32 + j) + i, p.o0.dtype, m_row[j]);
        }
      }
      ok = __syncthreads_and(ok);
    }
  } else if (ok && rowwarp) {
    // the given dA is stored transposed: my row i of dA is column i of the chunk's block
#pragma unroll 8
    for (int j = 0; j < 32; ++j) {
      const int jj = half * 32 + j;
      m_row[j] = (live && jj < i) ? ld_any(p.a.p, row_off(p.a, b, hv, t0 + jj) + i, p.a.dtype) : 0.f;
    }
  }
  if (ok && p.wy_mode != 1) {
    float* wt = reinterpret_cast<float*>(smem + wyOffW);
    float dbeta = 0.f, row_w = 0.f;
    const float bi = beta_s[i], egi = __expf(gam_s[i]);
    if (rowwarp) {
      row32_to_hilo(smem + wyOffM, smem + wyOffMl, i, half, m_row);
      float s[32];
      tmem_ld32(trow + cS + half * 32, s);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        m_row[j] *= bi;
        const float w = m_row[j] * s[j];
        row_w += w;
        wt[i * kColTile + half * 32 + j] = w;
      }
      row32_to_hilo(smem + wyOffMb, smem + wyOffMbl, i, half, m_row);
      // dv = beta (X^T du) and its part of dbeta (my 64 of the 128 value columns); this frees the accumulator for dA k
      bf16* dst = static_cast<bf16*>(const_cast<void*>(p.o1.p)) + row_off(p.o1, b, hv, t0 + i);
      {
        float r[64];
        tmem_ld_row64(trow + cVb + half * 64, r);
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          float vv[8];
          unpack_bf16x8(*reinterpret_cast<const uint4*>(smem + wyOffV + half * 8192 + panel_chunk_off(i, ch)), vv);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            dbeta += r[ch * 8 + j] * vv[j];
            r[ch * 8 + j] *= bi;
          }
        }
        if (live) {
#pragma unroll
          for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(dst + half * 64 + ch * 8) = pack8(r + ch * 8);
        }
      }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      mma_tile(tbase + cVb, opM, opKn, 128, 128, 4, false);      // dA k
      mma_tile(tbase + cVb, opMl, opKn, 128, 128, 4, true);
      mma_tile(tbase + cT2, opMbt, opKn, 128, 128, 4, false);    // (beta dA)^T k = dA^T (k beta)
      mma_tile(tbase + cT2, opMblt, opKn, 128, 128, 4, true);
      mma_commit(&mma_bar);
    }
    float col_w = 0.f;
    if (rowwarp) {   // column i of W, my 32 of its 64 rows
#pragma unroll 8
      for (int r = 0; r < 32; ++r) col_w += wt[(half * 32 + r) * kColTile + i];
    }
    ok = mbar_wait(&mma_bar, mphase, p.status, FLA_ERR_TIMEOUT);
    mphase ^= 1;
    tc_fence_after();
    float kdk = 0.f, kdkbg = 0.f;
    const float f2 = bi * egi;
    if (rowwarp && ok) {
      {   // my 64 of the 128 key columns
        float t1[64], acc[64];
        tmem_ld_row64(trow + cVb + half * 64, t1);
        tmem_ld_row64(trow + cT2 + half * 64, acc);
        float kb[64];
        tmem_ld_row64(trow + cKbg + half * 64, kb);
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          float kv[8];
          unpack_bf16x8(*reinterpret_cast<const uint4*>(smem + wyOffK + half * 8192 + panel_chunk_off(i, ch)), kv);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int q = ch * 8 + j;
            kdk += t1[q] * kv[j];
            kdkbg += kb[q] * kv[j];
            acc[q] += bi * t1[q] + f2 * kb[q];
          }
        }
        if (live) {
          if (p.ws_dq) {
            float* dst = p.ws_dq + ((int64_t(b) * p.H + hv) * p.T + (t0 + i)) * kK + half * 64;
#pragma unroll
            for (int j = 0; j < 64; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
          } else {
            bf16* dst = static_cast<bf16*>(const_cast<void*>(p.o0.p)) + row_off(p.o0, b, hk, t0 + i) + half * 64;
#pragma unroll
            for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(dst + ch * 8) = pack8(acc + ch * 8);
          }
        }
      }
    }
    // the two column halves add their row sums: the second half publishes, the first finishes the row
    if (rowwarp && half == 1) {
      part_s[0][i] = row_w; part_s[1][i] = dbeta; part_s[2][i] = col_w; part_s[3][i] = kdk; part_s[4][i] = kdkbg;
    }
    __syncthreads();
    if (rowwarp && half == 0 && ok && live) {
      row_w += part_s[0][i]; dbeta += part_s[1][i]; col_w += part_s[2][i]; kdk += part_s[3][i]; kdkbg += part_s[4][i];
      st_any(const_cast<void*>(p.o2.p), row_off(p.o2, b, hv, t0 + i), p.o2.dtype, dbeta + kdk + egi * kdkbg);
      st_any(const_cast<void*>(p.o3.p), row_off(p.o3, b, hv, t0 + i), p.o3.dtype, f2 * kdkbg + row_w - col_w);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 512);
}

}  // namespace fla

using namespace fla;

// ----------------------------------------------------------------------------- host side
namespace {

// [B, H, T, D] (nd == 4) or [B, H, T] (nd == 3) view; D contiguous; rows 16-byte aligned when `vec` is set
int make_view(const fla_tensor_t& t, int nd, bool vec, StageView* v) {
  if (!t.data) return FLA_ERR_NULL;
  if (t.ndim != nd) return FLA_ERR_SHAPE;
  if (nd == 4 && t.shape[3] > 1 && t.stride[3] != 1) return FLA_ERR_LAYOUT;
  v->p = t.data;
  v->sb = t.stride[0]; v->sh = t.stride[1]; v->st = t.stride[2];
  v->dtype = t.dtype;
  if (vec) {
    const int es = t.dtype == FLA_F32 ? 4 : 2;
    if (!aligned16(t.data) || (v->sb * es) % 16 || (v->sh * es) % 16 || (v->st * es) % 16) return FLA_ERR_LAYOUT;
  }
  return FLA_OK;
}

struct Geometry {
  int64_t B, H, T;
  int N, nt_max;
  int64_t total_chunks;
};

int geometry(const fla_chunk_stage_args* a, const fla_tensor_t& ref, Geometry* gm, StageParams* p) {
  if (a->chunk_size != kC) return FLA_ERR_VALUE;
  gm->B = ref.shape[0]; gm->H = ref.shape[1]; gm->T = ref.shape[2];
  if (gm->B <= 0 || gm->H <= 0 || gm->T <= 0) return FLA_ERR_SHAPE;
  gm->N = int(gm->B);
  int max_len = int(gm->T);
  gm->total_chunks = gm->B * ((gm->T + kC - 1) / kC);
  p->cu_seqlens = nullptr;
  p->chunk_offsets = nullptr;
  if (a->cu_seqlens.data) {
    if (gm->B != 1 || a->cu_seqlens.dtype != FLA_I32 || a->cu_seqlens.ndim != 1 || a->cu_seqlens.shape[0] < 2) return FLA_ERR_SHAPE;
    gm->N = int(a->cu_seqlens.shape[0] - 1);
    if (!a->chunk_offsets.data || a->chunk_offsets.dtype != FLA_I32 || a->chunk_offsets.shape[0] != gm->N + 1) return FLA_ERR_SHAPE;
    if (a->max_seqlen <= 0 || a->max_seqlen > gm->T || a->total_chunks <= 0) return FLA_ERR_VALUE;
    max_len = a->max_seqlen;
    gm->total_chunks = a->total_chunks;
    p->cu_seqlens = static_cast<const int32_t*>(a->cu_seqlens.data);
    p->chunk_offsets = static_cast<const int32_t*>(a->chunk_offsets.data);
  }
  gm->nt_max = (max_len + kC - 1) / kC;
  p->T = int(gm->T);
  p->H = int(gm->H);
  return FLA_OK;
}

bool same_bht(const fla_tensor_t& t, const Geometry& gm, int64_t heads) {
  return t.shape[0] == gm.B && t.shape[1] == heads && t.shape[2] == gm.T;
}

int prepare_status(void* workspace, uint64_t bytes, cudaStream_t cs, StageParams* p) {
  if (!workspace || bytes < 256 || !aligned16(workspace)) return FLA_ERR_WORKSPACE;
  if (cudaMemsetAsync(workspace, 0, 256, cs) != cudaSuccess) return FLA_ERR_CUDA;
  p->status = static_cast<int*>(workspace);
  return FLA_OK;
}

// 64-token x 64-column bf16 tiles of a [B, H, T, D] tensor
int token_tile_map(const fla_tensor_t& t, CUtensorMap* map) {
  return make_bhtd_tile_map(map, t.data, 2, uint64_t(t.shape[3]), uint64_t(t.shape[2]), uint64_t(t.shape[1]), uint64_t(t.shape[0]),
                            uint64_t(t.stride[2]), uint64_t(t.stride[1]), uint64_t(t.stride[0]), 64, 64);
}

template <typename Kern>
int opt_in_smem(Kern kern, uint32_t bytes) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes)) == cudaSuccess ? FLA_OK : FLA_ERR_CUDA;
}

}  // namespace

// Every stage needs the same workspace: the status word of the bounded device-side waits.
#define FLA_STAGE_WORKSPACE(op)                                                                              \
  extern "C" FLA_API int fla_b200_##op##_workspace_size(const fla_chunk_stage_args* a, uint64_t* bytes) {     \
    if (!a || !bytes) return FLA_ERR_NULL;                                                                   \
    *bytes = 256;                                                                                            \
    return FLA_OK;                                                                                           \
  }
FLA_STAGE_WORKSPACE(chunk_local_cumsum)
FLA_STAGE_WORKSPACE(chunk_scaled_dot_kkt)
FLA_STAGE_WORKSPACE(solve_tri)
FLA_STAGE_WORKSPACE(recompute_w_u_fwd)
FLA_STAGE_WORKSPACE(chunk_gated_delta_rule_fwd_h)
FLA_STAGE_WORKSPACE(chunk_fwd_o)
FLA_STAGE_WORKSPACE(chunk_bwd_dv_local)
FLA_STAGE_WORKSPACE(chunk_gated_delta_rule_bwd_dhu)

extern "C" FLA_API int fla_b200_chunk_local_cumsum(const fla_chunk_stage_args* a, void* workspace, uint64_t workspace_bytes,
                                                   void* stream) {
  if (!a) return FLA_ERR_NULL;
  (void)workspace; (void)workspace_bytes;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  StageParams p{};
  Geometry gm;
  int st;
  const int nd = a->g.ndim;
  if (nd != 3 && nd != 4) return FLA_ERR_SHAPE;
  if ((st = geometry(a, a->g, &gm, &p))) return st;
  if ((st = make_view(a->g, nd, false, &p.g)) || (st = make_view(a->out0, nd, false, &p.o0))) return st;
  for (int i = 0; i < nd; ++i)
    if (a->out0.shape[i] != a->g.shape[i]) return FLA_ERR_SHAPE;
  p.D = nd == 4 ? int(a->g.shape[3]) : 1;
  if (p.D < 1 || p.D > 1024) return FLA_ERR_SHAPE;
  p.reverse = a->reverse;
  p.scale = a->scale;
  p.gate_mode = a->gate_mode;
  if (a->gate_mode < 0 || a->gate_mode > 2) return FLA_ERR_VALUE;
  if (a->gate_mode) {   // per-channel gate activation: A_log [H] in `q`, dt_bias [H, D] (optional) in `k`, both f32
    if (nd != 4) return FLA_ERR_SHAPE;
    const fla_tensor_t &al = a->q, &db = a->k;
    if (!al.data) return FLA_ERR_NULL;
    if (al.dtype != FLA_F32 || numel(al) != gm.H || !is_contig_last(al)) return FLA_ERR_SHAPE;
    if (db.data && (db.dtype != FLA_F32 || numel(db) != gm.H * p.D || !is_contig_last(db))) return FLA_ERR_SHAPE;
    p.a_log = static_cast<const float*>(al.data);
    p.dt_bias = static_cast<const float*>(db.data);
    p.lower_bound = a->lower_bound;
  }
  const int threads = p.D == 1 ? 64 : ((std::min(p.D, 128) + 31) / 32) * 32;
  KernelTimer kt("chunk_local_cumsum", cs);
  stage_cumsum_kernel<<<dim3(gm.nt_max, unsigned(gm.H), gm.N), threads, 0, cs>>>(p);
  return cuda_status(cudaGetLastError());
}

extern "C" FLA_API int fla_b200_chunk_scaled_dot_kkt(const fla_chunk_stage_args* a, void* workspace, uint64_t workspace_bytes,
                                                     void* stream) {
  if (!a) return FLA_ERR_NULL;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  StageParams p{};
  Geometry gm;
  int st;
  if (a->g.ndim != 3) return FLA_ERR_SHAPE;
  if ((st = geometry(a, a->g, &gm, &p))) return st;
  if ((st = make_view(a->k, 4, true, &p.k)) || (st = make_view(a->g, 3, false, &p.g)) || (st = make_view(a->beta, 3, false, &p.beta)) ||
      (st = make_view(a->out0, 4, true, &p.o0)))
    return st;
  const int64_t HK = a->k.shape[1];
  if (a->k.dtype != FLA_BF16 || a->out0.dtype != FLA_F32) return FLA_ERR_DTYPE;
  if (HK <= 0 || gm.H % HK || a->k.shape[0] != gm.B || a->k.shape[2] != gm.T || a->k.shape[3] != kK) return FLA_ERR_SHAPE;
  if (!same_bht(a->beta, gm, gm.H) || !same_bht(a->out0, gm, gm.H) || a->out0.shape[3] != kC) return FLA_ERR_SHAPE;
  p.HK = int(HK);
  if ((st = prepare_status(workspace, workspace_bytes, cs, &p))) return st;
  if ((st = opt_in_smem(stage_kkt_kernel, kKktSmem + 1024))) return st;
  KernelTimer kt("chunk_scaled_dot_kkt", cs);
  stage_kkt_kernel<<<dim3((gm.nt_max + 1) / 2, unsigned(HK), gm.N), 128, kKktSmem + 1024, cs>>>(p);
  return cuda_status(cudaGetLastError());
}

extern "C" FLA_API int fla_b200_solve_tri(const fla_chunk_stage_args* a, void* workspace, uint64_t workspace_bytes, void* stream) {
  if (!a) return FLA_ERR_NULL;
  (void)workspace; (void)workspace_bytes;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  StageParams p{};
  Geometry gm;
  int st;
  if (a->A.ndim != 4) return FLA_ERR_SHAPE;
  if ((st = geometry(a, a->A, &gm, &p))) return st;
  if ((st = make_view(a->A, 4, false, &p.a)) || (st = make_view(a->out0, 4, false, &p.o0))) return st;
  if (a->A.shape[3] != kC || !same_bht(a->out0, gm, gm.H) || a->out0.shape[3] != kC) return FLA_ERR_SHAPE;
  const uint32_t smem = kSolveTiles * kC * kSolveStride * sizeof(float);
  if ((st = opt_in_smem(stage_solve_tri_kernel, smem))) return st;
  KernelTimer kt("solve_tri", cs);
  stage_solve_tri_kernel<<<dim3(gm.nt_max, unsigned((gm.H + kSolveTiles - 1) / kSolveTiles), gm.N), 64 * kSolveTiles, smem, cs>>>(p);
  return cuda_status(cudaGetLastError());
}

extern "C" FLA_API int fla_b200_recompute_w_u_fwd(const fla_chunk_stage_args* a, void* workspace, uint64_t workspace_bytes,
                                                  void* stream) {
  if (!a) return FLA_ERR_NULL;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  StageParams p{};
  Geometry gm;
  int st;
  if (a->v.ndim != 4) return FLA_ERR_SHAPE;
  if ((st = geometry(a, a->v, &gm, &p))) return st;
  if ((st = make_view(a->k, 4, true, &p.k)) || (st = make_view(a->v, 4, true, &p.v)) || (st = make_view(a->A, 4, true, &p.a)) ||
      (st = make_view(a->g, 3, false, &p.g)) || (st = make_view(a->beta, 3, false, &p.beta)) ||
      (st = make_view(a->out0, 4, true, &p.o0)) || (st = make_view(a->out1, 4, true, &p.o1)))
    return st;
  const int64_t HK = a->k.shape[1];
  for (const fla_tensor_t* t : {&a->k, &a->v, &a->A, &a->out0, &a->out1})
    if (t->dtype != FLA_BF16) return FLA_ERR_DTYPE;
  if (HK <= 0 || gm.H % HK || a->k.shape[0] != gm.B || a->k.shape[2] != gm.T || a->k.shape[3] != kK || a->v.shape[3] != kV) return FLA_ERR_SHAPE;
  if (!same_bht(a->A, gm, gm.H) || a->A.shape[3] != kC || !same_bht(a->g, gm, gm.H) || !same_bht(a->beta, gm, gm.H)) return FLA_ERR_SHAPE;
  if (!same_bht(a->out0, gm, gm.H) || a->out0.shape[3] != kK || !same_bht(a->out1, gm, gm.H) || a->out1.shape[3] != kV) return FLA_ERR_SHAPE;
  p.HK = int(HK);
  if ((st = prepare_status(workspace, workspace_bytes, cs, &p))) return st;
  if ((st = opt_in_smem(stage_wu_kernel, kWuSmem + 1024))) return st;
  CUtensorMap tm_k, tm_v, tm_x;
  if (token_tile_map(a->k, &tm_k) || token_tile_map(a->v, &tm_v) || token_tile_map(a->A, &tm_x)) return FLA_ERR_CUDA;
  KernelTimer kt("recompute_w_u_fwd", cs);
  stage_wu_kernel<<<dim3(gm.nt_max, unsigned(gm.H), gm.N), 256, kWuSmem + 1024, cs>>>(p, tm_k, tm_v, tm_x);
  return cuda_status(cudaGetLastError());
}

extern "C" FLA_API int fla_b200_chunk_gated_delta_rule_fwd_h(const fla_chunk_stage_args* a, void* workspace, uint64_t workspace_bytes,
                                                             void* stream) {
  if (!a) return FLA_ERR_NULL;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  StageParams p{};
  Geometry gm;
  int st;
  if (a->u.ndim != 4) return FLA_ERR_SHAPE;
  if ((st = geometry(a, a->u, &gm, &p))) return st;
  if ((st = make_view(a->k, 4, true, &p.k)) || (st = make_view(a->w, 4, true, &p.w)) || (st = make_view(a->u, 4, true, &p.u)) ||
      (st = make_view(a->g, 3, false, &p.g)) || (st = make_view(a->out1, 4, true, &p.o1)))
    return st;
  const int64_t HK = a->k.shape[1];
  for (const fla_tensor_t* t : {&a->k, &a->w, &a->u, &a->out0, &a->out1})
    if (t->dtype != FLA_BF16) return FLA_ERR_DTYPE;
  if (HK <= 0 || gm.H % HK || a->k.shape[0] != gm.B || a->k.shape[2] != gm.T || a->k.shape[3] != kK || a->u.shape[3] != kV) return FLA_ERR_SHAPE;
  if (!same_bht(a->w, gm, gm.H) || a->w.shape[3] != kK || !same_bht(a->g, gm, gm.H) || !same_bht(a->out1, gm, gm.H) || a->out1.shape[3] != kV)
    return FLA_ERR_SHAPE;
  // h [B, H, NT, K, V], dense
  const fla_tensor_t& h = a->out0;
  const int64_t NT = gm.total_chunks / gm.B;
  if (!h.data) return FLA_ERR_NULL;
  if (h.ndim != 5 || h.shape[0] != gm.B || h.shape[1] != gm.H || h.shape[2] != NT || h.shape[3] != kK || h.shape[4] != kV) return FLA_ERR_SHAPE;
  if (h.stride[4] != 1 || h.stride[3] != kV || h.stride[2] != kK * kV || h.stride[1] != NT * kK * kV || !aligned16(h.data)) return FLA_ERR_LAYOUT;
  p.o0.p = h.data;
  p.o0.sh = NT;    // chunks per (batch row, head)
  for (const fla_tensor_t* s : {&a->initial_state, &a->out2}) {
    if (!s->data) continue;
    if (s->dtype != FLA_F32) return FLA_ERR_DTYPE;
    if (s->ndim != 4 || s->shape[0] != gm.N || s->shape[1] != gm.H || s->shape[2] != kK || s->shape[3] != kV) return FLA_ERR_SHAPE;
    if (s->stride[3] != 1 || s->stride[2] != kV || s->stride[1] != kK * kV || s->stride[0] != gm.H * kK * kV || !aligned16(s->data))
      return FLA_ERR_LAYOUT;
  }
  p.h0.p = a->initial_state.data;
  p.o2.p = a->out2.data;
  p.want_final = a->out2.data != nullptr;
  p.HK = int(HK);
  if ((st = prepare_status(workspace, workspace_bytes, cs, &p))) return st;
  if ((st = opt_in_smem(stage_fwd_h_kernel, kFwdHSmem + 1024))) return st;
  CUtensorMap tm_w, tm_k, tm_u;
  if (token_tile_map(a->w, &tm_w) || token_tile_map(a->k, &tm_k) || token_tile_map(a->u, &tm_u)) return FLA_ERR_CUDA;
  KernelTimer kt("chunk_fwd_h", cs);
  stage_fwd_h_kernel<<<dim3(kV / 64, unsigned(gm.H), gm.N), 128, kFwdHSmem + 1024, cs>>>(p, tm_w, tm_k, tm_u);
  return cuda_status(cudaGetLastError());
}

extern "C" FLA_API int fla_b200_chunk_fwd_o(const fla_chunk_stage_args* a, void* workspace, uint64_t workspace_bytes, void* stream) {
  if (!a) return FLA_ERR_NULL;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  StageParams p{};
  Geometry gm;
  int st;
  if (a->v.ndim != 4) return FLA_ERR_SHAPE;
  if ((st = geometry(a, a->v, &gm, &p))) return st;
  if ((st = make_view(a->q, 4, true, &p.q)) || (st = make_view(a->k, 4, true, &p.k)) || (st = make_view(a->v, 4, true, &p.v)) ||
      (st = make_view(a->g, 3, false, &p.g)) || (st = make_view(a->out0, 4, true, &p.o0)))
    return st;
  const int64_t HK = a->k.shape[1];
  for (const fla_tensor_t* t : {&a->q, &a->k, &a->v, &a->h, &a->out0})
    if (t->dtype != FLA_BF16) return FLA_ERR_DTYPE;
  if (HK <= 0 || gm.H % HK || a->k.shape[0] != gm.B || a->k.shape[2] != gm.T || a->k.shape[3] != kK || a->v.shape[3] != kV) return FLA_ERR_SHAPE;
  if (a->q.shape[0] != gm.B || a->q.shape[1] != HK || a->q.shape[2] != gm.T || a->q.shape[3] != kK) return FLA_ERR_SHAPE;
  if (!same_bht(a->g, gm, gm.H) || !same_bht(a->out0, gm, gm.H) || a->out0.shape[3] != kV) return FLA_ERR_SHAPE;
  const fla_tensor_t& h = a->h;
  const int64_t NT = gm.total_chunks / gm.B;
  if (!h.data) return FLA_ERR_NULL;
  if (h.ndim != 5 || h.shape[0] != gm.B || h.shape[1] != gm.H || h.shape[2] != NT || h.shape[3] != kK || h.shape[4] != kV) return FLA_ERR_SHAPE;
  if (h.stride[4] != 1 || h.stride[3] != kV || h.stride[2] != kK * kV || h.stride[1] != NT * kK * kV || !aligned16(h.data)) return FLA_ERR_LAYOUT;
  p.h.p = h.data;
  p.h.sh = NT;
  p.HK = int(HK);
  p.scale = a->scale;
  if (!(a->scale == a->scale)) return FLA_ERR_VALUE;
  if ((st = prepare_status(workspace, workspace_bytes, cs, &p))) return st;
  if ((st = opt_in_smem(stage_fwd_o_kernel, kFwdOSmem + 1024))) return st;
  CUtensorMap tm_q, tm_k, tm_v, tm_h;
  if (token_tile_map(a->q, &tm_q) || token_tile_map(a->k, &tm_k) || token_tile_map(a->v, &tm_v) ||
      make_bhtd_tile_map(&tm_h, h.data, 2, kV, uint64_t(gm.B) * gm.H * NT * kK, 1, 1, kV, 0, 0, 64, 128))
    return FLA_ERR_CUDA;
  KernelTimer kt("chunk_fwd_o", cs);
  stage_fwd_o_kernel<<<dim3(gm.nt_max, unsigned(gm.H), gm.N), 256, kFwdOSmem + 1024, cs>>>(p, tm_q, tm_k, tm_v, tm_h);
  return cuda_status(cudaGetLastError());
}

extern "C" FLA_API int fla_b200_chunk_bwd_dv_local(const fla_chunk_stage_args* a, void* workspace, uint64_t workspace_bytes,
                                                   void* stream) {
  if (!a) return FLA_ERR_NULL;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  StageParams p{};
  Geometry gm;
  int st;
  const fla_tensor_t& d_o = a->v;
  if (d_o.ndim != 4) return FLA_ERR_SHAPE;
  if ((st = geometry(a, d_o, &gm, &p))) return st;
  StageView vq, vk, vdo;
  if ((st = make_view(a->q, 4, true, &vq)) || (st = make_view(a->k, 4, true, &vk)) || (st = make_view(d_o, 4, true, &vdo)) ||
      (st = make_view(a->g, 3, false, &p.g)) || (st = make_view(a->out0, 4, true, &p.o0)))
    return st;
  const int64_t HK = a->k.shape[1];
  for (const fla_tensor_t* t : {&a->q, &a->k, &d_o, &a->out0})
    if (t->dtype != FLA_BF16) return FLA_ERR_DTYPE;
  if (HK <= 0 || gm.H % HK || a->k.shape[0] != gm.B || a->k.shape[2] != gm.T || a->k.shape[3] != kK || d_o.shape[3] != kV) return FLA_ERR_SHAPE;
  if (a->q.shape[0] != gm.B || a->q.shape[1] != HK || a->q.shape[2] != gm.T || a->q.shape[3] != kK) return FLA_ERR_SHAPE;
  if (!same_bht(a->g, gm, gm.H) || !same_bht(a->out0, gm, gm.H) || a->out0.shape[3] != kV) return FLA_ERR_SHAPE;
  p.HK = int(HK);
  p.scale = a->scale;
  if (!(a->scale == a->scale)) return FLA_ERR_VALUE;
  if ((st = prepare_status(workspace, workspace_bytes, cs, &p))) return st;
  if ((st = opt_in_smem(stage_dv_local_kernel, kDvLocalSmem + 1024))) return st;
  CUtensorMap tm_q, tm_k, tm_do;
  if (token_tile_map(a->q, &tm_q) || token_tile_map(a->k, &tm_k) || token_tile_map(d_o, &tm_do)) return FLA_ERR_CUDA;
  KernelTimer kt("chunk_bwd_dv_local", cs);
  stage_dv_local_kernel<<<dim3(gm.nt_max, unsigned(gm.H), gm.N), 256, kDvLocalSmem + 1024, cs>>>(p, tm_q, tm_k, tm_do);
  return cuda_status(cudaGetLastError());
}

extern "C" FLA_API int fla_b200_chunk_gated_delta_rule_bwd_dhu(const fla_chunk_stage_args* a, void* workspace,
                                                               uint64_t workspace_bytes, void* stream) {
  if (!a) return FLA_ERR_NULL;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  StageParams p{};
  Geometry gm;
  int st;
  const fla_tensor_t &d_o = a->u, &dv = a->v;
  if (dv.ndim != 4) return FLA_ERR_SHAPE;
  if ((st = geometry(a, dv, &gm, &p))) return st;
  StageView tmp;
  if ((st = make_view(a->q, 4, true, &tmp)) || (st = make_view(a->k, 4, true, &tmp)) || (st = make_view(a->w, 4, true, &tmp)) ||
      (st = make_view(d_o, 4, true, &tmp)) || (st = make_view(dv, 4, true, &tmp)) || (st = make_view(a->g, 3, false, &p.g)) ||
      (st = make_view(a->out1, 4, true, &p.o1)))
    return st;
  const int64_t HK = a->k.shape[1];
  for (const fla_tensor_t* t : {&a->q, &a->k, &a->w, &d_o, &dv, &a->out0, &a->out1})
    if (t->dtype != FLA_BF16) return FLA_ERR_DTYPE;
  if (HK <= 0 || gm.H % HK || a->k.shape[0] != gm.B || a->k.shape[2] != gm.T || a->k.shape[3] != kK || dv.shape[3] != kV) return FLA_ERR_SHAPE;
  if (a->q.shape[0] != gm.B || a->q.shape[1] != HK || a->q.shape[2] != gm.T || a->q.shape[3] != kK) return FLA_ERR_SHAPE;
  if (!same_bht(a->w, gm, gm.H) || a->w.shape[3] != kK || !same_bht(d_o, gm, gm.H) || d_o.shape[3] != kV) return FLA_ERR_SHAPE;
  if (!same_bht(a->g, gm, gm.H) || !same_bht(a->out1, gm, gm.H) || a->out1.shape[3] != kV) return FLA_ERR_SHAPE;
  const fla_tensor_t& h = a->out0;
  const int64_t NT = gm.total_chunks / gm.B;
  if (!h.data) return FLA_ERR_NULL;
  if (h.ndim != 5 || h.shape[0] != gm.B || h.shape[1] != gm.H || h.shape[2] != NT || h.shape[3] != kK || h.shape[4] != kV) return FLA_ERR_SHAPE;
  if (h.stride[4] != 1 || h.stride[3] != kV || h.stride[2] != kK * kV || h.stride[1] != NT * kK * kV || !aligned16(h.data)) return FLA_ERR_LAYOUT;
  p.o0.p = h.data;
  p.o0.sh = NT;
  for (const fla_tensor_t* s : {&a->initial_state, &a->out2}) {
    if (!s->data) continue;
    if (s->dtype != FLA_F32) return FLA_ERR_DTYPE;
    if (s->ndim != 4 || s->shape[0] != gm.N || s->shape[1] != gm.H || s->shape[2] != kK || s->shape[3] != kV) return FLA_ERR_SHAPE;
    if (s->stride[3] != 1 || s->stride[2] != kV || s->stride[1] != kK * kV || s->stride[0] != gm.H * kK * kV || !aligned16(s->data))
      return FLA_ERR_LAYOUT;
  }
  p.h0.p = a->initial_state.data;   // dht
  p.o2.p = a->out2.data;            // dh0
  p.want_final = a->out2.data != nullptr;
  p.HK = int(HK);
  p.scale = a->scale;
  if (!(a->scale == a->scale)) return FLA_ERR_VALUE;
  if ((st = prepare_status(workspace, workspace_bytes, cs, &p))) return st;
  if ((st = opt_in_smem(stage_bwd_dhu_kernel, kBwdDhuSmem + 1024))) return st;
  CUtensorMap tm_q, tm_k, tm_w, tm_do, tm_dv;
  if (token_tile_map(a->q, &tm_q) || token_tile_map(a->k, &tm_k) || token_tile_map(a->w, &tm_w) || token_tile_map(d_o, &tm_do) ||
      token_tile_map(dv, &tm_dv))
    return FLA_ERR_CUDA;
  KernelTimer kt("chunk_bwd_dhu", cs);
  stage_bwd_dhu_kernel<<<dim3(kV / 64, unsigned(gm.H), gm.N), 128, kBwdDhuSmem + 1024, cs>>>(p, tm_q, tm_k, tm_w, tm_do, tm_dv);
  return cuda_status(cudaGetLastError());
}

static uint64_t dqkwg_scratch_bytes(const fla_chunk_stage_args* a) {
  const fla_tensor_t &q = a->q, &v = a->v;
  if (q.ndim != 4 || v.ndim != 4 || q.shape[1] <= 0 || v.shape[1] == q.shape[1]) return 0;
  return 2ull * uint64_t(v.shape[0]) * v.shape[1] * v.shape[2] * kK * sizeof(float);
}

extern "C" FLA_API int fla_b200_chunk_bwd_dqkwg_workspace_size(const fla_chunk_stage_args* a, uint64_t* bytes) {
  if (!a || !bytes) return FLA_ERR_NULL;
  *bytes = 256 + dqkwg_scratch_bytes(a);
  return FLA_OK;
}

extern "C" FLA_API int fla_b200_chunk_bwd_dqkwg(const fla_chunk_stage_args* a, void* workspace, uint64_t workspace_bytes, void* stream) {
  if (!a) return FLA_ERR_NULL;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  StageParams p{};
  Geometry gm;
  int st;
  const fla_tensor_t &d_o = a->u, &dv = a->w, &dh = a->A;
  if (a->v.ndim != 4) return FLA_ERR_SHAPE;
  if ((st = geometry(a, a->v, &gm, &p))) return st;
  StageView tmp;
  if ((st = make_view(a->q, 4, true, &tmp)) || (st = make_view(a->k, 4, true, &tmp)) || (st = make_view(a->v, 4, true, &tmp)) ||
      (st = make_view(d_o, 4, true, &tmp)) || (st = make_view(dv, 4, true, &tmp)) || (st = make_view(a->g, 3, false, &p.g)) ||
      (st = make_view(a->out0, 4, true, &p.o0)) || (st = make_view(a->out1, 4, true, &p.o1)) || (st = make_view(a->out3, 3, false, &p.o3)))
    return st;
  if (a->out2.data && (st = make_view(a->out2, 4, true, &p.o2))) return st;
  const int64_t HK = a->k.shape[1];
  for (const fla_tensor_t* t : {&a->q, &a->k, &a->v, &d_o, &dv, &a->h, &dh, &a->out0, &a->out1})
    if (t->dtype != FLA_BF16) return FLA_ERR_DTYPE;
  if (a->out2.data && a->out2.dtype != FLA_BF16) return FLA_ERR_DTYPE;
  if (HK <= 0 || gm.H % HK || a->v.shape[3] != kV) return FLA_ERR_SHAPE;
  for (const fla_tensor_t* t : {&a->q, &a->k, &a->out0, &a->out1})
    if (t->shape[0] != gm.B || t->shape[1] != HK || t->shape[2] != gm.T || t->shape[3] != kK) return FLA_ERR_SHAPE;
  for (const fla_tensor_t* t : {&d_o, &dv})
    if (!same_bht(*t, gm, gm.H) || t->shape[3] != kV) return FLA_ERR_SHAPE;
  if (a->out2.data && (!same_bht(a->out2, gm, gm.H) || a->out2.shape[3] != kK)) return FLA_ERR_SHAPE;
  if (!same_bht(a->g, gm, gm.H) || !same_bht(a->out3, gm, gm.H)) return FLA_ERR_SHAPE;
  const int64_t NT = gm.total_chunks / gm.B;
  for (const fla_tensor_t* h : {&a->h, &dh}) {
    if (!h->data) return FLA_ERR_NULL;
    if (h->ndim != 5 || h->shape[0] != gm.B || h->shape[1] != gm.H || h->shape[2] != NT || h->shape[3] != kK || h->shape[4] != kV) return FLA_ERR_SHAPE;
    if (h->stride[4] != 1 || h->stride[3] != kV || h->stride[2] != kK * kV || h->stride[1] != NT * kK * kV || !aligned16(h->data)) return FLA_ERR_LAYOUT;
  }
  p.h.sh = NT;
  p.HK = int(HK);
  p.scale = a->scale;
  if (!(a->scale == a->scale)) return FLA_ERR_VALUE;
  const uint64_t scratch = dqkwg_scratch_bytes(a);
  if (!workspace || workspace_bytes < 256 + scratch) return FLA_ERR_WORKSPACE;
  if ((st = prepare_status(workspace, workspace_bytes, cs, &p))) return st;
  if (scratch) {
    p.ws_dq = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + 256);
    p.ws_dk = p.ws_dq + scratch / 8;
  }
  if ((st = opt_in_smem(stage_dqkwg_kernel, kDqkwgSmem + 1024))) return st;
  CUtensorMap tm_q, tm_k, tm_v, tm_do, tm_dv, tm_h, tm_dh;
  const uint64_t hrows = uint64_t(gm.B) * gm.H * NT * kK;
  if (token_tile_map(a->q, &tm_q) || token_tile_map(a->k, &tm_k) || token_tile_map(a->v, &tm_v) || token_tile_map(d_o, &tm_do) ||
      token_tile_map(dv, &tm_dv) || make_bhtd_tile_map(&tm_h, a->h.data, 2, kV, hrows, 1, 1, kV, 0, 0, 64, 128) ||
      make_bhtd_tile_map(&tm_dh, dh.data, 2, kV, hrows, 1, 1, kV, 0, 0, 64, 128))
    return FLA_ERR_CUDA;
  {
    KernelTimer kt("chunk_bwd_dqkwg", cs);
    stage_dqkwg_kernel<<<dim3(gm.nt_max, unsigned(gm.H), gm.N), 256, kDqkwgSmem + 1024, cs>>>(p, tm_q, tm_k, tm_v, tm_do, tm_dv, tm_h, tm_dh);
  }
  if (cudaGetLastError() != cudaSuccess) return FLA_ERR_CUDA;
  if (scratch) {
    KernelTimer kt("chunk_bwd_dqkwg_group_sum", cs);
    stage_group_sum_kernel<<<148 * 8, 256, 0, cs>>>(p, int(gm.B), 2);
  }
  return cuda_status(cudaGetLastError());
}

static uint64_t wy_scratch_bytes(const fla_chunk_stage_args* a) {
  const fla_tensor_t &k = a->k, &v = a->v;
  if (k.ndim != 4 || v.ndim != 4 || k.shape[1] <= 0 || v.shape[1] == k.shape[1]) return 0;
  return uint64_t(v.shape[0]) * v.shape[1] * v.shape[2] * kK * sizeof(float);
}

static int wy_bwd_launch(const fla_chunk_stage_args* a, void* workspace, uint64_t workspace_bytes, void* stream, int mode) {
  if (!a) return FLA_ERR_NULL;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  StageParams p{};
  Geometry gm;
  int st;
  const fla_tensor_t &dw = a->w, &du = a->u, &dA = a->q;
  if (a->v.ndim != 4) return FLA_ERR_SHAPE;
  if ((st = geometry(a, a->v, &gm, &p))) return st;
  StageView tmp;
  if ((st = make_view(a->k, 4, true, &tmp)) || (st = make_view(a->v, 4, true, &tmp)) || (st = make_view(a->A, 4, true, &tmp)) ||
      (st = make_view(dw, 4, true, &tmp)) || (st = make_view(du, 4, true, &tmp)) || (st = make_view(a->g, 3, false, &p.g)) ||
      (st = make_view(a->beta, 3, false, &p.beta)))
    return st;
  const int64_t HK = a->k.shape[1];
  for (const fla_tensor_t* t : {&a->k, &a->v, &a->A, &dw, &du})
    if (t->dtype != FLA_BF16) return FLA_ERR_DTYPE;
  if (HK <= 0 || gm.H % HK || a->k.shape[0] != gm.B || a->k.shape[2] != gm.T || a->k.shape[3] != kK || a->v.shape[3] != kV) return FLA_ERR_SHAPE;
  if (!same_bht(a->A, gm, gm.H) || a->A.shape[3] != kC || !same_bht(dw, gm, gm.H) || dw.shape[3] != kK || !same_bht(du, gm, gm.H) ||
      du.shape[3] != kV || !same_bht(a->g, gm, gm.H) || !same_bht(a->beta, gm, gm.H))
    return FLA_ERR_SHAPE;
  uint64_t scratch = 0;
  if (mode == 1) {
    if ((st = make_view(a->out0, 4, false, &p.o0))) return st;
    if (!same_bht(a->out0, gm, gm.H) || a->out0.shape[3] != kC) return FLA_ERR_SHAPE;
  } else {
    if ((st = make_view(a->out0, 4, true, &p.o0)) || (st = make_view(a->out1, 4, true, &p.o1)) || (st = make_view(a->out2, 3, false, &p.o2)) ||
        (st = make_view(a->out3, 3, false, &p.o3)))
      return st;
    if (a->out0.dtype != FLA_BF16 || a->out1.dtype != FLA_BF16) return FLA_ERR_DTYPE;
    if (a->out0.shape[0] != gm.B || a->out0.shape[1] != HK || a->out0.shape[2] != gm.T || a->out0.shape[3] != kK) return FLA_ERR_SHAPE;
    if (!same_bht(a->out1, gm, gm.H) || a->out1.shape[3] != kV || !same_bht(a->out2, gm, gm.H) || !same_bht(a->out3, gm, gm.H)) return FLA_ERR_SHAPE;
    if (mode == 2) {
      if ((st = make_view(dA, 4, false, &p.a))) return st;
      if (!same_bht(dA, gm, gm.H) || dA.shape[3] != kC) return FLA_ERR_SHAPE;
    }
    scratch = wy_scratch_bytes(a);
  }
  p.HK = int(HK);
  p.wy_mode = mode;
  if (!workspace || workspace_bytes < 256 + scratch) return FLA_ERR_WORKSPACE;
  if ((st = prepare_status(workspace, workspace_bytes, cs, &p))) return st;
  if (scratch) p.ws_dq = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + 256);
  if ((st = opt_in_smem(stage_wy_bwd_kernel, kWySmem + 1024))) return st;
  CUtensorMap tm_x, tm_k, tm_v, tm_dw, tm_du;
  if (token_tile_map(a->A, &tm_x) || token_tile_map(a->k, &tm_k) || token_tile_map(a->v, &tm_v) || token_tile_map(dw, &tm_dw) ||
      token_tile_map(du, &tm_du))
    return FLA_ERR_CUDA;
  {
    KernelTimer kt("prepare_wy_repr_bwd", cs);
    stage_wy_bwd_kernel<<<dim3(gm.nt_max, unsigned(gm.H), gm.N), 256, kWySmem + 1024, cs>>>(p, tm_x, tm_k, tm_v, tm_dw, tm_du);
  }
  if (cudaGetLastError() != cudaSuccess) return FLA_ERR_CUDA;
  if (scratch) {
    KernelTimer kt("prepare_wy_repr_bwd_group_sum", cs);
    stage_group_sum_kernel<<<148 * 8, 256, 0, cs>>>(p, int(gm.B), 1);
  }
  return cuda_status(cudaGetLastError());
}

#define FLA_WY_ENTRY(op, mode)                                                                                              \
  extern "C" FLA_API int fla_b200_##op##_workspace_size(const fla_chunk_stage_args* a, uint64_t* bytes) {                    \
    if (!a || !bytes) return FLA_ERR_NULL;                                                                                  \
    *bytes = 256 + ((mode) == 1 ? 0 : wy_scratch_bytes(a));                                                                 \
    return FLA_OK;                                                                                                          \
  }                                                                                                                         \
  extern "C" FLA_API int fla_b200_##op(const fla_chunk_stage_args* a, void* workspace, uint64_t workspace_bytes, void* stream) { \
    return wy_bwd_launch(a, workspace, workspace_bytes, stream, mode);                                                      \
  }
FLA_WY_ENTRY(prepare_wy_repr_bwd, 0)
FLA_WY_ENTRY(prepare_wy_repr_bwd_da, 1)
FLA_WY_ENTRY(prepare_wy_repr_bwd_full, 2)

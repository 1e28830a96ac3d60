// Chunked Kimi-Delta-Attention forward (per-channel log gate g[t, h, :], chunk = 64, K = V = 128).
//
//   gk = chunk-local cumsum(gate(g));   with a per-channel anchor a = gk at the middle token of the chunk:
//   Qp = Q * e^{gk - a}   Kp = K * e^{gk - a}   Kn = K * e^{a - gk}        (all finite for any realistic decay)
//   Aqk = tril(Qp Kn^T)   Akk = strict_tril(beta_i Kp Kn^T)   X = (I + Akk)^-1
//   per chunk, Sa = diag(e^a) S:   v_new = X (beta * (V - Kp Sa))
//                                  o     = scale (Qp Sa + Aqk v_new)
//                                  S    <- diag(e^{gk_L - a}) (Sa + Kn^T v_new)
// which equals the reference's chunk_kda_fwd stages (gate cumsum -> Prepare -> Post-WU -> FwdH -> Finalize,
// fla/ops/ascendc/kda/chunk_kda_fwd/docs/design.md:11-78; golden tests/atk/chunk_kda_fwd/executor_chunk_kda_fwd.py:402-530)
// with w, u folded away.  The decay sits inside the K reduction, so the scaled operands cannot be the exact
// bf16 inputs: kda_prep_kernel (parallel over chunks) builds them once as bf16 hi + residual operand panels,
// computes both score tiles on tcgen05 and the inverse on CUDA cores, and stores everything as ready-to-load
// panel images; kda_fwd_kernel (sequential over chunks, fp32 state in TMEM) only bulk-loads them.
#include "gdn_common.cuh"
#include "fla_b200_internal.h"
#include "kernel_timer.h"
#include "tri_inverse.h"
#include "kda_common.cuh"
#include "tensor_map.h"

namespace fla {

// --------------------------------------------------------------------------------------------- prep
constexpr uint32_t pOffQKH = 0, pOffQKL = 32768, pOffKNH = 65536, pOffKNL = 81920;
constexpr uint32_t kKdaPrepSmem = 98304;           // operand panels only

__device__ __forceinline__ float kda_gate(float g, int mode, float eig, float bias, float lower_bound) {
  if (mode == 0) return g;
  const float raw = g + bias;
  if (mode == 1) {  // -exp(A_log) * softplus(g + dt_bias)
    const float sp = raw > 20.f ? raw : log1pf(__expf(raw));
    return -eig * sp;
  }
  return lower_bound / (1.f + __expf(-eig * raw));  // lower_bound * sigmoid(exp(A_log) (g + dt_bias))
}

// Thread layout of the elementwise phases: 16 channel groups (8 channels each) x 16 token segments (4 tokens each).
// The raw q and k rows arrive as TMA tiles in the residual panels (where each thread later overwrites exactly the
// 16-byte pieces it read), so their latency is hidden behind the gate phases.
__global__ void __launch_bounds__(256, 2) kda_prep_kernel(KdaParams p, const __grid_constant__ CUtensorMap tm_q,
                                                          const __grid_constant__ CUtensorMap tm_k) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ float tot_s[16][kK];          // gate sum of each token segment, per channel
  __shared__ float anchor_s[kK], last_s[kK];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t bar, qk_bar;

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int hv = blockIdx.y, n = blockIdx.z;
  const int hk = hv / (p.HV / p.HK);
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  const int c = blockIdx.x;
  if (c >= sq.nt) return;
  const int t0 = c * kC;
  const int rows = min(kC, sq.len - t0);
  const int64_t tok0 = int64_t(sq.bos) + t0;
  const int64_t cidx = (int64_t(sq.cbase) + c) * p.HV + hv;
  const int cg = tid & 15, seg = tid >> 4, r0 = cg * 8;

  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 64);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(&bar, 1);
    mbar_init(&qk_bar, 1);
    mbar_init_fence();
    const uint32_t sbq = smem_u32(smem);
    const int row0 = int(tok0);
    mbar_arrive_expect_tx(&qk_bar, 4 * 8192);
    tma_load_tile(sbq + pOffQKL, &tm_q, 0, hk, row0, &qk_bar);                  // q rows -> rows 0-63 of the lo panels
    tma_load_tile(sbq + pOffQKL + 16384, &tm_q, 64, hk, row0, &qk_bar);
    tma_load_tile(sbq + pOffQKL + 8192, &tm_k, 0, hk, row0, &qk_bar);           // k rows -> rows 64-127
    tma_load_tile(sbq + pOffQKL + 16384 + 8192, &tm_k, 64, hk, row0, &qk_bar);
  }
  // 1. activated gates of my 4 tokens x 8 channels, prefix-summed inside the segment (zero past the sequence end)
  float gk[4][8];
  {
    const float eig = (p.gate_mode && p.a_log) ? __expf(p.a_log[hv]) : 1.f;
    float bias[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) bias[j] = (p.gate_mode && p.dt_bias) ? p.dt_bias[hv * kK + r0 + j] : 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = seg * 4 + i;
      float raw[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) raw[j] = 0.f;
      if (t < rows) {
        const int64_t off = (tok0 + t) * p.g_st + hv * p.g_sh + r0;
        if (p.g_is_f32) {
          const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(p.g) + off);
          const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(p.g) + off + 4);
          raw[0] = a.x; raw[1] = a.y; raw[2] = a.z; raw[3] = a.w; raw[4] = b.x; raw[5] = b.y; raw[6] = b.z; raw[7] = b.w;
        } else {
          unpack_bf16x8(*reinterpret_cast<const uint4*>(static_cast<const bf16*>(p.g) + off), raw);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gv = t < rows ? kda_gate(raw[j], p.gate_mode, eig, bias[j], p.lower_bound) : 0.f;
        gk[i][j] = gv + (i ? gk[i - 1][j] : 0.f);
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) tot_s[seg][r0 + j] = gk[3][j];
  }
  __syncthreads();
  // 2. add the totals of the earlier segments; publish the anchor row (middle token) and the last valid row
  {
    float off[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) off[j] = 0.f;
    for (int sgm = 0; sgm < seg; ++sgm) {
#pragma unroll
      for (int j = 0; j < 8; ++j) off[j] += tot_s[sgm][r0 + j];
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) gk[i][j] += off[j];
    const int ta = min(kC / 2 - 1, rows - 1), tl = rows - 1;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = seg * 4 + i;
      if (t == ta) {
#pragma unroll
        for (int j = 0; j < 8; ++j) anchor_s[r0 + j] = gk[i][j];
      }
      if (t == tl) {
#pragma unroll
        for (int j = 0; j < 8; ++j) last_s[r0 + j] = gk[i][j];
      }
    }
  }
  __syncthreads();
  if (tid < kK) {
    const float a = anchor_s[tid];
    p.vec[cidx * kKdaVecs * kK + tid] = __expf(a);
    p.vec[cidx * kKdaVecs * kK + kK + tid] = __expf(last_s[tid] - a);
    p.vec[cidx * kKdaVecs * kK + 2 * kK + tid] = a;
  }
  // 3. scaled operands as split bf16 panels
  {
    float an[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) an[j] = anchor_s[r0 + j];
    const uint32_t pan = (cg / 8) * 16384, pan64 = (cg / 8) * 8192;
    const bool landed = mbar_wait(&qk_bar, 0, p.status, FLA_ERR_TIMEOUT);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = seg * 4 + i;
      float qv[8], kv[8], qp[8], kp[8], kn[8];
      uint4 qraw = make_uint4(0, 0, 0, 0), kraw = qraw;
      if (t < rows && landed) {   // rows past the end of the sequence hold foreign tokens in the tile: use zeros
        qraw = *reinterpret_cast<const uint4*>(smem + pOffQKL + pan + panel_chunk_off(t, cg % 8));
        kraw = *reinterpret_cast<const uint4*>(smem + pOffQKL + pan + panel_chunk_off(64 + t, cg % 8));
      }
      unpack_bf16x8(qraw, qv);
      unpack_bf16x8(kraw, kv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = gk[i][j] - an[j];
        const float e1 = __expf(d), e2 = __expf(-d);
        qp[j] = qv[j] * e1; kp[j] = kv[j] * e1; kn[j] = kv[j] * e2;
      }
      if (p.gk_out && t < rows) {
        float* dst = p.gk_out + ((tok0 + t) * p.HV + hv) * kK + r0;
        *reinterpret_cast<float4*>(dst) = make_float4(gk[i][0], gk[i][1], gk[i][2], gk[i][3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(gk[i][4], gk[i][5], gk[i][6], gk[i][7]);
      }
      uint4 hi, lo;
      const uint32_t o1 = panel_chunk_off(t, cg % 8), o2 = panel_chunk_off(64 + t, cg % 8);
      split8(qp, hi, lo);
      *reinterpret_cast<uint4*>(smem + pOffQKH + pan + o1) = hi;
      *reinterpret_cast<uint4*>(smem + pOffQKL + pan + o1) = lo;
      split8(kp, hi, lo);
      *reinterpret_cast<uint4*>(smem + pOffQKH + pan + o2) = hi;
      *reinterpret_cast<uint4*>(smem + pOffQKL + pan + o2) = lo;
      split8(kn, hi, lo);
      *reinterpret_cast<uint4*>(smem + pOffKNH + pan64 + o1) = hi;
      *reinterpret_cast<uint4*>(smem + pOffKNL + pan64 + o1) = lo;
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = tmem_base_s;
  const uint32_t sb = smem_u32(smem);
  // 4. save the operand images; both score tiles in one M = 128 product: rows 0-63 Qp Kn^T, rows 64-127 Kp Kn^T
  if (tid == 0) {
    bulk_store(p.qk_img + cidx * kKdaQkImg, sb + pOffQKH, 65536);
    bulk_store(p.kn_img + cidx * kKdaKnImg, sb + pOffKNH, 32768);
    bulk_commit();
    const Operand aH{sb + pOffQKH, 16384, 0}, aL{sb + pOffQKL, 16384, 0};
    const Operand bH{sb + pOffKNH, 8192, 0}, bL{sb + pOffKNL, 8192, 0};
    mma_tile(tbase, aH, bH, 128, 64, 8, false);
    mma_tile(tbase, aH, bL, 128, 64, 8, true);
    mma_tile(tbase, aL, bH, 128, 64, 8, true);
    mma_commit(&bar);
  }
  // 5. q-side rows: P = tril(Aqk) written straight into its split panel image;
  //    k-side rows: Akk^T = (beta_i Kp Kn^T)^T for the inverse kernel (coalesced along i)
  const int quad = warp & 3, half = warp >> 2, row = quad * 32 + lane, tok = row & 63;
  // requested before the product is waited for
  const float bi = (quad >= 2 && tok < rows) ? ld_scalar(p.beta, (tok0 + tok) * p.beta_st + hv, p.beta_is_f32) : 0.f;
  const bool ok = mbar_wait(&bar, 0, p.status, FLA_ERR_TIMEOUT);
  tc_fence_after();
  if (ok) {
    float sc[32];
    tmem_ld32(tmem_addr(tbase, quad * 32, half * 32), sc);
    tmem_ld_wait();
    if (quad < 2) {
#pragma unroll
      for (int jj = 0; jj < 32; ++jj) sc[jj] = (half * 32 + jj <= tok) ? sc[jj] : 0.f;   // select: masked entries may be inf
      uint8_t* img = reinterpret_cast<uint8_t*>(p.p_img + cidx * kKdaPImg);
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint4 hi, lo;
        split8(sc + ch * 8, hi, lo);
        const uint32_t off = panel_chunk_off(tok, half * 4 + ch);
        *reinterpret_cast<uint4*>(img + off) = hi;
        *reinterpret_cast<uint4*>(img + 8192 + off) = lo;
      }
    } else {
      float* at = p.at + cidx * (kC * kC);
#pragma unroll
      for (int jj = 0; jj < 32; ++jj) {
        const int j = half * 32 + jj;
        if (j < tok) at[j * kC + tok] = bi * sc[jj];
      }
    }
  }
  if (tid == 0) bulk_wait_all();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 64);
}

// --------------------------------------------------------------------------------------------- forward
constexpr uint32_t fOffQKH = 0, fOffQKL = 32768, fOffKNH = 65536, fOffKNL = 81920;
constexpr uint32_t fOffPH = 98304, fOffPL = 106496, fOffX = 114688, fOffXL = 122880;
constexpr uint32_t fOffSH = 131072, fOffSL = 147456, fOffZH = 163840, fOffZL = 172032;
constexpr uint32_t kKdaFwdSmem = 180224;
constexpr uint32_t fColS = 0, fColRQ = 64, fColPV = 128, fColVN = 192;

__global__ void __launch_bounds__(256, 1) kda_fwd_kernel(KdaParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ float vec_s[2][2][kK];     // [chunk parity][e^a | e^{gk_L - a}][channel]
  __shared__ float beta_s[2][kC];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t mma_bar, load1_bar, load2_bar;

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int vb = blockIdx.x, hv = blockIdx.y, n = blockIdx.z;
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  const int quad = warp & 3, half = warp >> 2;
  const bool kside = quad >= 2;
  const int row = quad * 32 + lane, tok = row & 63, c0 = half * 32;

  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 256);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(&mma_bar, 1);
    mbar_init(&load1_bar, 1);
    mbar_init(&load2_bar, 1);
    mbar_init_fence();
  }
  __syncthreads();
  const uint32_t tbase = tmem_base_s;
  const uint32_t trow = tmem_addr(tbase, quad * 32, c0);
  const uint32_t sb = smem_u32(smem);
  uint32_t mphase = 0, l1phase = 0, l2phase = 0;
  bool dead = false;

  auto issue_load1 = [&](int c) {   // [Qp; Kp] hi + lo
    const int64_t cidx = (int64_t(sq.cbase) + c) * p.HV + hv;
    mbar_arrive_expect_tx(&load1_bar, 65536);
    bulk_load(sb + fOffQKH, p.qk_img + cidx * kKdaQkImg, 65536, &load1_bar);
  };
  auto issue_load2 = [&](int c) {   // Kn hi + lo, P hi + lo, X
    const int64_t cidx = (int64_t(sq.cbase) + c) * p.HV + hv;
    mbar_arrive_expect_tx(&load2_bar, 32768 + 16384 + 16384);
    bulk_load(sb + fOffKNH, p.kn_img + cidx * kKdaKnImg, 32768, &load2_bar);
    bulk_load(sb + fOffPH, p.p_img + cidx * kKdaPImg, 16384, &load2_bar);
    bulk_load(sb + fOffX, p.x_img + cidx * kKdaXImg, 16384, &load2_bar);
  };
  if (tid == 0 && sq.nt > 0) {   // a sequence without tokens requests nothing: its final state is its initial state
    issue_load1(0);
    issue_load2(0);
  }

  const Operand opQKH{sb + fOffQKH, 16384, 0}, opQKL{sb + fOffQKL, 16384, 0};
  const Operand opKNTh{sb + fOffKNH, 8192, 1}, opKNTl{sb + fOffKNL, 8192, 1};   // Kn^T: M = 128 key dims
  const Operand opSH{sb + fOffSH, 16384, 1}, opSL{sb + fOffSL, 16384, 1};
  const Operand opZH{sb + fOffZH, 8192, 1}, opZL{sb + fOffZL, 8192, 1};
  const Operand opX{sb + fOffX - 8192, 16384, 0};               // rows 64..127 of this tile are X
  const Operand opXL{sb + fOffXL - 8192, 16384, 0};             // ... and of this one its bf16 residual
  const Operand opPH{sb + fOffPH, 16384, 0}, opPL{sb + fOffPL, 16384, 0};       // rows 0..63 are P

  // per-chunk scalars / vectors / value rows are staged through registers one chunk ahead
  float pf_vec = 0.f, pf_beta = 0.f;
  uint4 pf_v[4], vcur[4];
  auto prefetch_load = [&](int c) {
    const int t0 = c * kC;
    const int rows = min(kC, sq.len - t0);
    const int64_t tok0 = int64_t(sq.bos) + t0;
    const int64_t cidx = (int64_t(sq.cbase) + c) * p.HV + hv;
    pf_vec = p.vec[cidx * kKdaVecs * kK + tid];                       // 256 threads: e^a then e^{gk_L - a}
    if (kside) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        pf_v[i] = make_uint4(0, 0, 0, 0);
        if (tok < rows) pf_v[i] = *reinterpret_cast<const uint4*>(p.v + (tok0 + tok) * p.v_st + hv * p.v_sh + vb * kBV + c0 + i * 8);
      }
      pf_beta = tok < rows ? ld_scalar(p.beta, (tok0 + tok) * p.beta_st + hv, p.beta_is_f32) : 0.f;
    }
  };
  auto store_scalars = [&](int c) {   // double-buffered by chunk parity: safe to write while chunk c-1 is in flight
    vec_s[c & 1][tid / kK][tid % kK] = pf_vec;
    if (kside && half == 0) beta_s[c & 1][tok] = pf_beta;
  };
  auto take_values = [&]() {
#pragma unroll
    for (int i = 0; i < 4; ++i) vcur[i] = pf_v[i];
  };

  float srow[32];
  if (sq.nt > 0) {
    prefetch_load(0);
    store_scalars(0);
    take_values();
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
  __syncthreads();

  for (int c = 0; c < sq.nt; ++c) {
    const int cur = c & 1;
    const int t0 = c * kC;
    const int rows = min(kC, sq.len - t0);
    const int64_t tok0 = int64_t(sq.bos) + t0;

    // ---- stage 0: Sa = diag(e^a) S as split copy and as the fp32 master in TMEM
    {
      const float ea = vec_s[cur][0][row];
#pragma unroll
      for (int i = 0; i < 32; ++i) srow[i] *= ea;
      row32_to_hilo(smem + fOffSH, smem + fOffSL, row, half, srow);
      tmem_st16(trow + fColS, srow);
      tmem_st16(trow + fColS + 16, srow + 16);
      tmem_st_wait();
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    // ---- stage 1: [Qp; Kp] Sa
    if (!dead && !mbar_wait(&load1_bar, l1phase, p.status, FLA_ERR_TIMEOUT)) dead = true;
    l1phase ^= 1;
    if (tid == 0) {
      if (p.s_img) {
        const int64_t cidx = (int64_t(sq.cbase) + c) * p.HV + hv;
        bulk_store(p.s_img + (cidx * p.nvb + vb) * 16384, sb + fOffSH, 32768);
        bulk_commit();
      }
      mma_tile(tbase + fColRQ, opQKH, opSH, 128, 64, 8, false);
      mma_tile(tbase + fColRQ, opQKH, opSL, 128, 64, 8, true);
      mma_tile(tbase + fColRQ, opQKL, opSH, 128, 64, 8, true);
      mma_commit(&mma_bar);
    }
    if (c + 1 < sq.nt) {
      prefetch_load(c + 1);
      store_scalars(c + 1);
    }
    if (!dead && !mbar_wait(&mma_bar, mphase, p.status, FLA_ERR_TIMEOUT)) dead = true;
    mphase ^= 1;
    tc_fence_after();
    if (tid == 0 && c + 1 < sq.nt) issue_load1(c + 1);   // the [Qp; Kp] buffers are free again

    // ---- stage 2: k-side rows: Z = beta (V - Kp Sa)
    float acc[32];
    if (kside) {
      tmem_ld32(trow + fColRQ, acc);
      tmem_ld_wait();
      const float bi = beta_s[cur][tok];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float vv[8];
        unpack_bf16x8(vcur[i], vv);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i * 8 + j] = bi * (vv[j] - acc[i * 8 + j]);
      }
      row32_to_hilo(smem + fOffZH, smem + fOffZL, tok, half, acc);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    // ---- stage 3: v_new = X Z
    if (!dead && !mbar_wait(&load2_bar, l2phase, p.status, FLA_ERR_TIMEOUT)) dead = true;
    l2phase ^= 1;
    if (tid == 0) {
      mma_tile(tbase + fColVN, opX, opZH, 128, 64, 4, false);
      mma_tile(tbase + fColVN, opX, opZL, 128, 64, 4, true);
      mma_tile(tbase + fColVN, opXL, opZH, 128, 64, 4, true);
      mma_commit(&mma_bar);
    }
    if (!dead && !mbar_wait(&mma_bar, mphase, p.status, FLA_ERR_TIMEOUT)) dead = true;
    mphase ^= 1;
    tc_fence_after();

    // ---- stage 4: k-side rows publish v_new
    if (kside) {
      tmem_ld32(trow + fColVN, acc);
      tmem_ld_wait();
      row32_to_hilo(smem + fOffZH, smem + fOffZL, tok, half, acc);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    // ---- stage 5: Aqk v_new and the state update Sa += Kn^T v_new
    if (tid == 0) {
      if (p.vn_img) {
        const int64_t cidx = (int64_t(sq.cbase) + c) * p.HV + hv;
        bulk_store(p.vn_img + (cidx * p.nvb + vb) * 8192, sb + fOffZH, 16384);
        bulk_commit();
      }
      mma_tile(tbase + fColPV, opPH, opZH, 128, 64, 4, false);
      mma_tile(tbase + fColPV, opPH, opZL, 128, 64, 4, true);
      mma_tile(tbase + fColPV, opPL, opZH, 128, 64, 4, true);
      mma_tile(tbase + fColS, opKNTh, opZH, 128, 64, 4, true);
      mma_tile(tbase + fColS, opKNTh, opZL, 128, 64, 4, true);
      mma_tile(tbase + fColS, opKNTl, opZH, 128, 64, 4, true);
      mma_commit(&mma_bar);
    }
    if (!dead && !mbar_wait(&mma_bar, mphase, p.status, FLA_ERR_TIMEOUT)) dead = true;
    mphase ^= 1;
    tc_fence_after();
    if (tid == 0 && c + 1 < sq.nt) issue_load2(c + 1);
    if (p.s_img || p.vn_img) {   // the saved images must have left the S / v_new panels before they are rewritten
      if (tid == 0) bulk_wait_read();
      __syncthreads();
    }

    // ---- stage 6: output rows; next state S = diag(e^{gk_L - a}) (Sa + Kn^T v_new)
    if (!kside) {
      float qs[32];
      tmem_ld32(trow + fColRQ, qs);
      tmem_ld32(trow + fColPV, acc);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = p.scale * (qs[i] + acc[i]);
      if (tok < rows && p.o) {
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
    tmem_ld32(trow + fColS, srow);
    tmem_ld_wait();
    {
      const float el = vec_s[cur][1][row];
#pragma unroll
      for (int i = 0; i < 32; ++i) srow[i] *= el;
    }
    if (c + 1 < sq.nt) take_values();
  }

  if (!dead && p.ht) {
    float* dst = p.ht + ((int64_t(n) * p.HV + hv) * kK + row) * p.V + vb * kBV + c0;
#pragma unroll
    for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(srow[i], srow[i + 1], srow[i + 2], srow[i + 3]);
  }
  if (tid == 0) bulk_wait_all();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 256);
}

// The two 64 x 64 score blocks of every chunk as plain tensors, for callers of the reference's low-level forward
// (npu_chunk_kda_fwd returns them): Aqk = scale tril(q k^T 2^{gk_i - gk_j}) from the P image and Akk = the chunk inverse
// from the X image (value + residual panels summed), rows and columns past a short chunk as zeros.
struct KdaExportParams {
  const bf16* img[2];
  void* out[2];
  int is_f32[2];
  int64_t sb[2], st[2], sh[2];
  const int32_t* cu_seqlens;
  const int32_t* chunk_offsets;
  int T, HV;
  float scale;
};
__global__ void __launch_bounds__(128) kda_export_scores_kernel(KdaExportParams p) {
  const int n = blockIdx.z, hv = blockIdx.y, c = blockIdx.x;
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  if (c >= sq.nt) return;
  const int rows = min(kC, sq.len - c * kC);
  const int64_t b = p.cu_seqlens ? 0 : n;
  const int64_t t0 = (p.cu_seqlens ? sq.bos : 0) + c * kC;
  const int64_t cidx = (int64_t(sq.cbase) + c) * p.HV + hv;
  for (int which = 0; which < 2; ++which) {
    if (!p.out[which]) continue;
    const uint8_t* hi = reinterpret_cast<const uint8_t*>(p.img[which] + cidx * 8192);
    const uint8_t* lo = hi + 8192;
    const float f = which ? 1.f : p.scale;
    for (int idx = threadIdx.x; idx < kC * 8; idx += 128) {
      const int r = idx >> 3, ch = idx & 7;
      if (r >= rows) continue;
      float a[8], l[8];
      unpack_bf16x8(*reinterpret_cast<const uint4*>(hi + panel_chunk_off(r, ch)), a);
      unpack_bf16x8(*reinterpret_cast<const uint4*>(lo + panel_chunk_off(r, ch)), l);
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = (ch * 8 + j < rows && ch * 8 + j <= r) ? f * (a[j] + l[j]) : 0.f;
      const int64_t off = b * p.sb[which] + (t0 + r) * p.st[which] + hv * p.sh[which] + ch * 8;
      if (p.is_f32[which]) {
        float* dst = static_cast<float*>(p.out[which]) + off;
        *reinterpret_cast<float4*>(dst) = make_float4(a[0], a[1], a[2], a[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(a[4], a[5], a[6], a[7]);
      } else {
        *reinterpret_cast<uint4*>(static_cast<bf16*>(p.out[which]) + off) = pack8(a);
      }
    }
  }
}

}  // namespace fla

using namespace fla;

uint64_t fla::kda_ws_layout(int64_t total_chunks, int64_t HV, uint64_t off[6]) {
  uint64_t o = 256;
  const uint64_t per = uint64_t(total_chunks) * HV;
  off[0] = o; o += align_up(per * kKdaQkImg * 2, 256);
  off[1] = o; o += align_up(per * kKdaKnImg * 2, 256);
  off[2] = o; o += align_up(per * kKdaPImg * 2, 256);
  off[3] = o; o += align_up(per * kKdaXImg * 2, 256);
  off[4] = o; o += align_up(per * kKdaVecs * kK * 4, 256);
  off[5] = o; o += align_up(per * kC * kC * 4, 256);
  return o;
}

uint64_t fla::kda_saved_layout(int64_t total_chunks, int64_t HV, int64_t nvb, int64_t tokens, uint64_t off[4]) {
  uint64_t fo[6];
  const uint64_t per = uint64_t(total_chunks) * HV;
  uint64_t o = 0;
  off[0] = o; o += align_up(kda_ws_layout(total_chunks, HV, fo), 256);
  off[1] = o; o += align_up(uint64_t(tokens) * HV * kK * 4, 256);
  off[2] = o; o += align_up(per * nvb * kKdaSImg * 2, 256);
  off[3] = o; o += align_up(per * nvb * kKdaVnImg * 2, 256);
  return o;
}

static int kda_geometry(const fla_kda_chunk_fwd_args* a, int64_t* total_chunks, int* N, int* max_len) {
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

extern "C" FLA_API int fla_b200_kda_chunk_fwd_workspace_size(const fla_kda_chunk_fwd_args* a, uint64_t* bytes) {
  if (!a || !bytes) return FLA_ERR_NULL;
  int64_t total_chunks; int N, max_len;
  const int st = kda_geometry(a, &total_chunks, &N, &max_len);
  if (st) return st;
  uint64_t off[6];
  *bytes = a->saved.data ? 256 : kda_ws_layout(total_chunks, a->v.shape[2], off);
  return FLA_OK;
}

extern "C" FLA_API int fla_b200_kda_chunk_saved_size(const fla_kda_chunk_fwd_args* a, uint64_t* bytes) {
  if (!a || !bytes) return FLA_ERR_NULL;
  int64_t total_chunks; int N, max_len;
  const int st = kda_geometry(a, &total_chunks, &N, &max_len);
  if (st) return st;
  uint64_t off[4];
  const int64_t V = a->v.shape[3];
  if (V != kV && V != 2 * kV) return FLA_ERR_SHAPE;
  *bytes = kda_saved_layout(total_chunks, a->v.shape[2], V / kBV, a->q.shape[0] * a->q.shape[1], off);
  return FLA_OK;
}

static int kda_check_tok(const fla_tensor_t& t, int64_t B, int64_t T, int64_t heads, int64_t dim, bool allow_f32) {
  if (!t.data) return FLA_ERR_NULL;
  if (t.ndim != 4 || t.shape[0] != B || t.shape[1] != T || t.shape[2] != heads || t.shape[3] != dim) return FLA_ERR_SHAPE;
  if (t.dtype != FLA_BF16 && !(allow_f32 && t.dtype == FLA_F32)) return FLA_ERR_DTYPE;
  const int64_t esz = t.dtype == FLA_F32 ? 4 : 2;
  if (t.stride[3] != 1 || (t.stride[2] * esz) % 16 || (t.stride[1] * esz) % 16 || !aligned16(t.data)) return FLA_ERR_LAYOUT;
  if (B > 1 && t.stride[0] != T * t.stride[1]) return FLA_ERR_LAYOUT;
  return FLA_OK;
}

extern "C" FLA_API int fla_b200_kda_chunk_fwd(const fla_kda_chunk_fwd_args* a, void* workspace, uint64_t workspace_bytes,
                                              void* stream) {
  if (!a) return FLA_ERR_NULL;
  int64_t total_chunks; int N, max_len;
  int st = kda_geometry(a, &total_chunks, &N, &max_len);
  if (st) return st;
  const int64_t B = a->q.shape[0], T = a->q.shape[1], HK = a->q.shape[2], HV = a->v.shape[2];
  if (HK <= 0 || HV <= 0 || HV % HK) return FLA_ERR_SHAPE;
  const int64_t V = a->v.shape[3];
  if (V != kV && V != 2 * kV) return FLA_ERR_SHAPE;
  if ((st = kda_check_tok(a->q, B, T, HK, kK, false))) return st;
  if ((st = kda_check_tok(a->k, B, T, HK, kK, false))) return st;
  if ((st = kda_check_tok(a->v, B, T, HV, V, false))) return st;
  if ((st = kda_check_tok(a->g, B, T, HV, kK, true))) return st;
  if ((st = kda_check_tok(a->o, B, T, HV, V, true))) return st;
  const fla_tensor_t& be = a->beta;
  if (!be.data) return FLA_ERR_NULL;
  if (be.ndim != 3 || be.shape[0] != B || be.shape[1] != T || be.shape[2] != HV || be.stride[2] != 1 ||
      (B > 1 && be.stride[0] != T * be.stride[1]))
    return FLA_ERR_SHAPE;
  if (be.dtype != FLA_F32 && be.dtype != FLA_BF16) return FLA_ERR_DTYPE;
  for (const fla_tensor_t* s : {&a->initial_state, &a->final_state}) {
    if (!s->data) continue;
    if (s->dtype != FLA_F32) return FLA_ERR_DTYPE;
    if (s->ndim != 4 || s->shape[0] != N || s->shape[1] != HV || s->shape[2] != kK || s->shape[3] != V) return FLA_ERR_SHAPE;
    if (s->stride[3] != 1 || s->stride[2] != V || s->stride[1] != kK * V || s->stride[0] != HV * kK * V || !aligned16(s->data))
      return FLA_ERR_LAYOUT;
  }
  if (a->gate_mode < 0 || a->gate_mode > 2) return FLA_ERR_VALUE;
  if (a->gate_mode) {
    if (!a->a_log.data || a->a_log.dtype != FLA_F32 || a->a_log.ndim != 1 || a->a_log.shape[0] != HV || a->a_log.stride[0] != 1)
      return FLA_ERR_SHAPE;
    if (a->dt_bias.data && (a->dt_bias.dtype != FLA_F32 || a->dt_bias.ndim != 2 || a->dt_bias.shape[0] != HV ||
                            a->dt_bias.shape[1] != kK || a->dt_bias.stride[1] != 1 || a->dt_bias.stride[0] != kK))
      return FLA_ERR_SHAPE;
  }
  if (a->gk.data) {
    const fla_tensor_t& gk = a->gk;
    if (gk.dtype != FLA_F32 || gk.ndim != 4 || gk.shape[0] != B || gk.shape[1] != T || gk.shape[2] != HV || gk.shape[3] != kK ||
        gk.stride[3] != 1 || gk.stride[2] != kK || gk.stride[1] != HV * kK || (B > 1 && gk.stride[0] != T * HV * kK))
      return FLA_ERR_SHAPE;
  }
  if (a->chunk_size != kC) return FLA_ERR_VALUE;
  uint64_t off[6];
  uint64_t need = kda_ws_layout(total_chunks, HV, off);
  uint8_t* images = static_cast<uint8_t*>(workspace);   // where the operand images go
  uint64_t soff[4] = {0, 0, 0, 0};
  if (a->saved.data) {
    const uint64_t sbytes = kda_saved_layout(total_chunks, HV, V / kBV, B * T, soff);
    if (a->saved.dtype != FLA_BF16 || a->saved.ndim != 1 || uint64_t(a->saved.shape[0]) * 2 < sbytes || !aligned16(a->saved.data))
      return FLA_ERR_SHAPE;
    if (a->gate_mode != 0 || a->gk.data) return FLA_ERR_VALUE;
    images = static_cast<uint8_t*>(a->saved.data) + soff[0];
    need = 256;
  }
  if (!workspace || workspace_bytes < need || !aligned16(workspace)) return FLA_ERR_WORKSPACE;

  KdaParams p{};
  p.q = static_cast<const bf16*>(a->q.data); p.k = static_cast<const bf16*>(a->k.data); p.v = static_cast<const bf16*>(a->v.data);
  p.g = a->g.data; p.beta = be.data;
  p.a_log = static_cast<const float*>(a->a_log.data); p.dt_bias = static_cast<const float*>(a->dt_bias.data);
  p.gk_out = static_cast<float*>(a->gk.data);
  uint8_t* ws = images;
  p.status = reinterpret_cast<int*>(workspace);
  if (a->saved.data) {
    uint8_t* sv = static_cast<uint8_t*>(a->saved.data);
    p.gk_out = reinterpret_cast<float*>(sv + soff[1]);
    p.s_img = reinterpret_cast<bf16*>(sv + soff[2]);
    p.vn_img = reinterpret_cast<bf16*>(sv + soff[3]);
  }
  p.qk_img = reinterpret_cast<bf16*>(ws + off[0]); p.kn_img = reinterpret_cast<bf16*>(ws + off[1]);
  p.p_img = reinterpret_cast<bf16*>(ws + off[2]); p.x_img = reinterpret_cast<bf16*>(ws + off[3]);
  p.vec = reinterpret_cast<float*>(ws + off[4]);
  p.at = reinterpret_cast<float*>(ws + off[5]);
  p.h0 = static_cast<const float*>(a->initial_state.data); p.ht = static_cast<float*>(a->final_state.data);
  p.o = a->o.data;
  p.cu_seqlens = static_cast<const int32_t*>(a->cu_seqlens.data);
  p.chunk_offsets = static_cast<const int32_t*>(a->chunk_offsets.data);
  p.q_st = a->q.stride[1]; p.q_sh = a->q.stride[2]; p.k_st = a->k.stride[1]; p.k_sh = a->k.stride[2];
  p.v_st = a->v.stride[1]; p.v_sh = a->v.stride[2]; p.o_st = a->o.stride[1]; p.o_sh = a->o.stride[2];
  p.g_st = a->g.stride[1]; p.g_sh = a->g.stride[2]; p.beta_st = be.stride[1];
  p.N = N; p.T = int(T); p.HK = int(HK); p.HV = int(HV); p.total_tokens = B * T; p.V = int(V); p.nvb = int(V / kBV);
  p.g_is_f32 = a->g.dtype == FLA_F32; p.beta_is_f32 = be.dtype == FLA_F32; p.o_is_f32 = a->o.dtype == FLA_F32;
  p.gate_mode = a->gate_mode; p.scale = a->scale; p.lower_bound = a->lower_bound;

  KdaExportParams ep{};
  for (int which = 0; which < 2; ++which) {
    const fla_tensor_t& t = which ? a->akk : a->aqk;
    if (!t.data) continue;
    if (t.ndim != 4 || t.shape[0] != B || t.shape[1] != T || t.shape[2] != HV || t.shape[3] != kC) return FLA_ERR_SHAPE;
    if (t.dtype != FLA_BF16 && t.dtype != FLA_F32) return FLA_ERR_DTYPE;
    if (t.stride[3] != 1 || !aligned16(t.data) || (t.stride[0] % 8) || (t.stride[1] % 8) || (t.stride[2] % 8)) return FLA_ERR_LAYOUT;
    ep.out[which] = t.data; ep.is_f32[which] = t.dtype == FLA_F32;
    ep.sb[which] = t.stride[0]; ep.st[which] = t.stride[1]; ep.sh[which] = t.stride[2];
  }

  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(workspace, 0, 256, cs) != cudaSuccess) return FLA_ERR_CUDA;
  const int nt_max = (max_len + kC - 1) / kC;
  st = kda_launch_forward(p, nt_max, cs);
  if (st || (!ep.out[0] && !ep.out[1])) return st;
  ep.img[0] = p.p_img; ep.img[1] = p.x_img;
  ep.cu_seqlens = p.cu_seqlens; ep.chunk_offsets = p.chunk_offsets; ep.T = p.T; ep.HV = p.HV; ep.scale = p.scale;
  KernelTimer kt("kda_export_scores", cs);
  kda_export_scores_kernel<<<dim3(nt_max, unsigned(p.HV), p.N), 128, 0, cs>>>(ep);
  return cuda_status(cudaGetLastError());
}

int fla::kda_launch_forward(const KdaParams& p, int nt_max, cudaStream_t cs) {
  static std::atomic<bool> attr_done_dev[64] = {};   // per device ordinal; setting the attributes twice is harmless
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FLA_ERR_CUDA;
  if (!attr_done_dev[dev]) {
    if (cudaFuncSetAttribute(kda_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kKdaPrepSmem) + 1024) != cudaSuccess) return FLA_ERR_CUDA;
    if (cudaFuncSetAttribute(kda_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kKdaFwdSmem) + 1024) != cudaSuccess) return FLA_ERR_CUDA;
    attr_done_dev[dev] = true;
  }
  CUtensorMap tm_q, tm_k;
  if (make_row_tile_map(&tm_q, p.q, kK, uint64_t(p.HK), uint64_t(p.total_tokens), uint64_t(p.q_sh), uint64_t(p.q_st)) ||
      make_row_tile_map(&tm_k, p.k, kK, uint64_t(p.HK), uint64_t(p.total_tokens), uint64_t(p.k_sh), uint64_t(p.k_st)))
    return FLA_ERR_CUDA;
  {
    KernelTimer kt("kda_prep", cs);
    kda_prep_kernel<<<dim3(nt_max, unsigned(p.HV), p.N), 256, kKdaPrepSmem + 1024, cs>>>(p, tm_q, tm_k);
  }
  if (cudaGetLastError() != cudaSuccess) return FLA_ERR_CUDA;
  {
    KernelTimer kt("tri_inverse", cs);
    TriInverseParams tp{p.at, nullptr, nullptr, p.x_img, p.x_img + kC * kC, p.cu_seqlens, p.chunk_offsets, p.T, p.HV, int(kKdaXImg)};
    if (launch_tri_inverse(tp, nt_max, p.N, cs)) return FLA_ERR_CUDA;
  }
  {
    KernelTimer kt("kda_fwd", cs);
    kda_fwd_kernel<<<dim3(unsigned(p.nvb), unsigned(p.HV), p.N), 256, kKdaFwdSmem + 1024, cs>>>(p);
  }
  return cuda_status(cudaGetLastError());
}

// Chunked Kimi-Delta-Attention backward (per-channel log gate, chunk = 64, K = V = 128).
//
// The reference ships only the intra-chunk piece of this backward (chunk_kda_bwd_intra,
// torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:1534-1783) and defers the rest to a third-party
// package; the gradients here are those of the recurrence itself
// (tests/atk/recurrent_kda/executor_recurrent_kda.py:63-83), derived for the anchored chunk form of the forward:
//   gk = chunk cumsum(g), a = gk at the middle token, Qp = Q e^{gk-a}, Kp = K e^{gk-a}, Kn = K e^{a-gk},
//   P = tril(Qp Kn^T), M = strict_tril(Kp Kn^T), X = (I + beta M)^-1, Sa = diag(e^a) S, D = e^{gk_L-a}:
//   Vn = X (beta (V - Kp Sa)),  O = scale (Qp Sa + P Vn),  S' = diag(D) (Sa + Kn^T Vn).
// The entry point recomputes the forward (prep -> inverse -> forward scan, saving Sa and Vn as panel images) and runs
//
//  kda_bwd_dhu_kernel  (reverse-sequential over chunks, one CTA per (sequence, value head, 64-column block of V)):
//      dS'a = diag(D) dS'          dVn = scale P^T dO + Kn dS'a          dZ = X^T dVn          dV = beta dZ
//      dSa  = dS'a + Qp^T (scale dO) + Kp^T (-beta dZ)                   dS = diag(e^a) dSa    dh0 = dS after the first chunk
//  kda_bwd_par_kernel  (parallel over chunks, one CTA per (chunk, q/k head), looping over the value heads of the group):
//      dP = scale tril(dO Vn^T)     dA = -strict_tril(dZ Vn^T)     dM = beta dA
//      dQp = scale dO Sa^T + dP Kn          dKp = -beta dZ Sa^T + dM Kn          dKn = Vn dS'a^T + dP^T Qp + dM^T Kp
//      dq = dQp e^{gk-a}     dk = dKp e^{gk-a} + dKn e^{a-gk}     dbeta = sum_v dZ V - Kp.(dZ Sa^T) + sum_j dA M
//      dgk = Qp dQp + Kp dKp - Kn dKn;  dgk_L += sum_v dS'a Sa + sum_i Kn_i (Vn dS'a^T)_i;  dg = reverse chunk cumsum(dgk)
//
// Every operand that is not an exact bf16 input travels as bf16 hi + bf16 residual (three tcgen05.mma passes);
// accumulation is fp32 in TMEM.
#include "gdn_common.cuh"
#include "fla_b200_internal.h"
#include "kernel_timer.h"
#include "aux_stream.h"
#include "kda_common.cuh"
#include "tensor_map.h"

namespace fla {

struct KdaBwdParams {
  const bf16* v; const bf16* dO; const void* beta;
  const bf16* qk_img; const bf16* kn_img; const bf16* p_img; const bf16* x_img;
  const float* vec; const float* gk;
  const bf16* s_img; const bf16* vn_img;
  bf16* ds_img;        // [chunks, HV, V/64, {hi, lo}, 128x64]  dS'a entering each chunk
  bf16* dz_img;        // [chunks, HV, V/64, {64x64 dO, 64x64 dZ hi, 64x64 dZ lo}]
  float* bz;           // [V/32, tokens, HV] partial sums of dZ * V over the 32-column slices of V
  const float* dht; float* dh0;
  void* dq; void* dk; void* dv; void* dg; void* dbeta;
  const int32_t* cu_seqlens; const int32_t* chunk_offsets;
  int64_t v_st, v_sh, do_st, do_sh, beta_st;
  int64_t dq_st, dq_sh, dk_st, dk_sh, dv_st, dv_sh, dg_st, dg_sh;
  int64_t total_tokens;
  int N, T, HK, HV, beta_is_f32, grads_f32;
  int n0;              // first sequence of this launch (the backward may be launched as two halves of the batch)
  int V, nvb;          // value head dim (128 or 256) and its number of 64-column blocks
  float scale;
  int* status;
};

constexpr int64_t kKdaDsImg = 16384, kKdaDzImg = 12288;   // bf16 elements per (chunk, head, 64-column block of V)

// ============================================================================================= dhu
constexpr uint32_t dOffQKH = 0, dOffQKL = 32768, dOffKNH = 65536, dOffKNL = 81920;
constexpr uint32_t dOffDSH = 98304, dOffDSL = 114688;     // dS'a hi / lo, later rows 0-63 scale dO, rows 64-127 -beta dZ
constexpr uint32_t dOffDO = 131072;                        // raw dO rows of this V block
constexpr uint32_t dOffPH = 139264, dOffPL = 147456;      // P, then dVn, then dZ (hi / lo)
constexpr uint32_t dOffXH = 155648, dOffXL = 163840;
constexpr uint32_t kKdaDhuSmem = 172032;
constexpr uint32_t dColDS = 0, dColW1 = 64, dColDZ = 128, dColU1 = 192;

__global__ void __launch_bounds__(256, 1) kda_bwd_dhu_kernel(KdaBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ float vec_s[2][2][kK];     // [chunk parity][e^a | e^{gk_L - a}][channel]
  __shared__ float beta_s[2][kC];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t bar, pbar, qk_bar, kn_bar, x_bar;

  const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
  const int vb = blockIdx.x, hv = blockIdx.y, n = blockIdx.z + p.n0;
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  const int quad = warp & 3, half = warp >> 2;   // TMEM lane quadrant; which 32 of the tile's 64 columns
  const bool kside = quad >= 2;
  const int row = quad * 32 + lane, tok = row & 63, c0 = half * 32;

  if (warp == 0) {
    tmem_alloc(&tmem_base_s, 256);
    tmem_relinquish();
  }
  if (tid == 0) {
    mbar_init(&bar, 1);
    mbar_init(&pbar, 1);
    mbar_init(&qk_bar, 1);
    mbar_init(&kn_bar, 1);
    mbar_init(&x_bar, 1);
    mbar_init_fence();
  }
  __syncthreads();
  const uint32_t tbase = tmem_base_s;
  const uint32_t trow = tmem_addr(tbase, quad * 32, c0);
  uint32_t phase = 0, pphase = 0, qkphase = 0, knphase = 0, xphase = 0;
  bool dead = false;
  const uint32_t sb = smem_u32(smem);
  auto chunk_head = [&](int c) { return (int64_t(sq.cbase) + c) * p.HV + hv; };
  auto issue_p_load = [&](int c) {
    mbar_arrive_expect_tx(&pbar, 16384);
    bulk_load(sb + dOffPH, p.p_img + chunk_head(c) * kKdaPImg, 16384, &pbar);
  };
  auto issue_qk_load = [&](int c) {
    mbar_arrive_expect_tx(&qk_bar, 65536);
    bulk_load(sb + dOffQKH, p.qk_img + chunk_head(c) * kKdaQkImg, 65536, &qk_bar);
  };
  auto issue_kn_load = [&](int c) {
    mbar_arrive_expect_tx(&kn_bar, 32768);
    bulk_load(sb + dOffKNH, p.kn_img + chunk_head(c) * kKdaKnImg, 32768, &kn_bar);
  };
  auto issue_x_load = [&](int c) {
    mbar_arrive_expect_tx(&x_bar, 16384);
    bulk_load(sb + dOffXH, p.x_img + chunk_head(c) * kKdaXImg, 16384, &x_bar);
  };

  // per-chunk vectors, beta and my dO / v row travel through registers one chunk ahead
  float pf_vec = 0.f, pf_beta = 0.f;
  uint4 pf_row[4], rcur[4];
  auto prefetch_load = [&](int c) {
    const int t0 = c * kC;
    const int rows = min(kC, sq.len - t0);
    const int64_t tok0 = int64_t(sq.bos) + t0;
    pf_vec = p.vec[chunk_head(c) * kKdaVecs * kK + tid];      // 256 threads: e^a then e^{gk_L - a}
    const bf16* rsrc = kside ? p.v + (tok0 + tok) * p.v_st + hv * p.v_sh + vb * kBV + c0
                             : p.dO + (tok0 + tok) * p.do_st + hv * p.do_sh + vb * kBV + c0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      pf_row[i] = make_uint4(0, 0, 0, 0);
      if (tok < rows) pf_row[i] = *reinterpret_cast<const uint4*>(rsrc + i * 8);
    }
    if (kside) pf_beta = tok < rows ? ld_scalar(p.beta, (tok0 + tok) * p.beta_st + hv, p.beta_is_f32) : 0.f;
  };
  auto prefetch_store = [&](int c) {
    vec_s[c & 1][tid / kK][tid % kK] = pf_vec;
#pragma unroll
    for (int i = 0; i < 4; ++i) rcur[i] = pf_row[i];
    if (kside) {
      if (half == 0) beta_s[c & 1][tok] = pf_beta;
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(smem + dOffDO + panel_chunk_off(tok, half * 4 + i)) = pf_row[i];
    }
  };

  const Operand opKnAh{sb + dOffKNH - 8192, 8192, 0}, opKnAl{sb + dOffKNL - 8192, 8192, 0};   // Kn as A, valid rows 64..127
  const Operand opDSH{sb + dOffDSH, 16384, 1}, opDSL{sb + dOffDSL, 16384, 1};
  const Operand opPTh{sb + dOffPH - 8192, 8192, 1}, opPTl{sb + dOffPL - 8192, 8192, 1};       // P^T, valid rows 64..127
  const Operand opDO{sb + dOffDO, 8192, 1};
  const Operand opXTh{sb + dOffXH - 8192, 8192, 1}, opXTl{sb + dOffXL - 8192, 8192, 1};       // X^T, valid rows 64..127
  const Operand opDVh{sb + dOffPH, 8192, 1}, opDVl{sb + dOffPL, 8192, 1};
  const Operand opQKTh{sb + dOffQKH, 16384, 1}, opQKTl{sb + dOffQKL, 16384, 1};               // [Qp^T | Kp^T]

  float srow[32];   // this thread's 32 columns of the fp32 state-gradient row (row = key channel)
  const int c_last = sq.nt - 1;
  if (sq.nt > 0) {   // a sequence without tokens requests nothing: dh0 = dht below
    if (tid == 0) {
      issue_kn_load(c_last);
      issue_p_load(c_last);
      issue_x_load(c_last);
      issue_qk_load(c_last);
    }
    prefetch_load(c_last);
    prefetch_store(c_last);
  }
  if (p.dht) {
    const float* src = p.dht + ((int64_t(n) * p.HV + hv) * kK + row) * p.V + vb * kBV + c0;
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

  for (int c = c_last; c >= 0; --c) {
    const int cur = c & 1;
    const int t0 = c * kC;
    const int rows = min(kC, sq.len - t0);
    const int64_t tok0 = int64_t(sq.bos) + t0;
    const int64_t cidx = chunk_head(c);

    // ---- stage 0: dS'a = diag(e^{gk_L - a}) dS' as split copy (MMA operand and image) and as the fp32 master in TMEM
    {
      const float el = vec_s[cur][1][row];
#pragma unroll
      for (int i = 0; i < 32; ++i) srow[i] *= el;
      row32_to_hilo(smem + dOffDSH, smem + dOffDSL, row, half, srow);
      tmem_st_row32(trow + dColDS, srow);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    // ---- stage 1: W1 = Kn dS'a  and  U1 = P^T dO  (valid accumulator rows 64..127)
    if (tid == 0) {
      bulk_store(p.ds_img + (cidx * p.nvb + vb) * 16384, sb + dOffDSH, 32768);
      bulk_commit();
      if (!mbar_wait(&kn_bar, knphase, p.status, FLA_ERR_TIMEOUT)) dead = true;
      mma_tile(tbase + dColW1, opKnAh, opDSH, 128, 64, 8, false);
      mma_tile(tbase + dColW1, opKnAh, opDSL, 128, 64, 8, true);
      mma_tile(tbase + dColW1, opKnAl, opDSH, 128, 64, 8, true);
      if (!mbar_wait(&pbar, pphase, p.status, FLA_ERR_TIMEOUT)) dead = true;
      mma_tile(tbase + dColU1, opPTh, opDO, 128, 64, 4, false);
      mma_tile(tbase + dColU1, opPTl, opDO, 128, 64, 4, true);
      mma_commit(&bar);
    }
    knphase ^= 1;
    pphase ^= 1;
    wait_or_mark(&bar, phase, dead, p.status);
    tc_fence_after();
    if (tid == 0 && c > 0) issue_kn_load(c - 1);   // the Kn panels are free again

    // ---- stage 2: k-side rows: dVn = scale U1 + W1
    float acc[32];
    if (kside) {
      float w1[32];
      tmem_ld32(trow + dColW1, w1);
      tmem_ld32(trow + dColU1, acc);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = p.scale * acc[i] + w1[i];
      row32_to_hilo(smem + dOffPH, smem + dOffPL, tok, half, acc);
    }
    if (tid == 0) bulk_wait_read();  // the dS'a images have left shared memory (it is reused in stage 4)
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    // ---- stage 3: dZ = X^T dVn  (valid accumulator rows 64..127)
    if (tid == 0) {
      if (!mbar_wait(&x_bar, xphase, p.status, FLA_ERR_TIMEOUT)) dead = true;
      mma_tile(tbase + dColDZ, opXTh, opDVh, 128, 64, 4, false);
      mma_tile(tbase + dColDZ, opXTh, opDVl, 128, 64, 4, true);
      mma_tile(tbase + dColDZ, opXTl, opDVh, 128, 64, 4, true);
      mma_commit(&bar);
    }
    xphase ^= 1;
    wait_or_mark(&bar, phase, dead, p.status);
    tc_fence_after();
    if (tid == 0 && c > 0) issue_x_load(c - 1);

    // ---- stage 4: k-side rows: dV, sum_v dZ*V, dZ images, -beta dZ;  q-side rows: scale dO
    if (kside) {
      tmem_ld_row32(trow + dColDZ, acc);
      const float bi = beta_s[cur][tok];
      float bzsum = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float vv[8];
        unpack_bf16x8(rcur[i], vv);
#pragma unroll
        for (int j = 0; j < 8; ++j) bzsum += acc[i * 8 + j] * vv[j];
      }
      row32_to_hilo(smem + dOffPH, smem + dOffPL, tok, half, acc);
      if (tok < rows) {
        p.bz[(int64_t(vb * 2 + half) * p.total_tokens + tok0 + tok) * p.HV + hv] = bzsum;
        const int64_t off = (tok0 + tok) * p.dv_st + hv * p.dv_sh + vb * kBV + c0;
        if (p.grads_f32) {
          float* dst = static_cast<float*>(p.dv) + off;
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            *reinterpret_cast<float4*>(dst + i) = make_float4(bi * acc[i], bi * acc[i + 1], bi * acc[i + 2], bi * acc[i + 3]);
        } else {
          bf16* dst = static_cast<bf16*>(p.dv) + off;
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            float t[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) t[j] = bi * acc[ch * 8 + j];
            *reinterpret_cast<uint4*>(dst + ch * 8) = pack8(t);
          }
        }
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] *= -bi;
      row32_to_hilo(smem + dOffDSH, smem + dOffDSL, 64 + tok, half, acc);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float vv[8];
        unpack_bf16x8(rcur[i], vv);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i * 8 + j] = p.scale * vv[j];
      }
      row32_to_hilo(smem + dOffDSH, smem + dOffDSL, tok, half, acc);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    // ---- stage 5: dSa += [Qp^T | Kp^T] [scale dO ; -beta dZ]
    if (tid == 0) {
      bf16* dst = p.dz_img + (cidx * p.nvb + vb) * 12288;
      bulk_store(dst, sb + dOffDO, 8192);            // dO
      bulk_store(dst + 4096, sb + dOffPH, 16384);    // dZ hi, dZ lo
      bulk_commit();
      if (!mbar_wait(&qk_bar, qkphase, p.status, FLA_ERR_TIMEOUT)) dead = true;
      mma_tile(tbase + dColDS, opQKTh, opDSH, 128, 64, 8, true);
      mma_tile(tbase + dColDS, opQKTh, opDSL, 128, 64, 8, true);
      mma_tile(tbase + dColDS, opQKTl, opDSH, 128, 64, 8, true);
      mma_commit(&bar);
    }
    qkphase ^= 1;
    if (c > 0) prefetch_load(c - 1);
    wait_or_mark(&bar, phase, dead, p.status);
    tc_fence_after();
    if (tid == 0 && c > 0) issue_qk_load(c - 1);

    // ---- stage 6: dS = diag(e^a) dSa to registers; next chunk's operands
    tmem_ld_row32(trow + dColDS, srow);
    {
      const float ea = vec_s[cur][0][row];
#pragma unroll
      for (int i = 0; i < 32; ++i) srow[i] *= ea;
    }
    if (tid == 0) {
      bulk_wait_read();                  // the dO / dZ images have left the panels
      if (c > 0) issue_p_load(c - 1);    // ... which now receive the next chunk's P
    }
    tc_fence_before();
    __syncthreads();
    if (c > 0) {
      prefetch_store(c - 1);
      __syncthreads();
    }
  }

  if (!dead && p.dh0) {
    float* dst = p.dh0 + ((int64_t(n) * p.HV + hv) * kK + row) * p.V + vb * kBV + c0;
#pragma unroll
    for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(srow[i], srow[i + 1], srow[i + 2], srow[i + 3]);
  }
  if (tid == 0) bulk_wait_all();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 256);
}

// ============================================================================================= par
constexpr uint32_t qOffQKH = 0, qOffQKL = 32768, qOffKNH = 65536, qOffKNL = 81920;       // per-head operand images
constexpr uint32_t qOffAH = 98304;              // [dO ; dZ_hi] rows of one V block (128 rows)
constexpr uint32_t qOffAL = 114688;             // rows 0-63 zero, rows 64-127 dZ_lo
constexpr uint32_t qOffVNH = 131072, qOffVNL = 139264;
constexpr uint32_t qOffSH = 147456, qOffSL = 163840, qOffDSH = 180224, qOffDSL = 196608;
constexpr uint32_t qOffPAH = qOffAH, qOffPAL = qOffAL;   // [dP ; dM] hi / lo reuse the [dO ; dZ] panels
constexpr uint32_t qOffTile = qOffAH;           // two fp32 [64][132] tiles of the dg assembly reuse the step buffers
constexpr uint32_t kKdaParSmem = 212992;
constexpr int kTileStride = 132;   // 16-byte aligned rows; float4 row stores and scalar column reads are both conflict-free
constexpr uint32_t kTileBytes = kC * kTileStride * 4;
constexpr uint32_t qOffGk = 165888;             // the chunk's gk rows: four 64 x 32 fp32 TMA tiles (swizzled), 32 KB
static_assert(qOffTile + 2 * kTileBytes <= qOffGk && qOffGk % 1024 == 0 && qOffGk + 32768 <= kKdaParSmem &&
              qOffGk >= qOffSL, "dg tiles and the gk tile must fit in the phase-1 step buffers behind the [dP; dM] panels");
constexpr uint32_t qColQK = 0, qColDV = 64, qColTA = 128, qColTB1 = 256, qColTB2 = 384;
constexpr uint32_t kKdaStepBytes = 16384 + 8192 + 16384 + 32768 + 32768;

// sum over 8 columns of (hi + lo panel values) * x
__device__ __forceinline__ void chunk_vals(const uint8_t* pan_hi, const uint8_t* pan_lo, int row, int ch, float* f) {
  float lo[8];
  unpack_bf16x8(*reinterpret_cast<const uint4*>(pan_hi + panel_chunk_off(row, ch)), f);
  unpack_bf16x8(*reinterpret_cast<const uint4*>(pan_lo + panel_chunk_off(row, ch)), lo);
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] += lo[j];
}


// Sum over the 32 lanes (rows) of each of 32 per-lane values (columns): lane l ends up with the total of column l.
// Recursive halving: at every step a lane keeps one half of its values and hands the other half to its partner.
__device__ __forceinline__ float warp_column_sums32(const float* v, int lane) {
  float a[16], b[8], c[4], d[2];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float send = (lane & 16) ? v[i] : v[16 + i], keep = (lane & 16) ? v[16 + i] : v[i];
    a[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float send = (lane & 8) ? a[i] : a[8 + i], keep = (lane & 8) ? a[8 + i] : a[i];
    b[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float send = (lane & 4) ? b[i] : b[4 + i], keep = (lane & 4) ? b[4 + i] : b[i];
    c[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const float send = (lane & 2) ? c[i] : c[2 + i], keep = (lane & 2) ? c[2 + i] : c[i];
    d[i] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
  }
  const float send = (lane & 1) ? d[0] : d[1], keep = (lane & 1) ? d[1] : d[0];
  return keep + __shfl_xor_sync(0xffffffffu, send, 1);
}

// The chunk's gk rows arrive as TMA tiles once the phase-1 buffers are free; the last epilogue reads them from
// shared memory (their global loads used to sit, one round trip each, on the critical path).
template <int NVB>   // 64-column blocks of V per head (2 or 4): a compile-time trip count keeps the block loop unrolled
__global__ void __launch_bounds__(256, 1) kda_bwd_par_kernel(KdaBwdParams p, const __grid_constant__ CUtensorMap tm_gk) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ float beta_s[kC], anchor_s[kK];
  __shared__ float red[2][2][kC];      // rkG, ma : [half][row]
  __shared__ float sds_s[2][kK];       // sum_v dS'a * Sa per key channel, by column half
  __shared__ float colsum_s[2][kK];    // per 32-row part: column sums of the dgk tiles
  __shared__ float t1col_s[2][kK];     // per 32-row quadrant: sum_i Kn_i (Vn dS'a^T)_i of the last-row term
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) uint64_t mma_bar, load_bar, img_bar, gk_bar;

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
  if (tid == 0) {
    mbar_init(&mma_bar, 1);
    mbar_init(&load_bar, 1);
    mbar_init(&img_bar, 1);
    mbar_init(&gk_bar, 1);
    mbar_init_fence();
    tma_prefetch_descriptor(&tm_gk);
  }
  __syncthreads();
  const uint32_t tbase = tmem_base_s;
  const uint32_t trow = tmem_addr(tbase, quad * 32, 0);
  const uint32_t sb = smem_u32(smem);
  uint32_t mphase = 0, lphase = 0, iphase = 0, gphase = 0;
  bool ok = true;

  auto issue_images = [&](int hv) {           // one thread: [Qp; Kp] and Kn of one value head
    const int64_t cidx = (int64_t(sq.cbase) + c) * p.HV + hv;
    mbar_arrive_expect_tx(&img_bar, 65536 + 32768);
    bulk_load(sb + qOffQKH, p.qk_img + cidx * kKdaQkImg, 65536, &img_bar);
    bulk_load(sb + qOffKNH, p.kn_img + cidx * kKdaKnImg, 32768, &img_bar);
  };
  auto issue_loads = [&](int hv, int vb) {    // one thread: operands of one (value head, V block) step
    const int64_t cidx = (int64_t(sq.cbase) + c) * p.HV + hv;
    mbar_arrive_expect_tx(&load_bar, kKdaStepBytes);
    const bf16* dz = p.dz_img + (cidx * NVB + vb) * 12288;
    bulk_load(sb + qOffAH, dz, 16384, &load_bar);
    bulk_load(sb + qOffAL + 8192, dz + 8192, 8192, &load_bar);
    bulk_load(sb + qOffVNH, p.vn_img + (cidx * NVB + vb) * 8192, 16384, &load_bar);
    bulk_load(sb + qOffSH, p.s_img + (cidx * NVB + vb) * 16384, 32768, &load_bar);
    bulk_load(sb + qOffDSH, p.ds_img + (cidx * NVB + vb) * 16384, 32768, &load_bar);
  };

  const Operand opQKh{sb + qOffQKH, 16384, 0}, opQKl{sb + qOffQKL, 16384, 0};           // [Qp; Kp], reduction over key dims
  const Operand opQKnh{sb + qOffQKH, 16384, 1}, opQKnl{sb + qOffQKL, 16384, 1};         // as B, N = 128 key dims, reduction over 128 rows
  const Operand opKNbh{sb + qOffKNH, 8192, 0}, opKNbl{sb + qOffKNL, 8192, 0};           // Kn as B, N = 64 tokens
  const Operand opKNnh{sb + qOffKNH, 8192, 1}, opKNnl{sb + qOffKNL, 8192, 1};           // Kn as B, N = 128 key dims, reduction over tokens
  const Operand opAH{sb + qOffAH, 16384, 0}, opAL{sb + qOffAL, 16384, 0};
  const Operand opVNbH{sb + qOffVNH, 8192, 0}, opVNbL{sb + qOffVNL, 8192, 0};           // Vn as B (N = 64 tokens)
  const Operand opVNaH{sb + qOffVNH - 8192, 8192, 0}, opVNaL{sb + qOffVNL - 8192, 8192, 0};  // Vn as A, valid rows 64..127
  const Operand opSH{sb + qOffSH, 16384, 0}, opSL{sb + qOffSL, 16384, 0};               // Sa block as B (N = 128 key dims)
  const Operand opDSH{sb + qOffDSH, 16384, 0}, opDSL{sb + qOffDSL, 16384, 0};
  const Operand opPAH{sb + qOffPAH, 16384, 0}, opPAL{sb + qOffPAL, 16384, 0};           // [dP; dM], reduction over j
  const Operand opPATh{sb + qOffPAH - 8192, 8192, 1}, opPATl{sb + qOffPAL - 8192, 8192, 1};  // its transpose, valid rows 64..127

  float acc_out[64];  // running dq (q-side rows) or dk (k-side rows), this thread's 64 key-dim columns
#pragma unroll
  for (int i = 0; i < 64; ++i) acc_out[i] = 0.f;
  float* tile_q = reinterpret_cast<float*>(smem + qOffTile);
  float* tile_k = reinterpret_cast<float*>(smem + qOffTile + kTileBytes);

  for (int h = 0; h < G && ok; ++h) {
    const int hv = hk * G + h;
    const int64_t cidx = (int64_t(sq.cbase) + c) * p.HV + hv;
    // zero rows of the lo operand (dO has no residual), this head's scalars, then the loads
    for (int idx = tid; idx < 512; idx += 256) *reinterpret_cast<uint4*>(smem + qOffAL + idx * 16) = make_uint4(0, 0, 0, 0);
    if (tid < kC) beta_s[tid] = tid < rows ? ld_scalar(p.beta, (tok0 + tid) * p.beta_st + hv, p.beta_is_f32) : 0.f;
    if (tid >= 128) anchor_s[tid - 128] = p.vec[cidx * kKdaVecs * kK + 2 * kK + tid - 128];
    fence_async_smem();
    __syncthreads();
    if (tid == 0) {
      issue_images(hv);
      issue_loads(hv, 0);
    }
    float sds = 0.f;   // my key channel (tid & 127), my 32 columns (tid >> 7) of sum_v dS'a * Sa
    for (int vb = 0; vb < NVB; ++vb) {
      if (vb == 0) {
        ok = mbar_wait(&img_bar, iphase, p.status, FLA_ERR_TIMEOUT);
        iphase ^= 1;
      }
      ok = mbar_wait(&load_bar, lphase, p.status, FLA_ERR_TIMEOUT) && ok;
      lphase ^= 1;
      if (!__syncthreads_and(ok)) { ok = false; break; }
      if (tid == 0) {
        tc_fence_after();
        if (vb == 0) {
          mma_tile(tbase + qColQK, opQKh, opKNbh, 128, 64, 8, false);
          mma_tile(tbase + qColQK, opQKh, opKNbl, 128, 64, 8, true);
          mma_tile(tbase + qColQK, opQKl, opKNbh, 128, 64, 8, true);
        }
        const bool accf = vb > 0;
        // [dO; dZ] . [Vn_lo | Sa_hi]^T as one N = 192 product: the two images are neighbours in shared memory and their
        // accumulators neighbours in tensor memory, so the A operand is read once for both
        static_assert(qOffVNL + 8192 == qOffSH && qColDV + 64 == qColTA, "the N = 192 product needs both pairs adjacent");
        mma_tile(tbase + qColDV, opAH, opVNbL, 128, 192, 4, accf);
        mma_tile(tbase + qColDV, opAH, opVNbH, 128, 64, 4, true);
        mma_tile(tbase + qColDV, opAL, opVNbH, 128, 64, 4, true);
        mma_tile(tbase + qColTA, opAH, opSL, 128, 128, 4, true);
        mma_tile(tbase + qColTA, opAL, opSH, 128, 128, 4, true);
        mma_tile(tbase + qColTB1, opVNaH, opDSH, 128, 128, 4, accf);
        mma_tile(tbase + qColTB1, opVNaH, opDSL, 128, 128, 4, true);
        mma_tile(tbase + qColTB1, opVNaL, opDSH, 128, 128, 4, true);
        mma_commit(&mma_bar);
      }
      // sum_v dS'a * Sa per key channel over this V block while the MMAs run (elementwise on the panel images)
      {
        const int kr = tid & 127, hf = tid >> 7;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          float s[8], d[8];
          chunk_vals(smem + qOffSH, smem + qOffSL, kr, hf * 4 + ch, s);
          chunk_vals(smem + qOffDSH, smem + qOffDSL, kr, hf * 4 + ch, d);
#pragma unroll
          for (int j = 0; j < 8; ++j) sds += s[j] * d[j];
        }
      }
      ok = mbar_wait(&mma_bar, mphase, p.status, FLA_ERR_TIMEOUT);
      mphase ^= 1;
      if (!__syncthreads_and(ok)) { ok = false; break; }   // also: every thread is done reading the step's buffers
      tc_fence_after();
      if (tid == 0) {
        if (vb + 1 < NVB) {
          issue_loads(hv, vb + 1);
        } else {   // the phase-1 buffers are free: this head's gk rows, channels 32 b .. 32 b + 31 in tile b
          mbar_arrive_expect_tx(&gk_bar, 4 * 8192);
#pragma unroll
          for (int b = 0; b < 4; ++b) tma_load_tile(sb + qOffGk + b * 8192, &tm_gk, 32 * b, hv, int(tok0), &gk_bar);
        }
      }
    }
    if (!ok) break;
    sds_s[tid >> 7][tid & 127] = sds;

    // ---- epilogue 1: score-tile gradients -> [dP; dM] operand; row scaling of the first TA product in place
    const float beta_i = beta_s[tok];
    float ma_part = 0.f, rkG = 0.f;
    {
      float sc[32], dvv[32];
      tmem_ld32(trow + qColQK + half * 32, sc);
      tmem_ld32(trow + qColDV + half * 32, dvv);
      tmem_ld_wait();
      if (!kside) {
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) dvv[jj] = (half * 32 + jj <= tok) ? p.scale * dvv[jj] : 0.f;
      } else {
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) {
          const bool keep = half * 32 + jj < tok;
          const float dA = keep ? -dvv[jj] : 0.f;
          ma_part += keep ? dA * sc[jj] : 0.f;      // select: entries above the diagonal of M may be huge
          dvv[jj] = dA * beta_i;
        }
      }
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        uint4 hi, lo;
        split8(dvv + ch * 8, hi, lo);
        const uint32_t off = panel_chunk_off(row, half * 4 + ch);
        *reinterpret_cast<uint4*>(smem + qOffPAH + off) = hi;
        *reinterpret_cast<uint4*>(smem + qOffPAL + off) = lo;
      }
    }
    {
      float ta[64];
      tmem_ld_row64(trow + qColTA + half * 64, ta);
      float f = p.scale;
      if (kside) {
        // Kp_i . (dZ Sa^T)_i over my 64 key dims
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          float kp[8];
          chunk_vals(smem + qOffQKH + half * 16384, smem + qOffQKL + half * 16384, 64 + tok, ch, kp);
#pragma unroll
          for (int j = 0; j < 8; ++j) rkG += kp[j] * ta[ch * 8 + j];
        }
        f = -beta_i;
      }
#pragma unroll
      for (int i = 0; i < 64; ++i) ta[i] *= f;
      tmem_st_row64(trow + qColTA + half * 64, ta);
    }
    if (kside) {
      red[0][half][tok] = rkG;
      red[1][half][tok] = ma_part;
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();

    // ---- TA += [dP; dM] Kn   and   TB2 = [dP^T | dM^T] [Qp; Kp]
    if (tid == 0) {
      tc_fence_after();
      mma_tile(tbase + qColTA, opPAH, opKNnh, 128, 128, 4, true);
      mma_tile(tbase + qColTA, opPAH, opKNnl, 128, 128, 4, true);
      mma_tile(tbase + qColTA, opPAL, opKNnh, 128, 128, 4, true);
      mma_tile(tbase + qColTB2, opPATh, opQKnh, 128, 128, 8, false);
      mma_tile(tbase + qColTB2, opPATh, opQKnl, 128, 128, 8, true);
      mma_tile(tbase + qColTB2, opPATl, opQKnh, 128, 128, 8, true);
      mma_commit(&mma_bar);
    }
    // dbeta while the MMAs run
    if (tid < rows) {
      const int i = tid;
      const int64_t gidx = (tok0 + i) * p.HV + hv;
      const int64_t bzs = p.total_tokens * p.HV;
      float bz = 0.f;
      for (int s = 0; s < NVB; ++s) bz += p.bz[(2 * s) * bzs + gidx] + p.bz[(2 * s + 1) * bzs + gidx];
      const float db = bz - (red[0][0][i] + red[0][1][i]) + (red[1][0][i] + red[1][1][i]);
      if (p.grads_f32) static_cast<float*>(p.dbeta)[gidx] = db;
      else static_cast<bf16*>(p.dbeta)[gidx] = __float2bfloat16_rn(db);
    }
    ok = mbar_wait(&mma_bar, mphase, p.status, FLA_ERR_TIMEOUT);
    mphase ^= 1;
    if (!__syncthreads_and(ok)) { ok = false; break; }
    tc_fence_after();

    // ---- epilogue 2: dq / dk rows of this head and the three dg tiles (the step buffers are free now)
    {
      const int pan = half;   // my 64 key dims are panel `half` of the 128-wide images
      const bool live = tok < rows;
      ok = mbar_wait(&gk_bar, gphase, p.status, FLA_ERR_TIMEOUT) && ok;
      gphase ^= 1;
#pragma unroll
      for (int sub = 0; sub < 2; ++sub) {
        float x[32];
        tmem_ld32(trow + qColTA + half * 64 + sub * 32, x);
        tmem_ld_wait();
        if (!kside) {
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            float qp[8];
            chunk_vals(smem + qOffQKH + pan * 16384, smem + qOffQKL + pan * 16384, tok, sub * 4 + ch, qp);
            const uint8_t* gt = smem + qOffGk + (half * 2 + sub) * 8192 + tok * 128;
            const float4 g0 = *reinterpret_cast<const float4*>(gt + (((2 * ch) ^ (tok & 7)) << 4));
            const float4 g1 = *reinterpret_cast<const float4*>(gt + (((2 * ch + 1) ^ (tok & 7)) << 4));
            const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
            float tq[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int col = sub * 32 + ch * 8 + j;
              const float xv = x[ch * 8 + j];
              const float e1 = __expf(gv[j] - anchor_s[half * 64 + col]);
              acc_out[col] += live ? xv * e1 : 0.f;
              tq[j] = live ? qp[j] * xv : 0.f;
            }
            float* dq_ = tile_q + tok * kTileStride + half * 64 + sub * 32 + ch * 8;
            *reinterpret_cast<float4*>(dq_) = make_float4(tq[0], tq[1], tq[2], tq[3]);
            *reinterpret_cast<float4*>(dq_ + 4) = make_float4(tq[4], tq[5], tq[6], tq[7]);
          }
        } else {
          float y1[32], y2[32], t1v[32];
          tmem_ld32(trow + qColTB1 + half * 64 + sub * 32, y1);
          tmem_ld32(trow + qColTB2 + half * 64 + sub * 32, y2);
          tmem_ld_wait();
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {
            float kp[8], kn[8];
            chunk_vals(smem + qOffQKH + pan * 16384, smem + qOffQKL + pan * 16384, 64 + tok, sub * 4 + ch, kp);
            chunk_vals(smem + qOffKNH + pan * 8192, smem + qOffKNL + pan * 8192, tok, sub * 4 + ch, kn);
            const uint8_t* gt = smem + qOffGk + (half * 2 + sub) * 8192 + tok * 128;
            const float4 g0 = *reinterpret_cast<const float4*>(gt + (((2 * ch) ^ (tok & 7)) << 4));
            const float4 g1 = *reinterpret_cast<const float4*>(gt + (((2 * ch + 1) ^ (tok & 7)) << 4));
            const float gv[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
            float tk[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int col = sub * 32 + ch * 8 + j;
              const float d = gv[j] - anchor_s[half * 64 + col];
              const float e1 = __expf(d), e2 = __expf(-d);
              const float dkp = x[ch * 8 + j], t1 = y1[ch * 8 + j], dkn = t1 + y2[ch * 8 + j];
              acc_out[col] += live ? dkp * e1 + dkn * e2 : 0.f;
              tk[j] = live ? kp[j] * dkp - kn[j] * dkn : 0.f;
              t1v[ch * 8 + j] = live ? kn[j] * t1 : 0.f;
            }
            float* dk_ = tile_k + tok * kTileStride + half * 64 + sub * 32 + ch * 8;
            *reinterpret_cast<float4*>(dk_) = make_float4(tk[0], tk[1], tk[2], tk[3]);
            *reinterpret_cast<float4*>(dk_ + 4) = make_float4(tk[4], tk[5], tk[6], tk[7]);
          }
          // last-row term: column sums of Kn * (Vn dS'a^T) over my warp's 32 rows
          t1col_s[quad - 2][half * 64 + sub * 32 + lane] = warp_column_sums32(t1v, lane);
        }
      }
    }
    tc_fence_before();
    if (!__syncthreads_and(ok)) { ok = false; break; }
    // dg = reverse chunk-local cumulative sum of dgk; the last row additionally carries
    // sum_v dS'a Sa + sum_i Kn_i (Vn dS'a^T)_i, which therefore reaches every row.
    {
      // Two threads per key channel, 32 rows each: local totals first, then the suffix sums.  Each group of eight rows is
      // read into registers before any of its results is stored: a global store between two shared-memory loads would keep
      // the compiler from overlapping them (it cannot tell the generic pointers apart).
      const int kc = tid & (kK - 1), part = tid >> 7, r0 = part * 32;
      float tot = 0.f;
#pragma unroll 8
      for (int i = 0; i < 32; ++i) tot += tile_q[(r0 + i) * kTileStride + kc] + tile_k[(r0 + i) * kTileStride + kc];   // rows past the end hold zeros
      colsum_s[part][kc] = tot;
      __syncthreads();
      float run = sds_s[0][kc] + sds_s[1][kc] + t1col_s[0][kc] + t1col_s[1][kc] + (part == 0 ? colsum_s[1][kc] : 0.f);
      const int64_t base = tok0 * p.dg_st + hv * p.dg_sh + kc;
      for (int blk = 3; blk >= 0; --blk) {
        float vals[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int t = r0 + blk * 8 + j;
          vals[j] = tile_q[t * kTileStride + kc] + tile_k[t * kTileStride + kc];
        }
#pragma unroll
        for (int j = 7; j >= 0; --j) {
          run += vals[j];
          vals[j] = run;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int t = r0 + blk * 8 + j;
          if (t < rows) {
            if (p.grads_f32) static_cast<float*>(p.dg)[base + t * p.dg_st] = vals[j];
            else static_cast<bf16*>(p.dg)[base + t * p.dg_st] = __float2bfloat16_rn(vals[j]);
          }
        }
      }
    }
    __syncthreads();
  }

  if (ok && tok < rows) {
    void* base = kside ? p.dk : p.dq;
    const int64_t off = kside ? (tok0 + tok) * p.dk_st + hk * p.dk_sh + half * 64 : (tok0 + tok) * p.dq_st + hk * p.dq_sh + half * 64;
    if (p.grads_f32) {
      float* dst = static_cast<float*>(base) + off;
#pragma unroll
      for (int i = 0; i < 64; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(acc_out[i], acc_out[i + 1], acc_out[i + 2], acc_out[i + 3]);
    } else {
      bf16* dst = static_cast<bf16*>(base) + off;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(dst + ch * 8) = pack8(acc_out + ch * 8);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 512);
}

}  // namespace fla

using namespace fla;

// Workspace: status | [forward workspace | gk | s_img | vn_img unless the caller passes the forward's saved buffer] | ds_img | dz_img | bz
static uint64_t kda_bwd_ws_layout(int64_t total_chunks, int64_t HV, int64_t nvb, int64_t tokens, bool have_saved, uint64_t* off_saved,
                                  uint64_t off[3]) {
  const uint64_t per = uint64_t(total_chunks) * HV;
  uint64_t o = 256, so[4];
  *off_saved = o;
  if (!have_saved) o += align_up(kda_saved_layout(total_chunks, HV, nvb, tokens, so), 256);
  off[0] = o; o += align_up(per * nvb * kKdaDsImg * 2, 256);
  off[1] = o; o += align_up(per * nvb * kKdaDzImg * 2, 256);
  off[2] = o; o += align_up(uint64_t(2 * nvb) * tokens * HV * 4, 256);
  return o;
}

static int kda_bwd_geometry(const fla_kda_chunk_bwd_args* a, int64_t* total_chunks, int* N, int* max_len) {
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

extern "C" FLA_API int fla_b200_kda_chunk_bwd_workspace_size(const fla_kda_chunk_bwd_args* a, uint64_t* bytes) {
  if (!a || !bytes) return FLA_ERR_NULL;
  int64_t total_chunks; int N, max_len;
  const int st = kda_bwd_geometry(a, &total_chunks, &N, &max_len);
  if (st) return st;
  uint64_t off[3], off_saved;
  const int64_t V = a->v.shape[3];
  if (V != kV && V != 2 * kV) return FLA_ERR_SHAPE;
  *bytes = kda_bwd_ws_layout(total_chunks, a->v.shape[2], V / kBV, a->q.shape[0] * a->q.shape[1], a->saved.data != nullptr, &off_saved, off);
  return FLA_OK;
}

static int kda_bwd_check_tok(const fla_tensor_t& t, int64_t B, int64_t T, int64_t heads, int64_t dim, bool allow_f32) {
  if (!t.data) return FLA_ERR_NULL;
  if (t.ndim != 4 || t.shape[0] != B || t.shape[1] != T || t.shape[2] != heads || t.shape[3] != dim) return FLA_ERR_SHAPE;
  if (t.dtype != FLA_BF16 && !(allow_f32 && t.dtype == FLA_F32)) return FLA_ERR_DTYPE;
  const int64_t esz = t.dtype == FLA_F32 ? 4 : 2;
  if (t.stride[3] != 1 || (t.stride[2] * esz) % 16 || (t.stride[1] * esz) % 16 || !aligned16(t.data)) return FLA_ERR_LAYOUT;
  if (B > 1 && t.stride[0] != T * t.stride[1]) return FLA_ERR_LAYOUT;
  return FLA_OK;
}
static int kda_bwd_check_tok3(const fla_tensor_t& t, int64_t B, int64_t T, int64_t heads, bool dense) {
  if (!t.data) return FLA_ERR_NULL;
  if (t.ndim != 3 || t.shape[0] != B || t.shape[1] != T || t.shape[2] != heads) return FLA_ERR_SHAPE;
  if (t.dtype != FLA_BF16 && t.dtype != FLA_F32) return FLA_ERR_DTYPE;
  if (t.stride[2] != 1 || (B > 1 && t.stride[0] != T * t.stride[1])) return FLA_ERR_LAYOUT;
  if (dense && t.stride[1] != heads) return FLA_ERR_LAYOUT;
  return FLA_OK;
}

extern "C" FLA_API int fla_b200_kda_chunk_bwd(const fla_kda_chunk_bwd_args* a, void* workspace, uint64_t workspace_bytes,
                                              void* stream) {
  if (!a) return FLA_ERR_NULL;
  int64_t total_chunks; int N, max_len;
  int st = kda_bwd_geometry(a, &total_chunks, &N, &max_len);
  if (st) return st;
  const int64_t B = a->q.shape[0], T = a->q.shape[1], HK = a->q.shape[2], HV = a->v.shape[2];
  if (HK <= 0 || HV <= 0 || HV % HK) return FLA_ERR_SHAPE;
  const int64_t V = a->v.shape[3], nvb = V / kBV;
  if (V != kV && V != 2 * kV) return FLA_ERR_SHAPE;
  if ((st = kda_bwd_check_tok(a->q, B, T, HK, kK, false))) return st;
  if ((st = kda_bwd_check_tok(a->k, B, T, HK, kK, false))) return st;
  if ((st = kda_bwd_check_tok(a->v, B, T, HV, V, false))) return st;
  if ((st = kda_bwd_check_tok(a->g, B, T, HV, kK, true))) return st;
  if ((st = kda_bwd_check_tok(a->d_o, B, T, HV, V, false))) return st;
  if ((st = kda_bwd_check_tok(a->dq, B, T, HK, kK, true))) return st;
  if ((st = kda_bwd_check_tok(a->dk, B, T, HK, kK, true))) return st;
  if ((st = kda_bwd_check_tok(a->dv, B, T, HV, V, true))) return st;
  if ((st = kda_bwd_check_tok(a->dg, B, T, HV, kK, true))) return st;
  if ((st = kda_bwd_check_tok3(a->beta, B, T, HV, false))) return st;
  if ((st = kda_bwd_check_tok3(a->dbeta, B, T, HV, true))) return st;
  const int gdt = a->dq.dtype;
  if (a->dk.dtype != gdt || a->dv.dtype != gdt || a->dg.dtype != gdt || a->dbeta.dtype != gdt) return FLA_ERR_DTYPE;
  for (const fla_tensor_t* s : {&a->initial_state, &a->dht, &a->dh0}) {
    if (!s->data) continue;
    if (s->dtype != FLA_F32) return FLA_ERR_DTYPE;
    if (s->ndim != 4 || s->shape[0] != N || s->shape[1] != HV || s->shape[2] != kK || s->shape[3] != V) return FLA_ERR_SHAPE;
    if (s->stride[3] != 1 || s->stride[2] != V || s->stride[1] != kK * V || s->stride[0] != HV * kK * V || !aligned16(s->data))
      return FLA_ERR_LAYOUT;
  }
  if (a->chunk_size != kC) return FLA_ERR_VALUE;
  uint64_t off[3], off_saved, so[4], fo[6];
  const bool have_saved = a->saved.data != nullptr;
  const uint64_t need = kda_bwd_ws_layout(total_chunks, HV, nvb, B * T, have_saved, &off_saved, off);
  if (!workspace || workspace_bytes < need || !aligned16(workspace)) return FLA_ERR_WORKSPACE;
  const uint64_t sbytes = kda_saved_layout(total_chunks, HV, nvb, B * T, so);
  if (have_saved && (a->saved.dtype != FLA_BF16 || a->saved.ndim != 1 || uint64_t(a->saved.shape[0]) * 2 < sbytes ||
                     !aligned16(a->saved.data)))
    return FLA_ERR_SHAPE;
  kda_ws_layout(total_chunks, HV, fo);

  uint8_t* ws = static_cast<uint8_t*>(workspace);
  uint8_t* sv = have_saved ? static_cast<uint8_t*>(a->saved.data) : ws + off_saved;
  uint8_t* fws = sv + so[0];
  KdaParams f{};
  f.q = static_cast<const bf16*>(a->q.data); f.k = static_cast<const bf16*>(a->k.data); f.v = static_cast<const bf16*>(a->v.data);
  f.g = a->g.data; f.beta = a->beta.data;
  f.gk_out = reinterpret_cast<float*>(sv + so[1]);
  f.status = reinterpret_cast<int*>(ws);
  f.qk_img = reinterpret_cast<bf16*>(fws + fo[0]); f.kn_img = reinterpret_cast<bf16*>(fws + fo[1]);
  f.p_img = reinterpret_cast<bf16*>(fws + fo[2]); f.x_img = reinterpret_cast<bf16*>(fws + fo[3]);
  f.vec = reinterpret_cast<float*>(fws + fo[4]); f.at = reinterpret_cast<float*>(fws + fo[5]);
  f.s_img = reinterpret_cast<bf16*>(sv + so[2]); f.vn_img = reinterpret_cast<bf16*>(sv + so[3]);
  f.h0 = static_cast<const float*>(a->initial_state.data);
  f.cu_seqlens = static_cast<const int32_t*>(a->cu_seqlens.data);
  f.chunk_offsets = static_cast<const int32_t*>(a->chunk_offsets.data);
  f.q_st = a->q.stride[1]; f.q_sh = a->q.stride[2]; f.k_st = a->k.stride[1]; f.k_sh = a->k.stride[2];
  f.v_st = a->v.stride[1]; f.v_sh = a->v.stride[2];
  f.g_st = a->g.stride[1]; f.g_sh = a->g.stride[2]; f.beta_st = a->beta.stride[1];
  f.N = N; f.T = int(T); f.HK = int(HK); f.HV = int(HV); f.total_tokens = B * T; f.V = int(V); f.nvb = int(nvb);
  f.g_is_f32 = a->g.dtype == FLA_F32; f.beta_is_f32 = a->beta.dtype == FLA_F32;
  f.gate_mode = 0; f.scale = a->scale;

  KdaBwdParams p{};
  p.v = f.v; p.dO = static_cast<const bf16*>(a->d_o.data); p.beta = a->beta.data;
  p.qk_img = f.qk_img; p.kn_img = f.kn_img; p.p_img = f.p_img; p.x_img = f.x_img; p.vec = f.vec; p.gk = f.gk_out;
  p.s_img = f.s_img; p.vn_img = f.vn_img;
  p.ds_img = reinterpret_cast<bf16*>(ws + off[0]); p.dz_img = reinterpret_cast<bf16*>(ws + off[1]);
  p.bz = reinterpret_cast<float*>(ws + off[2]);
  p.dht = static_cast<const float*>(a->dht.data); p.dh0 = static_cast<float*>(a->dh0.data);
  p.dq = a->dq.data; p.dk = a->dk.data; p.dv = a->dv.data; p.dg = a->dg.data; p.dbeta = a->dbeta.data;
  p.cu_seqlens = f.cu_seqlens; p.chunk_offsets = f.chunk_offsets;
  p.v_st = f.v_st; p.v_sh = f.v_sh; p.do_st = a->d_o.stride[1]; p.do_sh = a->d_o.stride[2]; p.beta_st = f.beta_st;
  p.dq_st = a->dq.stride[1]; p.dq_sh = a->dq.stride[2]; p.dk_st = a->dk.stride[1]; p.dk_sh = a->dk.stride[2];
  p.dv_st = a->dv.stride[1]; p.dv_sh = a->dv.stride[2]; p.dg_st = a->dg.stride[1]; p.dg_sh = a->dg.stride[2];
  p.total_tokens = B * T;
  p.N = N; p.T = int(T); p.HK = int(HK); p.HV = int(HV); p.V = int(V); p.nvb = int(nvb);
  p.beta_is_f32 = f.beta_is_f32; p.grads_f32 = gdt == FLA_F32;
  p.scale = a->scale;
  p.status = f.status;

  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(workspace, 0, 256, cs) != cudaSuccess) return FLA_ERR_CUDA;
  const int nt_max = (max_len + kC - 1) / kC;
  if (!have_saved && (st = kda_launch_forward(f, nt_max, cs))) return st;
  static std::atomic<bool> attr_done_dev[64] = {};   // per device ordinal; setting the attributes twice is harmless
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FLA_ERR_CUDA;
  if (!attr_done_dev[dev]) {
    if (cudaFuncSetAttribute(kda_bwd_dhu_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kKdaDhuSmem) + 1024) != cudaSuccess) return FLA_ERR_CUDA;
    if (cudaFuncSetAttribute(kda_bwd_par_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kKdaParSmem) + 1024) != cudaSuccess) return FLA_ERR_CUDA;
    if (cudaFuncSetAttribute(kda_bwd_par_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kKdaParSmem) + 1024) != cudaSuccess) return FLA_ERR_CUDA;
    attr_done_dev[dev] = true;
  }
  CUtensorMap tm_gk;
  if (make_row_tile_map_f32(&tm_gk, p.gk, kK, uint64_t(HV), uint64_t(B * T), uint64_t(kK), uint64_t(HV) * kK)) return FLA_ERR_CUDA;
  auto launch_scan = [&](const KdaBwdParams& pp, int nseq, cudaStream_t st_) {
    kda_bwd_dhu_kernel<<<dim3(unsigned(nvb), unsigned(HV), nseq), 256, kKdaDhuSmem + 1024, st_>>>(pp);
  };
  auto launch_par = [&](const KdaBwdParams& pp, int nseq, cudaStream_t st_) {
    if (nvb == 2) kda_bwd_par_kernel<2><<<dim3(nt_max, unsigned(HK), nseq), 256, kKdaParSmem + 1024, st_>>>(pp, tm_gk);
    else kda_bwd_par_kernel<4><<<dim3(nt_max, unsigned(HK), nseq), 256, kKdaParSmem + 1024, st_>>>(pp, tm_gk);
  };
  // more scan chains (one CTA per SM each) than SMs: two halves of the batch on two streams, so that the chunk-parallel
  // kernel of the first half fills the SMs the second half's scan leaves idle (aux_stream.h)
  AuxStream* aux = nullptr;
  if (N >= 2 && int64_t(nvb) * HV * N > sm_count(dev) && !kernel_timing_enabled()) aux = aux_stream_for(dev, cs);
  if (aux) {
    std::lock_guard<std::mutex> lk(aux->mu);
    const int n1 = N / 2;
    KdaBwdParams p2 = p;
    p2.n0 = n1;
    if (cudaEventRecord(aux->fork, cs) != cudaSuccess || cudaStreamWaitEvent(aux->s, aux->fork, 0) != cudaSuccess) return FLA_ERR_CUDA;
    launch_scan(p, n1, cs);
    launch_scan(p2, N - n1, aux->s);
    launch_par(p, n1, cs);
    launch_par(p2, N - n1, aux->s);
    if (cudaEventRecord(aux->join, aux->s) != cudaSuccess || cudaStreamWaitEvent(cs, aux->join, 0) != cudaSuccess) return FLA_ERR_CUDA;
    return cuda_status(cudaGetLastError());
  }
  {
    KernelTimer kt("kda_bwd_dhu", cs);
    launch_scan(p, N, cs);
  }
  if (cudaGetLastError() != cudaSuccess) return FLA_ERR_CUDA;
  {
    KernelTimer kt("kda_bwd_par", cs);
    launch_par(p, N, cs);
  }
  return cuda_status(cudaGetLastError());
}


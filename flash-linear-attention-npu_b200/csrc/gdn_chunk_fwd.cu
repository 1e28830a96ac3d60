// Chunked gated-delta-rule forward (chunk = 64 tokens, K = V = 128) as two kernels:
//
//  gdn_prep_kernel   (parallel over chunks): gam = chunk-local cumsum(g);
//                    A[i,j] = beta_i exp(gam_i - gam_j) k_i.k_j (j < i);  X = (I + A)^-1
//                    KK^T on tcgen05 (shared by the value heads of a GVA group); the unit-lower
//                    triangular inverse runs in tri_inverse_kernel (fp32 forward substitution on CUDA cores).
//                    Replaces chunk_local_cumsum + chunk_scaled_dot_kkt + solve_tri of the reference
//                    (examples/flash_gated_delta_rule.py:811-838).
//  gdn_scan_fwd_kernel (gdn_scan_fwd.cuh; sequential over chunks, one CTA per (sequence, value head, 128-column block of V)):
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
  bf16* X;             // [chunks, HV, 2, 8 x 64 x 8]  the chunk's (I + A)^-1 as value + residual strips (saved for backward)
  float* at;           // [chunks, HV, 64, 64] scratch: A^T handed to the triangular-inverse kernel
  bf16* p_img;         // [chunks, HV, kPImg]: tril(Q K^T * decay) as value / residual strips, then the chunk's factor record (reused by backward)
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

}  // namespace fla
#include "gdn_scan_fwd.cuh"
namespace fla {

// --------------------------------------------------------------------------------------------- prep
// One CTA per (chunk, q/k head).  One M = 128 product [q; k] k^T leaves Q K^T in TMEM lanes 0..63 and K K^T in
// lanes 64..127.  Eight warps: warp w reads lane quadrant w % 4 and the half w / 4 of the 64 columns, so a thread keeps
// half a row (32 values) in registers; per value head of the GVA group the q-side threads emit their half of
// P = tril(Q K^T * e^{gam_i - gam_j}) as split operand panels and the k-side threads their half of A^T.  (With four warps
// and whole rows per thread the kernel took 0.245 ms at the benchmark shape: it is a chain of latencies, and half the
// work per thread at twice the warps per SM shortens it.)
constexpr int kPrepThreads = 256;
__global__ void __launch_bounds__(kPrepThreads, 4) gdn_prep_kernel(GdnFwdParams p) {
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
    uint4 val[8];   // all loads in flight before the first one is consumed
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = tid + i * kPrepThreads, r = (idx / 16) & 63, ch = idx % 16;
      const bool isk = idx >= 1024;
      val[i] = make_uint4(0, 0, 0, 0);
      if (r < rows) {
        const bf16* src = isk ? p.k + (tok0 + r) * p.k_st + hk * p.k_sh : p.q + (tok0 + r) * p.q_st + hk * p.q_sh;
        val[i] = *reinterpret_cast<const uint4*>(src + ch * 8);
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int idx = tid + i * kPrepThreads, r = ((idx / 16) & 63) + (idx >= 1024 ? 64 : 0), ch = idx % 16;
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
  const int quad = warp & 3, half = warp >> 2;
  const int row = quad * 32 + lane;                 // accumulator row == TMEM lane
  const bool kside = row >= 64;
  const int tok = row & 63;
  const int j0 = half * 32;                         // my 32 columns
  // the gate / beta values of a head are requested one head ahead (and those of the first head before the product is waited for)
  auto fetch_g = [&](int hv) { return (warp < 2 && tok < rows) ? ld_scalar(p.g, (tok0 + tok) * p.g_st + hv, p.g_is_f32) : 0.f; };
  auto fetch_b = [&](int hv) { return (kside && tok < rows) ? ld_scalar(p.beta, (tok0 + tok) * p.beta_st + hv, p.beta_is_f32) : 0.f; };
  float g_next = fetch_g(hk * G), b_next = fetch_b(hk * G);
  const bool ok = mbar_wait(&bar, 0, p.status, FLA_ERR_TIMEOUT);
  tc_fence_after();
  float sc[32];   // my half of row `tok` of Q K^T (q side) or K K^T (k side)
  if (ok) {
    tmem_ld32(tmem_addr(tbase, quad * 32, j0), sc);
    tmem_ld_wait();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 64);
  if (!ok) return;

  for (int h = 0; h < G; ++h) {
    const int hv = hk * G + h;
    const int64_t cidx = (int64_t(sq.cbase) + blockIdx.x) * p.HV + hv;
    // chunk-local cumulative sum of g (warps 0 and 1: the q-side rows of the first column half)
    float gv = g_next;
    const float bi = b_next;
    if (h + 1 < G) {
      g_next = fetch_g(hv + 1);
      b_next = fetch_b(hv + 1);
    }
    if (warp < 2) {
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, gv, o);
        if (lane >= o) gv += up;
      }
      if (lane == 31) wsum_s[warp] = gv;
    }
    __syncthreads();
    if (warp < 2) {
      if (warp == 1) gv += wsum_s[0];
      gam_s[tok] = gv;
      if (tok < rows) p.gam[(tok0 + tok) * p.HV + hv] = gv;
    }
    __syncthreads();
    const float gam_i = gam_s[tok];
    if (!kside) {
      // my half of the P row as split bf16, in strips of 8 columns ([j / 8][row i][16 bytes], value then residual): the 16
      // bytes a thread stores for a strip lie next to its neighbours' (512 contiguous bytes per warp store), and the scans
      // read the image as an operand with the reduction along j (forward) or along i (reverse) by the descriptor alone
      uint8_t* img = reinterpret_cast<uint8_t*>(p.p_img + cidx * kPImg);
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        float t[8];
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          const int j = j0 + ch * 8 + jj;
          const float e = __expf(fminf(gam_i - gam_s[j], 0.f));
          t[jj] = sc[ch * 8 + jj] * ((j <= tok) ? e : 0.f);
        }
        uint4 hi, lo;
        split8(t, hi, lo);
        const uint32_t off = uint32_t(half * 4 + ch) * 1024u + uint32_t(tok) * 16u;
        *reinterpret_cast<uint4*>(img + off) = hi;
        *reinterpret_cast<uint4*>(img + 8192 + off) = lo;
      }
    } else {
      if (half == 0) {   // the chunk's per-token factors for the scans, behind the P tile (rows past the end: beta = 0, gam = gam_L)
        ScanFactors* f = reinterpret_cast<ScanFactors*>(reinterpret_cast<uint8_t*>(p.p_img + cidx * kPImg) + kPTileBytes);
        const float eg = __expf(gam_i), gl = gam_s[rows - 1];
        f->b[tok] = bi;
        f->bg[tok] = bi * eg;
        f->se[tok] = p.scale * eg;
        f->dk[tok] = __expf(gl - gam_i);
        if (tok == 0) f->dl = __expf(gl);
      }
      // A^T[j][i] = beta_i exp(gam_i - gam_j) (k_i . k_j) for j < i, written coalesced along i
      float* at = p.at + cidx * (kC * kC);
#pragma unroll
      for (int jl = 0; jl < 32; ++jl) {
        const int j = j0 + jl;
        if (j < tok) at[j * kC + tok] = bi * __expf(gam_i - gam_s[j]) * sc[jl];
      }
    }
    __syncthreads();
  }
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
  *bytes = 256 + uint64_t(chunks) * a->v.shape[2] * (kC * kC * 4 + (a->p_img.data ? 0 : kPImgBytes));
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
  if (X.dtype != FLA_BF16 || X.ndim != 1 || X.shape[0] != total_chunks * HV * 8192 || !aligned16(X.data))
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
    if (workspace_bytes < 256 + per * (kC * kC * 4 + (a->p_img.data ? 0 : kPImgBytes))) return FLA_ERR_WORKSPACE;
    p.at = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + 256);
    if (a->p_img.data) {
      const fla_tensor_t& pi = a->p_img;
      if (pi.dtype != FLA_BF16 || pi.ndim != 1 || pi.shape[0] != int64_t(per) * kPImg || !aligned16(pi.data)) return FLA_ERR_SHAPE;
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
    if (cudaFuncSetAttribute(gdn_scan_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kScanFwdSmem) + 1024) != cudaSuccess) return FLA_ERR_CUDA;
    if (cudaFuncSetAttribute(gdn_scan_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kScanFwdSmem) + 1024) != cudaSuccess) return FLA_ERR_CUDA;
    attr_done = true;
  }
  const int nt_max = (max_len + kC - 1) / kC;
  {
    KernelTimer kt("gdn_prep", cs);
    gdn_prep_kernel<<<dim3(nt_max, unsigned(HK), N), kPrepThreads, prep_smem, cs>>>(p);
  }
  if (cudaGetLastError() != cudaSuccess) return FLA_ERR_CUDA;
  {
    KernelTimer kt("tri_inverse", cs);
    TriInverseParams tp{p.at, nullptr, p.X, nullptr, nullptr, p.cu_seqlens, p.chunk_offsets, p.T, p.HV, 0};
    if (launch_tri_inverse(tp, nt_max, N, cs)) return FLA_ERR_CUDA;
  }
  CUtensorMap tm_q, tm_k;
  if (make_row_tile_map(&tm_q, p.q, kK, uint64_t(HK), uint64_t(B * T), uint64_t(p.q_sh), uint64_t(p.q_st)) ||
      make_row_tile_map(&tm_k, p.k, kK, uint64_t(HK), uint64_t(B * T), uint64_t(p.k_sh), uint64_t(p.k_st)))
    return FLA_ERR_CUDA;
  CUtensorMap tm_v;
  if (make_row_tile_map(&tm_v, p.v, uint64_t(V), uint64_t(HV), uint64_t(B * T), uint64_t(p.v_sh), uint64_t(p.v_st))) return FLA_ERR_CUDA;
  {
    KernelTimer kt("gdn_fwd", cs);
    const dim3 grid(unsigned(V / 128), unsigned(HV), N);
    if (p.s_img) gdn_scan_fwd_kernel<true><<<grid, kFwdThreads, kScanFwdSmem + 1024, cs>>>(p, tm_q, tm_k, tm_v);
    else gdn_scan_fwd_kernel<false><<<grid, kFwdThreads, kScanFwdSmem + 1024, cs>>>(p, tm_q, tm_k, tm_v);
  }
  return cuda_status(cudaGetLastError());
}



// The head-major intermediates of the reference's low-level KDA forward, npu_chunk_kda_fwd with disable_recompute /
// return_intermediate_states (torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:1066-1265, visibility rule
// _kda_policy.py:15-37; definitions in the golden tests/atk/chunk_kda_fwd/executor_chunk_kda_fwd.py:447-492):
//     qg = q 2^{gk}      kg = k 2^{gk_last - gk}      w = Akk (beta k 2^{gk})      u = Akk (beta v)
//     v_new = u - w S    h  = S, the state at the start of each chunk
// The fused forward never forms w and u and keeps S, v_new only as operand images of its `saved` buffer.  This kernel
// runs after it, chunk-parallel on CUDA cores in fp32: w and u from the inverse image (value + residual panels), v_new
// and h read back from the saved images (h = diag(e^-a) Sa undoes the per-channel anchor the forward applies), qg and kg
// from q, k and the saved cumulative gate.  An export path: nothing of it runs unless a caller asks for these tensors.
#include <cuda_fp16.h>
#include <atomic>
#include "gdn_common.cuh"
#include "fla_b200_internal.h"
#include "kernel_timer.h"
#include "kda_common.cuh"

namespace fla {
namespace {

struct OutView {
  void* p; int dtype; int64_t sb, st, sh;
};
struct InView {
  const bf16* p; int64_t sb, st, sh;
};

struct KdaInterParams {
  InView q, k, v;
  const void* beta; int beta_is_f32; int64_t beta_sb, beta_st, beta_sh;
  const float* gk;        // [tokens, HV, K] chunk-local cumulative gate (natural log) of the saved buffer
  const bf16* x_img;      // (I + Akk)^-1 per (chunk, head): value + residual panels
  const float* vec;       // per (chunk, head): e^a, e^{gk_L - a}, a
  const bf16* s_img;      // Sa = diag(e^a) S per (chunk, head, 64-column block of V): value + residual panels
  const bf16* vn_img;     // v_new per (chunk, head, block): value + residual panels
  OutView w, u, qg, kg, vn;
  void* h; int h_dtype, h_vfirst;
  const int32_t* cu_seqlens; const int32_t* chunk_offsets;
  int T, HK, HV, V, nvb;
};

__device__ __forceinline__ void put(void* p, int dtype, int64_t idx, float x) {
  if (dtype == FLA_F32) static_cast<float*>(p)[idx] = x;
  else if (dtype == FLA_F16) static_cast<__half*>(p)[idx] = __float2half_rn(x);
  else static_cast<bf16*>(p)[idx] = __float2bfloat16_rn(x);
}
__device__ __forceinline__ float panel_val(const uint8_t* hi, uint32_t lo_off, int row, int col) {
  const uint32_t o = panel_off(row, col);
  return __bfloat162float(*reinterpret_cast<const bf16*>(hi + o)) + __bfloat162float(*reinterpret_cast<const bf16*>(hi + lo_off + o));
}

constexpr int kInterSmem = (kC * kC + kC * 128) * 4;   // X^T and one 64 x 128 right-hand side, fp32

// out[i][c] = sum_j X[i][j] rhs[j][c] for this thread's column c and 32 rows; X is lower triangular (zeros above it are stored)
__device__ __forceinline__ void tri_apply(const float* xt, const float* rhs, int c, int ih, float* acc) {
#pragma unroll
  for (int r = 0; r < 32; ++r) acc[r] = 0.f;
  for (int j = 0; j < kC; ++j) {
    const float b = rhs[j * 128 + c];
    const float4* xr = reinterpret_cast<const float4*>(xt + j * kC + ih * 32);
#pragma unroll
    for (int r4 = 0; r4 < 8; ++r4) {
      const float4 x4 = xr[r4];
      acc[4 * r4] += x4.x * b; acc[4 * r4 + 1] += x4.y * b; acc[4 * r4 + 2] += x4.z * b; acc[4 * r4 + 3] += x4.w * b;
    }
  }
}

__global__ void __launch_bounds__(256) kda_intermediates_kernel(KdaInterParams p) {
  extern __shared__ float inter_smem[];
  float* xt = inter_smem;               // xt[j * 64 + i] = X[i][j]
  float* rhs = inter_smem + kC * kC;    // rhs[j * 128 + c]
  __shared__ float beta_s[kC], ea_s[kK];
  const int tid = threadIdx.x;
  const int n = blockIdx.z, hv = blockIdx.y, c = blockIdx.x;
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  if (c >= sq.nt) return;
  const int rows = min(kC, sq.len - c * kC);
  const int hk = hv / (p.HV / p.HK);
  const int64_t b = p.cu_seqlens ? 0 : n;
  const int64_t t0 = (p.cu_seqlens ? sq.bos : 0) + c * kC;      // first token of the chunk inside batch row b
  const int64_t flat0 = b * p.T + t0;                           // the same in the saved buffer's flat token order
  const int64_t chunk = int64_t(sq.cbase) + c;
  const int64_t cidx = chunk * p.HV + hv;
  const bool full = p.w.p || p.u.p || p.qg.p || p.kg.p;

  if (full) {
    const uint8_t* xi = reinterpret_cast<const uint8_t*>(p.x_img + cidx * kKdaXImg);
    for (int idx = tid; idx < kC * kC; idx += 256) {
      const int i = idx & 63, j = idx >> 6;
      xt[j * kC + i] = (i < rows && j < rows) ? panel_val(xi, 8192, i, j) : 0.f;
    }
    if (tid < kC)
      beta_s[tid] = tid < rows ? ld_scalar(p.beta, b * p.beta_sb + (t0 + tid) * p.beta_st + hv * p.beta_sh, p.beta_is_f32) : 0.f;
  }
  if (p.h && tid < kK) ea_s[tid] = expf(-p.vec[cidx * kKdaVecs * kK + 2 * kK + tid]);
  __syncthreads();

  const int col = tid & 127, ih = tid >> 7;
  if (full) {
    // qg, kg and the right-hand side beta k 2^{gk} of w
    const float* gkc = p.gk + (flat0 * p.HV + hv) * kK + col;
    const float g_last = gkc[int64_t(rows - 1) * p.HV * kK];
    for (int s = 0; s < 32; ++s) {
      const int t = ih + 2 * s;
      float r = 0.f;
      if (t < rows) {
        const float g = gkc[int64_t(t) * p.HV * kK];
        const float e = expf(g);
        const float qv = __bfloat162float(p.q.p[b * p.q.sb + (t0 + t) * p.q.st + hk * p.q.sh + col]);
        const float kv = __bfloat162float(p.k.p[b * p.k.sb + (t0 + t) * p.k.st + hk * p.k.sh + col]);
        if (p.qg.p) put(p.qg.p, p.qg.dtype, b * p.qg.sb + (t0 + t) * p.qg.st + hv * p.qg.sh + col, qv * e);
        if (p.kg.p) put(p.kg.p, p.kg.dtype, b * p.kg.sb + (t0 + t) * p.kg.st + hv * p.kg.sh + col, kv * expf(g_last - g));
        r = beta_s[t] * kv * e;
      }
      rhs[t * 128 + col] = r;
    }
    __syncthreads();
    float acc[32];
    if (p.w.p) {
      tri_apply(xt, rhs, col, ih, acc);
#pragma unroll
      for (int r = 0; r < 32; ++r)
        if (ih * 32 + r < rows) put(p.w.p, p.w.dtype, b * p.w.sb + (t0 + ih * 32 + r) * p.w.st + hv * p.w.sh + col, acc[r]);
    }
    if (p.u.p) {
      for (int vh = 0; vh < p.V / 128; ++vh) {   // u = Akk (beta v), 128 value channels at a time
        __syncthreads();
        for (int s = 0; s < 32; ++s) {
          const int t = ih + 2 * s;
          rhs[t * 128 + col] = t < rows ? beta_s[t] * __bfloat162float(p.v.p[b * p.v.sb + (t0 + t) * p.v.st + hv * p.v.sh + vh * 128 + col]) : 0.f;
        }
        __syncthreads();
        tri_apply(xt, rhs, col, ih, acc);
#pragma unroll
        for (int r = 0; r < 32; ++r)
          if (ih * 32 + r < rows)
            put(p.u.p, p.u.dtype, b * p.u.sb + (t0 + ih * 32 + r) * p.u.st + hv * p.u.sh + vh * 128 + col, acc[r]);
      }
    }
  }
  // v_new and h straight from the saved images
  for (int vb = 0; vb < p.nvb; ++vb) {
    if (p.vn.p) {
      const uint8_t* img = reinterpret_cast<const uint8_t*>(p.vn_img + (cidx * p.nvb + vb) * kKdaVnImg);
      for (int idx = tid; idx < kC * 64; idx += 256) {
        const int t = idx >> 6, ch = idx & 63;
        if (t < rows) put(p.vn.p, p.vn.dtype, b * p.vn.sb + (t0 + t) * p.vn.st + hv * p.vn.sh + vb * 64 + ch, panel_val(img, 8192, t, ch));
      }
    }
    if (p.h) {
      const uint8_t* img = reinterpret_cast<const uint8_t*>(p.s_img + (cidx * p.nvb + vb) * kKdaSImg);
      for (int idx = tid; idx < kK * 64; idx += 256) {
        const int kd = idx >> 6, ch = idx & 63;
        const float x = panel_val(img, 16384, kd, ch) * ea_s[kd];
        const int64_t o = p.h_vfirst ? (cidx * p.V + vb * 64 + ch) * kK + kd : (cidx * kK + kd) * p.V + vb * 64 + ch;
        put(p.h, p.h_dtype, o, x);
      }
    }
  }
}

bool in_view(const fla_tensor_t& t, int64_t B, int64_t T, int64_t H, int64_t D, InView* v) {
  if (!t.data || t.ndim != 4 || t.dtype != FLA_BF16 || t.shape[0] != B || t.shape[1] != T || t.shape[2] != H || t.shape[3] != D ||
      t.stride[3] != 1)
    return false;
  *v = InView{static_cast<const bf16*>(t.data), t.stride[0], t.stride[1], t.stride[2]};
  return true;
}
int out_view(const fla_tensor_t& t, int64_t B, int64_t T, int64_t H, int64_t D, OutView* v) {
  *v = OutView{nullptr, 0, 0, 0, 0};
  if (!t.data) return FLA_OK;
  if (t.ndim != 4 || t.shape[0] != B || t.shape[1] != T || t.shape[2] != H || t.shape[3] != D || t.stride[3] != 1) return FLA_ERR_SHAPE;
  if (t.dtype != FLA_BF16 && t.dtype != FLA_F16 && t.dtype != FLA_F32) return FLA_ERR_DTYPE;
  *v = OutView{t.data, t.dtype, t.stride[0], t.stride[1], t.stride[2]};
  return FLA_OK;
}

}  // namespace
}  // namespace fla

extern "C" FLA_API int fla_b200_kda_chunk_intermediates(const fla_kda_intermediates_args* a, void* stream) {
  using namespace fla;
  if (!a) return FLA_ERR_NULL;
  if (!a->q.data || !a->k.data || !a->v.data || !a->beta.data || !a->saved.data) return FLA_ERR_NULL;
  if (a->q.ndim != 4 || a->v.ndim != 4) return FLA_ERR_SHAPE;
  const int64_t B = a->q.shape[0], T = a->q.shape[1], HK = a->q.shape[2], HV = a->v.shape[2], V = a->v.shape[3];
  if (a->q.shape[3] != kK || (V != 128 && V != 256) || HK <= 0 || HV % HK) return FLA_ERR_SHAPE;
  KdaInterParams p{};
  if (!in_view(a->q, B, T, HK, kK, &p.q) || !in_view(a->k, B, T, HK, kK, &p.k) || !in_view(a->v, B, T, HV, V, &p.v)) return FLA_ERR_SHAPE;
  const fla_tensor_t& be = a->beta;
  if (be.ndim != 3 || be.shape[0] != B || be.shape[1] != T || be.shape[2] != HV) return FLA_ERR_SHAPE;
  if (be.dtype != FLA_F32 && be.dtype != FLA_BF16) return FLA_ERR_DTYPE;
  p.beta = be.data; p.beta_is_f32 = be.dtype == FLA_F32; p.beta_sb = be.stride[0]; p.beta_st = be.stride[1]; p.beta_sh = be.stride[2];
  int N = int(B), max_len = int(T);
  int64_t total_chunks = B * ((T + kC - 1) / kC);
  if (a->cu_seqlens.data) {
    if (B != 1 || a->cu_seqlens.dtype != FLA_I32 || a->cu_seqlens.ndim != 1 || a->cu_seqlens.shape[0] < 2) return FLA_ERR_SHAPE;
    N = int(a->cu_seqlens.shape[0] - 1);
    if (!a->chunk_offsets.data || a->chunk_offsets.dtype != FLA_I32 || a->chunk_offsets.shape[0] != N + 1) return FLA_ERR_SHAPE;
    if (a->max_seqlen <= 0 || a->max_seqlen > T || a->total_chunks <= 0) return FLA_ERR_VALUE;
    max_len = a->max_seqlen;
    total_chunks = a->total_chunks;
  }
  const int64_t nvb = V / 64;
  uint64_t soff[4], woff[6];
  const uint64_t sbytes = kda_saved_layout(total_chunks, HV, nvb, B * T, soff);
  kda_ws_layout(total_chunks, HV, woff);
  if (a->saved.dtype != FLA_BF16 || a->saved.ndim != 1 || uint64_t(a->saved.shape[0]) * 2 < sbytes || !aligned16(a->saved.data))
    return FLA_ERR_SHAPE;
  const uint8_t* sv = static_cast<const uint8_t*>(a->saved.data);
  p.x_img = reinterpret_cast<const bf16*>(sv + soff[0] + woff[3]);
  p.vec = reinterpret_cast<const float*>(sv + soff[0] + woff[4]);
  p.gk = reinterpret_cast<const float*>(sv + soff[1]);
  p.s_img = reinterpret_cast<const bf16*>(sv + soff[2]);
  p.vn_img = reinterpret_cast<const bf16*>(sv + soff[3]);
  int st;
  if ((st = out_view(a->w, B, T, HV, kK, &p.w)) || (st = out_view(a->u, B, T, HV, V, &p.u)) || (st = out_view(a->qg, B, T, HV, kK, &p.qg)) ||
      (st = out_view(a->kg, B, T, HV, kK, &p.kg)) || (st = out_view(a->v_new, B, T, HV, V, &p.vn)))
    return st;
  if (a->h.data) {
    const fla_tensor_t& h = a->h;
    const int64_t r = a->state_v_first ? V : kK, cdim = a->state_v_first ? kK : V;
    if (h.ndim != 4 || h.shape[0] != total_chunks || h.shape[1] != HV || h.shape[2] != r || h.shape[3] != cdim) return FLA_ERR_SHAPE;
    if (h.stride[3] != 1 || h.stride[2] != cdim || h.stride[1] != r * cdim || h.stride[0] != HV * r * cdim) return FLA_ERR_LAYOUT;
    if (h.dtype != FLA_BF16 && h.dtype != FLA_F16 && h.dtype != FLA_F32) return FLA_ERR_DTYPE;
    p.h = h.data; p.h_dtype = h.dtype; p.h_vfirst = a->state_v_first != 0;
  }
  if (!p.w.p && !p.u.p && !p.qg.p && !p.kg.p && !p.vn.p && !p.h) return FLA_OK;
  p.cu_seqlens = static_cast<const int32_t*>(a->cu_seqlens.data);
  p.chunk_offsets = static_cast<const int32_t*>(a->chunk_offsets.data);
  p.T = int(T); p.HK = int(HK); p.HV = int(HV); p.V = int(V); p.nvb = int(nvb);

  static std::atomic<bool> attr_done_dev[64] = {};   // per device ordinal; setting the attribute twice is harmless
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FLA_ERR_CUDA;
  if (!attr_done_dev[dev]) {
    if (cudaFuncSetAttribute(kda_intermediates_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kInterSmem) != cudaSuccess) return FLA_ERR_CUDA;
    attr_done_dev[dev] = true;
  }
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const int nt_max = (max_len + kC - 1) / kC;
  KernelTimer kt("kda_intermediates", cs);
  kda_intermediates_kernel<<<dim3(nt_max, unsigned(HV), N), 256, kInterSmem, cs>>>(p);
  return cuda_status(cudaGetLastError());
}

// ------------------------------------------------------------------------------------------------------------------
// Score blocks of 128-token chunks from those of the 64-token chunks the kernels work in (npu_chunk_kda_fwd takes
// chunk_size 64 or 128, _aclnn_ctypes.py:1094-1096).  With A the first and B the second half of a 128-token chunk,
// gk the 64-token cumulative gate and L = gk at the last token of A (per channel):
//     gk128 = gk on A, gk + L on B
//     Aqk128 = [[Aqk_A, 0], [scale qg_B kg_A^T, Aqk_B]]          qg = q e^{gk},  kg = k e^{L - gk}  (all exponents <= 0)
//     Akk128 = [[X_A, 0], [-X_B M X_A, X_B]],  M = beta_B (k e^{gk})_B kg_A^T   (the inverse of a block-triangular matrix)
// One CTA per (128-token chunk, head), fp32 on CUDA cores: an export path like the kernel above.
namespace fla {
namespace {

struct KdaMergeParams {
  InView q, k;
  const void* beta; int beta_is_f32; int64_t beta_sb, beta_st, beta_sh;
  const float* gk;                 // [tokens, HV, K] cumulative gate of the 64-token chunks, dense
  float gk_unit;                   // 1 for a natural-log gate, ln 2 for a base-2 gate
  const float* aqk64; const float* akk64; int64_t a_sb, a_st, a_sh;   // [B, T, HV, 64] views, fp32
  OutView aqk, akk;                // [B, T, HV, 128] views
  float* gk_out; int64_t g_sb, g_st, g_sh;   // [B, T, HV, K] view, fp32, base 2
  const int32_t* cu_seqlens; const int32_t* chunk_offsets;
  int T, HK, HV;
  float scale;
};

constexpr int kMergeSmem = (3 * kC * kK + 4 * kC * kC) * 4;   // kgA, qgB, kqB rows; M, T, X_A, X_B tiles

__global__ void __launch_bounds__(256) kda_merge_blocks_kernel(KdaMergeParams p) {
  extern __shared__ float merge_smem[];
  float* kga = merge_smem;                 // [64][128]
  float* qgb = kga + kC * kK;
  float* kqb = qgb + kC * kK;
  float* m_kk = kqb + kC * kK;             // [64][64]  beta_i (k e^gk)_i . kg_j
  float* tmp = m_kk + kC * kC;             // [64][64]  M X_A
  float* xa = tmp + kC * kC;               // [64][64]
  float* xb = xa + kC * kC;
  __shared__ float beta_s[kC];
  const int tid = threadIdx.x;
  const int n = blockIdx.z, hv = blockIdx.y, c2 = blockIdx.x;
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  if (2 * c2 >= sq.nt) return;
  const int hk = hv / (p.HV / p.HK);
  const int64_t b = p.cu_seqlens ? 0 : n;
  const int64_t t0 = (p.cu_seqlens ? sq.bos : 0) + int64_t(c2) * 128;   // first token of the 128-token chunk in batch row b
  const int64_t flat0 = b * p.T + t0;
  const int len = min(128, sq.len - c2 * 128);
  const int ra = min(kC, len), rb = len - ra;                            // tokens in the two halves
  const int col = tid & 127, par = tid >> 7;

  // gk128, and the operands of the two products
  const float* gkc = p.gk + (flat0 * p.HV + hv) * kK + col;
  const float L = gkc[int64_t(ra - 1) * p.HV * kK] * p.gk_unit;
  for (int s = 0; s < 64; ++s) {
    const int t = par + 2 * s;            // 0..127
    if (t >= len) break;
    const float g = gkc[int64_t(t) * p.HV * kK] * p.gk_unit;
    const float g128 = t < kC ? g : g + L;
    if (p.gk_out) p.gk_out[b * p.g_sb + (t0 + t) * p.g_st + hv * p.g_sh + col] = g128 * 1.4426950408889634f;
    const float kv = __bfloat162float(p.k.p[b * p.k.sb + (t0 + t) * p.k.st + hk * p.k.sh + col]);
    if (t < kC) {
      kga[t * kK + col] = kv * expf(L - g);
    } else {
      const float e = expf(g);
      qgb[(t - kC) * kK + col] = __bfloat162float(p.q.p[b * p.q.sb + (t0 + t) * p.q.st + hk * p.q.sh + col]) * e;
      kqb[(t - kC) * kK + col] = kv * e;
    }
  }
  if (tid < kC) beta_s[tid] = tid < rb ? ld_scalar(p.beta, b * p.beta_sb + (t0 + kC + tid) * p.beta_st + hv * p.beta_sh, p.beta_is_f32) : 0.f;
  // the 64-token blocks (zero outside the valid rows / columns)
  for (int idx = tid; idx < kC * kC; idx += 256) {
    const int i = idx >> 6, j = idx & 63;
    xa[idx] = (i < ra && j < ra) ? p.akk64[b * p.a_sb + (t0 + i) * p.a_st + hv * p.a_sh + j] : 0.f;
    xb[idx] = (i < rb && j < rb) ? p.akk64[b * p.a_sb + (t0 + kC + i) * p.a_st + hv * p.a_sh + j] : 0.f;
  }
  __syncthreads();

  // rows of the first half: [block | 0]
  for (int idx = tid; idx < kC * 128; idx += 256) {
    const int i = idx >> 7, j = idx & 127;
    if (i >= ra) continue;
    const int64_t o = b * p.aqk.sb + (t0 + i) * p.aqk.st + hv * p.aqk.sh + j;
    const int64_t o2 = b * p.akk.sb + (t0 + i) * p.akk.st + hv * p.akk.sh + j;
    put(p.aqk.p, p.aqk.dtype, o, (j < ra) ? p.aqk64[b * p.a_sb + (t0 + i) * p.a_st + hv * p.a_sh + j] : 0.f);
    put(p.akk.p, p.akk.dtype, o2, (j < ra) ? xa[i * kC + j] : 0.f);
  }
  if (rb <= 0) return;

  // off-diagonal blocks: thread (j = tid & 63, rows i = (tid >> 6) * 16 .. + 16)
  {
    const int j = tid & 63, i0 = (tid >> 6) * 16;
    float aq[16], ak[16];
#pragma unroll
    for (int r = 0; r < 16; ++r) aq[r] = ak[r] = 0.f;
    for (int k = 0; k < kK; ++k) {
      const float kg = kga[j * kK + ((k + j) & 127)];     // rotated channel order: the 32 lanes read 32 different banks
      const int kk = (k + j) & 127;
#pragma unroll
      for (int r = 0; r < 16; ++r) {
        aq[r] += qgb[(i0 + r) * kK + kk] * kg;
        ak[r] += kqb[(i0 + r) * kK + kk] * kg;
      }
    }
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      const int i = i0 + r;
      const bool live = i < rb && j < ra;
      m_kk[i * kC + j] = live ? beta_s[i] * ak[r] : 0.f;
      if (i < rb) put(p.aqk.p, p.aqk.dtype, b * p.aqk.sb + (t0 + kC + i) * p.aqk.st + hv * p.aqk.sh + j, live ? p.scale * aq[r] : 0.f);
    }
  }
  __syncthreads();
  // tmp = M X_A, then X_21 = -X_B tmp
  {
    const int j = tid & 63, i0 = (tid >> 6) * 16;
    float acc[16];
#pragma unroll
    for (int r = 0; r < 16; ++r) acc[r] = 0.f;
    for (int k = 0; k < kC; ++k) {
      const float x = xa[k * kC + j];
#pragma unroll
      for (int r = 0; r < 16; ++r) acc[r] += m_kk[(i0 + r) * kC + k] * x;
    }
#pragma unroll
    for (int r = 0; r < 16; ++r) tmp[(i0 + r) * kC + j] = acc[r];
    __syncthreads();
#pragma unroll
    for (int r = 0; r < 16; ++r) acc[r] = 0.f;
    for (int k = 0; k < kC; ++k) {
      const float x = tmp[k * kC + j];
#pragma unroll
      for (int r = 0; r < 16; ++r) acc[r] += xb[(i0 + r) * kC + k] * x;
    }
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      const int i = i0 + r;
      if (i < rb) put(p.akk.p, p.akk.dtype, b * p.akk.sb + (t0 + kC + i) * p.akk.st + hv * p.akk.sh + j, j < ra ? -acc[r] : 0.f);
    }
  }
  // rows of the second half, columns 64..127: the block of the second 64-token chunk
  for (int idx = tid; idx < kC * kC; idx += 256) {
    const int i = idx >> 6, j = idx & 63;
    if (i >= rb) continue;
    put(p.aqk.p, p.aqk.dtype, b * p.aqk.sb + (t0 + kC + i) * p.aqk.st + hv * p.aqk.sh + kC + j,
        (j < rb) ? p.aqk64[b * p.a_sb + (t0 + kC + i) * p.a_st + hv * p.a_sh + j] : 0.f);
    put(p.akk.p, p.akk.dtype, b * p.akk.sb + (t0 + kC + i) * p.akk.st + hv * p.akk.sh + kC + j, (j < rb) ? xb[i * kC + j] : 0.f);
  }
}

}  // namespace
}  // namespace fla

extern "C" FLA_API int fla_b200_kda_merge_score_blocks(const fla_kda_merge_blocks_args* a, void* stream) {
  using namespace fla;
  if (!a) return FLA_ERR_NULL;
  if (!a->q.data || !a->k.data || !a->beta.data || !a->gk.data || !a->aqk64.data || !a->akk64.data || !a->aqk.data || !a->akk.data)
    return FLA_ERR_NULL;
  if (a->q.ndim != 4 || a->gk.ndim != 4) return FLA_ERR_SHAPE;
  const int64_t B = a->q.shape[0], T = a->q.shape[1], HK = a->q.shape[2], HV = a->gk.shape[2];
  if (a->q.shape[3] != kK || HK <= 0 || HV % HK) return FLA_ERR_SHAPE;
  KdaMergeParams p{};
  if (!in_view(a->q, B, T, HK, kK, &p.q) || !in_view(a->k, B, T, HK, kK, &p.k)) return FLA_ERR_SHAPE;
  const fla_tensor_t& be = a->beta;
  if (be.ndim != 3 || be.shape[0] != B || be.shape[1] != T || be.shape[2] != HV) return FLA_ERR_SHAPE;
  if (be.dtype != FLA_F32 && be.dtype != FLA_BF16) return FLA_ERR_DTYPE;
  p.beta = be.data; p.beta_is_f32 = be.dtype == FLA_F32; p.beta_sb = be.stride[0]; p.beta_st = be.stride[1]; p.beta_sh = be.stride[2];
  const fla_tensor_t& gk = a->gk;
  if (gk.dtype != FLA_F32 || gk.shape[0] != B || gk.shape[1] != T || gk.shape[3] != kK || gk.stride[3] != 1 || gk.stride[2] != kK ||
      gk.stride[1] != HV * kK || (B > 1 && gk.stride[0] != T * HV * kK))
    return FLA_ERR_SHAPE;
  p.gk = static_cast<const float*>(gk.data);
  p.gk_unit = a->gk_base2 ? 0.6931471805599453f : 1.f;
  for (const fla_tensor_t* t : {&a->aqk64, &a->akk64}) {
    if (t->dtype != FLA_F32 || t->ndim != 4 || t->shape[0] != B || t->shape[1] != T || t->shape[2] != HV || t->shape[3] != kC || t->stride[3] != 1)
      return FLA_ERR_SHAPE;
  }
  if (a->aqk64.stride[0] != a->akk64.stride[0] || a->aqk64.stride[1] != a->akk64.stride[1] || a->aqk64.stride[2] != a->akk64.stride[2])
    return FLA_ERR_LAYOUT;
  p.aqk64 = static_cast<const float*>(a->aqk64.data); p.akk64 = static_cast<const float*>(a->akk64.data);
  p.a_sb = a->aqk64.stride[0]; p.a_st = a->aqk64.stride[1]; p.a_sh = a->aqk64.stride[2];
  int st;
  if ((st = out_view(a->aqk, B, T, HV, 128, &p.aqk)) || (st = out_view(a->akk, B, T, HV, 128, &p.akk))) return st;
  if (a->gk_out.data) {
    const fla_tensor_t& g = a->gk_out;
    if (g.dtype != FLA_F32 || g.ndim != 4 || g.shape[0] != B || g.shape[1] != T || g.shape[2] != HV || g.shape[3] != kK || g.stride[3] != 1)
      return FLA_ERR_SHAPE;
    p.gk_out = static_cast<float*>(g.data); p.g_sb = g.stride[0]; p.g_st = g.stride[1]; p.g_sh = g.stride[2];
  }
  int N = int(B), max_len = int(T);
  if (a->cu_seqlens.data) {
    if (B != 1 || a->cu_seqlens.dtype != FLA_I32 || a->cu_seqlens.ndim != 1 || a->cu_seqlens.shape[0] < 2) return FLA_ERR_SHAPE;
    N = int(a->cu_seqlens.shape[0] - 1);
    if (!a->chunk_offsets.data || a->chunk_offsets.dtype != FLA_I32 || a->chunk_offsets.shape[0] != N + 1) return FLA_ERR_SHAPE;
    if (a->max_seqlen <= 0 || a->max_seqlen > T) return FLA_ERR_VALUE;
    max_len = a->max_seqlen;
  }
  p.cu_seqlens = static_cast<const int32_t*>(a->cu_seqlens.data);
  p.chunk_offsets = static_cast<const int32_t*>(a->chunk_offsets.data);
  p.T = int(T); p.HK = int(HK); p.HV = int(HV); p.scale = a->scale;
  static std::atomic<bool> attr_done_dev[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FLA_ERR_CUDA;
  if (!attr_done_dev[dev]) {
    if (cudaFuncSetAttribute(kda_merge_blocks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMergeSmem) != cudaSuccess) return FLA_ERR_CUDA;
    attr_done_dev[dev] = true;
  }
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const int nt128 = (max_len + 127) / 128;
  KernelTimer kt("kda_merge_score_blocks", cs);
  kda_merge_blocks_kernel<<<dim3(nt128, unsigned(HV), N), 256, kMergeSmem, cs>>>(p);
  return cuda_status(cudaGetLastError());
}

// ------------------------------------------------------------------------------------------------------------------
// w, u, qg, kg of 128-token chunks from those of their 64-token halves A, B (same notation as above, XM = X_B M):
//     qg128 = qg on A, qg e^L on B                 kg128 = kg e^{gk_B,last} on A, kg on B
//     w128  = w on A,  w e^L - XM w_A on B          u128  = u on A,  u - XM u_A on B
// (row block B of Akk128 is [-X_B M X_A, X_B], and X_A applied to the right-hand sides of A is w_A, u_A.)
// v_new does not depend on the blocking and h keeps every second state, so neither passes through here.
namespace fla {
namespace {

struct F32View {
  const float* p; int64_t sb, st, sh;
};
struct KdaMergeInterParams {
  InView k;
  const void* beta; int beta_is_f32; int64_t beta_sb, beta_st, beta_sh;
  const float* gk; float gk_unit;
  F32View akk64, w64, u64, qg64, kg64;
  OutView w, u, qg, kg;
  const int32_t* cu_seqlens; const int32_t* chunk_offsets;
  int T, HK, HV, V;
};

constexpr int kMergeInterSmem = (2 * kC * kK + 3 * kC * kC) * 4;   // a 64 x 128 tile twice; M, X_B, XM

__global__ void __launch_bounds__(256) kda_merge_intermediates_kernel(KdaMergeInterParams p) {
  extern __shared__ float mi_smem[];
  float* ta = mi_smem;                  // [64][128]: kg_A, then the right-hand sides w_A / u_A
  float* tb = ta + kC * kK;             // [64][128]: (k e^{gk})_B
  float* m_kk = tb + kC * kK;           // [64][64]
  float* xb = m_kk + kC * kC;
  float* xm = xb + kC * kC;
  __shared__ float beta_s[kC], el_s[kK], eb_s[kK];
  const int tid = threadIdx.x;
  const int n = blockIdx.z, hv = blockIdx.y, c2 = blockIdx.x;
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  if (2 * c2 >= sq.nt) return;
  const int hk = hv / (p.HV / p.HK);
  const int64_t b = p.cu_seqlens ? 0 : n;
  const int64_t t0 = (p.cu_seqlens ? sq.bos : 0) + int64_t(c2) * 128;
  const int64_t flat0 = b * p.T + t0;
  const int len = min(128, sq.len - c2 * 128);
  const int ra = min(kC, len), rb = len - ra;
  const int col = tid & 127, par = tid >> 7;
  auto at = [&](const F32View& v, int t, int c) { return v.p[b * v.sb + (t0 + t) * v.st + hv * v.sh + c]; };
  auto to = [&](const OutView& v, int t, int c, float x) { put(v.p, v.dtype, b * v.sb + (t0 + t) * v.st + hv * v.sh + c, x); };

  const float* gkc = p.gk + (flat0 * p.HV + hv) * kK + col;
  if (tid < kK) {
    el_s[tid] = expf(gkc[int64_t(ra - 1) * p.HV * kK] * p.gk_unit);
    eb_s[tid] = rb > 0 ? expf(gkc[int64_t(len - 1) * p.HV * kK] * p.gk_unit) : 1.f;
  }
  if (tid < kC) beta_s[tid] = tid < rb ? ld_scalar(p.beta, b * p.beta_sb + (t0 + kC + tid) * p.beta_st + hv * p.beta_sh, p.beta_is_f32) : 0.f;
  for (int s = 0; s < 64; ++s) {
    const int t = par + 2 * s;
    if (t >= len) break;
    if (t < kC) {
      ta[t * kK + col] = at(p.kg64, t, col);
    } else {
      const float g = gkc[int64_t(t) * p.HV * kK] * p.gk_unit;
      tb[(t - kC) * kK + col] = __bfloat162float(p.k.p[b * p.k.sb + (t0 + t) * p.k.st + hk * p.k.sh + col]) * expf(g);
    }
  }
  for (int idx = tid; idx < kC * kC; idx += 256) {
    const int i = idx >> 6, j = idx & 63;
    xb[idx] = (i < rb && j < rb) ? at(p.akk64, kC + i, j) : 0.f;
  }
  __syncthreads();
  // the elementwise parts and the rows of A
  for (int s = 0; s < 64; ++s) {
    const int t = par + 2 * s;
    if (t >= len) break;
    if (p.qg.p) to(p.qg, t, col, at(p.qg64, t, col) * (t < kC ? 1.f : el_s[col]));
    if (p.kg.p) to(p.kg, t, col, at(p.kg64, t, col) * (t < kC ? eb_s[col] : 1.f));
    if (t < kC) {
      if (p.w.p) to(p.w, t, col, at(p.w64, t, col));
      if (p.u.p)
        for (int vh = 0; vh < p.V / 128; ++vh) to(p.u, t, vh * 128 + col, at(p.u64, t, vh * 128 + col));
    }
  }
  if (rb <= 0 || (!p.w.p && !p.u.p)) return;
  // M = beta_B (k e^gk)_B kg_A^T, then XM = X_B M
  {
    const int j = tid & 63, i0 = (tid >> 6) * 16;
    float ak[16];
#pragma unroll
    for (int r = 0; r < 16; ++r) ak[r] = 0.f;
    for (int k = 0; k < kK; ++k) {
      const int kk = (k + j) & 127;
      const float kg = ta[j * kK + kk];
#pragma unroll
      for (int r = 0; r < 16; ++r) ak[r] += tb[(i0 + r) * kK + kk] * kg;
    }
#pragma unroll
    for (int r = 0; r < 16; ++r) m_kk[(i0 + r) * kC + j] = (i0 + r < rb && j < ra) ? beta_s[i0 + r] * ak[r] : 0.f;
    __syncthreads();
    float acc[16];
#pragma unroll
    for (int r = 0; r < 16; ++r) acc[r] = 0.f;
    for (int k = 0; k < kC; ++k) {
      const float x = m_kk[k * kC + j];
#pragma unroll
      for (int r = 0; r < 16; ++r) acc[r] += xb[(i0 + r) * kC + k] * x;
    }
#pragma unroll
    for (int r = 0; r < 16; ++r) xm[(i0 + r) * kC + j] = acc[r];
  }
  // rows of B: out = own - XM rhs_A, 128 columns at a time (w first, then u)
  const int passes = (p.w.p ? 1 : 0) + (p.u.p ? p.V / 128 : 0);
  for (int ps = 0; ps < passes; ++ps) {
    const bool is_w = p.w.p && ps == 0;
    const int vh = ps - (p.w.p ? 1 : 0);
    __syncthreads();     // XM complete / the previous pass has read `ta`
    for (int s = 0; s < 32; ++s) {
      const int t = par + 2 * s;
      ta[t * kK + col] = t < ra ? (is_w ? at(p.w64, t, col) : at(p.u64, t, vh * 128 + col)) : 0.f;
    }
    __syncthreads();
    float acc[32];
#pragma unroll
    for (int r = 0; r < 32; ++r) acc[r] = 0.f;
    for (int j = 0; j < kC; ++j) {
      const float rj = ta[j * kK + col];
#pragma unroll
      for (int r = 0; r < 32; ++r) acc[r] += xm[(par * 32 + r) * kC + j] * rj;
    }
#pragma unroll
    for (int r = 0; r < 32; ++r) {
      const int i = par * 32 + r;
      if (i >= rb) continue;
      if (is_w) to(p.w, kC + i, col, at(p.w64, kC + i, col) * el_s[col] - acc[r]);
      else to(p.u, kC + i, vh * 128 + col, at(p.u64, kC + i, vh * 128 + col) - acc[r]);
    }
  }
}

bool f32_view(const fla_tensor_t& t, int64_t B, int64_t T, int64_t H, int64_t D, F32View* v) {
  if (!t.data || t.dtype != FLA_F32 || t.ndim != 4 || t.shape[0] != B || t.shape[1] != T || t.shape[2] != H || t.shape[3] != D || t.stride[3] != 1)
    return false;
  *v = F32View{static_cast<const float*>(t.data), t.stride[0], t.stride[1], t.stride[2]};
  return true;
}

}  // namespace
}  // namespace fla

extern "C" FLA_API int fla_b200_kda_merge_intermediates(const fla_kda_merge_inter_args* a, void* stream) {
  using namespace fla;
  if (!a) return FLA_ERR_NULL;
  if (!a->k.data || !a->beta.data || !a->gk.data || !a->akk64.data || !a->w64.data || !a->u64.data || !a->qg64.data || !a->kg64.data)
    return FLA_ERR_NULL;
  if (a->k.ndim != 4 || a->gk.ndim != 4 || a->u64.ndim != 4) return FLA_ERR_SHAPE;
  const int64_t B = a->k.shape[0], T = a->k.shape[1], HK = a->k.shape[2], HV = a->gk.shape[2], V = a->u64.shape[3];
  if (a->k.shape[3] != kK || HK <= 0 || HV % HK || (V != 128 && V != 256)) return FLA_ERR_SHAPE;
  KdaMergeInterParams p{};
  if (!in_view(a->k, B, T, HK, kK, &p.k)) return FLA_ERR_SHAPE;
  const fla_tensor_t& be = a->beta;
  if (be.ndim != 3 || be.shape[0] != B || be.shape[1] != T || be.shape[2] != HV) return FLA_ERR_SHAPE;
  if (be.dtype != FLA_F32 && be.dtype != FLA_BF16) return FLA_ERR_DTYPE;
  p.beta = be.data; p.beta_is_f32 = be.dtype == FLA_F32; p.beta_sb = be.stride[0]; p.beta_st = be.stride[1]; p.beta_sh = be.stride[2];
  const fla_tensor_t& gk = a->gk;
  if (gk.dtype != FLA_F32 || gk.shape[0] != B || gk.shape[1] != T || gk.shape[3] != kK || gk.stride[3] != 1 || gk.stride[2] != kK ||
      gk.stride[1] != HV * kK || (B > 1 && gk.stride[0] != T * HV * kK))
    return FLA_ERR_SHAPE;
  p.gk = static_cast<const float*>(gk.data);
  p.gk_unit = a->gk_base2 ? 0.6931471805599453f : 1.f;
  if (!f32_view(a->akk64, B, T, HV, kC, &p.akk64) || !f32_view(a->w64, B, T, HV, kK, &p.w64) || !f32_view(a->u64, B, T, HV, V, &p.u64) ||
      !f32_view(a->qg64, B, T, HV, kK, &p.qg64) || !f32_view(a->kg64, B, T, HV, kK, &p.kg64))
    return FLA_ERR_SHAPE;
  int st;
  if ((st = out_view(a->w, B, T, HV, kK, &p.w)) || (st = out_view(a->u, B, T, HV, V, &p.u)) || (st = out_view(a->qg, B, T, HV, kK, &p.qg)) ||
      (st = out_view(a->kg, B, T, HV, kK, &p.kg)))
    return st;
  int N = int(B), max_len = int(T);
  if (a->cu_seqlens.data) {
    if (B != 1 || a->cu_seqlens.dtype != FLA_I32 || a->cu_seqlens.ndim != 1 || a->cu_seqlens.shape[0] < 2) return FLA_ERR_SHAPE;
    N = int(a->cu_seqlens.shape[0] - 1);
    if (!a->chunk_offsets.data || a->chunk_offsets.dtype != FLA_I32 || a->chunk_offsets.shape[0] != N + 1) return FLA_ERR_SHAPE;
    if (a->max_seqlen <= 0 || a->max_seqlen > T) return FLA_ERR_VALUE;
    max_len = a->max_seqlen;
  }
  p.cu_seqlens = static_cast<const int32_t*>(a->cu_seqlens.data);
  p.chunk_offsets = static_cast<const int32_t*>(a->chunk_offsets.data);
  p.T = int(T); p.HK = int(HK); p.HV = int(HV); p.V = int(V);
  static std::atomic<bool> attr_done_dev[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FLA_ERR_CUDA;
  if (!attr_done_dev[dev]) {
    if (cudaFuncSetAttribute(kda_merge_intermediates_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMergeInterSmem) != cudaSuccess)
      return FLA_ERR_CUDA;
    attr_done_dev[dev] = true;
  }
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  KernelTimer kt("kda_merge_intermediates", cs);
  kda_merge_intermediates_kernel<<<dim3((max_len + 127) / 128, unsigned(HV), N), 256, kMergeInterSmem, cs>>>(p);
  return cuda_status(cudaGetLastError());
}

// Gate activation of Kimi Delta Attention and its gradient, for the differentiable path of chunk_kda with
// use_gate_in_kernel (semantics: fla/ops/ascendc/kda/chunk_kda_fwd/docs/api.md:103-115; the reference activates the gate
// inside aclnnKdaGateCumsum, torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:1268-1296):
//     mode 1:  gate = -e^{A_log[h]} softplus(g + dt_bias[h, :])
//     mode 2:  gate = lower_bound sigmoid(e^{A_log[h]} (g + dt_bias[h, :]))
// The inference path activates the gate inside kda_prep_kernel.  With gradients required the activated gate has to exist
// as a tensor (the backward kernels take it as given and return its gradient), so it is made here in one pass, and the
// backward turns d(gate) into d(g), d(A_log) and d(dt_bias) in one pass plus a fixed-order reduction (deterministic).
// Elementwise and HBM-bound: one CTA walks 256 tokens of one head, a thread owns one channel of every other token.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <algorithm>
#include "gdn_common.cuh"
#include "fla_b200_internal.h"
#include "kernel_timer.h"

namespace fla {
namespace {

constexpr int kGateTile = 256;   // tokens per CTA

struct KdaGateParams {
  const void* g; int g_dtype; int64_t g_st, g_sh;   // [tokens, HV, K] view of the raw gate
  const float* a_log; const float* dt_bias;
  float* gate;                                      // fwd out, [tokens, HV, K] dense
  const float* d_gate; int64_t dg_st, dg_sh;        // bwd in
  void* d_g; int d_g_dtype;                         // bwd out, dense, dtype of g
  float* partial;                                   // bwd scratch [tiles, HV, K + 1]: per-tile sums for dt_bias and A_log
  int64_t tokens;
  int HV, mode;
  float lower_bound;
};

__device__ __forceinline__ float load_any(const void* p, int dtype, int64_t i) {
  if (dtype == FLA_F32) return static_cast<const float*>(p)[i];
  if (dtype == FLA_F16) return __half2float(static_cast<const __half*>(p)[i]);
  return __bfloat162float(static_cast<const bf16*>(p)[i]);
}
__device__ __forceinline__ void store_any(void* p, int dtype, int64_t i, float x) {
  if (dtype == FLA_F32) static_cast<float*>(p)[i] = x;
  else if (dtype == FLA_F16) static_cast<__half*>(p)[i] = __float2half_rn(x);
  else static_cast<bf16*>(p)[i] = __float2bfloat16_rn(x);
}

template <bool BWD>
__global__ void __launch_bounds__(256) kda_gate_kernel(KdaGateParams p) {
  __shared__ float red[2][kK];
  __shared__ float red_a[8];
  const int tid = threadIdx.x, col = tid & (kK - 1), par = tid >> 7;
  const int hv = blockIdx.y;
  const int64_t t_begin = int64_t(blockIdx.x) * kGateTile;
  const int64_t t_end = min(t_begin + kGateTile, p.tokens);
  const float eig = expf(p.a_log[hv]);
  const float bias = p.dt_bias ? p.dt_bias[hv * kK + col] : 0.f;
  float sum_r = 0.f, sum_a = 0.f;
  for (int64_t t = t_begin + par; t < t_end; t += 2) {
    const float raw = load_any(p.g, p.g_dtype, t * p.g_st + hv * p.g_sh + col) + bias;
    const int64_t o = (t * p.HV + hv) * kK + col;
    if (p.mode == 1) {
      const float sp = raw > 20.f ? raw : log1pf(expf(raw));
      if (!BWD) {
        p.gate[o] = -eig * sp;
      } else {
        const float dgt = p.d_gate[t * p.dg_st + hv * p.dg_sh + col];
        const float sg = raw > 20.f ? 1.f : 1.f / (1.f + expf(-raw));
        const float dr = -eig * sg * dgt;
        store_any(p.d_g, p.d_g_dtype, o, dr);
        sum_r += dr;
        sum_a += dgt * (-eig * sp);              // d gate / d A_log = gate
      }
    } else {
      const float s = 1.f / (1.f + expf(-eig * raw));
      if (!BWD) {
        p.gate[o] = p.lower_bound * s;
      } else {
        const float dgt = p.d_gate[t * p.dg_st + hv * p.dg_sh + col];
        const float dz = p.lower_bound * s * (1.f - s) * dgt;   // d / d(e^{A_log} raw)
        const float dr = dz * eig;
        store_any(p.d_g, p.d_g_dtype, o, dr);
        sum_r += dr;
        sum_a += dz * eig * raw;
      }
    }
  }
  if (BWD) {
    red[par][col] = sum_r;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum_a += __shfl_xor_sync(0xffffffffu, sum_a, o);
    if ((tid & 31) == 0) red_a[tid >> 5] = sum_a;
    __syncthreads();
    float* out = p.partial + (int64_t(blockIdx.x) * p.HV + hv) * (kK + 1);
    if (tid < kK) out[tid] = red[0][tid] + red[1][tid];
    if (tid == 0) {
      float a = 0.f;
      for (int w = 0; w < 8; ++w) a += red_a[w];
      out[kK] = a;
    }
  }
}

// d_dt_bias[h, k] and d_A_log[h]: the per-tile sums added in tile order
__global__ void __launch_bounds__(kK + 32) kda_gate_reduce_kernel(const float* partial, int tiles, int HV, float* d_dt_bias, float* d_a_log) {
  const int hv = blockIdx.x, tid = threadIdx.x;
  if (tid > kK) return;
  float acc = 0.f;
  for (int i = 0; i < tiles; ++i) acc += partial[(int64_t(i) * HV + hv) * (kK + 1) + tid];
  if (tid < kK) {
    if (d_dt_bias) d_dt_bias[hv * kK + tid] = acc;
  } else if (d_a_log) {
    d_a_log[hv] = acc;
  }
}

int fill(const fla_kda_gate_args* a, KdaGateParams* p, bool bwd) {
  const fla_tensor_t& g = a->g;
  if (!g.data || !a->a_log.data) return FLA_ERR_NULL;
  if (g.ndim != 4 || g.shape[3] != kK || g.stride[3] != 1) return FLA_ERR_SHAPE;
  if (g.dtype != FLA_F32 && g.dtype != FLA_BF16 && g.dtype != FLA_F16) return FLA_ERR_DTYPE;
  const int64_t B = g.shape[0], T = g.shape[1], HV = g.shape[2];
  if (B > 1 && g.stride[0] != T * g.stride[1]) return FLA_ERR_LAYOUT;   // batch rows back to back: one flat token index
  if (a->a_log.dtype != FLA_F32 || a->a_log.ndim != 1 || a->a_log.shape[0] != HV || a->a_log.stride[0] != 1) return FLA_ERR_SHAPE;
  if (a->dt_bias.data && (a->dt_bias.dtype != FLA_F32 || a->dt_bias.ndim != 2 || a->dt_bias.shape[0] != HV || a->dt_bias.shape[1] != kK ||
                          a->dt_bias.stride[1] != 1 || a->dt_bias.stride[0] != kK))
    return FLA_ERR_SHAPE;
  if (a->gate_mode != 1 && a->gate_mode != 2) return FLA_ERR_VALUE;
  auto dense_f32 = [&](const fla_tensor_t& t) {
    return t.data && t.dtype == FLA_F32 && t.ndim == 4 && t.shape[0] == B && t.shape[1] == T && t.shape[2] == HV && t.shape[3] == kK &&
           t.stride[3] == 1 && t.stride[2] == kK && t.stride[1] == HV * kK && (B == 1 || t.stride[0] == T * HV * kK);
  };
  p->g = g.data; p->g_dtype = g.dtype; p->g_st = g.stride[1]; p->g_sh = g.stride[2];
  p->a_log = static_cast<const float*>(a->a_log.data);
  p->dt_bias = static_cast<const float*>(a->dt_bias.data);
  p->tokens = B * T; p->HV = int(HV); p->mode = a->gate_mode; p->lower_bound = a->lower_bound;
  if (!bwd) {
    if (!dense_f32(a->gate)) return FLA_ERR_SHAPE;
    p->gate = static_cast<float*>(a->gate.data);
    return FLA_OK;
  }
  const fla_tensor_t& dg = a->d_gate;
  if (!dg.data || dg.dtype != FLA_F32 || dg.ndim != 4 || dg.shape[0] != B || dg.shape[1] != T || dg.shape[2] != HV || dg.shape[3] != kK ||
      dg.stride[3] != 1 || (B > 1 && dg.stride[0] != T * dg.stride[1]))
    return FLA_ERR_SHAPE;
  p->d_gate = static_cast<const float*>(dg.data); p->dg_st = dg.stride[1]; p->dg_sh = dg.stride[2];
  const fla_tensor_t& o = a->d_g;
  if (!o.data || o.ndim != 4 || o.shape[0] != B || o.shape[1] != T || o.shape[2] != HV || o.shape[3] != kK || o.stride[3] != 1 ||
      o.stride[2] != kK || o.stride[1] != HV * kK || (B > 1 && o.stride[0] != T * HV * kK))
    return FLA_ERR_SHAPE;
  if (o.dtype != FLA_F32 && o.dtype != FLA_BF16 && o.dtype != FLA_F16) return FLA_ERR_DTYPE;
  p->d_g = o.data; p->d_g_dtype = o.dtype;
  return FLA_OK;
}

}  // namespace
}  // namespace fla

extern "C" FLA_API int fla_b200_kda_gate_fwd(const fla_kda_gate_args* a, void* stream) {
  using namespace fla;
  if (!a) return FLA_ERR_NULL;
  KdaGateParams p{};
  if (int st = fill(a, &p, false)) return st;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const unsigned tiles = unsigned((p.tokens + kGateTile - 1) / kGateTile);
  KernelTimer kt("kda_gate_fwd", cs);
  kda_gate_kernel<false><<<dim3(tiles, unsigned(p.HV)), 256, 0, cs>>>(p);
  return cuda_status(cudaGetLastError());
}

extern "C" FLA_API int fla_b200_kda_gate_bwd_workspace_size(const fla_kda_gate_args* a, uint64_t* bytes) {
  using namespace fla;
  if (!a || !bytes) return FLA_ERR_NULL;
  if (!a->g.data || a->g.ndim != 4) return FLA_ERR_SHAPE;
  const int64_t tokens = a->g.shape[0] * a->g.shape[1], HV = a->g.shape[2];
  *bytes = uint64_t((tokens + kGateTile - 1) / kGateTile) * HV * (kK + 1) * 4;
  return FLA_OK;
}

extern "C" FLA_API int fla_b200_kda_gate_bwd(const fla_kda_gate_args* a, void* workspace, uint64_t workspace_bytes, void* stream) {
  using namespace fla;
  if (!a) return FLA_ERR_NULL;
  KdaGateParams p{};
  if (int st = fill(a, &p, true)) return st;
  const unsigned tiles = unsigned((p.tokens + kGateTile - 1) / kGateTile);
  if (!workspace || workspace_bytes < uint64_t(tiles) * p.HV * (kK + 1) * 4) return FLA_ERR_WORKSPACE;
  for (const fla_tensor_t* t : {&a->d_a_log, &a->d_dt_bias}) {
    if (!t->data) continue;
    if (t->dtype != FLA_F32) return FLA_ERR_DTYPE;
  }
  if (a->d_a_log.data && (a->d_a_log.ndim != 1 || a->d_a_log.shape[0] != p.HV || a->d_a_log.stride[0] != 1)) return FLA_ERR_SHAPE;
  if (a->d_dt_bias.data && (a->d_dt_bias.ndim != 2 || a->d_dt_bias.shape[0] != p.HV || a->d_dt_bias.shape[1] != kK ||
                            a->d_dt_bias.stride[1] != 1 || a->d_dt_bias.stride[0] != kK))
    return FLA_ERR_SHAPE;
  p.partial = static_cast<float*>(workspace);
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  KernelTimer kt("kda_gate_bwd", cs);
  kda_gate_kernel<true><<<dim3(tiles, unsigned(p.HV)), 256, 0, cs>>>(p);
  if (cudaGetLastError() != cudaSuccess) return FLA_ERR_CUDA;
  if (a->d_a_log.data || a->d_dt_bias.data)
    kda_gate_reduce_kernel<<<unsigned(p.HV), kK + 32, 0, cs>>>(p.partial, int(tiles), p.HV, static_cast<float*>(a->d_dt_bias.data),
                                                                static_cast<float*>(a->d_a_log.data));
  return cuda_status(cudaGetLastError());
}

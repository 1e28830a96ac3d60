// Row-wise L2 normalisation used by the use_qk_l2norm_in_kernel option:
//   forward   y = x * rstd,  rstd = rsqrt(sum x^2 + eps)                      (saved: rstd)
//   backward  dx = dy * rstd - (sum dy * y) * y * rstd
// Follows the reference's l2norm_fwd / l2norm_bwd (fla/ops/triton/triton_core/l2norm.py:131-234).
// Pure HBM streaming: 16 lanes own one row, 16-byte vector loads, fp32 math, shuffle reduction.
#include <cuda_bf16.h>
#include "fla_b200_internal.h"
#include "kernel_timer.h"

namespace fla {

struct L2Params {
  const void* x; void* y; float* rstd; const void* dy; void* dx;
  int64_t rows, x_stride, y_stride, dy_stride, dx_stride;
  int D, x_f32, y_f32, dy_f32, dx_f32;
  float eps;
};

__device__ __forceinline__ void load8(const void* base, int64_t off, int is_f32, float* f) {
  if (is_f32) {
    const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + off);
    const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(base) + off + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  } else {
    const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(base) + off);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __low2float(h[i]); f[2 * i + 1] = __high2float(h[i]); }
  }
}
__device__ __forceinline__ void store8(void* base, int64_t off, int is_f32, const float* f) {
  if (is_f32) {
    float* p = static_cast<float*>(base) + off;
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
  } else {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(base) + off) = raw;
  }
}
__device__ __forceinline__ float group16_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr int kL2MaxVec = 8;  // up to 16 lanes * 8 vectors * 8 elements = 1024 columns

template <bool BWD>
__global__ void __launch_bounds__(256) l2norm_kernel(L2Params p) {
  const int64_t row = (int64_t(blockIdx.x) * 256 + threadIdx.x) / 16;
  const int sub = threadIdx.x % 16;
  if (row >= p.rows) return;   // whole 16-lane groups leave together
  const int nvec = p.D / 8;
  float v[kL2MaxVec][8], w[BWD ? kL2MaxVec : 1][8];
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < kL2MaxVec; ++i) {
    const int vi = sub + i * 16;
    if (vi < nvec) {
      if constexpr (!BWD) {
        load8(p.x, row * p.x_stride + vi * 8, p.x_f32, v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += v[i][j] * v[i][j];
      } else {
        load8(p.y, row * p.y_stride + vi * 8, p.y_f32, v[i]);
        load8(p.dy, row * p.dy_stride + vi * 8, p.dy_f32, w[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc += v[i][j] * w[i][j];
      }
    }
  }
  acc = group16_sum(acc);
  if constexpr (!BWD) {
    const float r = rsqrtf(acc + p.eps);
    if (sub == 0) p.rstd[row] = r;
#pragma unroll
    for (int i = 0; i < kL2MaxVec; ++i) {
      const int vi = sub + i * 16;
      if (vi < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] *= r;
        store8(p.y, row * p.y_stride + vi * 8, p.y_f32, v[i]);
      }
    }
  } else {
    const float r = p.rstd[row];
#pragma unroll
    for (int i = 0; i < kL2MaxVec; ++i) {
      const int vi = sub + i * 16;
      if (vi < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) w[i][j] = (w[i][j] - acc * v[i][j]) * r;
        store8(p.dx, row * p.dx_stride + vi * 8, p.dx_f32, w[i]);
      }
    }
  }
}

}  // namespace fla

using namespace fla;

static int l2_check(const fla_tensor_t& t, int64_t rows, int64_t D, bool need) {
  if (!t.data) return need ? FLA_ERR_NULL : FLA_OK;
  if (t.ndim != 2 || t.shape[0] != rows || t.shape[1] != D) return FLA_ERR_SHAPE;
  if (t.dtype != FLA_BF16 && t.dtype != FLA_F32) return FLA_ERR_DTYPE;
  const int64_t esz = t.dtype == FLA_F32 ? 4 : 2;
  if (t.stride[1] != 1 || (t.stride[0] * esz) % 16 || !aligned16(t.data)) return FLA_ERR_LAYOUT;
  return FLA_OK;
}

extern "C" FLA_API int fla_b200_l2norm_fwd(const fla_l2norm_args* a, void* stream) {
  if (!a) return FLA_ERR_NULL;
  const fla_tensor_t& x = a->x;
  if (!x.data || x.ndim != 2) return FLA_ERR_SHAPE;
  const int64_t rows = x.shape[0], D = x.shape[1];
  if (D <= 0 || D % 8 || D > 16 * 8 * kL2MaxVec) return FLA_ERR_SHAPE;
  int st;
  if ((st = l2_check(x, rows, D, true)) || (st = l2_check(a->y, rows, D, true))) return st;
  if (!a->rstd.data || a->rstd.dtype != FLA_F32 || a->rstd.ndim != 1 || a->rstd.shape[0] != rows || a->rstd.stride[0] != 1)
    return FLA_ERR_SHAPE;
  if (rows == 0) return FLA_OK;
  L2Params p{};
  p.x = x.data; p.y = a->y.data; p.rstd = static_cast<float*>(a->rstd.data);
  p.rows = rows; p.x_stride = x.stride[0]; p.y_stride = a->y.stride[0];
  p.D = int(D); p.x_f32 = x.dtype == FLA_F32; p.y_f32 = a->y.dtype == FLA_F32; p.eps = a->eps;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  KernelTimer kt("l2norm_fwd", cs);
  l2norm_kernel<false><<<unsigned((rows * 16 + 255) / 256), 256, 0, cs>>>(p);
  return cuda_status(cudaGetLastError());
}

extern "C" FLA_API int fla_b200_l2norm_bwd(const fla_l2norm_args* a, void* stream) {
  if (!a) return FLA_ERR_NULL;
  const fla_tensor_t& y = a->y;
  if (!y.data || y.ndim != 2) return FLA_ERR_SHAPE;
  const int64_t rows = y.shape[0], D = y.shape[1];
  if (D <= 0 || D % 8 || D > 16 * 8 * kL2MaxVec) return FLA_ERR_SHAPE;
  int st;
  if ((st = l2_check(y, rows, D, true)) || (st = l2_check(a->dy, rows, D, true)) || (st = l2_check(a->dx, rows, D, true))) return st;
  if (!a->rstd.data || a->rstd.dtype != FLA_F32 || a->rstd.ndim != 1 || a->rstd.shape[0] != rows || a->rstd.stride[0] != 1)
    return FLA_ERR_SHAPE;
  if (rows == 0) return FLA_OK;
  L2Params p{};
  p.y = y.data; p.rstd = static_cast<float*>(a->rstd.data); p.dy = a->dy.data; p.dx = a->dx.data;
  p.rows = rows; p.y_stride = y.stride[0]; p.dy_stride = a->dy.stride[0]; p.dx_stride = a->dx.stride[0];
  p.D = int(D); p.y_f32 = y.dtype == FLA_F32; p.dy_f32 = a->dy.dtype == FLA_F32; p.dx_f32 = a->dx.dtype == FLA_F32;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  KernelTimer kt("l2norm_bwd", cs);
  l2norm_kernel<true><<<unsigned((rows * 16 + 255) / 256), 256, 0, cs>>>(p);
  return cuda_status(cudaGetLastError());
}

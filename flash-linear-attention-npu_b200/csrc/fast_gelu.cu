// FastGELU  y = x / (1 + exp(-1.702 x))  and its backward  dx = dy * (s + 1.702 x s (1 - s)),  s = sigmoid(1.702 x).
// Replaces the reference operators npu_fast_gelu_custom / npu_fast_gelu_custom_backward (aclnnFastGelu /
// aclnnFastGeluBackward as bound in torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:224-239; the forward
// formula is the golden of torch_custom/fla_npu/test/test_npu_fast_gelu_custom.py:22-24, the backward is its exact
// derivative).  Elementwise and HBM-bound: 16-byte loads and stores over a flat contiguous buffer, fp32 arithmetic.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "fla_b200_internal.h"
#include "kernel_timer.h"

namespace fla {
namespace {

constexpr float kGeluAlpha = 1.702f;

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

template <bool BWD>
__device__ __forceinline__ float gelu_elem(float x, float dy) {
  const float s = 1.f / (1.f + __expf(-kGeluAlpha * x));
  if (!BWD) return x * s;
  return dy * (s + kGeluAlpha * x * s * (1.f - s));
}

// One thread handles one 16-byte vector (4 fp32 or 8 half-precision elements) per grid-stride step.
template <typename T, bool BWD>
__global__ void __launch_bounds__(256) fast_gelu_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ out,
                                                        int64_t n) {
  constexpr int VEC = 16 / sizeof(T);
  const int64_t nvec = n / VEC;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const uint4 xr = reinterpret_cast<const uint4*>(x)[i];
    uint4 gr = make_uint4(0, 0, 0, 0);
    if (BWD) gr = reinterpret_cast<const uint4*>(dy)[i];
    const T* xv = reinterpret_cast<const T*>(&xr);
    const T* gv = reinterpret_cast<const T*>(&gr);
    uint4 o;
    T* ov = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < VEC; ++j) ov[j] = from_f<T>(gelu_elem<BWD>(to_f<T>(xv[j]), BWD ? to_f<T>(gv[j]) : 0.f));
    reinterpret_cast<uint4*>(out)[i] = o;
  }
  // tail (fewer than VEC elements)
  const int64_t t = nvec * VEC + int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t < n) out[t] = from_f<T>(gelu_elem<BWD>(to_f<T>(x[t]), BWD ? to_f<T>(dy[t]) : 0.f));
}

bool flat_contiguous(const fla_tensor_t& t, int64_t* n) {
  if (!t.data || t.ndim < 1 || t.ndim > FLA_MAX_DIMS) return false;
  int64_t expect = 1;
  for (int d = t.ndim - 1; d >= 0; --d) {
    if (t.shape[d] <= 0) return false;
    if (t.shape[d] != 1 && t.stride[d] != expect) return false;
    expect *= t.shape[d];
  }
  *n = expect;
  return true;
}

template <bool BWD>
int launch(const fla_fast_gelu_args* a, void* stream) {
  if (!a) return FLA_ERR_NULL;
  const fla_tensor_t &x = a->x, &o = BWD ? a->dx : a->y;
  if (!x.data || !o.data || (BWD && !a->dy.data)) return FLA_ERR_NULL;
  int64_t n = 0, no = 0, ng = 0;
  if (!flat_contiguous(x, &n) || !flat_contiguous(o, &no) || n != no) return FLA_ERR_LAYOUT;
  if (BWD && (!flat_contiguous(a->dy, &ng) || ng != n)) return FLA_ERR_LAYOUT;
  if (o.dtype != x.dtype || (BWD && a->dy.dtype != x.dtype)) return FLA_ERR_DTYPE;
  if (!aligned16(x.data) || !aligned16(o.data) || (BWD && !aligned16(a->dy.data))) return FLA_ERR_LAYOUT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t nvec = (n + 3) / 4;
  const unsigned grid = unsigned(std::min<int64_t>((nvec + 255) / 256, 148 * 16));
  KernelTimer kt(BWD ? "fast_gelu_bwd" : "fast_gelu", st);
  switch (x.dtype) {
    case FLA_F32:
      fast_gelu_kernel<float, BWD><<<grid, 256, 0, st>>>(static_cast<const float*>(x.data), static_cast<const float*>(a->dy.data),
                                                         static_cast<float*>(o.data), n);
      break;
    case FLA_BF16:
      fast_gelu_kernel<__nv_bfloat16, BWD><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x.data),
                                                                 static_cast<const __nv_bfloat16*>(a->dy.data),
                                                                 static_cast<__nv_bfloat16*>(o.data), n);
      break;
    case FLA_F16:
      fast_gelu_kernel<__half, BWD><<<grid, 256, 0, st>>>(static_cast<const __half*>(x.data), static_cast<const __half*>(a->dy.data),
                                                          static_cast<__half*>(o.data), n);
      break;
    default:
      return FLA_ERR_DTYPE;
  }
  return cuda_status(cudaGetLastError());
}

}  // namespace
}  // namespace fla

extern "C" FLA_API int fla_b200_fast_gelu(const fla_fast_gelu_args* a, void* stream) { return fla::launch<false>(a, stream); }
extern "C" FLA_API int fla_b200_fast_gelu_bwd(const fla_fast_gelu_args* a, void* stream) { return fla::launch<true>(a, stream); }

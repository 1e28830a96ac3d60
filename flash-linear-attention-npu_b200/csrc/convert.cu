// Elementwise conversion between f32, bf16 and f16 tensors (round to nearest even), with re-layout: source and destination
// are addressed through their strides, so a head-first view is converted and made token-major in one pass.
// The chunk operators multiply bf16 operands on the tensor cores; the reference also takes fp16 tensors
// (examples/flash_gated_delta_rule.py:1161-1162 rejects only fp32).  fp16 inputs enter through this kernel, rounded
// from 11 to 8 significant bits, and results leave through it as fp16.  HBM-bound: 16-byte loads where the rows allow.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <algorithm>
#include "fla_b200_internal.h"
#include "kernel_timer.h"

namespace fla {
namespace {

template <typename T> __device__ __forceinline__ float cv_to_f(T v);
template <> __device__ __forceinline__ float cv_to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float cv_to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float cv_to_f<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T cv_from_f(float v);
template <> __device__ __forceinline__ float cv_from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 cv_from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half cv_from_f<__half>(float v) { return __float2half_rn(v); }

struct ConvertParams {
  const void* src; void* dst;
  int64_t n1, n2, d;            // logical shape [n0, n1, n2, d] (leading dims padded with 1); n0 is implied by `groups`
  int64_t ss[3], ds[3];         // element strides of the three outer dims
  int64_t groups;               // n0 * n1 * n2 * (d / 8)
};

// One thread converts 8 consecutive elements of a row per grid-stride step (d % 8 == 0).
template <typename S, typename D>
__global__ void __launch_bounds__(256) convert_kernel(ConvertParams p) {
  const int64_t per_row = p.d / 8;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < p.groups; i += stride) {
    const int64_t c = i % per_row;
    int64_t r = i / per_row;
    const int64_t i2 = r % p.n2; r /= p.n2;
    const int64_t i1 = r % p.n1;
    const int64_t i0 = r / p.n1;
    const S* s = static_cast<const S*>(p.src) + i0 * p.ss[0] + i1 * p.ss[1] + i2 * p.ss[2] + c * 8;
    D* d = static_cast<D*>(p.dst) + i0 * p.ds[0] + i1 * p.ds[1] + i2 * p.ds[2] + c * 8;
    __align__(16) S in[8];
    if (sizeof(S) == 2) {
      *reinterpret_cast<uint4*>(in) = *reinterpret_cast<const uint4*>(s);
    } else {
      *reinterpret_cast<uint4*>(in) = *reinterpret_cast<const uint4*>(s);
      *reinterpret_cast<uint4*>(in + 4) = *reinterpret_cast<const uint4*>(s + 4);
    }
    __align__(16) D out[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] = cv_from_f<D>(cv_to_f<S>(in[j]));
    if (sizeof(D) == 2) {
      *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(out);
    } else {
      *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(out);
      *reinterpret_cast<uint4*>(d + 4) = *reinterpret_cast<const uint4*>(out + 4);
    }
  }
}

// Rows that are not a multiple of 8 long, or not 16-byte aligned: one element per thread.
template <typename S, typename D>
__global__ void __launch_bounds__(256) convert_scalar_kernel(ConvertParams p, int64_t n) {
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t c = i % p.d;
    int64_t r = i / p.d;
    const int64_t i2 = r % p.n2; r /= p.n2;
    const int64_t i1 = r % p.n1;
    const int64_t i0 = r / p.n1;
    static_cast<D*>(p.dst)[i0 * p.ds[0] + i1 * p.ds[1] + i2 * p.ds[2] + c] =
        cv_from_f<D>(cv_to_f<S>(static_cast<const S*>(p.src)[i0 * p.ss[0] + i1 * p.ss[1] + i2 * p.ss[2] + c]));
  }
}

int elem_bytes(int dtype) { return dtype == FLA_F32 ? 4 : 2; }

bool rows_vectorisable(const fla_tensor_t& t, const int64_t* st) {
  const int64_t eb = elem_bytes(t.dtype);
  if (reinterpret_cast<uintptr_t>(t.data) % 16) return false;
  for (int i = 0; i < 3; ++i)
    if ((st[i] * eb) % 16) return false;
  return true;
}

template <typename S, typename D>
int run(const ConvertParams& p, int64_t n, bool vec, cudaStream_t st) {
  const int64_t work = vec ? p.groups : n;
  const unsigned grid = unsigned(std::max<int64_t>(1, std::min<int64_t>((work + 255) / 256, 148 * 16)));
  KernelTimer kt("convert", st);
  if (vec) convert_kernel<S, D><<<grid, 256, 0, st>>>(p);
  else convert_scalar_kernel<S, D><<<grid, 256, 0, st>>>(p, n);
  return cuda_status(cudaGetLastError());
}

template <typename S>
int dispatch_dst(int dst_dtype, const ConvertParams& p, int64_t n, bool vec, cudaStream_t st) {
  switch (dst_dtype) {
    case FLA_F32: return run<S, float>(p, n, vec, st);
    case FLA_BF16: return run<S, __nv_bfloat16>(p, n, vec, st);
    case FLA_F16: return run<S, __half>(p, n, vec, st);
    default: return FLA_ERR_DTYPE;
  }
}

}  // namespace
}  // namespace fla

extern "C" FLA_API int fla_b200_convert(const fla_tensor_t* src, const fla_tensor_t* dst, void* stream) {
  using namespace fla;
  if (!src || !dst || !src->data || !dst->data) return FLA_ERR_NULL;
  if (src->ndim < 1 || src->ndim > 4 || dst->ndim != src->ndim) return FLA_ERR_SHAPE;
  const int nd = src->ndim;
  for (int i = 0; i < nd; ++i)
    if (src->shape[i] != dst->shape[i] || src->shape[i] <= 0) return FLA_ERR_SHAPE;
  if ((src->shape[nd - 1] != 1 && (src->stride[nd - 1] != 1 || dst->stride[nd - 1] != 1))) return FLA_ERR_LAYOUT;
  if (src->dtype < FLA_F32 || src->dtype > FLA_F16 || dst->dtype < FLA_F32 || dst->dtype > FLA_F16) return FLA_ERR_DTYPE;
  ConvertParams p{};
  p.src = src->data;
  p.dst = dst->data;
  int64_t shp[3] = {1, 1, 1};
  for (int i = 0; i < 3; ++i) p.ss[i] = p.ds[i] = 0;
  for (int i = 0; i < nd - 1; ++i) {   // outer dims, right-aligned into the three slots
    const int slot = 3 - (nd - 1) + i;
    shp[slot] = src->shape[i];
    p.ss[slot] = src->stride[i];
    p.ds[slot] = dst->stride[i];
  }
  p.n1 = shp[1];
  p.n2 = shp[2];
  p.d = src->shape[nd - 1];
  const int64_t n = shp[0] * shp[1] * shp[2] * p.d;
  const bool vec = p.d % 8 == 0 && rows_vectorisable(*src, p.ss) && rows_vectorisable(*dst, p.ds);
  p.groups = vec ? n / 8 : 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (src->dtype) {
    case FLA_F32: return dispatch_dst<float>(dst->dtype, p, n, vec, st);
    case FLA_BF16: return dispatch_dst<__nv_bfloat16>(dst->dtype, p, n, vec, st);
    default: return dispatch_dst<__half>(dst->dtype, p, n, vec, st);
  }
}

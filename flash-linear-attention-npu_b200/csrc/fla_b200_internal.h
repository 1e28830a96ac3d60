// Internal helpers shared by the C-ABI translation units (not installed).
#pragma once
#include <atomic>
#include <cstdint>
#include <cuda_runtime.h>
#include "../../include/fla_b200.h"

namespace fla {

inline bool is_contig_last(const fla_tensor_t& t) { return t.ndim > 0 && t.stride[t.ndim - 1] == 1; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline int64_t numel(const fla_tensor_t& t) {
  int64_t n = 1;
  for (int i = 0; i < t.ndim; ++i) n *= t.shape[i];
  return n;
}
inline uint64_t align_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }

inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? FLA_OK : FLA_ERR_CUDA; }

}  // namespace fla

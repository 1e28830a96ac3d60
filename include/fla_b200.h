/* C ABI of libfla_b200.so: hand-written sm_100a CUDA kernels for the GDN / KDA linear-attention
 * hot path (chunked forward + backward, fused-recurrent decode, causal_conv1d forward / update).
 *
 * Calling convention (replaces the reference's two-phase aclnn calls, i.e. the pair
 * aclnn<Op>GetWorkspaceSize / aclnn<Op> driven from
 * torch_custom/fla_npu/fla_npu/ops/ascendc/_runtime.py:388-429):
 *   1. int fla_b200_<op>_workspace_size(const <op>_args*, uint64_t* bytes)
 *   2. int fla_b200_<op>(const <op>_args*, void* workspace, uint64_t workspace_bytes, void* stream)
 * Every tensor is described by fla_tensor_t (device pointer, dtype code, shape, element strides),
 * the analogue of the aclTensor descriptors built in _runtime.py:210-256.  The caller owns all
 * memory, including the workspace; the library allocates nothing and keeps no state between calls.
 * Launches are asynchronous on `stream` (a cudaStream_t).  Every entry point returns FLA_OK (0) or
 * a non-zero status and never aborts, like aclnnStatus (_runtime.py:410-411,427-428).
 * A NULL `data` pointer in an optional tensor means "absent" (_runtime.py:299-300).
 */
#ifndef FLA_B200_H_
#define FLA_B200_H_

#include <stdint.h>

#if defined(__GNUC__)
#define FLA_API __attribute__((visibility("default")))
#else
#define FLA_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum fla_status {
  FLA_OK = 0,
  FLA_ERR_NULL = 1,      /* required pointer missing */
  FLA_ERR_SHAPE = 2,     /* unsupported or inconsistent shape */
  FLA_ERR_DTYPE = 3,     /* unsupported dtype combination */
  FLA_ERR_LAYOUT = 4,    /* stride / alignment requirement not met */
  FLA_ERR_WORKSPACE = 5, /* workspace missing or too small */
  FLA_ERR_CUDA = 6,      /* a CUDA runtime call failed */
  FLA_ERR_VALUE = 7,     /* scalar argument out of range */
  FLA_ERR_TIMEOUT = 8    /* a bounded device-side wait ran out (read back from a kernel status word) */
};

enum fla_dtype { FLA_F32 = 0, FLA_BF16 = 1, FLA_F16 = 2, FLA_I32 = 3, FLA_I64 = 4 };

#define FLA_MAX_DIMS 6

typedef struct fla_tensor {
  void* data;                   /* device pointer to element [0,...,0]; NULL = tensor absent */
  int32_t dtype;                /* enum fla_dtype */
  int32_t ndim;
  int64_t shape[FLA_MAX_DIMS];
  int64_t stride[FLA_MAX_DIMS]; /* in elements */
} fla_tensor_t;

/* Library version (major * 10000 + minor * 100 + patch). */
FLA_API int fla_b200_version(void);

/* Hardware self-test of the tcgen05 tile-GEMM building block (no reference counterpart; it exists
 * because the kernels below stage every tensor-core operand through the same descriptors).
 * Computes D[M x N] (+)= A * B^T-or-B with bf16 operands read from row-major device buffers and
 * dumps the 128-lane TMEM accumulator into d[128][N].  err_flag: device int, set non-zero on timeout. */
FLA_API int fla_b200_selftest_mma(const void* a, const void* b, float* d, int M, int N, int K, int a_mn, int b_mn,
                          int d_lane_off, int prefill, int* err_flag, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLA_B200_H_ */

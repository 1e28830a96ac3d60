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
  FLA_ERR_TIMEOUT = 8,   /* a bounded device-side wait ran out (read back from a kernel status word) */
  FLA_ERR_TOO_LARGE = 9  /* the problem needs more scratch than an allocation-free entry point owns */
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

/* Optional per-kernel device timing (no reference counterpart; the reference relies on an external
 * profiler).  While enabled, every kernel launch of the library is bracketed by CUDA events on the
 * launching stream.  Enabling or disabling clears earlier records.  kernel_timing_read synchronises the
 * recorded events and returns the summed duration and the number of launches of `kernel_name`
 * (names: "gdn_prep", "tri_inverse", "kda_prep", "kda_fwd", "gdn_fwd", "gdn_bwd_dhu", "gdn_bwd_par", "recurrent_gdn", "causal_conv1d_fwd",
 * "causal_conv1d_update", "causal_conv1d_bwd", "kda_bwd_dhu", "kda_bwd_par", "chunk_local_cumsum", "chunk_scaled_dot_kkt",
 * "solve_tri", "recompute_w_u_fwd", "chunk_fwd_h", "chunk_fwd_o", "convert"). */
FLA_API int fla_b200_kernel_timing_enable(int enable);
FLA_API int fla_b200_kernel_timing_read(const char* kernel_name, float* total_ms, int* launches);

/* Hardware self-test of the tcgen05 tile-GEMM building block (no reference counterpart; it exists
 * because the kernels below stage every tensor-core operand through the same descriptors).
 * Computes D[M x N] (+)= A * B^T-or-B with bf16 operands read from row-major device buffers and
 * dumps the 128-lane TMEM accumulator into d[128][N].  err_flag: device int, set non-zero on timeout. */
FLA_API int fla_b200_selftest_mma(const void* a, const void* b, float* d, int M, int N, int K, int a_mn, int b_mn,
                          int d_lane_off, int prefill, int* err_flag, void* stream);
/* The same check for products whose A operand is read from tensor memory (M = 128): A [128][K] row-major bf16 is packed
 * into TMEM columns 256 + a_col_off .. by the kernel (two elements per 32-bit column), B as above, d[128][N] out. */
FLA_API int fla_b200_selftest_mma_ts(const void* a, const void* b, float* d, int N, int K, int b_mn, int a_col_off,
                             int* err_flag, void* stream);
/* The same check for operands in the un-swizzled strip layout ([M or N / 8][reduction rows][16 bytes]) in which the scan
 * kernels save their per-chunk operands: b is [K][N] row-major; variant 0 reads A [128][K] from tensor memory, variant 1
 * stages A in strips as well; variant 2 takes b as [N][K] row-major and stages it in strips along the reduction dim
 * ([K / 8][N rows][16 bytes]). */
FLA_API int fla_b200_selftest_mma_nosw(const void* a, const void* b, float* d, int N, int K, int variant, int* err_flag,
                               void* stream);

/* Device-side failure reporting (the counterpart of the non-zero aclnnStatus the reference turns into a
 * RuntimeError, torch_custom/fla_npu/fla_npu/ops/ascendc/_runtime.py:410-411,427-428).  Launches are
 * asynchronous, so a kernel cannot fail through the return value of its entry point: the chunk operators
 * (gdn_chunk_fwd / bwd, kda_chunk_fwd / bwd and the stage operators) keep an int32 status word at byte 0
 * of their workspace, cleared when the call is enqueued; a kernel whose bounded wait on a barrier runs out
 * writes FLA_ERR_TIMEOUT there, releases what it holds and returns (its outputs are then invalid).
 *   fla_b200_read_status_word  copies that word to the host after waiting for `stream`.  Call it while the
 *                              workspace is still alive and where a synchronisation is acceptable.
 *   fla_b200_selftest_wait_timeout  launches one CTA that allocates TMEM and waits, for at most `spin_limit`
 *                              polls (1 .. 2^20), on a barrier nobody arrives at, then records FLA_ERR_TIMEOUT in
 *                              *status_word (device int32), frees its TMEM and returns: the give-up path of
 *                              every kernel, exercised without hanging or faulting anything. */
FLA_API int fla_b200_read_status_word(const void* workspace, void* stream, int32_t* status_out);
FLA_API int fla_b200_selftest_wait_timeout(uint32_t spin_limit, void* status_word, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Fused-recurrent gated delta rule (decode step), in-place over a state pool.
 * Replaces aclnnRecurrentGatedDeltaRule as bound by npu_recurrent_gated_delta_rule
 * (torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:654-846; kernel
 * fla/ops/ascendc/gdn/recurrent_gdn/recurrent_gated_delta_rule/op_kernel/recurrent_gated_delta_rule.h:159-199).
 * Per token: S <- exp(g) S; d = beta (v - S^T k); S <- S + k d^T; o = S^T (scale q).
 *   q, k   [T, HK, K] bf16|f16      v   [T, HV, V], the same dtype (HV % HK == 0, head hv reads q/k head hv / (HV/HK));
 *          fp16 values are read exactly (the arithmetic is fp32 on CUDA cores)
 *   g      [T, HV] f32|bf16, optional (absent: no decay)        beta [T, HV] f32|bf16, optional (absent: 1)
 *   state_in / state_out [blocks, HV, K, V] (state_v_first = 0) or [blocks, HV, V, K] (= 1), f32|bf16,
 *          innermost two dims dense; the two may be the same tensor (in-place update)
 *   out    [T, HV, V] bf16|f16|f32
 *   cu_seqlens          int32 [N+1] device, token offsets of the N sequences; absent: every sequence has
 *                       `tokens_per_seq` tokens
 *   state_indices       int32 [T] device: the state after token t is written to block state_indices[t], and a
 *                       sequence starts from block state_indices[first token (+ accepted - 1)]; a negative
 *                       start index skips the sequence.  Absent: sequence n reads block n of state_in and its
 *                       final state is written to block n of state_out.
 *   num_accepted_tokens int32 [N] device, optional (needs state_indices)
 * Per-channel gate (the reference's recurrent KDA step, aclnnRecurrentKda as bound by npu_recurrent_kda,
 * _aclnn_ctypes.py:1298-1503; semantics fla/ops/ascendc/kda/recurrent_kda/docs/design.md:44-70):
 *   gk     [T, HV, K] f32|bf16, optional: S <- diag(exp(gate(gk))) S before the update, where gate is the identity
 *          (gate_mode 0), -exp(a_log[h]) softplus(gk + dt_bias[h, :]) (1) or lower_bound sigmoid(exp(a_log[h]) (gk + dt_bias)) (2)
 *   a_log  [HV] f32, dt_bias [HV, K] f32 (optional): gate parameters for gate_mode 1 / 2
 *   beta_mode 0: beta as given; 1: sigmoid(beta); 2: 2 sigmoid(beta)
 * K, V in {64, 128}.  No workspace. */
typedef struct fla_recurrent_gdn_args {
  fla_tensor_t q, k, v, g, beta, state_in, state_out, out;
  fla_tensor_t cu_seqlens, state_indices, num_accepted_tokens;
  fla_tensor_t gk, a_log, dt_bias;
  float scale;
  float lower_bound;
  int32_t tokens_per_seq;
  int32_t state_v_first;
  int32_t use_qk_l2norm; /* normalise q and k rows as x * rsqrt(sum x^2 + 1e-6) first */
  int32_t gate_mode;
  int32_t beta_mode;
} fla_recurrent_gdn_args;
FLA_API int fla_b200_recurrent_gdn_workspace_size(const fla_recurrent_gdn_args* args, uint64_t* bytes);
FLA_API int fla_b200_recurrent_gdn(const fla_recurrent_gdn_args* args, void* workspace, uint64_t workspace_bytes,
                                   void* stream);

/* ---------------------------------------------------------------------------------------------
 * causal_conv1d forward over whole sequences (prefill).
 * Replaces aclnnCausalConv1d with run_mode = 0 as bound by npu_causal_conv1d
 * (torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:951-985) and the composed entry
 * causal_conv1d_ascendc (examples/flash_gated_delta_rule.py:422-443).
 *   y[t, d] = act(bias[d] + sum_{j<W} weight[d, j] * x[t - (W-1) + j, d]) (+ residual[t, d])
 *   x, y, residual [B, T, D] bf16, D contiguous and a multiple of 8; y may instead be head-first, [B, H, T, D/H] with D/H a
 *          multiple of 8 (the reference's head_num output, _aclnn_ctypes.py:939-948): channel d goes to head d / (D/H)
 *   weight [D, W] bf16 (any strides: pass the reference's [W, D] tensor as a transposed view), W in {2,3,4}
 *   bias [D] bf16, optional
 *   initial_state / final_state [N, D, W-1] bf16 (any strides), optional: the last W-1 inputs before /
 *          after each sequence (zero-padded on the left when a sequence is shorter)
 *   cu_seqlens int32 [N+1] device, optional: packed variable-length sequences, requires B == 1
 *   activation_silu: 0 = none, 1 = SiLU.   No workspace. */
typedef struct fla_causal_conv1d_fwd_args {
  fla_tensor_t x, weight, bias, residual, initial_state, y, final_state, cu_seqlens;
  int32_t activation_silu;
} fla_causal_conv1d_fwd_args;
FLA_API int fla_b200_causal_conv1d_fwd_workspace_size(const fla_causal_conv1d_fwd_args* args, uint64_t* bytes);
FLA_API int fla_b200_causal_conv1d_fwd(const fla_causal_conv1d_fwd_args* args, void* workspace,
                                       uint64_t workspace_bytes, void* stream);

/* causal_conv1d backward (prefill form).
 * Replaces aclnnCausalConv1dBwd as bound by npu_causal_conv1d_bwd
 * (torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:988-1037; golden
 * torch_custom/fla_npu/test/test_npu_causal_conv1d_bwd.py:33-127).
 *   x, dy, dx [B, T, D] bf16;  weight [D, W] bf16 (any strides);  bias [D] bf16 optional (enters the recomputed
 *   pre-activation);  y_pre [B, T, D] bf16 optional: the forward's pre-activation, read instead of recomputed;
 *   initial_state, dht [N, D, W-1] bf16 optional (gradient of the final state);  dw [D, W] f32 (any strides);
 *   db [D] f32 optional;  dh0 [N, D, W-1] bf16|f32 optional;  cu_seqlens as in the forward.
 * Workspace: per-tile partial sums of dw / db (reduced in a fixed order: results are deterministic). */
typedef struct fla_causal_conv1d_bwd_args {
  fla_tensor_t x, weight, bias, dy, y_pre, initial_state, dht;
  fla_tensor_t dx, dw, db, dh0, cu_seqlens;
  int32_t activation_silu;
} fla_causal_conv1d_bwd_args;
FLA_API int fla_b200_causal_conv1d_bwd_workspace_size(const fla_causal_conv1d_bwd_args* args, uint64_t* bytes);
FLA_API int fla_b200_causal_conv1d_bwd(const fla_causal_conv1d_bwd_args* args, void* workspace,
                                       uint64_t workspace_bytes, void* stream);

/* causal_conv1d decode update: consumes T new tokens per sequence and shifts conv_state in place.
 * Replaces aclnnCausalConv1d with run_mode = 1 (same binding as above; kernel
 * fla/ops/ascendc/gdn/gdn_preprocess/causal_conv1d/op_kernel/causal_conv1d_update.h).
 *   x, y, residual [N, T, D] bf16 (T <= 16);  weight [D, W];  bias [D]
 *   conv_state [slots, D, S] bf16, any strides, S >= W-1, updated in place.  Fast paths: T == 1, S == W-1 and
 *          either channels contiguous ([slots, S, D] memory) or taps contiguous ([slots, D, S] memory).
 *   cache_indices int32 [N] device, optional: slot of each sequence; entries equal to pad_slot_id are skipped
 *   num_accepted_tokens int32 [N] device, optional: speculative decoding; history window starts at
 *          accepted-1 and S >= (W-1) + (T-1)
 * No workspace. */
typedef struct fla_causal_conv1d_update_args {
  fla_tensor_t x, weight, bias, residual, conv_state, y, cache_indices, num_accepted_tokens;
  int32_t activation_silu;
  int32_t pad_slot_id;
} fla_causal_conv1d_update_args;
FLA_API int fla_b200_causal_conv1d_update_workspace_size(const fla_causal_conv1d_update_args* args, uint64_t* bytes);
FLA_API int fla_b200_causal_conv1d_update(const fla_causal_conv1d_update_args* args, void* workspace,
                                          uint64_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Chunked gated delta rule, forward (chunk = 64, K = 128, V = 128 or 256).
 * Replaces the reference's forward chain chunk_local_cumsum -> chunk_scaled_dot_kkt -> solve_tri ->
 * recompute_w_u_fwd -> chunk_gated_delta_rule_fwd_h -> chunk_fwd_o as composed by
 * flash_chunk_gated_delta_rule_fwd (examples/flash_gated_delta_rule.py:796-881; per-op bindings
 * torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:875-936, 1786-1800, 618-651, 552-615, 517-549).
 *   q, k [B, T, HK, 128] bf16;  v [B, T, HV, V] bf16;  g, beta [B, T, HV] f32|bf16 (g = log decay per token)
 *   o [B, T, HV, V] bf16|f32
 *   initial_state / final_state [N, HV, 128(K), V] f32, optional
 *   gam   [B, T, HV] f32      out: chunk-local cumulative sum of g      (saved for backward)
 *   x_inv [chunks * HV * 8192] bf16 out: X = (I + strict_tril(beta_i exp(gam_i-gam_j) k_i.k_j))^-1 per (chunk, head), as a bf16 value
 *          and a bf16 residual (4096 elements each) in strips of 8 rows: element [r/8][c][r%8] = X[r][c]; rows past the chunk are zero
 *   s_img  [chunks * HV * (V/64) * 16384] bf16, optional out (for backward): per (chunk, head, 64-channel half of V) the state at
 *          chunk start as a bf16 value and a bf16 residual, each 128 key dims x 64 channels in strips of 8 key dims
 *          (element [k/8][channel][k%8])
 *   vn_img [chunks * HV * (V/64) * 8192] bf16, optional out (for backward): v_new per half, value and residual, each 64 tokens x
 *          64 channels in strips of 8 tokens (element [t/8][channel][t%8])
 *   p_img  [chunks * HV * 8768] bf16, optional out (for backward): per (chunk, head) tril(Q K^T * decay) as a bf16 value and a
 *          bf16 residual, each 64x64 in strips of 8 columns (element [j/8][i][j%8] = P[i][j]), followed by 1152 bytes that hold
 *          the chunk's per-token factors (beta, beta e^gam, e^{gam_L-gam}, scale e^gam as 64 floats each, then e^{gam_L});
 *          when absent the forward keeps these panels in its workspace
 *          (s_img, vn_img, p_img are opaque to the caller: produced here, consumed by fla_b200_gdn_chunk_bwd)
 *   cu_seqlens int32 [N+1] device (requires B == 1) with chunk_offsets int32 [N+1] device (prefix sum of
 *   ceil(len/64)), max_seqlen and total_chunks given by the host.  All four are ignored for dense batches.
 * Token tensors need a contiguous last dim, 16-byte aligned rows and batch rows laid out back to back.
 * Workspace: a 256-byte status block (first int32 becomes FLA_ERR_TIMEOUT if a device-side wait ran out)
 * followed by a 16 KB fp32 scratch tile per (chunk, value head) for the triangular inverse and, when p_img is
 * absent, 17,536 bytes per (chunk, value head) for the score tile and the chunk's factor record. */
typedef struct fla_gdn_chunk_fwd_args {
  fla_tensor_t q, k, v, g, beta, initial_state;
  fla_tensor_t o, final_state, gam, x_inv, s_img, vn_img, p_img;
  fla_tensor_t cu_seqlens, chunk_offsets;
  float scale;
  int32_t chunk_size;
  int32_t max_seqlen;
  int32_t total_chunks;
} fla_gdn_chunk_fwd_args;
FLA_API int fla_b200_gdn_chunk_fwd_workspace_size(const fla_gdn_chunk_fwd_args* args, uint64_t* bytes);
FLA_API int fla_b200_gdn_chunk_fwd(const fla_gdn_chunk_fwd_args* args, void* workspace, uint64_t workspace_bytes,
                                   void* stream);

/* ---------------------------------------------------------------------------------------------
 * Chunked gated delta rule, backward (chunk = 64, K = 128, V = 128 or 256).
 * Replaces the reference's backward chain chunk_bwd_dv_local -> chunk_gated_delta_rule_bwd_dhu -> chunk_bwd_dqkwg ->
 * prepare_wy_repr_bwd_da -> prepare_wy_repr_bwd_full -> reverse chunk_local_cumsum as composed by
 * flash_chunk_gated_delta_rule_bwd (examples/flash_gated_delta_rule.py:884-1023; per-op bindings
 * torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:397-427, 324-394, 463-514, 430-460, 242-281).
 * Unlike the reference's composition it also consumes the final-state cotangent dht and produces dh0.
 *   q, k, v, beta, gam, x_inv, s_img, vn_img, p_img: the forward's inputs and saved outputs (same shapes as there)
 *   d_o [B, T, HV, V] bf16;   dht [N, HV, 128, V] f32, optional
 *   dq, dk [B, T, HK, 128], dv [B, T, HV, V], dg, dbeta [B, T, HV]: all bf16 or all f32;  dh0 [N, HV, 128, V] f32, optional
 *   dq / dk are summed over the value heads of each GVA group inside the kernel (deterministic).
 * Workspace (size from the _workspace_size call): status block + state-gradient images + [dO; dZ] images + row sums. */
typedef struct fla_gdn_chunk_bwd_args {
  fla_tensor_t q, k, v, beta, gam, x_inv, s_img, vn_img, p_img, d_o, dht;
  fla_tensor_t dq, dk, dv, dg, dbeta, dh0;
  fla_tensor_t cu_seqlens, chunk_offsets;
  float scale;
  int32_t chunk_size;
  int32_t max_seqlen;
  int32_t total_chunks;
} fla_gdn_chunk_bwd_args;
FLA_API int fla_b200_gdn_chunk_bwd_workspace_size(const fla_gdn_chunk_bwd_args* args, uint64_t* bytes);
FLA_API int fla_b200_gdn_chunk_bwd(const fla_gdn_chunk_bwd_args* args, void* workspace, uint64_t workspace_bytes,
                                   void* stream);

/* Allocation-free backward (no counterpart in the reference, whose Python runtime always allocates the
 * workspace itself).  Same arguments and results as fla_b200_gdn_chunk_bwd, but the scratch is a fixed
 * 32 MiB array inside the library instead of a caller-provided workspace, and the call performs no
 * cudaMalloc / cudaFree and calls no allocating routine.  It is meant for callers that must not allocate
 * when they reach this call: runtimes that carved up one device arena at start-up and forbid later
 * allocations (a cudaMalloc can synchronise the device and stall the other streams of a serving process),
 * plugins that run inside another framework's callback and do not own its allocator, fixed-budget
 * real-time loops.
 *   - Limit: the scratch fla_b200_gdn_chunk_bwd_workspace_size reports for the arguments must not exceed
 *     fla_b200_gdn_chunk_bwd_static_scratch_bytes (32 MiB, about 290 (chunk, value-head) pairs, e.g. T = 512
 *     with HV = 32 or T = 1024 with HV = 16 for one sequence); larger problems return FLA_ERR_TOO_LARGE.
 *   - Every GPU whose context loads the library holds the 32 MiB until the process exits.
 *   - The first call on a device looks up the array's device address (with that device current); if the
 *     library's device code has not been loaded on that device yet, this lookup is also what loads it and
 *     places the 32 MiB (the CUDA runtime loads modules lazily), so the device's free memory drops once,
 *     at that call.  Make that first call before starting any stream capture.
 *   - All calls on one device share the array: two calls whose kernels can overlap on the GPU (different
 *     streams, or a second process thread) race on it.  Serialise them, or use the workspace entry point.
 *   - The status word of a call (see fla_b200_read_status_word) sits at the head of the built-in array,
 *     which the caller cannot address: fla_b200_gdn_chunk_bwd_noalloc_status waits for `stream` and returns
 *     the word left by the last call on the current device (FLA_OK when no call was made yet). */
FLA_API int fla_b200_gdn_chunk_bwd_static_scratch_bytes(uint64_t* bytes);
FLA_API int fla_b200_gdn_chunk_bwd_noalloc(const fla_gdn_chunk_bwd_args* args, void* stream);
FLA_API int fla_b200_gdn_chunk_bwd_noalloc_status(void* stream, int32_t* status_out);

/* ---------------------------------------------------------------------------------------------
 * Chunked Kimi Delta Attention, forward (per-channel log gate, chunk = 64, K = 128, V = 128 or 256).
 * Replaces aclnnKdaGateCumsum + aclnnChunkKdaFwd as bound by npu_kda_gate_cumsum / npu_chunk_kda_fwd
 * (torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:1268-1296, 1066-1265; stages in
 * fla/ops/ascendc/kda/chunk_kda_fwd/docs/design.md:11-78).
 *   q, k [B, T, HK, 128] bf16;  v [B, T, HV, V] bf16;  g [B, T, HV, 128] f32|bf16;  beta [B, T, HV] f32|bf16
 *   gate_mode 0: g is the log decay;  1: -exp(a_log[h]) * softplus(g + dt_bias[h, :]);
 *             2: lower_bound * sigmoid(exp(a_log[h]) * (g + dt_bias[h, :]))   (a_log [HV] f32, dt_bias [HV, 128] f32 optional)
 *   o [B, T, HV, 128] bf16|f32;  initial_state / final_state [N, HV, 128(K), 128(V)] f32, optional
 *   gk [B, T, HV, 128] f32, optional out: chunk-local cumulative sum of the activated gate (natural log units)
 *   cu_seqlens / chunk_offsets / max_seqlen / total_chunks: as in fla_gdn_chunk_fwd_args
 * Workspace: status block + per (chunk, head) operand images (about 121 KB each). */
typedef struct fla_kda_chunk_fwd_args {
  fla_tensor_t q, k, v, g, beta, a_log, dt_bias, initial_state;
  fla_tensor_t o, final_state, gk;
  fla_tensor_t cu_seqlens, chunk_offsets;
  fla_tensor_t saved;   /* optional out, 1-D bf16 of fla_b200_kda_chunk_saved_size bytes: what the backward otherwise recomputes */
  fla_tensor_t aqk, akk; /* optional out [B, T, HV, 64] bf16|f32 (any strides, e.g. head-first views): the per-chunk blocks
                            scale tril(q k^T 2^{gk_i-gk_j}) and (I + beta strict(k k^T 2^{gk_i-gk_j}))^-1 that npu_chunk_kda_fwd returns */
  float scale;
  float lower_bound;
  int32_t gate_mode;
  int32_t chunk_size;
  int32_t max_seqlen;
  int32_t total_chunks;
} fla_kda_chunk_fwd_args;
FLA_API int fla_b200_kda_chunk_fwd_workspace_size(const fla_kda_chunk_fwd_args* args, uint64_t* bytes);
/* Size of the `saved` buffer (the reference's disable_recompute=True mode of npu_chunk_kda_fwd, _aclnn_ctypes.py:1085,
 * keeps the forward's intermediates for the backward instead of recomputing them); gate_mode must be 0 with it. */
FLA_API int fla_b200_kda_chunk_saved_size(const fla_kda_chunk_fwd_args* args, uint64_t* bytes);
FLA_API int fla_b200_kda_chunk_fwd(const fla_kda_chunk_fwd_args* args, void* workspace, uint64_t workspace_bytes,
                                   void* stream);

/* The head-major intermediates of the reference's low-level KDA forward: what npu_chunk_kda_fwd returns in addition under
 * disable_recompute=True (w, u, qg, kg, v_new, h) or return_intermediate_states=True (h)
 * (torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:1066-1265, visibility _kda_policy.py:15-37, definitions
 * tests/atk/chunk_kda_fwd/executor_chunk_kda_fwd.py:447-492):
 *     qg = q 2^{gk}    kg = k 2^{gk_last - gk}    w = Akk (beta k 2^{gk})    u = Akk (beta v)    v_new = u - w S    h = S
 * with gk the chunk-local cumulative gate in base 2, Akk the chunk inverse and S the state at the start of each chunk.
 * Runs after fla_b200_kda_chunk_fwd on the `saved` buffer that call filled (same q, k, v, beta, cu_seqlens, chunk_offsets,
 * max_seqlen, total_chunks): a chunk-parallel fp32 pass on CUDA cores, outside the hot path.
 *   w, qg, kg [B, T, HV, K], u, v_new [B, T, HV, V]: optional out, bf16|f16|f32, any strides with a contiguous last dim
 *       (the reference's head-first [B, HV, T, .] tensors are passed as transposed views)
 *   h [total_chunks, HV, K, V] ([.., V, K] with state_v_first), dense, bf16|f16|f32, optional out
 * Single-phase (no workspace). */
typedef struct fla_kda_intermediates_args {
  fla_tensor_t q, k, v, beta;
  fla_tensor_t saved;
  fla_tensor_t cu_seqlens, chunk_offsets;
  fla_tensor_t w, u, qg, kg, v_new, h;
  int32_t max_seqlen;
  int32_t total_chunks;
  int32_t state_v_first;
} fla_kda_intermediates_args;
FLA_API int fla_b200_kda_chunk_intermediates(const fla_kda_intermediates_args* args, void* stream);

/* Score blocks of 128-token chunks (npu_chunk_kda_fwd takes chunk_size 64 or 128, _aclnn_ctypes.py:1094-1096) merged from
 * those of the 64-token chunks the kernels work in.  With A / B the halves of a 128-token chunk and L = gk at the end of A:
 *     gk128 = gk on A, gk + L on B;   Aqk128 = [[Aqk_A, 0], [scale (q e^{gk})_B (k e^{L-gk})_A^T, Aqk_B]];
 *     Akk128 = [[X_A, 0], [-X_B M X_A, X_B]],  M = beta_B (k e^{gk})_B (k e^{L-gk})_A^T
 *   q, k [B,T,HK,K] bf16, beta [B,T,HV] f32|bf16, gk [B,T,HV,K] f32 dense (cumulative gate of the 64-token chunks: natural log, the
 *   `gk` output of fla_b200_kda_chunk_fwd, or base 2 with gk_base2), aqk64 / akk64 [B,T,HV,64] f32 views (the forward's exports)
 *   aqk, akk [B,T,HV,128] out, bf16|f16|f32 views;  gk_out [B,T,HV,K] f32 view, optional out (base 2).
 * A chunk-parallel fp32 pass on CUDA cores, outside the hot path.  Single-phase (no workspace). */
typedef struct fla_kda_merge_blocks_args {
  fla_tensor_t q, k, beta, gk, aqk64, akk64;
  fla_tensor_t cu_seqlens, chunk_offsets;
  fla_tensor_t aqk, akk, gk_out;
  float scale;
  int32_t max_seqlen;
  int32_t gk_base2;   /* gk is given in base 2 (the output of fla_b200_chunk_local_cumsum with scale 1/ln 2) instead of natural log */
} fla_kda_merge_blocks_args;
FLA_API int fla_b200_kda_merge_score_blocks(const fla_kda_merge_blocks_args* args, void* stream);

/* w, u, qg, kg of 128-token chunks from those of their 64-token halves A, B (fla_b200_kda_chunk_intermediates with f32 outputs):
 *     qg128 = qg on A, qg e^L on B;   kg128 = kg e^{gk_B,last} on A, kg on B;
 *     w128 = w on A, w e^L - (X_B M) w_A on B;   u128 = u on A, u - (X_B M) u_A on B      (M as in the score-block merge)
 *   k [B,T,HK,K] bf16, beta [B,T,HV], gk [B,T,HV,K] f32 dense (natural log, or base 2 with gk_base2), akk64 [B,T,HV,64] f32 view,
 *   w64, qg64, kg64 [B,T,HV,K] and u64 [B,T,HV,V] f32 views;  w, u, qg, kg: out views of the same shapes, bf16|f16|f32, optional.
 * v_new does not depend on the blocking and h keeps every second state.  Single-phase (no workspace). */
typedef struct fla_kda_merge_inter_args {
  fla_tensor_t k, beta, gk, akk64, w64, u64, qg64, kg64;
  fla_tensor_t cu_seqlens, chunk_offsets;
  fla_tensor_t w, u, qg, kg;
  int32_t max_seqlen;
  int32_t gk_base2;
} fla_kda_merge_inter_args;
FLA_API int fla_b200_kda_merge_intermediates(const fla_kda_merge_inter_args* args, void* stream);

/* Gate activation of KDA as a tensor, and its gradient: what chunk_kda needs on its differentiable path when
 * use_gate_in_kernel is set (fla/ops/ascendc/kda/chunk_kda_fwd/docs/api.md:103-115; the inference path activates the gate
 * inside the forward kernels instead).
 *   gate_mode 1: gate = -e^{A_log[h]} softplus(g + dt_bias[h, :]);  2: gate = lower_bound sigmoid(e^{A_log[h]} (g + dt_bias[h, :]))
 *   g       [B, T, HV, K] f32|bf16|f16 (K = 128; batch rows back to back, contiguous channels)
 *   a_log   [HV] f32        dt_bias [HV, K] f32, optional
 *   fwd:  gate [B, T, HV, K] f32 dense, out
 *   bwd:  d_gate [B, T, HV, K] f32 in;  d_g [B, T, HV, K] dense, f32|bf16|f16, out;  d_a_log [HV] f32 and d_dt_bias [HV, K] f32,
 *         optional out (per-tile sums added in a fixed order: deterministic).  Workspace: the per-tile sums. */
typedef struct fla_kda_gate_args {
  fla_tensor_t g, a_log, dt_bias;
  fla_tensor_t gate;
  fla_tensor_t d_gate, d_g, d_a_log, d_dt_bias;
  float lower_bound;
  int32_t gate_mode;
} fla_kda_gate_args;
FLA_API int fla_b200_kda_gate_fwd(const fla_kda_gate_args* args, void* stream);
FLA_API int fla_b200_kda_gate_bwd_workspace_size(const fla_kda_gate_args* args, uint64_t* bytes);
FLA_API int fla_b200_kda_gate_bwd(const fla_kda_gate_args* args, void* workspace, uint64_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Chunked Kimi Delta Attention, backward (gate_mode 0: g is the per-channel log decay).
 * The reference has only the intra-chunk piece (aclnnChunkKdaBwdIntra as bound by npu_chunk_kda_bwd_intra,
 * torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:1534-1783) and defers the inter-chunk backward to a
 * third-party package; this entry computes the complete gradient of fla_b200_kda_chunk_fwd in one call.
 * It recomputes the forward internally (nothing has to be saved except the inputs) unless `saved` is given.
 *   q, k, v, g, beta, initial_state, cu_seqlens ...: the forward's inputs;  d_o [B, T, HV, 128] bf16;
 *   dht [N, HV, 128, 128] f32 optional (gradient of the final state);
 *   dq, dk [B, T, HK, 128] (summed over the value heads of a group), dv [B, T, HV, 128], dg [B, T, HV, 128],
 *   dbeta [B, T, HV]: all bf16 or all f32;  dh0 [N, HV, 128, 128] f32 optional.
 * Workspace: the forward's workspace plus about 250 KB per (chunk, value head). */
typedef struct fla_kda_chunk_bwd_args {
  fla_tensor_t q, k, v, g, beta, initial_state;
  fla_tensor_t d_o, dht;
  fla_tensor_t dq, dk, dv, dg, dbeta, dh0;
  fla_tensor_t cu_seqlens, chunk_offsets;
  fla_tensor_t saved;   /* optional in: the buffer the forward filled; skips the internal recomputation */
  float scale;
  int32_t chunk_size;
  int32_t max_seqlen;
  int32_t total_chunks;
} fla_kda_chunk_bwd_args;
FLA_API int fla_b200_kda_chunk_bwd_workspace_size(const fla_kda_chunk_bwd_args* args, uint64_t* bytes);
FLA_API int fla_b200_kda_chunk_bwd(const fla_kda_chunk_bwd_args* args, void* workspace, uint64_t workspace_bytes,
                                   void* stream);

/* ---------------------------------------------------------------------------------------------
 * Row-wise L2 normalisation (the q/k normalisation behind use_qk_l2norm_in_kernel).
 * Replaces the reference's Triton l2norm_fwd / l2norm_bwd (fla/ops/triton/triton_core/l2norm.py:131-234).
 *   fwd: x [rows, D] -> y [rows, D] = x * rstd, rstd [rows] f32 = rsqrt(sum x^2 + eps)
 *   bwd: y, rstd, dy -> dx = dy * rstd - (sum dy * y) * y * rstd
 * x, y, dy, dx bf16|f32 with contiguous columns and 16-byte aligned rows; D % 8 == 0, D <= 1024.
 * Single-phase (no workspace). */
typedef struct fla_l2norm_args {
  fla_tensor_t x, y, rstd, dy, dx;
  float eps;
} fla_l2norm_args;
FLA_API int fla_b200_l2norm_fwd(const fla_l2norm_args* args, void* stream);
FLA_API int fla_b200_l2norm_bwd(const fla_l2norm_args* args, void* stream);

/* ---------------------------------------------------------------------------------------------
 * FastGELU  y = x / (1 + exp(-1.702 x))  and its backward  dx = dy * (s + 1.702 x s (1 - s)), s = sigmoid(1.702 x).
 * Replaces npu_fast_gelu_custom / npu_fast_gelu_custom_backward (aclnnFastGelu / aclnnFastGeluBackward,
 * torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:224-239; golden formula
 * torch_custom/fla_npu/test/test_npu_fast_gelu_custom.py:22-24).
 *   x, y (fwd) / x, dy, dx (bwd): the same dtype (f32 | bf16 | f16) and element count, dense (contiguous) and 16-byte
 *   aligned; any rank up to FLA_MAX_DIMS.  Single-phase (no workspace). */
typedef struct fla_fast_gelu_args {
  fla_tensor_t x, y, dy, dx;
} fla_fast_gelu_args;
FLA_API int fla_b200_fast_gelu(const fla_fast_gelu_args* args, void* stream);
FLA_API int fla_b200_fast_gelu_bwd(const fla_fast_gelu_args* args, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Elementwise conversion between f32, bf16 and f16 tensors (round to nearest even) with re-layout.
 * The chunk and decode operators multiply bf16 operands; the reference also accepts fp16 tensors
 * (examples/flash_gated_delta_rule.py:1161-1162 rejects only fp32): the host wrappers route fp16 inputs and
 * results through this kernel (inputs are rounded from 11 to 8 significant bits).
 *   src, dst: the same shape, 1 to 4 dims, innermost dim contiguous, any other strides (a head-first view can be
 *   made token-major in the same pass).  Rows of a multiple of 8 elements at 16-byte aligned addresses take the
 *   vector path.  Single-phase (no workspace). */
FLA_API int fla_b200_convert(const fla_tensor_t* src, const fla_tensor_t* dst, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Stand-alone stages of the chunked gated-delta-rule forward: one entry point per low-level reference operator,
 * for call sites that drive the reference's stage-by-stage chain (examples/flash_gated_delta_rule.py:796-881)
 * instead of the fused fla_b200_gdn_chunk_fwd.  Token tensors are [B, H, T, D] and gate tensors [B, H, T], addressed
 * through their strides (the reference's head-first tensors, or sequence-first views of the same memory); D is
 * contiguous.  K = V = 128, chunk_size = 64.  GVA: HV % HK == 0, value head hv reads q/k head hv / (HV/HK).
 * cu_seqlens / chunk_offsets (int32 [N+1], device; B == 1): packed variable-length sequences; chunk_offsets[n] is the
 * index of sequence n's first chunk among all chunks; max_seqlen and total_chunks describe the packing.
 * All six share one argument block; each entry point reads the fields listed for it.
 *
 * fla_b200_chunk_local_cumsum   (aclnnChunkLocalCumsum, _aclnn_ctypes.py:875-904)
 *     g [B,H,T] or [B,H,T,D] f32|bf16|f16 -> out0 same shape, f32|bf16|f16:
 *     out0[t] = scale * sum of g over t's chunk up to t (reverse != 0: from t to the chunk's end).
 *     With a 4-D g and gate_mode != 0 this is aclnnKdaGateCumsum (:1268-1296; kda/chunk_kda_fwd/docs/api.md:103-115):
 *     the gate is activated first, -e^{A_log[h]} softplus(g + dt_bias[h,:]) (gate_mode 1) or
 *     lower_bound sigmoid(e^{A_log[h]} (g + dt_bias[h,:])) (gate_mode 2), with A_log [H] f32 passed in `q` and
 *     dt_bias [H,D] f32 (optional) in `k`; scale = 1/ln 2 gives the reference's base-2 gk.
 * fla_b200_chunk_scaled_dot_kkt (aclnnChunkScaledDotKkt, :907-936; golden test_npu_chunk_scaled_dot_kkt.py:60-103)
 *     k [B,HK,T,128] bf16, g (chunk-local cumulative gate) and beta [B,HV,T] -> out0 [B,HV,T,64] f32:
 *     out0[i,j] = beta_i exp(clamp(g_i - g_j, -50, 50)) k_i.k_j for j < i inside a chunk, else 0.
 * fla_b200_solve_tri            (aclnnSolveTri, :1786-1800; solve_tri/README.md:9-13)
 *     A [B,H,T,64] f32|bf16|f16 -> out0 same shape and dtype: per chunk (I + strict_lower(A))^-1.
 * fla_b200_recompute_w_u_fwd    (aclnnRecomputeWUFwd, :618-651; golden test_npu_recompute_w_u_fwd.py:38-145)
 *     k [B,HK,T,128], v [B,HV,T,128], A [B,HV,T,64] bf16 (the inverse), beta, g [B,HV,T]
 *     -> out0 = w [B,HV,T,128], out1 = u [B,HV,T,128] bf16:  w = A (k beta e^g),  u = A (v beta).
 * fla_b200_chunk_gated_delta_rule_fwd_h (aclnnChunkGatedDeltaRuleFwdH, :552-615; golden
 *     tests/atk/chunk_gated_delta_rule_fwd_h/executor_chunk_gated_delta_rule_fwd_h.py:79-135)
 *     k, w [B,HV,T,128], u [B,HV,T,128] bf16, g [B,HV,T], initial_state [N,HV,128,128] f32 (optional)
 *     -> out0 = h [B,HV,NT,128,128] bf16 dense (state at the start of every chunk), out1 = v_new [B,HV,T,128] bf16,
 *        out2 = final_state [N,HV,128,128] f32 (optional).
 * fla_b200_chunk_fwd_o          (aclnnChunkFwdO, :517-549; golden chunk_fwd_o/tests/pta/test_fwd_o.py:52-128)
 *     q, k [B,HK,T,128], v (= v_new) [B,HV,T,128], h [B,HV,NT,128,128] bf16, g [B,HV,T]
 *     -> out0 = o [B,HV,T,128] bf16:  o = scale (e^{g_i} q h_c + tril(q k^T e^{g_i - g_j}) v).
 * Two stages of the backward chain use the same block:
 * fla_b200_chunk_bwd_dv_local   (aclnnChunkBwdDvLocal, :397-427; golden
 *     fla/ops/ascendc/gdn/chunk_gdn_bwd/chunk_bwd_dv_local/tests/ATK/executor_chunk_bwd_dv_local.py:57-130)
 *     q, k [B,HK,T,128], v = d_o [B,HV,T,128] bf16, g [B,HV,T], scale
 *     -> out0 = dv [B,HV,T,128] bf16:  dv_j = sum_{i >= j in chunk} scale (k_j.q_i) e^{g_i - g_j} d_o_i.
 * fla_b200_chunk_gated_delta_rule_bwd_dhu (aclnnChunkGatedDeltaRuleBwdDhu, :324-394; golden
 *     torch_custom/fla_npu/test/test_bwd_dhu.py:61-290)
 *     q, k [B,HK,T,128], w [B,HV,T,128], u = d_o, v = dv [B,HV,T,128] bf16, g [B,HV,T], scale,
 *     initial_state = dht [N,HV,128,128] f32 (optional cotangent of the final state; the reference ignores it)
 *     -> out0 = dh [B,HV,NT,128,128] bf16 dense (gradient of the state at the END of every chunk), out1 = dv2 bf16,
 *        out2 = dh0 [N,HV,128,128] f32 (optional).  Reverse over chunks: dh_c = dS; dv2 = dv + e^{g_last - g} (k dS);
 *        dS <- e^{g_last} dS + q^T (scale e^g d_o) - w^T dv2.
 * fla_b200_chunk_bwd_dqkwg      (aclnnChunkBwdDqkwg, :463-514; golden tests/atk/chunk_bwd_dqkwg/scripts/chunk_bwd_dqkwg_cpu.py:66-409)
 *     q, k [B,HK,T,128], v = v_new, u = d_o, w = dv (the dv2 of the reverse pass) [B,HV,T,128] bf16, g [B,HV,T],
 *     h and A = dh [B,HV,NT,128,128] bf16 dense, scale
 *     -> out0 = dq, out1 = dk [B,HK,T,128] bf16 (summed over the value heads of a group), out2 = dw [B,HV,T,128] bf16
 *        (optional), out3 = dg [B,HV,T] (before the reverse cumulative sum, the chunk's last row carrying the state terms).
 *     Workspace: 256 bytes, plus 2 * B*HV*T*128 fp32 when HV > HK (fla_b200_chunk_bwd_dqkwg_workspace_size).
 * fla_b200_prepare_wy_repr_bwd_da   (aclnnPrepareWyReprBwdDa, :430-460; golden test_npu_prepare_wy_repr_bwd_da.py:166-291)
 *     k [B,HK,T,128], v [B,HV,T,128], A (the inverse) [B,HV,T,64], w = dw, u = du [B,HV,T,128] bf16, beta, g [B,HV,T]
 *     -> out0 = dA [B,HV,T,64] (any float dtype), stored transposed within each chunk:
 *        dA^T = strict_lower(-(A^T strict_lower(dw (k beta e^g)^T + du (v beta)^T) A^T) * e^{g_i - g_j}).
 * fla_b200_prepare_wy_repr_bwd_full (aclnnPrepareWyReprBwdFull, :242-281; goldens test_npu_prepare_wy_repr_bwd_full.py:47-428)
 *     the same inputs plus q = dA (as produced above)
 *     -> out0 = dk [B,HK,T,128] bf16 (summed over the value heads of a group), out1 = dv [B,HV,T,128] bf16,
 *        out2 = dbeta, out3 = dg [B,HV,T].
 * fla_b200_prepare_wy_repr_bwd      (aclnnPrepareWyReprBwd, :284-321): both steps in one launch, dA never leaves the chip.
 *     Workspace of the last two: 256 bytes, plus B*HV*T*128 fp32 when HV > HK.
 * Workspace of the others: 256 bytes (status word of the bounded device-side waits). */
typedef struct fla_chunk_stage_args {
  fla_tensor_t q, k, v, w, u, g, beta, A, h, initial_state;
  fla_tensor_t out0, out1, out2, out3;
  fla_tensor_t cu_seqlens, chunk_offsets;
  float scale;
  int32_t chunk_size;
  int32_t max_seqlen;
  int32_t total_chunks;
  int32_t reverse;
  int32_t gate_mode;   /* chunk_local_cumsum of per-channel gates only */
  float lower_bound;
} fla_chunk_stage_args;
FLA_API int fla_b200_chunk_local_cumsum_workspace_size(const fla_chunk_stage_args* args, uint64_t* bytes);
FLA_API int fla_b200_chunk_scaled_dot_kkt_workspace_size(const fla_chunk_stage_args* args, uint64_t* bytes);
FLA_API int fla_b200_solve_tri_workspace_size(const fla_chunk_stage_args* args, uint64_t* bytes);
FLA_API int fla_b200_recompute_w_u_fwd_workspace_size(const fla_chunk_stage_args* args, uint64_t* bytes);
FLA_API int fla_b200_chunk_gated_delta_rule_fwd_h_workspace_size(const fla_chunk_stage_args* args, uint64_t* bytes);
FLA_API int fla_b200_chunk_fwd_o_workspace_size(const fla_chunk_stage_args* args, uint64_t* bytes);
FLA_API int fla_b200_chunk_local_cumsum(const fla_chunk_stage_args* args, void* workspace, uint64_t workspace_bytes, void* stream);
FLA_API int fla_b200_chunk_scaled_dot_kkt(const fla_chunk_stage_args* args, void* workspace, uint64_t workspace_bytes, void* stream);
FLA_API int fla_b200_solve_tri(const fla_chunk_stage_args* args, void* workspace, uint64_t workspace_bytes, void* stream);
FLA_API int fla_b200_recompute_w_u_fwd(const fla_chunk_stage_args* args, void* workspace, uint64_t workspace_bytes, void* stream);
FLA_API int fla_b200_chunk_gated_delta_rule_fwd_h(const fla_chunk_stage_args* args, void* workspace, uint64_t workspace_bytes,
                                                  void* stream);
FLA_API int fla_b200_chunk_fwd_o(const fla_chunk_stage_args* args, void* workspace, uint64_t workspace_bytes, void* stream);
FLA_API int fla_b200_chunk_bwd_dv_local_workspace_size(const fla_chunk_stage_args* args, uint64_t* bytes);
FLA_API int fla_b200_chunk_gated_delta_rule_bwd_dhu_workspace_size(const fla_chunk_stage_args* args, uint64_t* bytes);
FLA_API int fla_b200_prepare_wy_repr_bwd_workspace_size(const fla_chunk_stage_args* args, uint64_t* bytes);
FLA_API int fla_b200_prepare_wy_repr_bwd(const fla_chunk_stage_args* args, void* workspace, uint64_t workspace_bytes, void* stream);
FLA_API int fla_b200_prepare_wy_repr_bwd_da_workspace_size(const fla_chunk_stage_args* args, uint64_t* bytes);
FLA_API int fla_b200_prepare_wy_repr_bwd_da(const fla_chunk_stage_args* args, void* workspace, uint64_t workspace_bytes, void* stream);
FLA_API int fla_b200_prepare_wy_repr_bwd_full_workspace_size(const fla_chunk_stage_args* args, uint64_t* bytes);
FLA_API int fla_b200_prepare_wy_repr_bwd_full(const fla_chunk_stage_args* args, void* workspace, uint64_t workspace_bytes, void* stream);
FLA_API int fla_b200_chunk_bwd_dqkwg_workspace_size(const fla_chunk_stage_args* args, uint64_t* bytes);
FLA_API int fla_b200_chunk_bwd_dqkwg(const fla_chunk_stage_args* args, void* workspace, uint64_t workspace_bytes, void* stream);
FLA_API int fla_b200_chunk_bwd_dv_local(const fla_chunk_stage_args* args, void* workspace, uint64_t workspace_bytes, void* stream);
FLA_API int fla_b200_chunk_gated_delta_rule_bwd_dhu(const fla_chunk_stage_args* args, void* workspace, uint64_t workspace_bytes,
                                                    void* stream);

/* ---------------------------------------------------------------------------------------------
 * chunk_kda_bwd_intra: intra-chunk part of the KDA backward as a stand-alone, accumulating operator.
 * Replaces aclnnChunkKdaBwdIntra as bound by npu_chunk_kda_bwd_intra
 * (torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:1534-1783; golden
 * torch_custom/fla_npu/test/test_npu_chunk_kda_bwd_intra.py:7-91).  (fla_b200_kda_chunk_bwd computes the complete KDA
 * gradient without this split.)
 *   q, k [B,T,H,128] bf16; gk [B,T,H,128] f32 (base-2 chunk-local cumulative gate); beta [B,T,H] bf16|f32;
 *   d_aqk, d_akk [B,T,H,64] f32: gradients of the two score blocks, lower triangle with diagonal used;
 *   dq, dk, dg [B,T,H,128] f32 and db [B,T,H] f32 are updated IN PLACE (+=):
 *     dq_i += sum_{j<=i} d_aqk[i][j] k_j 2^{g_i-g_j};  lower_i = sum_{j<=i} d_akk[i][j] k_j 2^{g_i-g_j};
 *     upper_j = sum_{i>=j} (d_aqk[i][j] q_i + d_akk[i][j] beta_i k_i) 2^{g_i-g_j};
 *     dk_i += beta_i lower_i + upper_i;  db_i += lower_i.k_i;  dg_i += q_i*dq_delta_i + k_i*(beta_i lower_i - upper_i).
 *   Head-first tensors are passed as strided views; q, k, gk, dq, dk, dg share one set of strides, d_aqk and d_akk another,
 *   beta and db a third.  chunk_size = 64.  cu_seqlens / chunk_offsets as for the chunk operators.  No workspace. */
typedef struct fla_chunk_kda_bwd_intra_args {
  fla_tensor_t q, k, gk, beta, d_aqk, d_akk, dq, dk, db, dg;
  fla_tensor_t cu_seqlens, chunk_offsets;
  int32_t chunk_size;
  int32_t max_seqlen;
  int32_t total_chunks;
} fla_chunk_kda_bwd_intra_args;
FLA_API int fla_b200_chunk_kda_bwd_intra_workspace_size(const fla_chunk_kda_bwd_intra_args* args, uint64_t* bytes);
FLA_API int fla_b200_chunk_kda_bwd_intra(const fla_chunk_kda_bwd_intra_args* args, void* workspace, uint64_t workspace_bytes,
                                         void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLA_B200_H_ */

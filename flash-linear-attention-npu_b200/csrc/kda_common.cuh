// Parameter block and image sizes shared by the KDA chunk forward and backward translation units.
#pragma once
#include "gdn_common.cuh"

namespace fla {

struct KdaParams {
  const bf16* q; const bf16* k; const bf16* v;
  const void* g; const void* beta;
  const float* a_log; const float* dt_bias;   // optional gate parameters: [HV], [HV, K]
  float* gk_out;        // [tokens, HV, K] cumulative gate (optional)
  bf16* qk_img;         // [chunks, HV, {hi, lo}, 2 panels x 128 rows]  rows 0-63 Qp, rows 64-127 Kp
  bf16* kn_img;         // [chunks, HV, {hi, lo}, 2 panels x 64 rows]
  bf16* p_img;          // [chunks, HV, {hi, lo}, 64 x 64]   tril(Qp Kn^T)
  bf16* x_img;          // [chunks, HV, {hi, lo}, 64 x 64]   (I + Akk)^-1 (written by the inverse kernel)
  float* at;            // [chunks, HV, 64, 64] scratch: Akk^T for the inverse kernel
  float* vec;           // [chunks, HV, 3, K]  e^a, e^{gk_L - a}, a
  bf16* s_img;          // optional out for the backward: [chunks, HV, V/64, {hi, lo}, 128 x 64]  Sa = diag(e^a) S at chunk start
  bf16* vn_img;         // optional out for the backward: [chunks, HV, V/64, {hi, lo}, 64 x 64]   v_new
  const float* h0; float* ht;
  void* o;              // may be null when only the saved images are wanted
  const int32_t* cu_seqlens; const int32_t* chunk_offsets;
  int64_t q_st, q_sh, k_st, k_sh, v_st, v_sh, o_st, o_sh, g_st, g_sh, beta_st;
  int64_t total_tokens;   // rows of the flat [tokens, heads, dim] views
  int N, T, HK, HV, g_is_f32, beta_is_f32, o_is_f32, gate_mode;
  int V, nvb;           // value head dim (128 or 256) and its number of 64-column blocks
  float scale, lower_bound;
  int* status;
};

constexpr int64_t kKdaQkImg = 32768, kKdaKnImg = 16384, kKdaPImg = 8192, kKdaXImg = 8192;  // bf16 elements, hi + lo
constexpr int64_t kKdaSImg = 16384, kKdaVnImg = 8192;   // per 64-column block of V
constexpr int kKdaVecs = 3;

// Workspace layout of the forward (offsets of qk_img, kn_img, p_img, x_img, vec, at); returns the total size.
uint64_t kda_ws_layout(int64_t total_chunks, int64_t HV, uint64_t off[6]);
// Layout of the buffer a training forward leaves for the backward: the forward workspace (operand images), gk, the
// Sa images and the v_new images; returns the total size.
uint64_t kda_saved_layout(int64_t total_chunks, int64_t HV, int64_t nvb, int64_t tokens, uint64_t off[4]);
// prep -> inverse -> forward scan on `stream`; 0 or an FLA_ERR_* status.
int kda_launch_forward(const KdaParams& p, int nt_max, cudaStream_t stream);

}  // namespace fla

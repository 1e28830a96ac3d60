// chunk_kda_bwd_intra: the intra-chunk part of the KDA backward as a stand-alone operator
// (aclnnChunkKdaBwdIntra as bound by npu_chunk_kda_bwd_intra,
// torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:1534-1783; golden
// torch_custom/fla_npu/test/test_npu_chunk_kda_bwd_intra.py:7-91).
//
// Per chunk of 64 tokens and head, with base-2 per-channel cumulative gates gk and the gradients dAqk, dAkk of the two
// lower-triangular score blocks (diagonal included):
//   dq_i      += sum_{j<=i} dAqk[i][j] k_j 2^{g_i - g_j}
//   lower_i    = sum_{j<=i} dAkk[i][j] k_j 2^{g_i - g_j}
//   upper_j    = sum_{i>=j} (dAqk[i][j] q_i + dAkk[i][j] beta_i k_i) 2^{g_i - g_j}
//   dk_i      += beta_i lower_i + upper_i
//   db_i      += lower_i . k_i
//   dg_i      += q_i * dq_delta_i + k_i * (beta_i lower_i - upper_i)          (per channel)
// All arithmetic is fp32 on the CUDA cores (the operator's inputs and outputs are fp32 apart from q, k): like the
// reference golden, every exponent is taken relative to an anchor row inside a 16-row tile so that no power of two
// leaves the fp32 range for gates as steep as the safe-gate lower bound allows.
//
// One CTA per (chunk, head), 256 threads: thread (c, half) owns key channel c and the two 16-row tiles of its half
// of the chunk.  q, k, gk of the chunk and the two 64 x 64 blocks sit in shared memory; the score-gradient entries
// are read as warp-wide broadcasts.
#include "gdn_common.cuh"
#include "fla_b200_internal.h"
#include "kernel_timer.h"

namespace fla {

struct KdaIntraParams {
  const bf16* q;
  const bf16* k;
  const float* gk;
  const void* beta;
  int beta_is_f32;
  const float* daqk;
  const float* dakk;
  float* dq;
  float* dk;
  float* db;
  float* dg;
  // element strides of [B, T, H, .] tensors: batch, token, head
  int64_t sb, st, sh;          // q, k, gk, dq, dk, dg (128 channels contiguous)
  int64_t ab, at, ah;          // dAqk, dAkk (64 contiguous)
  int64_t bb, bt, bh;          // beta, db
  const int32_t* cu_seqlens;
  const int32_t* chunk_offsets;
  int T, H;
};

constexpr int kIntraTile = 16;
constexpr int kAStride = 68;     // fp32 row stride of the 64 x 64 blocks (16-byte aligned rows)
constexpr uint32_t kIntraSmem = (3 * kC * kK + 2 * kC * kAStride + kC) * sizeof(float);

__global__ void __launch_bounds__(256) kda_bwd_intra_kernel(KdaIntraParams p) {
  extern __shared__ float sm[];
  float* q_s = sm;                       // [64][128]
  float* k_s = q_s + kC * kK;
  float* g_s = k_s + kC * kK;
  float* aqk_s = g_s + kC * kK;          // [64][68], lower triangle incl. diagonal, zero elsewhere
  float* akk_s = aqk_s + kC * kAStride;
  float* beta_s = akk_s + kC * kAStride;
  const int tid = threadIdx.x;
  const int n = blockIdx.z, hh = blockIdx.y, chunk = blockIdx.x;
  const SeqInfo sq = seq_info(p.cu_seqlens, p.chunk_offsets, n, p.T);
  if (chunk >= sq.nt) return;
  const int rows = min(kC, sq.len - chunk * kC);
  const int64_t b = p.cu_seqlens ? 0 : n;
  const int64_t t0 = (p.cu_seqlens ? sq.bos : 0) + chunk * kC;

  // stage the chunk (rows past its end as zeros)
  for (int idx = tid; idx < kC * (kK / 8); idx += 256) {
    const int r = idx / (kK / 8), ch = idx % (kK / 8);
    float qv[8] = {0, 0, 0, 0, 0, 0, 0, 0}, kv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float4 g0 = make_float4(0.f, 0.f, 0.f, 0.f), g1 = g0;
    if (r < rows) {
      const int64_t off = b * p.sb + (t0 + r) * p.st + hh * p.sh + ch * 8;
      unpack_bf16x8(*reinterpret_cast<const uint4*>(p.q + off), qv);
      unpack_bf16x8(*reinterpret_cast<const uint4*>(p.k + off), kv);
      g0 = *reinterpret_cast<const float4*>(p.gk + off);
      g1 = *reinterpret_cast<const float4*>(p.gk + off + 4);
    }
    float* qd = q_s + r * kK + ch * 8;
    float* kd = k_s + r * kK + ch * 8;
    float* gd = g_s + r * kK + ch * 8;
    *reinterpret_cast<float4*>(qd) = make_float4(qv[0], qv[1], qv[2], qv[3]);
    *reinterpret_cast<float4*>(qd + 4) = make_float4(qv[4], qv[5], qv[6], qv[7]);
    *reinterpret_cast<float4*>(kd) = make_float4(kv[0], kv[1], kv[2], kv[3]);
    *reinterpret_cast<float4*>(kd + 4) = make_float4(kv[4], kv[5], kv[6], kv[7]);
    *reinterpret_cast<float4*>(gd) = g0;
    *reinterpret_cast<float4*>(gd + 4) = g1;
  }
  for (int idx = tid; idx < kC * (kC / 4); idx += 256) {
    const int r = idx / (kC / 4), c4 = idx % (kC / 4);
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f), k4 = a;
    if (r < rows) {
      const int64_t off = b * p.ab + (t0 + r) * p.at + hh * p.ah + c4 * 4;
      a = *reinterpret_cast<const float4*>(p.daqk + off);
      k4 = *reinterpret_cast<const float4*>(p.dakk + off);
    }
    const int j = c4 * 4;
    // keep the lower triangle (diagonal included) of the valid block
    a.x = (j <= r && j < rows) ? a.x : 0.f;         k4.x = (j <= r && j < rows) ? k4.x : 0.f;
    a.y = (j + 1 <= r && j + 1 < rows) ? a.y : 0.f; k4.y = (j + 1 <= r && j + 1 < rows) ? k4.y : 0.f;
    a.z = (j + 2 <= r && j + 2 < rows) ? a.z : 0.f; k4.z = (j + 2 <= r && j + 2 < rows) ? k4.z : 0.f;
    a.w = (j + 3 <= r && j + 3 < rows) ? a.w : 0.f; k4.w = (j + 3 <= r && j + 3 < rows) ? k4.w : 0.f;
    *reinterpret_cast<float4*>(aqk_s + r * kAStride + j) = a;
    *reinterpret_cast<float4*>(akk_s + r * kAStride + j) = k4;
  }
  if (tid < kC) beta_s[tid] = tid < rows ? ld_scalar(p.beta, b * p.bb + (t0 + tid) * p.bt + hh * p.bh, p.beta_is_f32) : 0.f;
  __syncthreads();

  const int c = tid & (kK - 1), half = tid >> 7;
  for (int tile = half * 2; tile < half * 2 + 2; ++tile) {
    const int row_begin = tile * kIntraTile;
    if (row_begin >= rows) break;
    const int row_end = min(row_begin + kIntraTile, rows);
    const int anchor = min(row_begin + 8, row_end - 1);
    const float ca = g_s[anchor * kK + c];

    // lower part: rows of this tile against all earlier rows (and themselves)
    float accq[kIntraTile], acck[kIntraTile];
#pragma unroll
    for (int r = 0; r < kIntraTile; ++r) accq[r] = acck[r] = 0.f;
    for (int j4 = 0; j4 < row_end; j4 += 4) {
      float lb[4];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int j = j4 + jj;
        lb[jj] = j < row_end ? k_s[j * kK + c] * exp2f(ca - g_s[j * kK + c]) : 0.f;
      }
#pragma unroll
      for (int r = 0; r < kIntraTile; ++r) {
        const float4 a = *reinterpret_cast<const float4*>(aqk_s + (row_begin + r) * kAStride + j4);   // zero above the diagonal
        const float4 k4 = *reinterpret_cast<const float4*>(akk_s + (row_begin + r) * kAStride + j4);
        accq[r] += a.x * lb[0] + a.y * lb[1] + a.z * lb[2] + a.w * lb[3];
        acck[r] += k4.x * lb[0] + k4.y * lb[1] + k4.z * lb[2] + k4.w * lb[3];
      }
    }
    // upper part: later rows (and themselves) against the rows of this tile
    float accu[kIntraTile];
#pragma unroll
    for (int r = 0; r < kIntraTile; ++r) accu[r] = 0.f;
    for (int i = row_begin; i < rows; ++i) {
      const float fw = exp2f(g_s[i * kK + c] - ca);
      const float uq = q_s[i * kK + c] * fw, uk = k_s[i * kK + c] * beta_s[i] * fw;
      const float* ar = aqk_s + i * kAStride + row_begin;
      const float* kr = akk_s + i * kAStride + row_begin;
#pragma unroll
      for (int r4 = 0; r4 < kIntraTile; r4 += 4) {
        const float4 a = *reinterpret_cast<const float4*>(ar + r4);     // zero where the column is later than row i
        const float4 k4 = *reinterpret_cast<const float4*>(kr + r4);
        accu[r4] += a.x * uq + k4.x * uk;
        accu[r4 + 1] += a.y * uq + k4.y * uk;
        accu[r4 + 2] += a.z * uq + k4.z * uk;
        accu[r4 + 3] += a.w * uq + k4.w * uk;
      }
    }
    // finish the rows of the tile
#pragma unroll
    for (int r = 0; r < kIntraTile; ++r) {
      const int i = row_begin + r;
      if (i < row_end) {
        const float gi = g_s[i * kK + c];
        const float rs = exp2f(gi - ca), ri = exp2f(ca - gi);
        const float dq_delta = accq[r] * rs, lower = acck[r] * rs, upper = accu[r] * ri;
        const float kk = k_s[i * kK + c], qq = q_s[i * kK + c], bl = beta_s[i] * lower;
        const int64_t off = b * p.sb + (t0 + i) * p.st + hh * p.sh + c;
        p.dq[off] += dq_delta;
        p.dk[off] += bl + upper;
        p.dg[off] += qq * dq_delta + kk * (bl - upper);
        // db: lower . k over the 128 channels = the four warps of this half
        float part = lower * kk;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
        if ((tid & 31) == 0) atomicAdd(p.db + b * p.bb + (t0 + i) * p.bt + hh * p.bh, part);
      }
    }
  }
}

}  // namespace fla

using namespace fla;

extern "C" FLA_API int fla_b200_chunk_kda_bwd_intra_workspace_size(const fla_chunk_kda_bwd_intra_args* a, uint64_t* bytes) {
  if (!a || !bytes) return FLA_ERR_NULL;
  *bytes = 0;
  return FLA_OK;
}

extern "C" FLA_API int fla_b200_chunk_kda_bwd_intra(const fla_chunk_kda_bwd_intra_args* a, void* workspace, uint64_t workspace_bytes,
                                                    void* stream) {
  if (!a) return FLA_ERR_NULL;
  (void)workspace; (void)workspace_bytes;
  cudaStream_t cs = static_cast<cudaStream_t>(stream);
  const fla_tensor_t& q = a->q;
  if (!q.data) return FLA_ERR_NULL;
  if (q.ndim != 4) return FLA_ERR_SHAPE;
  const int64_t B = q.shape[0], T = q.shape[1], H = q.shape[2];
  if (B <= 0 || T <= 0 || H <= 0 || q.shape[3] != kK) return FLA_ERR_SHAPE;
  if (a->chunk_size != kC) return FLA_ERR_VALUE;
  for (const fla_tensor_t* t : {&a->q, &a->k, &a->gk, &a->dq, &a->dk, &a->dg}) {
    if (!t->data) return FLA_ERR_NULL;
    if (t->ndim != 4 || t->shape[0] != B || t->shape[1] != T || t->shape[2] != H || t->shape[3] != kK) return FLA_ERR_SHAPE;
    for (int d = 0; d < 4; ++d)
      if (t->stride[d] != q.stride[d]) return FLA_ERR_LAYOUT;
    if (t->stride[3] != 1 || !aligned16(t->data) || (t->stride[0] % 8) || (t->stride[1] % 8) || (t->stride[2] % 8)) return FLA_ERR_LAYOUT;
  }
  if (a->q.dtype != FLA_BF16 || a->k.dtype != FLA_BF16) return FLA_ERR_DTYPE;
  for (const fla_tensor_t* t : {&a->gk, &a->dq, &a->dk, &a->dg, &a->d_aqk, &a->d_akk, &a->db})
    if (t->dtype != FLA_F32) return FLA_ERR_DTYPE;
  for (const fla_tensor_t* t : {&a->d_aqk, &a->d_akk}) {
    if (!t->data) return FLA_ERR_NULL;
    if (t->ndim != 4 || t->shape[0] != B || t->shape[1] != T || t->shape[2] != H || t->shape[3] != kC) return FLA_ERR_SHAPE;
    for (int d = 0; d < 4; ++d)
      if (t->stride[d] != a->d_aqk.stride[d]) return FLA_ERR_LAYOUT;
    if (t->stride[3] != 1 || !aligned16(t->data) || (t->stride[0] % 4) || (t->stride[1] % 4) || (t->stride[2] % 4)) return FLA_ERR_LAYOUT;
  }
  for (const fla_tensor_t* t : {&a->beta, &a->db}) {
    if (!t->data) return FLA_ERR_NULL;
    if (t->ndim != 3 || t->shape[0] != B || t->shape[1] != T || t->shape[2] != H) return FLA_ERR_SHAPE;
  }
  if (a->beta.dtype != FLA_BF16 && a->beta.dtype != FLA_F32) return FLA_ERR_DTYPE;
  // beta and db share one index computation only if their strides agree
  for (int d = 0; d < 3; ++d)
    if (a->beta.stride[d] != a->db.stride[d]) return FLA_ERR_LAYOUT;

  KdaIntraParams p{};
  p.q = static_cast<const bf16*>(a->q.data); p.k = static_cast<const bf16*>(a->k.data);
  p.gk = static_cast<const float*>(a->gk.data);
  p.beta = a->beta.data; p.beta_is_f32 = a->beta.dtype == FLA_F32;
  p.daqk = static_cast<const float*>(a->d_aqk.data); p.dakk = static_cast<const float*>(a->d_akk.data);
  p.dq = static_cast<float*>(a->dq.data); p.dk = static_cast<float*>(a->dk.data);
  p.db = static_cast<float*>(a->db.data); p.dg = static_cast<float*>(a->dg.data);
  p.sb = q.stride[0]; p.st = q.stride[1]; p.sh = q.stride[2];
  p.ab = a->d_aqk.stride[0]; p.at = a->d_aqk.stride[1]; p.ah = a->d_aqk.stride[2];
  p.bb = a->beta.stride[0]; p.bt = a->beta.stride[1]; p.bh = a->beta.stride[2];
  p.T = int(T); p.H = int(H);
  int N = int(B), max_len = int(T);
  if (a->cu_seqlens.data) {
    if (B != 1 || a->cu_seqlens.dtype != FLA_I32 || a->cu_seqlens.ndim != 1 || a->cu_seqlens.shape[0] < 2) return FLA_ERR_SHAPE;
    N = int(a->cu_seqlens.shape[0] - 1);
    if (!a->chunk_offsets.data || a->chunk_offsets.dtype != FLA_I32 || a->chunk_offsets.shape[0] != N + 1) return FLA_ERR_SHAPE;
    if (a->max_seqlen <= 0 || a->max_seqlen > T) return FLA_ERR_VALUE;
    max_len = a->max_seqlen;
    p.cu_seqlens = static_cast<const int32_t*>(a->cu_seqlens.data);
    p.chunk_offsets = static_cast<const int32_t*>(a->chunk_offsets.data);
  }
  static std::atomic<bool> attr_done_dev[64] = {};   // per device ordinal; setting the attributes twice is harmless
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FLA_ERR_CUDA;
  if (!attr_done_dev[dev]) {
    if (cudaFuncSetAttribute(kda_bwd_intra_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kIntraSmem)) != cudaSuccess)
      return FLA_ERR_CUDA;
    attr_done_dev[dev] = true;
  }
  KernelTimer kt("chunk_kda_bwd_intra", cs);
  kda_bwd_intra_kernel<<<dim3((max_len + kC - 1) / kC, unsigned(H), N), 256, kIntraSmem, cs>>>(p);
  return cuda_status(cudaGetLastError());
}

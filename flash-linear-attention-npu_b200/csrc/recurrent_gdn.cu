// Fused-recurrent gated delta rule (decode / short-sequence step) over a pool of per-sequence states.
//
// One CTA owns one (sequence, value-head) state matrix (128 of its value channels when V = 256), streams it from HBM once with 16-byte
// loads, applies up to a few tokens of
//     S <- exp(g) S  (scalar g per head and / or a per-key-channel gate gk: S <- diag(exp(gk)) S) ;
//     d = beta (v - S^T k) ;  S <- S + k d^T ;  o = S^T (scale q)
// entirely in registers (fp32), and streams it back.  The kernel is HBM-bound: per (seq, head) it
// moves K*V*sizeof(state) bytes in and out and a few hundred bytes of activations; no tensor cores.
// Replaces the reference operators recurrent_gated_delta_rule
// (fla/ops/ascendc/gdn/recurrent_gdn/recurrent_gated_delta_rule/op_kernel/recurrent_gated_delta_rule.h:159-199,364-402,445-513)
// and recurrent_kda (fla/ops/ascendc/kda/recurrent_kda/docs/design.md:44-70: per-channel gate with optional in-kernel
// gate activation and beta sigmoid).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "fla_b200_internal.h"
#include "kernel_timer.h"

namespace fla {

struct RecurrentParams {
  const void* q;           // [T, HK, K]  bf16, or fp16 when act_f16
  const void* k;           // [T, HK, K]
  const void* v;           // [T, HV, V]
  const void* g;           // [T, HV] or null
  const void* beta;        // [T, HV] or null
  const void* gk;          // [T, HV, K] per-channel log gate (raw when gate_mode != 0) or null
  const float* a_log;      // [HV] or null
  const float* dt_bias;    // [HV, K] or null
  const void* state_in;    // [blocks, HV, K, V] (or [.., V, K] when v-first)
  void* state_out;         // may alias state_in
  void* out;               // [T, HV, V]
  const int32_t* cu_seqlens;           // [N+1] or null (then every sequence has tokens_per_seq tokens)
  const int32_t* state_indices;        // [T] or null (then sequence n uses block n, written once at the end)
  const int32_t* num_accepted_tokens;  // [N] or null
  int64_t q_stride_t, q_stride_h, k_stride_t, k_stride_h, v_stride_t, v_stride_h;
  int64_t g_stride_t, beta_stride_t, out_stride_t, out_stride_h;
  int64_t state_in_stride_b, state_in_stride_h, state_out_stride_b, state_out_stride_h;
  int HK, HV, tokens_per_seq, nblocks_in, nblocks_out;
  int64_t gk_stride_t, gk_stride_h;
  int g_is_f32, beta_is_f32, out_is_f32, l2norm, gk_is_f32, gate_mode, beta_mode;
  int act_f16, out_is_f16;   // q, k, v are fp16 (read exactly: the arithmetic is fp32) / out is fp16
  float scale, lower_bound;
};

template <typename T>
__device__ __forceinline__ float4 load4(const T* p);
template <>
__device__ __forceinline__ float4 load4<float>(const float* p) {
  return *reinterpret_cast<const float4*>(p);
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
template <>
__device__ __forceinline__ float4 load4<__half>(const __half* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T>
__device__ __forceinline__ void store4(T* p, float4 x);
template <>
__device__ __forceinline__ void store4<__half>(__half* p, float4 x) {
  __half2 a = __floats2half2_rn(x.x, x.y), b = __floats2half2_rn(x.z, x.w);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&a);
  raw.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}
template <>
__device__ __forceinline__ void store4<float>(float* p, float4 x) {
  *reinterpret_cast<float4*>(p) = x;
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 x) {
  __nv_bfloat162 a = __floats2bfloat162_rn(x.x, x.y), b = __floats2bfloat162_rn(x.z, x.w);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&a);
  raw.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

// one activation element (q, k, v): bf16, or fp16 when f16
__device__ __forceinline__ float load_act(const void* p, int64_t idx, int f16) {
  return f16 ? __half2float(static_cast<const __half*>(p)[idx]) : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
}
__device__ __forceinline__ float load_scalar(const void* p, int64_t idx, int is_f32) {
  return is_f32 ? static_cast<const float*>(p)[idx] : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[idx]);
}

constexpr int kRecThreads = 256;

// ROWS x COLS state tile held by one CTA (COLS contiguous in memory, LD elements between rows).  The columns of V
// are independent recurrences, so a CTA owns VT of the V value channels: K-first ROWS = K, COLS = VT, LD = V;
// V-first ROWS = VT, COLS = K, LD = K.
template <int K, int V, int VT, typename ST, bool VFIRST>
__global__ void __launch_bounds__(kRecThreads, 3) recurrent_gdn_kernel(RecurrentParams p) {
  constexpr int ROWS = VFIRST ? VT : K;
  constexpr int COLS = VFIRST ? K : VT;
  constexpr int LD = VFIRST ? K : V;
  constexpr int NVB = V / VT;
  constexpr int TPR = COLS / 4;              // threads per row
  constexpr int RG = kRecThreads / TPR;      // row groups handled per pass
  constexpr int R = ROWS / RG;               // rows per thread
  static_assert(ROWS % RG == 0 && TPR <= 32, "unsupported head dims");

  __shared__ float k_s[K], q_s[K], dk_s[K];
  __shared__ __align__(16) float red[VFIRST ? 1 : RG][VFIRST ? 4 : COLS];
  __shared__ float norm_s[2];

  const int vb = blockIdx.x % NVB;
  const int seq = (blockIdx.x / NVB) / p.HV, hv = (blockIdx.x / NVB) % p.HV;
  const int v0 = vb * VT;                                   // first value channel of this CTA
  const int64_t tile_off = VFIRST ? int64_t(v0) * LD : v0;  // offset of the tile inside the stored K x V (V x K) matrix
  const int hk = hv / (p.HV / p.HK);
  const int tid = threadIdx.x;
  const int rg = tid / TPR, c0 = (tid % TPR) * 4;

  int t0, t1;
  if (p.cu_seqlens) {
    t0 = p.cu_seqlens[seq];
    t1 = p.cu_seqlens[seq + 1];
  } else {
    t0 = seq * p.tokens_per_seq;
    t1 = t0 + p.tokens_per_seq;
  }
  if (t1 <= t0) return;
  int blk = seq;
  if (p.state_indices) {
    int tok = t0;
    if (p.num_accepted_tokens) tok = t0 + p.num_accepted_tokens[seq] - 1;
    blk = p.state_indices[tok];
  }
  if (blk < 0 || blk >= p.nblocks_in) return;  // padded slot or bad index: leave everything untouched

  float4 s[R];
  {
    const ST* src = static_cast<const ST*>(p.state_in) + blk * p.state_in_stride_b + hv * p.state_in_stride_h;
#pragma unroll
    for (int i = 0; i < R; ++i) s[i] = load4<ST>(src + tile_off + int64_t(rg + i * RG) * LD + c0);
  }

  for (int t = t0; t < t1; ++t) {
    __syncthreads();  // previous token's readers of k_s/q_s/red are done
    if (tid < K) {
      k_s[tid] = load_act(p.k, t * p.k_stride_t + hk * p.k_stride_h + tid, p.act_f16);
    } else if (tid < 2 * K) {
      q_s[tid - K] = load_act(p.q, t * p.q_stride_t + hk * p.q_stride_h + (tid - K), p.act_f16);
    }
    if (p.gk && tid < K) {   // per-channel decay of this token: exp(gate(gk))
      float gate = load_scalar(p.gk, t * p.gk_stride_t + hv * p.gk_stride_h + tid, p.gk_is_f32);
      if (p.gate_mode) {
        const float eig = p.a_log ? __expf(p.a_log[hv]) : 1.f;
        const float raw = gate + (p.dt_bias ? p.dt_bias[hv * K + tid] : 0.f);
        if (p.gate_mode == 1) gate = -eig * (raw > 20.f ? raw : log1pf(__expf(raw)));
        else gate = p.lower_bound / (1.f + __expf(-eig * raw));
      }
      dk_s[tid] = __expf(gate);
    }
    const float decay = p.g ? expf(load_scalar(p.g, t * p.g_stride_t + hv, p.g_is_f32)) : 1.f;
    float beta = p.beta ? load_scalar(p.beta, t * p.beta_stride_t + hv, p.beta_is_f32) : 1.f;
    if (p.beta_mode) beta = float(p.beta_mode) / (1.f + __expf(-beta));
    __syncthreads();
    float kscale = 1.f, qscale = p.scale;
    if (p.l2norm) {
      if (tid < 64) {  // warp 0: |k|^2, warp 1: |q|^2
        const float* src = tid < 32 ? k_s : q_s;
        float acc = 0.f;
        for (int i = tid % 32; i < K; i += 32) acc += src[i] * src[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (tid % 32 == 0) norm_s[tid / 32] = rsqrtf(acc + 1e-6f);
      }
      __syncthreads();
      kscale = norm_s[0];
      qscale = p.scale * norm_s[1];
    }

    if (p.gk) {   // S <- diag(exp(gate)) S
      if constexpr (!VFIRST) {
#pragma unroll
        for (int i = 0; i < R; ++i) {
          const float d = dk_s[rg + i * RG];
          s[i].x *= d; s[i].y *= d; s[i].z *= d; s[i].w *= d;
        }
      } else {
        const float4 d = make_float4(dk_s[c0], dk_s[c0 + 1], dk_s[c0 + 2], dk_s[c0 + 3]);
#pragma unroll
        for (int i = 0; i < R; ++i) { s[i].x *= d.x; s[i].y *= d.y; s[i].z *= d.z; s[i].w *= d.w; }
      }
    }
    if constexpr (!VFIRST) {
      // rows are k, my 4 columns are v.  dot[v] = sum_k S[k][v] k[k]
      float4 part = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const float kk = k_s[rg + i * RG] * kscale;
        part.x += s[i].x * kk; part.y += s[i].y * kk; part.z += s[i].z * kk; part.w += s[i].w * kk;
      }
      *reinterpret_cast<float4*>(&red[rg][c0]) = part;
      __syncthreads();
      float4 dot = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < RG; ++r) {
        const float4 x = *reinterpret_cast<const float4*>(&red[r][c0]);
        dot.x += x.x; dot.y += x.y; dot.z += x.z; dot.w += x.w;
      }
      const int64_t voff = t * p.v_stride_t + hv * p.v_stride_h + v0 + c0;
      const float4 vv = p.act_f16 ? load4<__half>(static_cast<const __half*>(p.v) + voff)
                                  : load4<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(p.v) + voff);
      float4 d;
      d.x = beta * (vv.x - decay * dot.x); d.y = beta * (vv.y - decay * dot.y);
      d.z = beta * (vv.z - decay * dot.z); d.w = beta * (vv.w - decay * dot.w);
      float4 po = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const float kk = k_s[rg + i * RG] * kscale, qq = q_s[rg + i * RG] * qscale;
        s[i].x = decay * s[i].x + kk * d.x; s[i].y = decay * s[i].y + kk * d.y;
        s[i].z = decay * s[i].z + kk * d.z; s[i].w = decay * s[i].w + kk * d.w;
        po.x += s[i].x * qq; po.y += s[i].y * qq; po.z += s[i].z * qq; po.w += s[i].w * qq;
      }
      __syncthreads();  // everyone has consumed red[] for the dot
      *reinterpret_cast<float4*>(&red[rg][c0]) = po;
      __syncthreads();
      if (rg == 0) {
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < RG; ++r) {
          const float4 x = *reinterpret_cast<const float4*>(&red[r][c0]);
          o.x += x.x; o.y += x.y; o.z += x.z; o.w += x.w;
        }
        const int64_t off = t * p.out_stride_t + hv * p.out_stride_h + v0 + c0;
        if (p.out_is_f32) store4<float>(static_cast<float*>(p.out) + off, o);
        else if (p.out_is_f16) store4<__half>(static_cast<__half*>(p.out) + off, o);
        else store4<__nv_bfloat16>(static_cast<__nv_bfloat16*>(p.out) + off, o);
      }
    } else {
      // rows are v, my 4 columns are k.  Each row is reduced across the TPR lanes that share it.
      const float4 kk = make_float4(k_s[c0] * kscale, k_s[c0 + 1] * kscale, k_s[c0 + 2] * kscale, k_s[c0 + 3] * kscale);
      const float4 qq = make_float4(q_s[c0] * qscale, q_s[c0 + 1] * qscale, q_s[c0 + 2] * qscale, q_s[c0 + 3] * qscale);
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const int row = v0 + rg + i * RG;
        float dot = s[i].x * kk.x + s[i].y * kk.y + s[i].z * kk.z + s[i].w * kk.w;
#pragma unroll
        for (int o = TPR / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const float vv = load_act(p.v, t * p.v_stride_t + hv * p.v_stride_h + row, p.act_f16);
        const float d = beta * (vv - decay * dot);
        s[i].x = decay * s[i].x + d * kk.x; s[i].y = decay * s[i].y + d * kk.y;
        s[i].z = decay * s[i].z + d * kk.z; s[i].w = decay * s[i].w + d * kk.w;
        float o = s[i].x * qq.x + s[i].y * qq.y + s[i].z * qq.z + s[i].w * qq.w;
#pragma unroll
        for (int sft = TPR / 2; sft > 0; sft >>= 1) o += __shfl_xor_sync(0xffffffffu, o, sft);
        if (tid % TPR == 0) {
          const int64_t off = t * p.out_stride_t + hv * p.out_stride_h + row;
          if (p.out_is_f32) static_cast<float*>(p.out)[off] = o;
          else if (p.out_is_f16) static_cast<__half*>(p.out)[off] = __float2half_rn(o);
          else static_cast<__nv_bfloat16*>(p.out)[off] = __float2bfloat16_rn(o);
        }
      }
    }

    const bool last = (t == t1 - 1);
    int wblk = -1;
    if (p.state_indices) wblk = p.state_indices[t];
    else if (last) wblk = seq;
    if (wblk >= 0 && wblk < p.nblocks_out) {
      ST* dst = static_cast<ST*>(p.state_out) + wblk * p.state_out_stride_b + hv * p.state_out_stride_h;
#pragma unroll
      for (int i = 0; i < R; ++i) store4<ST>(dst + tile_off + int64_t(rg + i * RG) * LD + c0, s[i]);
    }
  }
}

template <int K, int V>
int launch_recurrent(const RecurrentParams& p, int nseq, bool state_f32, bool vfirst, cudaStream_t st) {
  constexpr int VT = V > 128 ? 128 : V;
  const dim3 grid(nseq * p.HV * (V / VT)), block(kRecThreads);
  KernelTimer kt("recurrent_gdn", st);
  if (state_f32) {
    if (vfirst) recurrent_gdn_kernel<K, V, VT, float, true><<<grid, block, 0, st>>>(p);
    else recurrent_gdn_kernel<K, V, VT, float, false><<<grid, block, 0, st>>>(p);
  } else {
    if (vfirst) recurrent_gdn_kernel<K, V, VT, __nv_bfloat16, true><<<grid, block, 0, st>>>(p);
    else recurrent_gdn_kernel<K, V, VT, __nv_bfloat16, false><<<grid, block, 0, st>>>(p);
  }
  return cuda_status(cudaGetLastError());
}

}  // namespace fla

extern "C" FLA_API int fla_b200_recurrent_gdn_workspace_size(const fla_recurrent_gdn_args* a, uint64_t* bytes) {
  if (!a || !bytes) return FLA_ERR_NULL;
  *bytes = 0;
  return FLA_OK;
}

extern "C" FLA_API int fla_b200_recurrent_gdn(const fla_recurrent_gdn_args* a, void* workspace, uint64_t workspace_bytes,
                                              void* stream) {
  using namespace fla;
  (void)workspace; (void)workspace_bytes;
  if (!a) return FLA_ERR_NULL;
  const fla_tensor_t &q = a->q, &k = a->k, &v = a->v, &si = a->state_in, &so = a->state_out, &o = a->out;
  if (!q.data || !k.data || !v.data || !si.data || !so.data || !o.data) return FLA_ERR_NULL;
  if (q.ndim != 3 || k.ndim != 3 || v.ndim != 3 || o.ndim != 3 || si.ndim != 4 || so.ndim != 4) return FLA_ERR_SHAPE;
  if ((q.dtype != FLA_BF16 && q.dtype != FLA_F16) || k.dtype != q.dtype || v.dtype != q.dtype) return FLA_ERR_DTYPE;
  if (si.dtype != so.dtype || (si.dtype != FLA_F32 && si.dtype != FLA_BF16)) return FLA_ERR_DTYPE;
  if (o.dtype != FLA_BF16 && o.dtype != FLA_F32 && o.dtype != FLA_F16) return FLA_ERR_DTYPE;
  const int64_t T = q.shape[0], HK = q.shape[1], K = q.shape[2], HV = v.shape[1], V = v.shape[2];
  if (T <= 0 || HK <= 0 || HV <= 0 || HV % HK) return FLA_ERR_SHAPE;
  for (int i = 0; i < 3; ++i)
    if (k.shape[i] != q.shape[i] || o.shape[i] != v.shape[i]) return FLA_ERR_SHAPE;
  if (v.shape[0] != T) return FLA_ERR_SHAPE;
  const bool vfirst = a->state_v_first != 0;
  const int64_t r = vfirst ? V : K, c = vfirst ? K : V;
  for (const fla_tensor_t* s : {&si, &so}) {
    if (s->shape[1] != HV || s->shape[2] != r || s->shape[3] != c) return FLA_ERR_SHAPE;
    if (s->stride[3] != 1 || s->stride[2] != c) return FLA_ERR_LAYOUT;
    if (!aligned16(s->data) || (s->stride[0] * (s->dtype == FLA_F32 ? 4 : 2)) % 16 ||
        (s->stride[1] * (s->dtype == FLA_F32 ? 4 : 2)) % 16)
      return FLA_ERR_LAYOUT;
  }
  if (q.stride[2] != 1 || k.stride[2] != 1 || v.stride[2] != 1 || o.stride[2] != 1) return FLA_ERR_LAYOUT;
  if ((reinterpret_cast<uintptr_t>(v.data) & 7) || v.stride[0] % 4 || v.stride[1] % 4) return FLA_ERR_LAYOUT;
  if (!aligned16(o.data) || o.stride[0] % 4 || o.stride[1] % 4) return FLA_ERR_LAYOUT;
  int nseq;
  if (a->cu_seqlens.data) {
    if (a->cu_seqlens.dtype != FLA_I32 || a->cu_seqlens.ndim != 1 || a->cu_seqlens.shape[0] < 2) return FLA_ERR_SHAPE;
    nseq = int(a->cu_seqlens.shape[0] - 1);
  } else {
    if (a->tokens_per_seq <= 0 || T % a->tokens_per_seq) return FLA_ERR_VALUE;
    nseq = int(T / a->tokens_per_seq);
  }
  if (a->state_indices.data && (a->state_indices.dtype != FLA_I32 || a->state_indices.shape[0] != T)) return FLA_ERR_SHAPE;
  if (a->num_accepted_tokens.data &&
      (a->num_accepted_tokens.dtype != FLA_I32 || a->num_accepted_tokens.shape[0] != nseq || !a->state_indices.data))
    return FLA_ERR_SHAPE;
  for (const fla_tensor_t* s : {&a->g, &a->beta}) {
    if (!s->data) continue;
    if (s->ndim != 2 || s->shape[0] != T || s->shape[1] != HV || s->stride[1] != 1) return FLA_ERR_SHAPE;
    if (s->dtype != FLA_F32 && s->dtype != FLA_BF16) return FLA_ERR_DTYPE;
  }
  if (!(a->scale == a->scale) || a->scale > 3.0e38f || a->scale < -3.0e38f) return FLA_ERR_VALUE;
  if (a->gate_mode < 0 || a->gate_mode > 2 || a->beta_mode < 0 || a->beta_mode > 2) return FLA_ERR_VALUE;
  if (a->gk.data) {
    const fla_tensor_t& gk = a->gk;
    if (gk.ndim != 3 || gk.shape[0] != T || gk.shape[1] != HV || gk.shape[2] != K || gk.stride[2] != 1) return FLA_ERR_SHAPE;
    if (gk.dtype != FLA_F32 && gk.dtype != FLA_BF16) return FLA_ERR_DTYPE;
    if (a->gate_mode) {
      if (!a->a_log.data || a->a_log.dtype != FLA_F32 || a->a_log.ndim != 1 || a->a_log.shape[0] != HV || a->a_log.stride[0] != 1)
        return FLA_ERR_SHAPE;
      if (a->dt_bias.data && (a->dt_bias.dtype != FLA_F32 || a->dt_bias.ndim != 2 || a->dt_bias.shape[0] != HV ||
                              a->dt_bias.shape[1] != K || a->dt_bias.stride[1] != 1 || a->dt_bias.stride[0] != K))
        return FLA_ERR_SHAPE;
    }
  } else if (a->gate_mode) {
    return FLA_ERR_VALUE;
  }

  RecurrentParams p{};
  p.q = q.data;
  p.k = k.data;
  p.v = v.data;
  p.act_f16 = q.dtype == FLA_F16; p.out_is_f16 = o.dtype == FLA_F16;
  p.g = a->g.data; p.beta = a->beta.data;
  p.state_in = si.data; p.state_out = so.data; p.out = o.data;
  p.cu_seqlens = static_cast<const int32_t*>(a->cu_seqlens.data);
  p.state_indices = static_cast<const int32_t*>(a->state_indices.data);
  p.num_accepted_tokens = static_cast<const int32_t*>(a->num_accepted_tokens.data);
  p.q_stride_t = q.stride[0]; p.q_stride_h = q.stride[1];
  p.k_stride_t = k.stride[0]; p.k_stride_h = k.stride[1];
  p.v_stride_t = v.stride[0]; p.v_stride_h = v.stride[1];
  p.g_stride_t = a->g.data ? a->g.stride[0] : 0;
  p.beta_stride_t = a->beta.data ? a->beta.stride[0] : 0;
  p.out_stride_t = o.stride[0]; p.out_stride_h = o.stride[1];
  p.state_in_stride_b = si.stride[0]; p.state_in_stride_h = si.stride[1];
  p.state_out_stride_b = so.stride[0]; p.state_out_stride_h = so.stride[1];
  p.HK = int(HK); p.HV = int(HV); p.tokens_per_seq = a->tokens_per_seq;
  p.nblocks_in = int(si.shape[0]); p.nblocks_out = int(so.shape[0]);
  p.g_is_f32 = a->g.dtype == FLA_F32; p.beta_is_f32 = a->beta.dtype == FLA_F32; p.out_is_f32 = o.dtype == FLA_F32;
  p.l2norm = a->use_qk_l2norm; p.scale = a->scale;
  p.gk = a->gk.data; p.a_log = static_cast<const float*>(a->a_log.data); p.dt_bias = static_cast<const float*>(a->dt_bias.data);
  p.gk_stride_t = a->gk.data ? a->gk.stride[0] : 0; p.gk_stride_h = a->gk.data ? a->gk.stride[1] : 0;
  p.gk_is_f32 = a->gk.dtype == FLA_F32; p.gate_mode = a->gate_mode; p.beta_mode = a->beta_mode; p.lower_bound = a->lower_bound;
  if (!a->state_indices.data && nseq > p.nblocks_in) return FLA_ERR_SHAPE;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool f32 = si.dtype == FLA_F32;
  if (K == 128 && V == 128) return launch_recurrent<128, 128>(p, nseq, f32, vfirst, st);
  if (K == 64 && V == 64) return launch_recurrent<64, 64>(p, nseq, f32, vfirst, st);
  if (K == 64 && V == 128) return launch_recurrent<64, 128>(p, nseq, f32, vfirst, st);
  if (K == 128 && V == 64) return launch_recurrent<128, 64>(p, nseq, f32, vfirst, st);
  if (K == 128 && V == 256) return launch_recurrent<128, 256>(p, nseq, f32, vfirst, st);
  if (K == 64 && V == 256) return launch_recurrent<64, 256>(p, nseq, f32, vfirst, st);
  return FLA_ERR_SHAPE;
}

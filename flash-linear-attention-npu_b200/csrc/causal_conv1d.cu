// Depthwise causal conv1d: prefill (forward over whole sequences) and decode update (in-place state).
//   y[t, d] = act(bias[d] + sum_{j<W} w[d, j] * x[t - (W-1) + j, d])   (+ residual[t, d])
// Inputs before a sequence's first token come from its initial state (the last W-1 inputs of the
// previous segment) or are zero.  Both kernels are pure HBM streaming: every thread owns 8 adjacent
// channels (one 16-byte bf16 vector), keeps the W-1 previous inputs in registers and accumulates in
// fp32; SiLU is evaluated in fp32 and the result is rounded once.
// Replaces the reference operator causal_conv1d, run_mode 0 and 1
// (fla/ops/ascendc/gdn/gdn_preprocess/causal_conv1d/op_kernel/causal_conv1d.h, causal_conv1d_update.h).
#include <cuda_bf16.h>
#include "fla_b200_internal.h"
#include "kernel_timer.h"

namespace fla {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ void unpack8(const uint4& raw, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __low2float(h[i]);
    f[2 * i + 1] = __high2float(h[i]);
  }
}
__device__ __forceinline__ uint4 pack8f(const float* f) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return raw;
}
// SiLU as 0.5 x (1 + tanh(0.5 x)): one MUFU op and two FP32 ops.  tanh.approx is accurate to about 2^-11
// relative, far below the rounding of the bf16 result.
__device__ __forceinline__ float silu(float x) {
  const float h = 0.5f * x;
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(h));
  return fmaf(h, t, h);
}

// weight element (d, j) at w[d * wsd + j * wsw]; returns taps for 8 channels starting at d0.
template <int W>
__device__ __forceinline__ void load_weights(const bf16* w, int64_t wsd, int64_t wsw, int d0, float (&out)[W][8]) {
  if (wsd == 1) {  // [W, D]: channels contiguous
#pragma unroll
    for (int j = 0; j < W; ++j) unpack8(*reinterpret_cast<const uint4*>(w + j * wsw + d0), out[j]);
  } else if (wsw == 1 && wsd == W && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
    // [D, W] dense: the 8 channels' taps are 8 * W contiguous elements = W 16-byte vectors
    float flat[W * 8];
#pragma unroll
    for (int j = 0; j < W; ++j) unpack8(*reinterpret_cast<const uint4*>(w + int64_t(d0) * W + j * 8), flat + j * 8);
#pragma unroll
    for (int c = 0; c < 8; ++c)
#pragma unroll
      for (int j = 0; j < W; ++j) out[j][c] = flat[c * W + j];
  } else {
#pragma unroll
    for (int j = 0; j < W; ++j)
#pragma unroll
      for (int c = 0; c < 8; ++c) out[j][c] = __bfloat162float(w[(d0 + c) * wsd + j * wsw]);
  }
}

struct ConvFwdParams {
  const bf16* x; bf16* y; const bf16* residual;
  const bf16* weight; const bf16* bias;
  const bf16* init; bf16* final_state;
  const int32_t* cu_seqlens;  // varlen: [N+1] token offsets into the single batch row
  int64_t x_sb, x_st, y_sb, y_st, r_sb, r_st, w_sd, w_sw;
  int64_t i_sn, i_sd, i_sw, f_sn, f_sd, f_sw;
  int64_t y_sh;       // head-first output [B, H, T, D/H]: stride between heads (0 with the [B, T, D] output)
  int y_hd;           // channels per head of the output (D with the [B, T, D] output)
  int B, T, D, nseq, silu;
};

constexpr int kConvTile = 64;     // tokens per CTA tile
constexpr int kConvGroup = 4;     // tokens processed per inner step (independent 16-byte loads in flight); 4 keeps 128 registers = 4 CTAs per SM
constexpr int kConvThreads = 128;

template <int W, bool HAS_RES, bool SILU>
__global__ void __launch_bounds__(kConvThreads, 4) conv_fwd_kernel(ConvFwdParams p) {
  constexpr int G = kConvGroup;
  const int d0 = (blockIdx.x * kConvThreads + threadIdx.x) * 8;
  if (d0 >= p.D) return;
  const int b = blockIdx.z;
  const int t_begin = blockIdx.y * kConvTile;
  const int t_end = min(p.T, t_begin + kConvTile);
  if (t_begin >= t_end) return;

  float w[W][8], bias[8];
  load_weights<W>(p.weight, p.w_sd, p.w_sw, d0, w);
  if (p.bias) unpack8(*reinterpret_cast<const uint4*>(p.bias + d0), bias);
  else {
#pragma unroll
    for (int c = 0; c < 8; ++c) bias[c] = 0.f;
  }

  // sequence containing t_begin
  int seq = b, seq_begin = 0, seq_end = p.T;
  if (p.cu_seqlens) {
    int lo = 0, hi = p.nseq - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (p.cu_seqlens[mid] <= t_begin) lo = mid; else hi = mid - 1;
    }
    seq = lo;
    seq_begin = p.cu_seqlens[seq];
    seq_end = p.cu_seqlens[seq + 1];
  }

  const bf16* xb = p.x + b * p.x_sb + d0;
  bf16* yb = p.y + b * p.y_sb + (d0 / p.y_hd) * p.y_sh + d0 % p.y_hd;   // a thread's 8 channels never straddle a head
  const bf16* rb = HAS_RES ? p.residual + b * p.r_sb + d0 : nullptr;

  // win[0 .. W-2] = the W-1 inputs before the group, win[W-1 + i] = input i of the group
  float win[W - 1 + G][8];
  int t = t_begin;
  while (t < t_end) {
    if (p.cu_seqlens) {
      while (seq_end <= t) {  // step over sequences that end at or before t (also skips empty ones)
        ++seq;
        seq_begin = seq_end;
        seq_end = p.cu_seqlens[seq + 1];
      }
    }
    const int seg_end = min(t_end, seq_end);
#pragma unroll
    for (int j = 1; j < W; ++j) {
      const int pos = t - j;
      if (pos >= seq_begin) {
        unpack8(*reinterpret_cast<const uint4*>(xb + pos * p.x_st), win[W - 1 - j]);
      } else {
        const int si = (W - 1) + (pos - seq_begin);  // index into the W-1 stored inputs
#pragma unroll
        for (int c = 0; c < 8; ++c)
          win[W - 1 - j][c] = (p.init && si >= 0) ? __bfloat162float(p.init[seq * p.i_sn + (d0 + c) * p.i_sd + si * p.i_sw]) : 0.f;
      }
    }
    uint4 xin[G], rin[HAS_RES ? G : 1];
    auto issue = [&](int tg) {
#pragma unroll
      for (int i = 0; i < G; ++i) {
        const int tt = tg + i;
        xin[i] = (tt < seg_end) ? *reinterpret_cast<const uint4*>(xb + tt * p.x_st) : make_uint4(0, 0, 0, 0);
        if constexpr (HAS_RES) rin[i] = (tt < seg_end) ? *reinterpret_cast<const uint4*>(rb + tt * p.r_st) : make_uint4(0, 0, 0, 0);
      }
    };
    issue(t);
    int nvalid = 0;
    for (int tg = t; tg < seg_end; tg += G) {
#pragma unroll
      for (int i = 0; i < G; ++i) unpack8(xin[i], win[W - 1 + i]);
      float res[HAS_RES ? G : 1][8];
      if constexpr (HAS_RES) {
#pragma unroll
        for (int i = 0; i < G; ++i) unpack8(rin[i], res[i]);
      }
      if (tg + G < seg_end) issue(tg + G);   // next group's loads fly while this one is computed
      nvalid = min(G, seg_end - tg);
#pragma unroll
      for (int i = 0; i < G; ++i) {
        if (i < nvalid) {
          float acc[8];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            float a = bias[c];
#pragma unroll
            for (int j = 0; j < W; ++j) a = fmaf(w[j][c], win[i + j][c], a);
            if constexpr (SILU) a = silu(a);
            if constexpr (HAS_RES) a += res[i][c];
            acc[c] = a;
          }
          *reinterpret_cast<uint4*>(yb + (tg + i) * p.y_st) = pack8f(acc);
        }
      }
      if (nvalid == G) {
#pragma unroll
        for (int j = 0; j < W - 1; ++j)
#pragma unroll
          for (int c = 0; c < 8; ++c) win[j][c] = win[G + j][c];
      }
    }
    if (nvalid != G) {  // partial last group: the W-1 newest inputs sit at win[nvalid .. nvalid + W-2]
#pragma unroll
      for (int i = 0; i < G; ++i) {
        if (i == nvalid) {
#pragma unroll
          for (int j = 0; j < W - 1; ++j)
#pragma unroll
            for (int c = 0; c < 8; ++c) win[j][c] = win[i + j][c];
        }
      }
    }
    if (p.final_state && seg_end == seq_end) {  // the sequence ended in this tile: its last W-1 inputs are the state
#pragma unroll
      for (int j = 0; j < W - 1; ++j)
#pragma unroll
        for (int c = 0; c < 8; ++c)
          p.final_state[seq * p.f_sn + (d0 + c) * p.f_sd + j * p.f_sw] = __float2bfloat16_rn(win[j][c]);
    }
    t = seg_end;
  }
}

struct ConvUpdParams {
  const bf16* x; bf16* y; const bf16* residual;
  const bf16* weight; const bf16* bias;
  bf16* state;
  const int32_t* cache_indices;        // [N] or null
  const int32_t* num_accepted_tokens;  // [N] or null
  int64_t x_sn, x_st, y_sn, y_st, r_sn, r_st, w_sd, w_sw, s_sn, s_sd, s_ss;
  int N, T, D, S, W, nslots, silu, pad_slot_id;
};

// Fast path: one token per sequence, state holds exactly W-1 inputs.
// STATE_DMAJOR: state is [slots, W-1, D] (channels contiguous); otherwise [slots, D, W-1] (taps contiguous).
template <int W, bool STATE_DMAJOR>
__global__ void __launch_bounds__(kConvThreads) conv_update1_kernel(ConvUpdParams p) {
  constexpr int S = W - 1;
  const int d0 = (blockIdx.x * kConvThreads + threadIdx.x) * 8;
  if (d0 >= p.D) return;
  const int n = blockIdx.y;
  int slot = n;
  if (p.cache_indices) slot = p.cache_indices[n];
  if (slot == p.pad_slot_id || slot < 0 || slot >= p.nslots) return;

  float w[W][8], acc[8], xv[8], h[S][8];
  load_weights<W>(p.weight, p.w_sd, p.w_sw, d0, w);
  if (p.bias) unpack8(*reinterpret_cast<const uint4*>(p.bias + d0), acc);
  else {
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = 0.f;
  }
  unpack8(*reinterpret_cast<const uint4*>(p.x + n * p.x_sn + d0), xv);
  bf16* st = p.state + slot * p.s_sn;
  if constexpr (STATE_DMAJOR) {
#pragma unroll
    for (int s = 0; s < S; ++s) unpack8(*reinterpret_cast<const uint4*>(st + s * p.s_ss + d0), h[s]);
  } else {
    // 8 channels x S taps are 8*S contiguous elements = S 16-byte vectors
    float flat[S * 8];
#pragma unroll
    for (int s = 0; s < S; ++s) unpack8(*reinterpret_cast<const uint4*>(st + int64_t(d0) * S + s * 8), flat + s * 8);
#pragma unroll
    for (int c = 0; c < 8; ++c)
#pragma unroll
      for (int s = 0; s < S; ++s) h[s][c] = flat[c * S + s];
  }
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    float a = acc[c] + w[W - 1][c] * xv[c];
#pragma unroll
    for (int s = 0; s < S; ++s) a += w[s][c] * h[s][c];
    acc[c] = p.silu ? silu(a) : a;
  }
  if (p.residual) {
    float rv[8];
    unpack8(*reinterpret_cast<const uint4*>(p.residual + n * p.r_sn + d0), rv);
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] += rv[c];
  }
  *reinterpret_cast<uint4*>(p.y + n * p.y_sn + d0) = pack8f(acc);
  // new state = (h[1], ..., h[S-1], x)
  if constexpr (STATE_DMAJOR) {
#pragma unroll
    for (int s = 0; s < S; ++s)
      *reinterpret_cast<uint4*>(st + s * p.s_ss + d0) = (s + 1 < S) ? pack8f(h[s + 1]) : pack8f(xv);
  } else {
    float flat[S * 8];
#pragma unroll
    for (int c = 0; c < 8; ++c)
#pragma unroll
      for (int s = 0; s < S; ++s) flat[c * S + s] = (s + 1 < S) ? h[s + 1][c] : xv[c];
#pragma unroll
    for (int s = 0; s < S; ++s) *reinterpret_cast<uint4*>(st + int64_t(d0) * S + s * 8) = pack8f(flat + s * 8);
  }
}

// General path (several tokens per sequence, longer state windows, speculative-decode offsets,
// arbitrary strides): one thread per channel.
__global__ void conv_update_generic_kernel(ConvUpdParams p) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= p.D) return;
  const int n = blockIdx.y;
  int slot = n;
  if (p.cache_indices) slot = p.cache_indices[n];
  if (slot == p.pad_slot_id || slot < 0 || slot >= p.nslots) return;
  constexpr int kMaxW = 4, kMaxT = 16, kMaxS = 32;
  const int W = p.W, T = p.T, S = p.S;
  float w[kMaxW], full[kMaxW - 1 + kMaxT], old[kMaxS];
  for (int j = 0; j < W; ++j) w[j] = __bfloat162float(p.weight[d * p.w_sd + j * p.w_sw]);
  const float bias = p.bias ? __bfloat162float(p.bias[d]) : 0.f;
  bf16* st = p.state + slot * p.s_sn + d * p.s_sd;
  for (int s = 0; s < S; ++s) old[s] = __bfloat162float(st[s * p.s_ss]);
  const bool spec = p.num_accepted_tokens != nullptr;
  const int offset = spec ? p.num_accepted_tokens[n] - 1 : S - (W - 1);
  for (int j = 0; j < W - 1; ++j) full[j] = old[offset + j];
  for (int t = 0; t < T; ++t) full[W - 1 + t] = __bfloat162float(p.x[n * p.x_sn + t * p.x_st + d]);
  for (int t = 0; t < T; ++t) {
    float a = bias;
    for (int j = 0; j < W; ++j) a += w[j] * full[t + j];
    a = p.silu ? silu(a) : a;
    if (p.residual) a += __bfloat162float(p.residual[n * p.r_sn + t * p.r_st + d]);
    p.y[n * p.y_sn + t * p.y_st + d] = __float2bfloat16_rn(a);
  }
  if (spec) {
    const int keep = W - 2;
    for (int s = 0; s < keep; ++s) st[s * p.s_ss] = __float2bfloat16_rn(old[offset + 1 + s]);
    for (int t = 0; t < T; ++t) st[(keep + t) * p.s_ss] = __float2bfloat16_rn(full[W - 1 + t]);
  } else {
    // state <- last S entries of (old state, x)
    for (int s = 0; s < S; ++s) {
      const int src = s + T;  // index into concat(old[S], x[T])
      const float val = src < S ? old[src] : full[W - 1 + (src - S)];
      st[s * p.s_ss] = __float2bfloat16_rn(val);
    }
  }
}

}  // namespace fla

using namespace fla;

static bool vec_ok(const fla_tensor_t& t) {
  if (!aligned16(t.data) || t.stride[t.ndim - 1] != 1) return false;
  for (int i = 0; i < t.ndim - 1; ++i)
    if (t.stride[i] % 8) return false;
  return true;
}

extern "C" FLA_API int fla_b200_causal_conv1d_fwd_workspace_size(const fla_causal_conv1d_fwd_args* a, uint64_t* bytes) {
  if (!a || !bytes) return FLA_ERR_NULL;
  *bytes = 0;
  return FLA_OK;
}

extern "C" FLA_API int fla_b200_causal_conv1d_fwd(const fla_causal_conv1d_fwd_args* a, void* workspace,
                                                  uint64_t workspace_bytes, void* stream) {
  (void)workspace; (void)workspace_bytes;
  if (!a) return FLA_ERR_NULL;
  const fla_tensor_t &x = a->x, &y = a->y, &w = a->weight;
  if (!x.data || !y.data || !w.data) return FLA_ERR_NULL;
  if (x.ndim != 3 || (y.ndim != 3 && y.ndim != 4) || w.ndim != 2) return FLA_ERR_SHAPE;
  if (x.dtype != FLA_BF16 || y.dtype != FLA_BF16 || w.dtype != FLA_BF16) return FLA_ERR_DTYPE;
  const int64_t B = x.shape[0], T = x.shape[1], D = x.shape[2], W = w.shape[1];
  if (w.shape[0] != D || W < 2 || W > 4 || D % 8 || B <= 0 || T < 0) return FLA_ERR_SHAPE;
  if (y.ndim == 3) {
    for (int i = 0; i < 3; ++i)
      if (y.shape[i] != x.shape[i]) return FLA_ERR_SHAPE;
  } else if (y.shape[0] != B || y.shape[2] != T || y.shape[1] * y.shape[3] != D || y.shape[3] % 8) {
    return FLA_ERR_SHAPE;   // head-first output [B, H, T, D / H]
  }
  if (!vec_ok(x) || !vec_ok(y)) return FLA_ERR_LAYOUT;
  if (w.stride[0] == 1 && (!aligned16(w.data) || w.stride[1] % 8)) return FLA_ERR_LAYOUT;
  int nseq = int(B);
  if (a->cu_seqlens.data) {
    if (B != 1 || a->cu_seqlens.dtype != FLA_I32 || a->cu_seqlens.ndim != 1 || a->cu_seqlens.shape[0] < 2)
      return FLA_ERR_SHAPE;
    nseq = int(a->cu_seqlens.shape[0] - 1);
  }
  ConvFwdParams p{};
  p.x = static_cast<const bf16*>(x.data); p.y = static_cast<bf16*>(y.data);
  p.weight = static_cast<const bf16*>(w.data);
  p.x_sb = x.stride[0]; p.x_st = x.stride[1]; p.y_sb = y.stride[0]; p.y_st = y.stride[1];
  p.y_hd = int(D);
  if (y.ndim == 4) { p.y_sh = y.stride[1]; p.y_st = y.stride[2]; p.y_hd = int(y.shape[3]); }
  p.w_sd = w.stride[0]; p.w_sw = w.stride[1];
  if (a->residual.data) {
    const fla_tensor_t& r = a->residual;
    if (r.ndim != 3 || r.dtype != FLA_BF16 || !vec_ok(r)) return FLA_ERR_LAYOUT;
    for (int i = 0; i < 3; ++i)
      if (r.shape[i] != x.shape[i]) return FLA_ERR_SHAPE;
    p.residual = static_cast<const bf16*>(r.data); p.r_sb = r.stride[0]; p.r_st = r.stride[1];
  }
  if (a->bias.data) {
    if (a->bias.ndim != 1 || a->bias.shape[0] != D || a->bias.dtype != FLA_BF16 || !vec_ok(a->bias)) return FLA_ERR_SHAPE;
    p.bias = static_cast<const bf16*>(a->bias.data);
  }
  for (int which = 0; which < 2; ++which) {
    const fla_tensor_t& s = which ? a->final_state : a->initial_state;
    if (!s.data) continue;
    if (s.ndim != 3 || s.dtype != FLA_BF16 || s.shape[0] != nseq || s.shape[1] != D || s.shape[2] != W - 1)
      return FLA_ERR_SHAPE;
    if (which) { p.final_state = static_cast<bf16*>(s.data); p.f_sn = s.stride[0]; p.f_sd = s.stride[1]; p.f_sw = s.stride[2]; }
    else { p.init = static_cast<const bf16*>(s.data); p.i_sn = s.stride[0]; p.i_sd = s.stride[1]; p.i_sw = s.stride[2]; }
  }
  p.cu_seqlens = static_cast<const int32_t*>(a->cu_seqlens.data);
  p.B = int(B); p.T = int(T); p.D = int(D); p.nseq = nseq; p.silu = a->activation_silu;
  if (T == 0) return FLA_OK;
  const dim3 grid(unsigned((D / 8 + kConvThreads - 1) / kConvThreads), unsigned((T + kConvTile - 1) / kConvTile), unsigned(B));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  KernelTimer kt("causal_conv1d_fwd", st);
#define FLA_LAUNCH_FWD(WW)                                                                           \
  if (p.residual) {                                                                                  \
    if (p.silu) conv_fwd_kernel<WW, true, true><<<grid, kConvThreads, 0, st>>>(p);                   \
    else conv_fwd_kernel<WW, true, false><<<grid, kConvThreads, 0, st>>>(p);                         \
  } else {                                                                                           \
    if (p.silu) conv_fwd_kernel<WW, false, true><<<grid, kConvThreads, 0, st>>>(p);                  \
    else conv_fwd_kernel<WW, false, false><<<grid, kConvThreads, 0, st>>>(p);                        \
  }
  if (W == 4) { FLA_LAUNCH_FWD(4) } else if (W == 3) { FLA_LAUNCH_FWD(3) } else { FLA_LAUNCH_FWD(2) }
#undef FLA_LAUNCH_FWD
  return cuda_status(cudaGetLastError());
}

extern "C" FLA_API int fla_b200_causal_conv1d_update_workspace_size(const fla_causal_conv1d_update_args* a,
                                                                    uint64_t* bytes) {
  if (!a || !bytes) return FLA_ERR_NULL;
  *bytes = 0;
  return FLA_OK;
}

extern "C" FLA_API int fla_b200_causal_conv1d_update(const fla_causal_conv1d_update_args* a, void* workspace,
                                                     uint64_t workspace_bytes, void* stream) {
  (void)workspace; (void)workspace_bytes;
  if (!a) return FLA_ERR_NULL;
  const fla_tensor_t &x = a->x, &y = a->y, &w = a->weight, &s = a->conv_state;
  if (!x.data || !y.data || !w.data || !s.data) return FLA_ERR_NULL;
  if (x.ndim != 3 || y.ndim != 3 || w.ndim != 2 || s.ndim != 3) return FLA_ERR_SHAPE;
  if (x.dtype != FLA_BF16 || y.dtype != FLA_BF16 || w.dtype != FLA_BF16 || s.dtype != FLA_BF16) return FLA_ERR_DTYPE;
  const int64_t N = x.shape[0], T = x.shape[1], D = x.shape[2], W = w.shape[1], S = s.shape[2];
  if (w.shape[0] != D || s.shape[1] != D || W < 2 || W > 4 || N <= 0 || T <= 0 || T > 16 || S > 32) return FLA_ERR_SHAPE;
  for (int i = 0; i < 3; ++i)
    if (y.shape[i] != x.shape[i]) return FLA_ERR_SHAPE;
  if (x.stride[2] != 1 || y.stride[2] != 1) return FLA_ERR_LAYOUT;
  const bool spec = a->num_accepted_tokens.data != nullptr;
  if (S < W - 1 || (spec && S < (W - 1) + (T - 1))) return FLA_ERR_SHAPE;
  if (a->cache_indices.data && (a->cache_indices.dtype != FLA_I32 || a->cache_indices.shape[0] != N)) return FLA_ERR_SHAPE;
  if (spec && (a->num_accepted_tokens.dtype != FLA_I32 || a->num_accepted_tokens.shape[0] != N)) return FLA_ERR_SHAPE;
  if (!a->cache_indices.data && s.shape[0] < N) return FLA_ERR_SHAPE;

  ConvUpdParams p{};
  p.x = static_cast<const bf16*>(x.data); p.y = static_cast<bf16*>(y.data);
  p.weight = static_cast<const bf16*>(w.data); p.state = static_cast<bf16*>(s.data);
  p.x_sn = x.stride[0]; p.x_st = x.stride[1]; p.y_sn = y.stride[0]; p.y_st = y.stride[1];
  p.w_sd = w.stride[0]; p.w_sw = w.stride[1];
  p.s_sn = s.stride[0]; p.s_sd = s.stride[1]; p.s_ss = s.stride[2];
  bool vec = vec_ok(x) && vec_ok(y) && D % 8 == 0;
  if (a->residual.data) {
    const fla_tensor_t& r = a->residual;
    if (r.ndim != 3 || r.dtype != FLA_BF16 || r.stride[2] != 1) return FLA_ERR_LAYOUT;
    for (int i = 0; i < 3; ++i)
      if (r.shape[i] != x.shape[i]) return FLA_ERR_SHAPE;
    p.residual = static_cast<const bf16*>(r.data); p.r_sn = r.stride[0]; p.r_st = r.stride[1];
    vec = vec && vec_ok(r);
  }
  if (a->bias.data) {
    if (a->bias.ndim != 1 || a->bias.shape[0] != D || a->bias.dtype != FLA_BF16 || a->bias.stride[0] != 1) return FLA_ERR_SHAPE;
    p.bias = static_cast<const bf16*>(a->bias.data);
    vec = vec && aligned16(a->bias.data);
  }
  p.cache_indices = static_cast<const int32_t*>(a->cache_indices.data);
  p.num_accepted_tokens = static_cast<const int32_t*>(a->num_accepted_tokens.data);
  p.N = int(N); p.T = int(T); p.D = int(D); p.S = int(S); p.W = int(W); p.nslots = int(s.shape[0]);
  p.silu = a->activation_silu; p.pad_slot_id = a->pad_slot_id;
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  KernelTimer kt("causal_conv1d_update", st);
  const bool w_ok = w.stride[0] != 1 || (aligned16(w.data) && w.stride[1] % 8 == 0);
  const bool dmajor = s.stride[1] == 1 && s.stride[2] % 8 == 0 && s.stride[0] % 8 == 0 && aligned16(s.data);
  const bool smajor = s.stride[2] == 1 && s.stride[1] == S && s.stride[0] % 8 == 0 && aligned16(s.data);
  if (vec && w_ok && T == 1 && S == W - 1 && !spec && (dmajor || smajor)) {
    const dim3 grid(unsigned((D / 8 + kConvThreads - 1) / kConvThreads), unsigned(N));
#define FLA_LAUNCH_UPD(WW)                                                               \
  if (dmajor) conv_update1_kernel<WW, true><<<grid, kConvThreads, 0, st>>>(p);          \
  else conv_update1_kernel<WW, false><<<grid, kConvThreads, 0, st>>>(p);
    if (W == 4) { FLA_LAUNCH_UPD(4) } else if (W == 3) { FLA_LAUNCH_UPD(3) } else { FLA_LAUNCH_UPD(2) }
#undef FLA_LAUNCH_UPD
  } else {
    const dim3 grid(unsigned((D + 127) / 128), unsigned(N));
    conv_update_generic_kernel<<<grid, 128, 0, st>>>(p);
  }
  return cuda_status(cudaGetLastError());
}

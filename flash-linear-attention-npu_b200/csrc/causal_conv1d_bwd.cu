// Backward of the depthwise causal conv1d (prefill form):
//   p[t] = bias + sum_j w[j] x[t-(W-1)+j]        y[t] = act(p[t])        gr[t] = dy[t] * act'(p[t])
//   dx[s]  = sum_j w[j] gr[s+(W-1)-j]  (+ dht: the last W-1 inputs of a sequence are its final state)
//   dw[j]  = sum_t gr[t] x[t-(W-1)+j]      db = sum_t gr[t]      dh0[i] = sum_{t<=i} gr[t] w[i-t]
// Replaces the reference operator causal_conv1d_bwd (aclnnCausalConv1dBwd as bound by npu_causal_conv1d_bwd,
// torch_custom/fla_npu/fla_npu/ops/ascendc/_aclnn_ctypes.py:988-1037; golden
// torch_custom/fla_npu/test/test_npu_causal_conv1d_bwd.py:33-127).
// HBM streaming like the forward: a thread owns 8 adjacent channels, walks a tile of tokens once with the input
// and gradient windows in registers, recomputes the pre-activation (or reads it when the caller kept it) and
// leaves its dw / db partial sums in a workspace that a second, tiny kernel reduces in a fixed order.
// The arithmetic runs on channel pairs with the packed fp32x2 instructions of sm_100 (fma / mul / add .f32x2: two
// IEEE fp32 operations per issue slot), and the four-token windows live in a register ring with compile-time
// indices, so no register is moved when the window advances; the kernel is bound by instruction issue otherwise.
#include <cuda_bf16.h>
#include "fla_b200_internal.h"
#include "kernel_timer.h"

namespace fla {

using bf16 = __nv_bfloat16;

namespace {

__device__ __forceinline__ void unpack8b(const uint4& raw, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __low2float(h[i]);
    f[2 * i + 1] = __high2float(h[i]);
  }
}

struct ConvBwdParams {
  const bf16* x; const bf16* dy; const bf16* ypre; bf16* dx;
  const bf16* weight; const bf16* bias;
  const bf16* init; const bf16* dht;
  void* dh0;
  float* part;                 // [tiles][W + 1][D] partial dw (W rows) and db (1 row)
  const int32_t* cu_seqlens;
  int64_t x_sb, x_st, dy_sb, dy_st, yp_sb, yp_st, dx_sb, dx_st, w_sd, w_sw;
  int64_t i_sn, i_sd, i_sw, t_sn, t_sd, t_sw, h_sn, h_sd, h_sw;
  int B, T, D, nseq, dh0_is_f32, tiles_per_row;
};

constexpr int kBwdTile = 128;    // tokens per CTA tile
constexpr int kBwdThreads = 128;

// derivative of SiLU at pre-activation p: s (1 + p (1 - s)), s = sigmoid(p)
__device__ __forceinline__ float dsilu(float p) {
  float t;   // sigmoid(p) = 0.5 (1 + tanh(p / 2)): one MUFU op
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * p));
  const float s = fmaf(0.5f, t, 0.5f);
  return s * fmaf(p, 1.f - s, 1.f);
}

constexpr int kBwdGroup = 2;     // tokens per inner step
constexpr int kBwdAhead = 3;     // groups requested ahead of the one being processed (ring = 48 KB per CTA)
constexpr int kBwdRing = kBwdAhead + 1;
constexpr uint32_t kBwdSmem = kBwdRing * kBwdGroup * 3 * kBwdThreads * sizeof(uint4);   // x, dy, y_pre slots

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))), "l"(gsrc)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// weight element (d, j) at w[d * wsd + j * wsw]; taps of 8 channels starting at d0
template <int W>
__device__ __forceinline__ void load_taps(const bf16* w, int64_t wsd, int64_t wsw, int d0, float (&out)[W][8]) {
  if (wsd == 1 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 && wsw % 8 == 0) {  // [W, D]: channels contiguous
#pragma unroll
    for (int j = 0; j < W; ++j) unpack8b(*reinterpret_cast<const uint4*>(w + j * wsw + d0), out[j]);
  } else if (wsw == 1 && wsd == W && (reinterpret_cast<uintptr_t>(w) & 15) == 0) {
    float flat[W * 8];   // [D, W] dense: the 8 channels' taps are W consecutive 16-byte vectors
#pragma unroll
    for (int j = 0; j < W; ++j) unpack8b(*reinterpret_cast<const uint4*>(w + int64_t(d0) * W + j * 8), flat + j * 8);
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

// two fp32 values in one 64-bit register pair, operated on by the packed .f32x2 instructions
using f2 = unsigned long long;
__device__ __forceinline__ f2 mk2(float lo, float hi) {
  f2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void un2(f2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f2 fma2(f2 a, f2 b, f2 c) {
  f2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f2 mul2(f2 a, f2 b) {
  f2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f2 add2(f2 a, f2 b) {
  f2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f2 bf2_to_f2(uint32_t raw) { return mk2(__uint_as_float(raw << 16), __uint_as_float(raw & 0xffff0000u)); }
__device__ __forceinline__ uint32_t f2_to_bf2(f2 v) {
  float lo, hi;
  un2(v, lo, hi);
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ void unpack4p(const uint4& raw, f2* out) {
  out[0] = bf2_to_f2(raw.x); out[1] = bf2_to_f2(raw.y); out[2] = bf2_to_f2(raw.z); out[3] = bf2_to_f2(raw.w);
}
__device__ __forceinline__ void pairs_from(const float* f, f2* out) {
#pragma unroll
  for (int c = 0; c < 4; ++c) out[c] = mk2(f[2 * c], f[2 * c + 1]);
}
// derivative of SiLU on a channel pair, the same operations as dsilu() on each half
__device__ __forceinline__ f2 dsilu2(f2 p, f2 half2, f2 one2, f2 neg2) {
  float h0, h1, t0, t1;
  un2(mul2(half2, p), h0, h1);
  asm("tanh.approx.f32 %0, %1;" : "=f"(t0) : "f"(h0));
  asm("tanh.approx.f32 %0, %1;" : "=f"(t1) : "f"(h1));
  const f2 s = fma2(half2, mk2(t0, t1), half2);
  return mul2(s, fma2(p, fma2(neg2, s, one2), one2));
}

constexpr int kBwdRot = 4;   // tokens per rotation of the register windows (two groups)

template <int W, bool SILU>
__global__ void __launch_bounds__(kBwdThreads, 2) conv_bwd_kernel(ConvBwdParams p) {
  constexpr int G = kBwdGroup;
  static_assert(G == 2 && kBwdRot == 4 && W <= kBwdRot, "window ring layout");
  extern __shared__ uint4 ring[];
  const int d0 = (blockIdx.x * kBwdThreads + threadIdx.x) * 8;
  if (d0 >= p.D) return;
  const int b = blockIdx.z;
  const int s0 = blockIdx.y * kBwdTile;
  const int s1 = min(p.T, s0 + kBwdTile);
  const f2 half2 = mk2(0.5f, 0.5f), one2 = mk2(1.f, 1.f), neg2 = mk2(-1.f, -1.f), zero2 = mk2(0.f, 0.f);

  f2 w[W][4], bias[4];
  {
    float wf[W][8], bf[8];
    load_taps<W>(p.weight, p.w_sd, p.w_sw, d0, wf);
    if (p.bias) unpack8b(*reinterpret_cast<const uint4*>(p.bias + d0), bf);
    else {
#pragma unroll
      for (int c = 0; c < 8; ++c) bf[c] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < W; ++j) pairs_from(wf[j], w[j]);
    pairs_from(bf, bias);
  }

  f2 dw[W][4], db[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    db[c] = zero2;
#pragma unroll
    for (int j = 0; j < W; ++j) dw[j][c] = zero2;
  }

  int seq = b, seq_begin = 0, seq_end = p.T;
  if (p.cu_seqlens) {
    int lo = 0, hi = p.nseq - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (p.cu_seqlens[mid] <= s0) lo = mid; else hi = mid - 1;
    }
    seq = lo;
    seq_begin = p.cu_seqlens[seq];
    seq_end = p.cu_seqlens[seq + 1];
  }
  const bf16* xb = p.x + b * p.x_sb + d0;
  const bf16* gb = p.dy + b * p.dy_sb + d0;
  const bf16* yb = p.ypre ? p.ypre + b * p.yp_sb + d0 : nullptr;
  bf16* dxb = p.dx + b * p.dx_sb + d0;

  // input at position pos of the current sequence (initial state or zero before its first token)
  auto input_at = [&](int pos, float* out) {
    if (pos >= seq_begin) {
      unpack8b(*reinterpret_cast<const uint4*>(xb + pos * p.x_st), out);
    } else {
      const int si = (W - 1) + (pos - seq_begin);
#pragma unroll
      for (int c = 0; c < 8; ++c)
        out[c] = (p.init && si >= 0) ? __bfloat162float(p.init[seq * p.i_sn + (d0 + c) * p.i_sd + si * p.i_sw]) : 0.f;
    }
  };

  int t = s0;
  while (t < s1) {
    if (p.cu_seqlens) {
      while (seq_end <= t) {
        ++seq;
        seq_begin = seq_end;
        seq_end = p.cu_seqlens[seq + 1];
      }
    }
    const int seg_end = min(s1, seq_end);
    // Tokens u = t .. u_real_end-1 are read (the outputs of this segment need the gradients of the W-1 tokens after
    // it); steps up to u_stop-1 flush the window with zero gradient when the sequence ends first.
    const int u_real_end = min(seg_end + (W - 1), seq_end);
    const int u_stop = seg_end + (W - 1);
    // Register windows as rings of kBwdRot token slots: token u = t + n lives in slot n % 4, so while it is processed
    // x[u - (W-1) + j] and gr[u - (W-1) + k] sit in slots (n - (W-1) + j) % 4: every index below is a compile-time
    // constant of the unrolled rotation and nothing is shifted.
    f2 xr[kBwdRot][4], gr[kBwdRot][4];
#pragma unroll
    for (int j = 0; j < W - 1; ++j) {
      float xv[8];
      input_at(t - (W - 1) + j, xv);
      pairs_from(xv, xr[(j - (W - 1)) & 3]);
#pragma unroll
      for (int c = 0; c < 4; ++c) gr[(j - (W - 1)) & 3][c] = zero2;
    }
    // Loads run kBwdAhead groups ahead of the arithmetic as asynchronous copies into a per-thread ring in shared memory
    // (cp.async, 16 bytes each): they occupy no registers while in flight, so every thread keeps
    // kBwdAhead * G * (2 or 3) * 16 bytes on their way and the copies' latency is covered by the work on earlier groups.
    // A thread only ever reads the slots it wrote itself: cp.async.wait_group orders them, no barrier is needed.
    auto request = [&](int ug) {
      const int slot = ((ug - t) / G) % kBwdRing;
#pragma unroll
      for (int i = 0; i < G; ++i) {
        uint4* dst = ring + ((slot * G + i) * 3) * kBwdThreads + threadIdx.x;
        if (ug + i < u_real_end) {
          cp_async16(dst, xb + (ug + i) * p.x_st);
          cp_async16(dst + kBwdThreads, gb + (ug + i) * p.dy_st);
          if (SILU && yb) cp_async16(dst + 2 * kBwdThreads, yb + (ug + i) * p.yp_st);
        } else {
          dst[0] = make_uint4(0, 0, 0, 0);
          dst[kBwdThreads] = make_uint4(0, 0, 0, 0);
          dst[2 * kBwdThreads] = make_uint4(0, 0, 0, 0);
        }
      }
      cp_async_commit();
    };
#pragma unroll
    for (int a = 0; a < kBwdAhead; ++a) request(t + a * G);
    for (int ug = t; ug < u_stop; ug += kBwdRot) {
#pragma unroll
      for (int hg = 0; hg < kBwdRot / G; ++hg) {   // a second group past u_stop only sees zero gradients and stores nothing
        const int uh = ug + hg * G;
        request(uh + kBwdAhead * G);            // past the end: zeros, and an empty group keeps the count uniform
        cp_async_wait<kBwdAhead>();
        uint4 xin[G], gin[G], yin[G];
        {
          const int slot = ((uh - t) / G) % kBwdRing;
#pragma unroll
          for (int i = 0; i < G; ++i) {
            const uint4* src = ring + ((slot * G + i) * 3) * kBwdThreads + threadIdx.x;
            xin[i] = src[0];
            gin[i] = src[kBwdThreads];
            if (SILU) yin[i] = src[2 * kBwdThreads];
          }
        }
#pragma unroll
        for (int i = 0; i < G; ++i) {
          const int ii = hg * G + i;   // slot of this token
          const int u = uh + i;
          f2 g4[4];
          unpack4p(xin[i], xr[ii]);
          unpack4p(gin[i], g4);
          if constexpr (SILU) {
            f2 pre[4];
            if (yb) {
              unpack4p(yin[i], pre);
            } else {
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                f2 a = bias[c];
#pragma unroll
                for (int j = 0; j < W; ++j) a = fma2(w[j][c], xr[(ii - (W - 1) + j) & 3][c], a);
                pre[c] = a;
              }
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) g4[c] = mul2(g4[c], dsilu2(pre[c], half2, one2, neg2));   // zero beyond the last real token
          }
#pragma unroll
          for (int c = 0; c < 4; ++c) gr[ii][c] = g4[c];
          if (u < seg_end) {   // tokens of this segment own their dw / db contributions
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              db[c] = add2(db[c], g4[c]);
#pragma unroll
              for (int j = 0; j < W; ++j) dw[j][c] = fma2(g4[c], xr[(ii - (W - 1) + j) & 3][c], dw[j][c]);
            }
          }
          const int s = u - (W - 1);   // dx[s] = sum_k w[W-1-k] gr[s+k] is complete now
          if (s >= t && s < seg_end) {
            f2 o[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              f2 a = zero2;
#pragma unroll
              for (int k = 0; k < W; ++k) a = fma2(w[W - 1 - k][c], gr[(ii - (W - 1) + k) & 3][c], a);
              o[c] = a;
            }
            const int ti = s - (seq_end - (W - 1));   // index into the final state when s is one of the last W-1 inputs
            if (p.dht && ti >= 0) {
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                float lo, hi;
                un2(o[c], lo, hi);
                lo += __bfloat162float(p.dht[seq * p.t_sn + (d0 + 2 * c) * p.t_sd + ti * p.t_sw]);
                hi += __bfloat162float(p.dht[seq * p.t_sn + (d0 + 2 * c + 1) * p.t_sd + ti * p.t_sw]);
                o[c] = mk2(lo, hi);
              }
            }
            *reinterpret_cast<uint4*>(dxb + s * p.dx_st) = make_uint4(f2_to_bf2(o[0]), f2_to_bf2(o[1]), f2_to_bf2(o[2]), f2_to_bf2(o[3]));
          }
        }
      }
    }
    cp_async_wait<0>();     // the groups requested past the segment's end
    if (t == seq_begin && p.dh0) {
      // dh0[i] = sum_{rel <= i} gr[rel] w[i - rel]: the first W-1 tokens of the sequence, recomputed on their own
      const int len = seq_end - seq_begin;
      float dh[W - 1][8];
#pragma unroll
      for (int i = 0; i < W - 1; ++i)
#pragma unroll
        for (int c = 0; c < 8; ++c) dh[i][c] = 0.f;
#pragma unroll
      for (int rel = 0; rel < W - 1; ++rel) {
        if (rel < len) {
          const int u = seq_begin + rel;
          float g8[8];
          unpack8b(*reinterpret_cast<const uint4*>(gb + u * p.dy_st), g8);
          if constexpr (SILU) {
            float pre[8];
            if (yb) {
              unpack8b(*reinterpret_cast<const uint4*>(yb + u * p.yp_st), pre);
            } else {
#pragma unroll
              for (int c = 0; c < 4; ++c) un2(bias[c], pre[2 * c], pre[2 * c + 1]);
#pragma unroll
              for (int j = 0; j < W; ++j) {
                float xv[8], wj[8];
                input_at(u - (W - 1) + j, xv);
#pragma unroll
                for (int c = 0; c < 4; ++c) un2(w[j][c], wj[2 * c], wj[2 * c + 1]);
#pragma unroll
                for (int c = 0; c < 8; ++c) pre[c] = fmaf(wj[c], xv[c], pre[c]);
              }
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) g8[c] *= dsilu(pre[c]);
          }
#pragma unroll
          for (int i = rel; i < W - 1; ++i) {
            float wj[8];
#pragma unroll
            for (int c = 0; c < 4; ++c) un2(w[i - rel][c], wj[2 * c], wj[2 * c + 1]);
#pragma unroll
            for (int c = 0; c < 8; ++c) dh[i][c] = fmaf(g8[c], wj[c], dh[i][c]);
          }
        }
      }
#pragma unroll
      for (int i = 0; i < W - 1; ++i) {
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float v = dh[i][c];
          // a sequence shorter than W-1 hands part of its initial state on to the final state
          const int ti = i - len;
          if (p.dht && len < W - 1 && ti >= 0) v += __bfloat162float(p.dht[seq * p.t_sn + (d0 + c) * p.t_sd + ti * p.t_sw]);
          const int64_t off = seq * p.h_sn + (d0 + c) * p.h_sd + i * p.h_sw;
          if (p.dh0_is_f32) static_cast<float*>(p.dh0)[off] = v;
          else static_cast<bf16*>(p.dh0)[off] = __float2bfloat16_rn(v);
        }
      }
    }
    t = seg_end;
  }

  float* dst = p.part + (int64_t(b) * p.tiles_per_row + blockIdx.y) * (W + 1) * p.D + d0;
#pragma unroll
  for (int j = 0; j < W; ++j) {
    float f[8];
#pragma unroll
    for (int c = 0; c < 4; ++c) un2(dw[j][c], f[2 * c], f[2 * c + 1]);
    *reinterpret_cast<float4*>(dst + j * p.D) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(dst + j * p.D + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
  {
    float f[8];
#pragma unroll
    for (int c = 0; c < 4; ++c) un2(db[c], f[2 * c], f[2 * c + 1]);
    *reinterpret_cast<float4*>(dst + W * p.D) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(dst + W * p.D + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
}


struct ConvBwdReduceParams {
  const float* part; float* dw; float* db;
  int64_t dw_sd, dw_sw;
  int tiles, W, D;
};

__global__ void conv_bwd_reduce_kernel(ConvBwdReduceParams p) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  const int j = blockIdx.y;   // 0 .. W-1: dw tap, W: db
  if (d >= p.D) return;
  float acc = 0.f;
  for (int t = 0; t < p.tiles; ++t) acc += p.part[(int64_t(t) * (p.W + 1) + j) * p.D + d];
  if (j < p.W) p.dw[d * p.dw_sd + j * p.dw_sw] = acc;
  else if (p.db) p.db[d] = acc;
}

inline bool vec_ok3(const fla_tensor_t& t) {
  return t.stride[2] == 1 && aligned16(t.data) && t.stride[1] % 8 == 0 && t.stride[0] % 8 == 0;
}

int bwd_tiles(const fla_causal_conv1d_bwd_args* a) {
  return int((a->x.shape[1] + kBwdTile - 1) / kBwdTile);
}

}  // namespace
}  // namespace fla

using namespace fla;

extern "C" FLA_API int fla_b200_causal_conv1d_bwd_workspace_size(const fla_causal_conv1d_bwd_args* a, uint64_t* bytes) {
  if (!a || !bytes) return FLA_ERR_NULL;
  if (!a->x.data || a->x.ndim != 3 || !a->weight.data || a->weight.ndim != 2) return FLA_ERR_SHAPE;
  const int64_t B = a->x.shape[0], D = a->x.shape[2], W = a->weight.shape[1];
  *bytes = uint64_t(B) * bwd_tiles(a) * (W + 1) * D * 4;
  return FLA_OK;
}

extern "C" FLA_API int fla_b200_causal_conv1d_bwd(const fla_causal_conv1d_bwd_args* a, void* workspace,
                                                  uint64_t workspace_bytes, void* stream) {
  if (!a) return FLA_ERR_NULL;
  const fla_tensor_t &x = a->x, &dy = a->dy, &dx = a->dx, &w = a->weight, &dw = a->dw;
  if (!x.data || !dy.data || !dx.data || !w.data || !dw.data) return FLA_ERR_NULL;
  if (x.ndim != 3 || dy.ndim != 3 || dx.ndim != 3 || w.ndim != 2 || dw.ndim != 2) return FLA_ERR_SHAPE;
  if (x.dtype != FLA_BF16 || dy.dtype != FLA_BF16 || dx.dtype != FLA_BF16 || w.dtype != FLA_BF16 || dw.dtype != FLA_F32)
    return FLA_ERR_DTYPE;
  const int64_t B = x.shape[0], T = x.shape[1], D = x.shape[2], W = w.shape[1];
  if (w.shape[0] != D || dw.shape[0] != D || dw.shape[1] != W || W < 2 || W > 4 || D % 8 || B <= 0 || T <= 0) return FLA_ERR_SHAPE;
  for (int i = 0; i < 3; ++i)
    if (dy.shape[i] != x.shape[i] || dx.shape[i] != x.shape[i]) return FLA_ERR_SHAPE;
  if (!vec_ok3(x) || !vec_ok3(dy) || !vec_ok3(dx)) return FLA_ERR_LAYOUT;
  int nseq = int(B);
  if (a->cu_seqlens.data) {
    if (B != 1 || a->cu_seqlens.dtype != FLA_I32 || a->cu_seqlens.ndim != 1 || a->cu_seqlens.shape[0] < 2) return FLA_ERR_SHAPE;
    nseq = int(a->cu_seqlens.shape[0] - 1);
  }
  ConvBwdParams p{};
  p.x = static_cast<const bf16*>(x.data); p.dy = static_cast<const bf16*>(dy.data); p.dx = static_cast<bf16*>(dx.data);
  p.weight = static_cast<const bf16*>(w.data);
  p.x_sb = x.stride[0]; p.x_st = x.stride[1]; p.dy_sb = dy.stride[0]; p.dy_st = dy.stride[1];
  p.dx_sb = dx.stride[0]; p.dx_st = dx.stride[1]; p.w_sd = w.stride[0]; p.w_sw = w.stride[1];
  if (a->y_pre.data) {
    const fla_tensor_t& y = a->y_pre;
    if (y.ndim != 3 || y.dtype != FLA_BF16 || !vec_ok3(y)) return FLA_ERR_LAYOUT;
    for (int i = 0; i < 3; ++i)
      if (y.shape[i] != x.shape[i]) return FLA_ERR_SHAPE;
    p.ypre = static_cast<const bf16*>(y.data); p.yp_sb = y.stride[0]; p.yp_st = y.stride[1];
  }
  if (a->bias.data) {
    if (a->bias.ndim != 1 || a->bias.shape[0] != D || a->bias.dtype != FLA_BF16 || a->bias.stride[0] != 1 || !aligned16(a->bias.data)) return FLA_ERR_SHAPE;
    p.bias = static_cast<const bf16*>(a->bias.data);
  }
  float* db = nullptr;
  if (a->db.data) {
    if (a->db.ndim != 1 || a->db.shape[0] != D || a->db.dtype != FLA_F32 || a->db.stride[0] != 1) return FLA_ERR_SHAPE;
    db = static_cast<float*>(a->db.data);
  }
  for (int which = 0; which < 3; ++which) {
    const fla_tensor_t& s = which == 0 ? a->initial_state : which == 1 ? a->dht : a->dh0;
    if (!s.data) continue;
    if (s.ndim != 3 || s.shape[0] != nseq || s.shape[1] != D || s.shape[2] != W - 1) return FLA_ERR_SHAPE;
    if (which < 2 && s.dtype != FLA_BF16) return FLA_ERR_DTYPE;
    if (which == 2 && s.dtype != FLA_BF16 && s.dtype != FLA_F32) return FLA_ERR_DTYPE;
    if (which == 0) { p.init = static_cast<const bf16*>(s.data); p.i_sn = s.stride[0]; p.i_sd = s.stride[1]; p.i_sw = s.stride[2]; }
    else if (which == 1) { p.dht = static_cast<const bf16*>(s.data); p.t_sn = s.stride[0]; p.t_sd = s.stride[1]; p.t_sw = s.stride[2]; }
    else { p.dh0 = s.data; p.h_sn = s.stride[0]; p.h_sd = s.stride[1]; p.h_sw = s.stride[2]; p.dh0_is_f32 = s.dtype == FLA_F32; }
  }
  p.cu_seqlens = static_cast<const int32_t*>(a->cu_seqlens.data);
  const int tiles = bwd_tiles(a);
  p.B = int(B); p.T = int(T); p.D = int(D); p.nseq = nseq; p.tiles_per_row = tiles;
  const uint64_t need = uint64_t(B) * tiles * (W + 1) * D * 4;
  if (!workspace || workspace_bytes < need || !aligned16(workspace)) return FLA_ERR_WORKSPACE;
  p.part = static_cast<float*>(workspace);

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid(unsigned((D / 8 + kBwdThreads - 1) / kBwdThreads), unsigned(tiles), unsigned(B));
  {
    KernelTimer kt("causal_conv1d_bwd", st);
    const bool silu = a->activation_silu != 0;
#define FLA_LAUNCH_BWD(WW)                                                        \
  if (silu) conv_bwd_kernel<WW, true><<<grid, kBwdThreads, kBwdSmem, st>>>(p);    \
  else conv_bwd_kernel<WW, false><<<grid, kBwdThreads, kBwdSmem, st>>>(p);
    if (W == 4) { FLA_LAUNCH_BWD(4) } else if (W == 3) { FLA_LAUNCH_BWD(3) } else { FLA_LAUNCH_BWD(2) }
#undef FLA_LAUNCH_BWD
  }
  if (cudaGetLastError() != cudaSuccess) return FLA_ERR_CUDA;
  ConvBwdReduceParams r{p.part, static_cast<float*>(dw.data), db, dw.stride[0], dw.stride[1], int(B) * tiles, int(W), int(D)};
  conv_bwd_reduce_kernel<<<dim3(unsigned((D + 255) / 256), unsigned(W + 1)), 256, 0, st>>>(r);
  return cuda_status(cudaGetLastError());
}

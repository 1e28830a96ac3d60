// Shared pieces of the chunked GDN kernels: parameter block, sequence/chunk geometry and small
// row-wise helpers for moving fp32 accumulator rows between TMEM, registers and operand panels.
#pragma once
#include <cuda_fp16.h>
#include "common/sm100.cuh"

namespace fla {

using bf16 = __nv_bfloat16;

constexpr int kC = 64;     // chunk length (tokens)
constexpr int kK = 128;    // key head dim
constexpr int kV = 128;    // value head dim
constexpr int kBV = 64;    // value columns owned by one CTA of the sequential kernels

struct SeqInfo {
  int bos;   // first token (flat index) of the sequence
  int len;   // tokens in the sequence
  int nt;    // chunks in the sequence
  int cbase; // flat index of the sequence's first chunk (for per-chunk saved tensors)
};

// cu_seqlens == nullptr: sequence n is batch row n with T tokens.
__device__ __forceinline__ SeqInfo seq_info(const int32_t* cu_seqlens, const int32_t* chunk_offsets, int n, int T) {
  SeqInfo s;
  if (cu_seqlens) {
    s.bos = cu_seqlens[n];
    s.len = cu_seqlens[n + 1] - s.bos;
    s.cbase = chunk_offsets[n];
  } else {
    s.bos = n * T;
    s.len = T;
    s.cbase = n * ((T + kC - 1) / kC);
  }
  s.nt = (s.len + kC - 1) / kC;
  return s;
}

__device__ __forceinline__ float ld_scalar(const void* p, int64_t idx, int is_f32) {
  return is_f32 ? static_cast<const float*>(p)[idx] : __bfloat162float(static_cast<const bf16*>(p)[idx]);
}

// Load 64 consecutive fp32 accumulator columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld_row64(uint32_t taddr, float* v) {
  tmem_ld32(taddr, v);
  tmem_ld32(taddr + 32, v + 32);
  tmem_ld_wait();
}
__device__ __forceinline__ void tmem_st_row64(uint32_t taddr, const float* v) {
  tmem_st16(taddr, v);
  tmem_st16(taddr + 16, v + 16);
  tmem_st16(taddr + 32, v + 32);
  tmem_st16(taddr + 48, v + 48);
  tmem_st_wait();
}

// Write a 64-wide fp32 row as bf16 hi / lo residual rows of two panels.
__device__ __forceinline__ void row64_to_hilo(uint8_t* pan_hi, uint8_t* pan_lo, int row, const float* x) {
#pragma unroll
  for (int ch = 0; ch < 8; ++ch) {
    uint4 hi, lo;
    split8(x + ch * 8, hi, lo);
    const uint32_t off = panel_chunk_off(row, ch);
    *reinterpret_cast<uint4*>(pan_hi + off) = hi;
    *reinterpret_cast<uint4*>(pan_lo + off) = lo;
  }
}
__device__ __forceinline__ void row64_to_bf16(uint8_t* pan, int row, const float* x) {
#pragma unroll
  for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(pan + panel_chunk_off(row, ch)) = pack8(x + ch * 8);
}

__device__ __forceinline__ void unpack_bf16x8(const uint4& raw, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __low2float(h[i]);
    f[2 * i + 1] = __high2float(h[i]);
  }
}

// 32 consecutive fp32 accumulator columns of this thread's TMEM lane <-> registers / split bf16 panels.
__device__ __forceinline__ void tmem_ld_row32(uint32_t taddr, float* v) {
  tmem_ld32(taddr, v);
  tmem_ld_wait();
}
__device__ __forceinline__ void tmem_st_row32(uint32_t taddr, const float* v) {
  tmem_st16(taddr, v);
  tmem_st16(taddr + 16, v + 16);
  tmem_st_wait();
}
// columns [32*half, 32*half + 32) of `row`
__device__ __forceinline__ void row32_to_hilo(uint8_t* pan_hi, uint8_t* pan_lo, int row, int half, const float* x) {
#pragma unroll
  for (int ch = 0; ch < 4; ++ch) {
    uint4 hi, lo;
    split8(x + ch * 8, hi, lo);
    const uint32_t off = panel_chunk_off(row, half * 4 + ch);
    *reinterpret_cast<uint4*>(pan_hi + off) = hi;
    *reinterpret_cast<uint4*>(pan_lo + off) = lo;
  }
}


// columns [32*half, 32*half + 32) of `row` as fp16 (11-bit significand: enough for the state copy in one pass)
__device__ __forceinline__ void row32_to_f16(uint8_t* pan, int row, int half, const float* x) {
#pragma unroll
  for (int ch = 0; ch < 4; ++ch) {
    uint4 v;
    __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(x[ch * 8 + 2 * i], x[ch * 8 + 2 * i + 1]);
    *reinterpret_cast<uint4*>(pan + panel_chunk_off(row, half * 4 + ch)) = v;
  }
}
__device__ __forceinline__ void unpack_f16x8(const uint4& raw, float* f) {
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// A wait that gives up records the timeout once; afterwards the thread stops waiting so that the kernel
// still terminates quickly (its results are then invalid, which the status word tells the host).
__device__ __forceinline__ void wait_or_mark(uint64_t* bar, uint32_t& phase, bool& dead, int* status) {
  if (!dead && !mbar_wait(bar, phase, status, 8 /* FLA_ERR_TIMEOUT */)) dead = true;
  phase ^= 1;
}


}  // namespace fla

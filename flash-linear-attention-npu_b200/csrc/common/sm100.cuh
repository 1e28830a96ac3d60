// Hand-written sm_100a building blocks: mbarrier, tcgen05 (TMEM alloc / MMA / ld / st),
// shared-memory matrix descriptors and the 128-byte swizzled "panel" layout every tensor-core
// operand in this library is staged in.
//
// Panel layout.  A panel is R rows x 64 bf16 columns, one row = 128 bytes, rows contiguous,
// base address 1024-byte aligned.  Inside each 1024-byte group of 8 rows the 16-byte chunk
// index is XOR-ed with (row % 8)  (the hardware's SWIZZLE_128B pattern).  One panel can be fed
// to tcgen05.mma in two ways without moving data:
//   * "K-major":  rows index M (or N), columns index the MMA reduction dim.  One MMA consumes
//     16 columns (32 bytes); consecutive k-steps advance the start address by 32 bytes, and a
//     tile wider than 64 columns continues in the next panel.
//   * "MN-major": columns index M (or N) (64 contiguous elements), rows index the reduction
//     dim.  One MMA consumes 16 rows (2048 bytes); M/N beyond 64 continues in the next panel
//     (leading byte offset = panel stride).
// All waits are bounded: a wait that runs out records an error code and returns false so the
// kernel can release its TMEM and exit instead of hanging the GPU.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

namespace fla {

constexpr uint32_t kSpinLimit = 20u * 1000u * 1000u;  // iterations before a wait gives up

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ----------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      " selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and leaves *err_flag = code) when `limit` polls have passed without the phase completing.
__device__ __forceinline__ bool mbar_wait_limit(uint64_t* bar, uint32_t parity, uint32_t limit, int* err_flag, int code) {
  for (uint32_t it = 0; it < limit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  if (err_flag) atomicExch(err_flag, code);
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err_flag, int code) {
  return mbar_wait_limit(bar, parity, kSpinLimit, err_flag, code);
}

// ----------------------------------------------------------------------------- bulk async copies
// 1-D bulk copies between global and shared memory (16-byte aligned addresses, size % 16 == 0).
// Loads complete on an mbarrier (transaction bytes); stores are tracked by bulk groups.  No multicast.
__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_dst),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// Asks for a global range to be brought into L2 (no completion to wait for): a later bulk_load of it then pays the L2 latency
// instead of the DRAM one.  For consumers that can only issue the load itself once their single buffer is free.
__device__ __forceinline__ void bulk_prefetch_l2(const void* gsrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gsrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, uint32_t smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_src), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// All committed bulk stores have finished READING shared memory (the source may be overwritten).
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// All committed bulk stores are complete.
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ----------------------------------------------------------------------------- fences
__device__ __forceinline__ void fence_async_smem() {  // generic-proxy smem writes -> async proxy (MMA/TMA)
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ----------------------------------------------------------------------------- TMEM
// Warp-collective.  ncols: power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// TMEM address of (lane, column) relative to an allocation base.
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t col) {
  return base + (lane << 16) + col;
}

// 32 lanes x 32-bit loads: thread i of the warp receives N consecutive columns of lane (base lane + i).
// The warp may only touch the 32-lane quadrant (warp_id % 4).
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float* v) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(
          taddr),
      "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
      "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
      "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
      "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])),
      "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ----------------------------------------------------------------------------- descriptors
// Instruction descriptor for tcgen05.mma.kind::f16 with fp32 accumulate.
// a_mn / b_mn: 0 = operand is K-major, 1 = MN-major.  fmt: 1 = bf16, 0 = fp16; A and B must use the SAME
// format (a bf16 x fp16 mix is rejected by the hardware as an illegal instruction).
__host__ __device__ constexpr uint32_t make_idesc(int M, int N, int a_mn, int b_mn, int a_fmt, int b_fmt) {
  return (1u << 4)                       // D format: f32
         | (uint32_t(a_fmt) << 7)        // A format
         | (uint32_t(b_fmt) << 10)       // B format
         | (uint32_t(a_mn) << 15)        // A major
         | (uint32_t(b_mn) << 16)        // B major
         | (uint32_t(N >> 3) << 17)      // N / 8
         | (uint32_t(M >> 4) << 24);     // M / 16
}
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N, int a_mn, int b_mn) {
  return make_idesc(M, N, a_mn, b_mn, 1, 1);
}

constexpr uint64_t kDescSw128 = (uint64_t(1) << 46) | (uint64_t(2) << 61);  // version 1, SWIZZLE_128B

// K-major view of a panel: 8-row groups 1024 bytes apart; leading offset unused under swizzle.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
  return kDescSw128 | uint64_t((saddr >> 4) & 0x3FFF) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32);
}
// MN-major view: next 64 M/N elements `panel_stride` bytes away, next 8 reduction rows 1024 bytes away.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr, uint32_t panel_stride) {
  return kDescSw128 | uint64_t((saddr >> 4) & 0x3FFF) | (uint64_t((panel_stride >> 4) & 0x3FFF) << 16) |
         (uint64_t(1024 >> 4) << 32);
}

// One tcgen05.mma (K = 16): D[tmem] (+)= A[smem] * B[smem].  Issued by a single thread.
// `leader` != 0 in the thread that issues: callers inside a branch that only one thread takes pass 1 (the default); callers
// whose whole warp runs the issuing code (so that descriptors stay warp-uniform values) pass elect_one().
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate, uint32_t leader = 1u) {
  asm volatile(
      "{\n"
      " .reg .pred p, q;\n"
      " setp.ne.b32 p, %4, 0;\n"
      " setp.ne.b32 q, %5, 0;\n"
      " @q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(leader)
      : "memory");
}
// One lane of the (converged) warp.
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      " .reg .pred p;\n"
      " elect.sync _|p, 0xffffffff;\n"
      " selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred;
}
// The same with the A operand in tensor memory: row m of A is TMEM lane m (M = 128), its 16-bit elements are packed two
// per 32-bit column (element 2c in the low half of column c), so one K = 16 step reads 8 columns starting at `a_tmem`.
// A written with tcgen05.st needs tcgen05.wait::st + tcgen05.fence::before_thread_sync + a barrier before this is issued.
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate, uint32_t leader = 1u) {
  asm volatile(
      "{\n"
      " .reg .pred p, q;\n"
      " setp.ne.b32 p, %4, 0;\n"
      " setp.ne.b32 q, %5, 0;\n"
      " @q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(leader)
      : "memory");
}
// Make the mbarrier observe completion of every MMA this thread issued so far.
__device__ __forceinline__ void mma_commit(uint64_t* bar, uint32_t leader = 1u) {
  asm volatile(
      "{\n"
      " .reg .pred q;\n"
      " setp.ne.b32 q, %1, 0;\n"
      " @q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
      "}\n" ::"r"(smem_u32(bar)), "r"(leader)
      : "memory");
}

// A tile operand in shared memory.
//   mn_major 0 / 1: 128-byte-swizzled panels (rows x 64 columns each, `panel_stride` bytes apart), read with the rows as
//                   M / N and the columns as the reduction dim (0) or the other way round (1).
//   mn_major 2:     the un-swizzled "strip" layout [M or N / 8][reduction rows][8 elements = 16 bytes]: the 8 x 16-byte core
//                   matrices are 128 contiguous bytes, strips are `panel_stride` bytes apart.  A writer whose threads each own
//                   one reduction row stores a strip piece as 16 bytes per thread at consecutive addresses (coalesced), which
//                   the swizzled panels cannot offer (their rows are 128 bytes apart).
//   mn_major 3:     the same memory read the other way round: [reduction / 8][M or N rows][16 bytes], i.e. strips of 8
//                   reduction elements and rows = M / N (what the swizzled panels do with one layout, strips do too).
struct Operand {
  uint32_t saddr;         // shared address of the operand
  uint32_t panel_stride;  // bytes between panels (mn_major 0 / 1) or between strips (2)
  int mn_major;
};
__device__ __forceinline__ uint64_t operand_desc(const Operand& o, int kstep) {
  if (o.mn_major) return desc_mnmajor(o.saddr + kstep * 2048, o.panel_stride);
  return desc_kmajor(o.saddr + (kstep >> 2) * o.panel_stride + (kstep & 3) * 32);
}
// Upper 32 bits of the swizzled descriptors: stride byte offset 1024, descriptor version 1, SWIZZLE_128B.
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
// Upper 32 bits: swizzled, or (strips) stride byte offset = strip stride, version 1, no swizzle.
__device__ __forceinline__ uint32_t operand_desc_hi(const Operand& o) {
  if (o.mn_major == 2) return ((o.panel_stride >> 4) & 0x3FFFu) | (1u << 14);   // stride offset = next strip of 8 M / N elements
  if (o.mn_major == 3) return (128u >> 4) | (1u << 14);                          // stride offset = next 8 rows (M / N)
  return kDescHi;
}
// Lower 32 bits at k-step 0: start address and leading byte offset (panel stride of swizzled MN-major views; for strips
// the 128 bytes between groups of 8 reduction rows).
__device__ __forceinline__ uint32_t operand_desc_lo(const Operand& o) {
  const uint32_t lbo = o.mn_major == 2 ? (128u >> 4)                               // next 8 reduction rows
                       : o.mn_major == 3 ? ((o.panel_stride >> 4) & 0x3FFFu)       // next strip of 8 reduction elements
                       : (o.mn_major ? ((o.panel_stride >> 4) & 0x3FFFu) : 1u);
  return ((o.saddr >> 4) & 0x3FFFu) | (lbo << 16);
}
// Start-address advance (in 16-byte units) of k-step `ks`
__device__ __forceinline__ uint32_t operand_kstep(const Operand& o, int ks) {
  if (o.mn_major == 3) return uint32_t(ks) * 2u * (o.panel_stride >> 4);  // two strips of 8 reduction elements
  if (o.mn_major == 2) return uint32_t(ks) * 16u;                       // 16 reduction rows of 16 bytes
  if (o.mn_major == 1) return uint32_t(ks) * 128u;                      // 16 rows of 128 bytes
  return uint32_t(ks >> 2) * (o.panel_stride >> 4) + uint32_t(ks & 3) * 2u;
}
// D (+)= A * B over `ksteps` MMAs of K = 16 each.  Single-thread call; call with a literal `ksteps` so the
// loop unrolls.  Issue cost matters (one thread feeds the tensor core): per k-step only the start-address
// field of each descriptor changes, by a constant, so each MMA costs two integer adds.
__device__ __forceinline__ void mma_tile(uint32_t d_tmem, const Operand& a, const Operand& b, int M, int N,
                                         int ksteps, bool accumulate, uint32_t leader = 1u) {
  const uint32_t idesc = make_idesc_bf16(M, N, a.mn_major == 1 || a.mn_major == 2, b.mn_major == 1 || b.mn_major == 2);
  const uint32_t alo = operand_desc_lo(a), blo = operand_desc_lo(b);
  const uint32_t ahi = operand_desc_hi(a), bhi = operand_desc_hi(b);
#pragma unroll
  for (int ks = 0; ks < ksteps; ++ks) {
    const uint64_t ad = (uint64_t(ahi) << 32) | uint64_t(alo + operand_kstep(a, ks));
    const uint64_t bd = (uint64_t(bhi) << 32) | uint64_t(blo + operand_kstep(b, ks));
    mma_ss(d_tmem, ad, bd, idesc, (accumulate || ks > 0) ? 1u : 0u, leader);
  }
}

// D (+)= A * B over `ksteps` MMAs of K = 16 with A in tensor memory at columns [a_tmem, a_tmem + 8 * ksteps).
__device__ __forceinline__ void mma_tile_ts(uint32_t d_tmem, uint32_t a_tmem, const Operand& b, int N, int ksteps,
                                            bool accumulate, uint32_t leader = 1u) {
  const uint32_t idesc = make_idesc_bf16(128, N, 0, b.mn_major == 1 || b.mn_major == 2);
  const uint32_t blo = operand_desc_lo(b), bhi = operand_desc_hi(b);
#pragma unroll
  for (int ks = 0; ks < ksteps; ++ks) {
    const uint64_t bd = (uint64_t(bhi) << 32) | uint64_t(blo + operand_kstep(b, ks));
    mma_ts(d_tmem, a_tmem + uint32_t(ks) * 8u, bd, idesc, (accumulate || ks > 0) ? 1u : 0u, leader);
  }
}

// ----------------------------------------------------------------------------- panel addressing
// Byte offset of element (row, col) (col in [0,64)) inside a panel.
__device__ __forceinline__ uint32_t panel_off(int row, int col) {
  return uint32_t(row) * 128u + ((uint32_t(col >> 3) ^ uint32_t(row & 7)) << 4) + uint32_t(col & 7) * 2u;
}
// Byte offset of 16-byte chunk `chunk` (0..7) of `row`.
__device__ __forceinline__ uint32_t panel_chunk_off(int row, int chunk) {
  return uint32_t(row) * 128u + ((uint32_t(chunk) ^ uint32_t(row & 7)) << 4);
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
// Split eight fp32 values into a bf16 "hi" vector and a bf16 "lo" residual vector (x ~= hi + lo).
// Per pair: one packed convert, the two hi values recovered by shift / mask, two subtractions, one packed convert.
__device__ __forceinline__ void split8(const float* x, uint4& hi, uint4& lo) {
  uint32_t h[4], l[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    h[i] = pack_bf16(x[2 * i], x[2 * i + 1]);
    const float h0 = __uint_as_float(h[i] << 16), h1 = __uint_as_float(h[i] & 0xffff0000u);
    l[i] = pack_bf16(x[2 * i] - h0, x[2 * i + 1] - h1);
  }
  hi = make_uint4(h[0], h[1], h[2], h[3]);
  lo = make_uint4(l[0], l[1], l[2], l[3]);
}
__device__ __forceinline__ uint4 pack8(const float* x) {
  return make_uint4(pack_bf16(x[0], x[1]), pack_bf16(x[2], x[3]), pack_bf16(x[4], x[5]), pack_bf16(x[6], x[7]));
}

}  // namespace fla

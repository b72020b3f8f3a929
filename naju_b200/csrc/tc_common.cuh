// tcgen05 / TMEM / TMA / mbarrier primitives (inline PTX, sm_100a) shared by the tensor-core
// kernels.  Every wait in here is bounded: it gives up after a fixed number of tries and reports it.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace naju {
namespace tcx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- shared-memory matrix descriptor: K-major, no swizzle, descriptor version 1 (sm_100).
// Core matrix = 8 rows x 16 bytes, stored as 128 contiguous bytes.  `lbo` = byte distance
// between core matrices adjacent in K, `sbo` = byte distance between 8-row groups.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

// ---- instruction descriptor: D fp32; A,B of `fmt` (0 f16, 1 bf16, 2 tf32), both K-major, dense
__device__ __forceinline__ uint32_t umma_idesc(int M, int N, uint32_t fmt) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] . B[smem]^T, bf16 operands, one K=16 slab
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t mbar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar)
               : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Asynchronous TMEM load: the registers are valid only after tmem_ld_wait16() on the same array.
__device__ __forceinline__ void tmem_ld16_async(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// Waits for every outstanding TMEM load of this thread; naming the registers keeps the compiler
// from using them before the wait.
__device__ __forceinline__ void tmem_ld_wait16(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;\n"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}

// Eight-column forms of the two above.
__device__ __forceinline__ void tmem_ld8_async(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld_wait8(uint32_t (&a)[8], uint32_t (&b)[8]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;\n"
               : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7]),
                 "+r"(b[0]), "+r"(b[1]), "+r"(b[2]), "+r"(b[3]), "+r"(b[4]), "+r"(b[5]), "+r"(b[6]), "+r"(b[7])
               :
               : "memory");
}
__device__ __forceinline__ void tmem_ld_wait8(uint32_t (&a)[8]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;\n"
               : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7])
               :
               : "memory");
}

// ---- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t mbar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t mbar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mbar) : "memory");
}
// One arrival for the whole (converged) warp: 32 lanes arriving on one barrier would be 32
// serialised updates of the same shared-memory word.  __syncwarp orders the lanes' earlier
// shared-memory writes before the elected lane's releasing arrival.  Barriers used with this are
// initialised with a count in WARPS.
__device__ __forceinline__ void mbar_arrive_warp(uint32_t mbar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(mbar);
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t mbar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"(bytes) : "memory");
}
// Bounded wait for the phase of parity `parity` to complete; false if the budget ran out.
// mbarrier.try_wait parks the warp in hardware (here for up to ~4 us per try) and wakes it when
// the phase completes, so the common case costs one instruction and no wake-up delay; only after
// 64 failed tries does the loop add a nanosleep, which bounds the whole wait to roughly
// [2^18 x 0.26 us, 2^18 x 4.3 us] = 0.07 .. 1.1 s.
// One try at the barrier (the hardware may park the thread for a short, bounded time before it
// answers): true if the phase of parity `parity` has completed.
__device__ __forceinline__ bool mbar_try_once(uint32_t mbar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(mbar), "r"(parity)
      : "memory");
  return ok != 0;
}

// (kept out of line: the retry loop is cold code, and the kernels' hot loops must stay small
// enough for the instruction caches)
static __device__ __noinline__ bool mbar_wait_slow(uint32_t mbar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      ".reg .u32 n;\n\t"
      "mov.u32 n, 0;\n"
      "NAJU_MBAR_TRY:\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "@p bra NAJU_MBAR_DONE;\n\t"
      "add.u32 n, n, 1;\n\t"
      "setp.gt.u32 q, n, 64;\n\t"
      "@q nanosleep.u32 256;\n\t"
      "setp.lt.u32 q, n, %4;\n\t"
      "@q bra NAJU_MBAR_TRY;\n"
      "NAJU_MBAR_DONE:\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(mbar), "r"(parity), "r"(4096u), "r"(1u << 18)
      : "memory");
  return ok != 0;
}
// (the common case -- the phase is already complete -- costs one try and one branch)
__device__ __forceinline__ bool mbar_wait(uint32_t mbar, uint32_t parity) {
  if (mbar_try_once(mbar, parity)) return true;
  return mbar_wait_slow(mbar, parity);
}

// (Waits that sleep between polls -- 32 ns to 1 us, for the roles with slack -- were measured in both
// walk kernels and are 1-4 % slower than parking every wait in try_wait.)

// ---- TMA: 3-D tiled load global -> shared, completion counted on an mbarrier.  Plain
// (single-destination) form only.  The innermost coordinate times the element size must be a
// multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* map, int c0, int c1,
                                            int c2, uint32_t mbar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(mbar)
      : "memory");
}

// 3-D tiled store shared -> global (bulk async-group completion).  The writers of the shared tile
// fence (fence_async_smem) and synchronise before one thread issues the store; rows and columns
// of the box that fall outside the tensor are not written.  Same 16-byte rule as the load.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, int c0, int c1, int c2, uint32_t smem_src) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
               ::"l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_src)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all earlier store groups of this thread have finished READING shared memory (the tile may be reused)
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all but the newest N store groups of this thread have finished reading shared memory
template <int N>
__device__ __forceinline__ void tma_store_wait_read_but() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// all earlier store groups of this thread are complete (before the kernel exits)
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---- named barrier over a subset of the CTA's warps
template <int ID, int COUNT>
__device__ __forceinline__ void bar_sync() {
  asm volatile("bar.sync %0, %1;" ::"n"(ID), "n"(COUNT) : "memory");
}
// barrier + OR-reduction of a predicate over the participating threads
template <int ID, int COUNT>
__device__ __forceinline__ bool bar_or(bool pred) {
  uint32_t out;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, %2, %3, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(out)
      : "r"(pred ? 1u : 0u), "n"(ID), "n"(COUNT)
      : "memory");
  return out != 0;
}

// ---- bf16 helpers
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {  // lo -> bits [0,16)
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float bf16lo_f32(uint32_t p) { return __uint_as_float(p << 16); }
__device__ __forceinline__ float bf16hi_f32(uint32_t p) { return __uint_as_float(p & 0xFFFF0000u); }

// Two-term bf16 split of a pair of floats: v ~= hi + lo with 16 mantissa bits kept.  Both terms
// are truncations (the first one's error is exactly what the second term carries), so the split
// costs only integer and FMA-pipe operations: the conversion instructions share the SFU pipe with
// ex2/rcp, which is the busiest pipe of the gate warps.  Residual <= 2^-16 relative.
__device__ __forceinline__ void split_bf16x2(float a, float b, uint32_t& hi, uint32_t& lo) {
  const uint32_t ua = __float_as_uint(a), ub = __float_as_uint(b);
  const uint32_t ha = ua & 0xFFFF0000u, hb = ub & 0xFFFF0000u;
  hi = __byte_perm(ha, hb, 0x7632);  // {hb[31:16], ha[31:16]}
  const uint32_t la = __float_as_uint(a - __uint_as_float(ha)), lb = __float_as_uint(b - __uint_as_float(hb));
  lo = __byte_perm(la, lb, 0x7632);
}

// shared-memory element -> fp32 without the conversion unit where the format allows it
__device__ __forceinline__ float ld_as_f32(const __nv_bfloat16* p, int i) {
  return __uint_as_float(static_cast<uint32_t>(reinterpret_cast<const unsigned short*>(p)[i]) << 16);
}
__device__ __forceinline__ float ld_as_f32(const __half* p, int i) { return __half2float(p[i]); }
__device__ __forceinline__ float ld_as_f32(const float* p, int i) { return p[i]; }
// two adjacent 16-bit elements (4-byte aligned) as floats, one 32-bit load
__device__ __forceinline__ float2 ld_pair_as_f32(const __nv_bfloat16* p) {
  const uint32_t pk = *reinterpret_cast<const uint32_t*>(p);
  return make_float2(bf16lo_f32(pk), bf16hi_f32(pk));
}
__device__ __forceinline__ float2 ld_pair_as_f32(const __half* p) {
  return __half22float2(*reinterpret_cast<const __half2*>(p));
}

// D(16x8, fp32) += A(16x16, bf16, row) . B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16_16x8x16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                 uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// byte offset of bf16 element (row, k) in a K-major no-swizzle operand (8 elements per chunk)
__device__ __forceinline__ uint32_t op_off16(int row, int k, uint32_t sbo) {
  return static_cast<uint32_t>(row >> 3) * sbo + static_cast<uint32_t>(k >> 3) * 128u +
         static_cast<uint32_t>(row & 7) * 16u + static_cast<uint32_t>(k & 7) * 2u;
}

}  // namespace tcx
}  // namespace naju

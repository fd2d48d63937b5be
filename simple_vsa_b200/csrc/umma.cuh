// sm_100a building blocks: mbarriers with bounded waits, TMA tile loads (plain: every CTA fetches its own boxes),
// tensor-memory allocation, tcgen05.mma with shared-memory operand descriptors, tcgen05.ld.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace vsa {
namespace umma {

// ---- mbarrier --------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait.  The limit is wall-clock (the global nanosecond timer), not an iteration count,
// because one try_wait may itself suspend the thread for a hardware-defined time.  A legitimate
// wait inside these kernels lasts microseconds; after kWaitLimitNs the wait gives up and returns
// false.  `abort_flag` (a device status word) is polled too, so that once any CTA has given up
// every other wait in flight returns at once instead of serving its own full limit.
constexpr unsigned long long kWaitLimitNs = 250ull * 1000ull * 1000ull;
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const volatile int* abort_flag,
                                          unsigned long long limit_ns = kWaitLimitNs) {
  // Called by ONE lane per warp (see warp_wait): hundreds of threads polling the same barrier word
  // measurably slowed the shared-memory pipe.  The clock and the abort flag live in global memory and
  // are looked at once per 64 unsuccessful tries only.
  unsigned long long t0 = 0;
#pragma unroll 1
  for (int i = 0; i < 32; ++i)
    if (mbar_try_wait(bar, parity)) return true;
#pragma unroll 1
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
      __nanosleep(20);   // measured with 0, 20, 100 and 400 ns: no difference in kernel time or board power
    }
    if (*abort_flag != 0) return false;
    const unsigned long long now = global_ns();
    if (t0 == 0) t0 = now;
    else if (now - t0 > limit_ns) return false;
  }
}
// Whole-warp wait: lane 0 polls (one try first: the common case is a barrier that has already flipped);
// the warp barrier orders the acquired data for the other lanes, the vote shares the result.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, const volatile int* abort_flag, int lane) {
  int ok = 1;
  if (lane == 0) {
    if (!mbar_try_wait(bar, parity)) ok = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
  }
  __syncwarp();
  return __all_sync(0xffffffffu, ok) != 0;
}
// Two barriers at once: lane 0 polls the first, lane 1 the second, in the same instruction stream, so the
// pair costs one shared-memory round trip instead of two back to back (each is ~180 cycles even when the
// barrier has long flipped, and the elementwise warps pay it once per pair of tiles).
__device__ __forceinline__ bool warp_wait2(uint32_t bar_a, uint32_t parity_a, uint32_t bar_b, uint32_t parity_b,
                                           const volatile int* abort_flag, int lane) {
  int ok = 1;
  if (lane < 2) {
    const uint32_t bar = lane == 0 ? bar_a : bar_b;
    const uint32_t parity = lane == 0 ? parity_a : parity_b;
    if (!mbar_try_wait(bar, parity)) ok = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
  }
  __syncwarp();
  return __all_sync(0xffffffffu, ok) != 0;
}

// Wait for barrier A and, in the same shared-memory round trip, LOOK at barrier B (mbarrier.test_wait: no
// suspension).  Returns false on a time-out of A; *b_done tells whether B's phase had completed.  For a second
// barrier that is needed a few hundred cycles later and has usually flipped by now: the later blocking wait (and
// its ~180-cycle round trip) is then skipped.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool warp_wait_and_test(uint32_t bar_a, uint32_t parity_a, uint32_t bar_b, uint32_t parity_b,
                                                   const volatile int* abort_flag, int lane, bool* b_done) {
  int ok = 1, done = 1;
  if (lane == 0) {
    if (!mbar_try_wait(bar_a, parity_a)) ok = mbar_wait(bar_a, parity_a, abort_flag) ? 1 : 0;
  } else if (lane == 1) {
    done = mbar_test(bar_b, parity_b) ? 1 : 0;
  }
  __syncwarp();
  *b_done = __all_sync(0xffffffffu, done) != 0;
  return __all_sync(0xffffffffu, ok) != 0;
}

// The executing thread's earlier cp.async copies arrive on the barrier when they have landed (the arrival is one
// of the barrier's expected count, not an extra one).
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- fences ----------------------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- TMA: one 2-D box global -> shared, completion counted on an mbarrier (plain form, one CTA) ------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}
// One 2-D box shared -> global (bulk async-group completion: commit, then wait for the reads of shared memory).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int x, int y, uint32_t src) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(src) : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_group0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Contiguous bytes global -> shared (16-byte aligned addresses, size a multiple of 16), completion on an mbarrier.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- tensor memory ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {   // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {       // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---- descriptors -------------------------------------------------------------------------------
// Shared-memory operand descriptor, 128-byte swizzle: start address, leading-dimension byte offset
// and stride byte offset in 16-byte units, descriptor version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor for kind::f16 with 16-bit inputs and fp32 accumulation.
// major: 0 = K-major operand, 1 = MN-major operand.  in_fmt: format of both inputs, 1 = bf16, 0 = fp16.
__host__ __device__ constexpr uint32_t instr_desc(int M, int N, int a_mn_major, int b_mn_major, uint32_t in_fmt = 1u) {
  return (1u << 4) | (in_fmt << 7) | (in_fmt << 10) | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16) |
         ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// The same descriptor split into its 32-bit halves, so that the issuing thread (a single lane, hence
// latency-bound on every dependent instruction) advances an operand with ONE 32-bit add per MMA:
// low word = start address and leading offset (both in 16-byte units), high word = stride offset,
// version and swizzle mode.
__device__ __forceinline__ uint32_t desc_lo(uint32_t addr, uint32_t lbo_bytes) {
  return ((addr & 0x3FFFFu) >> 4) | (((lbo_bytes >> 4) & 0x3FFFu) << 16);
}
__host__ __device__ constexpr uint32_t desc_hi(uint32_t sbo_bytes) {
  return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
}
// High word for an un-swizzled operand (layout type 0): core matrices of 8 rows x 16 bytes stored contiguously;
// for a K-major operand the leading offset (low word) is the distance between core matrices along K and the
// stride offset the distance between 8-row groups.
__host__ __device__ constexpr uint32_t desc_hi_noswizzle(uint32_t sbo_bytes) {
  return ((sbo_bytes >> 4) & 0x3FFFu) | (1u << 14);
}
__device__ __forceinline__ uint64_t desc_pack(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// mbarrier arrives once every tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 columns of 32-bit: thread i of the warp receives lane (lane_base+i), columns c..c+31.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
// 32 lanes x 16 columns.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld16(taddr, r); }
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld32(taddr, r); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

}  // namespace umma
}  // namespace vsa

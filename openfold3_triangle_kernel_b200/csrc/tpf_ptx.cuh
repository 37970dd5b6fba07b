// Thin inline-PTX layer for sm_100a: mbarrier, TMA tile loads, tcgen05 (UMMA)
// issue/commit, TMEM allocation and TMEM<->register moves, plus the shared-memory
// matrix descriptors and the instruction descriptor for bf16 x bf16 -> fp32.
//
// Every wait in this file is bounded: a wait that does not complete within
// TPF_WAIT_LIMIT_CYCLES SM cycles raises a per-CTA abort flag (all later waits of that CTA
// return at once) and records a non-zero code in a global status word that the
// host reads back through tpf_device_status().  Kernels therefore always run to
// their normal end, free their TMEM and return.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tpf {

#ifndef TPF_WAIT_LIMIT_CYCLES
#define TPF_WAIT_LIMIT_CYCLES 4000000000ll
#endif

enum StatusCode : int {
  kStatusOk = 0,
  kStatusWaitTimeout = 1,
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ----------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking probe (try_wait may suspend the thread for a while when the phase is still open).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Per-CTA abort state: `flag` lives in shared memory, `status` in global memory.
struct WaitCtx {
  volatile int* flag;
  int* status;
};

// Bounded wait.  The common case (a few polls) touches no timer; after that the SM cycle
// counter bounds the wait (TPF_WAIT_LIMIT_CYCLES, about two seconds at boost clock).
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& ctx) {
#pragma unroll 1
  for (int i = 0; i < 128; ++i)
    if (mbar_try_wait(bar, parity)) return;
  const long long t0 = clock64();
  uint32_t it = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (((++it) & 0xFF) == 0) {
      if (*ctx.flag) return;
      if (clock64() - t0 > (long long)TPF_WAIT_LIMIT_CYCLES) {
        *ctx.flag = 1;
        atomicCAS(ctx.status, 0, (int)kStatusWaitTimeout);
        return;
      }
    }
  }
}

// Waits on two / three barriers at once.  A probe answers only after 150+ cycles even when its phase
// completed long ago; probes issued back to back overlap, sequential waits would pay that latency each.
// The blocking waits are the fallback for the (rare) case that one of the phases is still open.
__device__ __forceinline__ void mbar_wait2(uint64_t* a, uint32_t pa, uint64_t* b, uint32_t pb, const WaitCtx& ctx) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred qa, qb;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 qa, [%1], %2;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 qb, [%3], %4;\n\t"
      "and.pred qa, qa, qb;\n\t"
      "selp.u32 %0, 1, 0, qa;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(a)), "r"(pa), "r"(smem_u32(b)), "r"(pb)
      : "memory");
  if (ok) return;
  mbar_wait(a, pa, ctx);
  mbar_wait(b, pb, ctx);
}
__device__ __forceinline__ void mbar_wait3(uint64_t* a, uint32_t pa, uint64_t* b, uint32_t pb, uint64_t* c, uint32_t pc,
                                           const WaitCtx& ctx) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred qa, qb, qc;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 qa, [%1], %2;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 qb, [%3], %4;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 qc, [%5], %6;\n\t"
      "and.pred qa, qa, qb;\n\t"
      "and.pred qa, qa, qc;\n\t"
      "selp.u32 %0, 1, 0, qa;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(a)), "r"(pa), "r"(smem_u32(b)), "r"(pb), "r"(smem_u32(c)), "r"(pc)
      : "memory");
  if (ok) return;
  mbar_wait(a, pa, ctx);
  mbar_wait(b, pb, ctx);
  mbar_wait(c, pc, ctx);
}

// ----------------------------------------------------------------------------
// Proxy / tcgen05 fences
// ----------------------------------------------------------------------------
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ----------------------------------------------------------------------------
// TMA tile loads (global -> this CTA's shared memory, completion on an mbarrier)
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
      "[%2];" ::"r"(smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ void tma_load_5d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, "
      "%7}], [%2];" ::"r"(smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}

// ----------------------------------------------------------------------------
// TMEM allocation (one full warp executes these)
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ----------------------------------------------------------------------------
// UMMA descriptors
// ----------------------------------------------------------------------------
// Shared-memory matrix descriptor (64 bit):
//   [ 0,14) start address >> 4        [16,30) leading byte offset >> 4
//   [32,46) stride byte offset >> 4   [46,48) version = 1 on sm_100
//   [61,64) swizzle mode: 0 none, 2 = 128 B, 4 = 64 B, 6 = 32 B
// K-major operand  (rows = M/N index, K contiguous, row pitch = swizzle width):
//   SBO = distance between 8-row groups, LBO unused (set to 16 B).
// MN-major operand (rows = K index, M/N contiguous in chunks of one swizzle width):
//   SBO = distance between 8-k-row groups, LBO = distance between M/N chunks.
__host__ __device__ constexpr uint32_t swizzle_mode_for_bytes(int bytes) {
  return bytes == 128 ? 2u : bytes == 64 ? 4u : bytes == 32 ? 6u : 0u;
}
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t swizzle_mode) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | ((uint64_t)swizzle_mode << 61);
}
// Instruction descriptor for kind::f16 with bf16 A/B and fp32 accumulate.
//   [4,6) D fmt (1 = f32)  [7,10) A fmt (1 = bf16)  [10,13) B fmt (1 = bf16)
//   [15] A is MN-major     [16] B is MN-major       [17,23) N >> 3   [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc_bf16(int M, int N, bool a_mn, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One k-block of UMMAs issued under two barrier probes.
// A barrier probe (test_wait / try_wait) answers after 150+ cycles even when the phase completed long ago,
// and the issuing thread's instruction stream is the critical path of the tensor pipe.  Here the probes of
// the barriers needed NEXT (the next stage's `full`, the next tile's accumulator) are issued first, then the
// four UMMAs of this k-block (descriptor j = base + j * STEP in the start-address field) and the commit that
// releases the stage; the probe answers are read only after all of that has been issued.
// Returns bit 0: probe_a done, bit 1: probe_b done.
template <int A_STEP, int B_STEP>
__device__ __forceinline__ uint32_t umma_ss_x4_probed(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                      uint32_t accumulate_first, uint64_t* commit_bar,
                                                      uint64_t* probe_a, uint32_t parity_a, uint64_t* probe_b,
                                                      uint32_t parity_b) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, qa, qb;\n\t.reg .b64 ad, bd;\n\t.reg .b32 ra, rb;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 qa, [%7], %8;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 qb, [%9], %10;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], %2, %3, %4, p;\n\t"
      "add.s64 ad, %2, %11;\n\t add.s64 bd, %3, %12;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], ad, bd, %4, 1;\n\t"
      "add.s64 ad, ad, %11;\n\t add.s64 bd, bd, %12;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], ad, bd, %4, 1;\n\t"
      "add.s64 ad, ad, %11;\n\t add.s64 bd, bd, %12;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], ad, bd, %4, 1;\n\t"
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%6];\n\t"
      "selp.u32 ra, 1, 0, qa;\n\t selp.u32 rb, 2, 0, qb;\n\t or.b32 %0, ra, rb;\n\t}"
      : "=r"(r)
      : "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate_first), "r"(smem_u32(commit_bar)),
        "r"(smem_u32(probe_a)), "r"(parity_a), "r"(smem_u32(probe_b)), "r"(parity_b), "n"(A_STEP), "n"(B_STEP)
      : "memory");
  return r;
}
// The same for a k-block computed with the operand roles exchanged: UMMAs (w, x) -> d0 and (w + W1_OFF, x) -> d1.
template <int STEP, int W1_OFF>
__device__ __forceinline__ uint32_t umma_ss_x4x2_probed(uint32_t d0, uint32_t d1, uint64_t wdesc, uint64_t xdesc,
                                                        uint32_t idesc, uint32_t accumulate_first, uint64_t* commit_bar,
                                                        uint64_t* probe_a, uint32_t parity_a, uint64_t* probe_b,
                                                        uint32_t parity_b) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, qa, qb;\n\t.reg .b64 wd, w1, xd;\n\t.reg .b32 ra, rb;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 qa, [%8], %9;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 qb, [%10], %11;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "add.s64 w1, %3, %13;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], %3, %4, %5, p;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%2], w1, %4, %5, p;\n\t"
      "add.s64 wd, %3, %12;\n\t add.s64 w1, w1, %12;\n\t add.s64 xd, %4, %12;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], wd, xd, %5, 1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%2], w1, xd, %5, 1;\n\t"
      "add.s64 wd, wd, %12;\n\t add.s64 w1, w1, %12;\n\t add.s64 xd, xd, %12;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], wd, xd, %5, 1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%2], w1, xd, %5, 1;\n\t"
      "add.s64 wd, wd, %12;\n\t add.s64 w1, w1, %12;\n\t add.s64 xd, xd, %12;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%1], wd, xd, %5, 1;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%2], w1, xd, %5, 1;\n\t"
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%7];\n\t"
      "selp.u32 ra, 1, 0, qa;\n\t selp.u32 rb, 2, 0, qb;\n\t or.b32 %0, ra, rb;\n\t}"
      : "=r"(r)
      : "r"(d0), "r"(d1), "l"(wdesc), "l"(xdesc), "r"(idesc), "r"(accumulate_first), "r"(smem_u32(commit_bar)),
        "r"(smem_u32(probe_a)), "r"(parity_a), "r"(smem_u32(probe_b)), "r"(parity_b), "n"(STEP), "n"(W1_OFF)
      : "memory");
  return r;
}
// Arrive on `bar` once every UMMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ----------------------------------------------------------------------------
// TMEM -> registers.  Shape 32x32b: lane i of the warp reads TMEM lane
// (32 * (warp_id % 4) + i), N consecutive 32-bit columns.
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t (&r)[4]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// TMEM address helpers: bits [31:16] lane, [15:0] column.
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t col) {
  return base + (lane << 16) + col;
}

// ----------------------------------------------------------------------------
// Small numeric helpers
// ----------------------------------------------------------------------------
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2_approx(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Programmatic dependent launch: returns once the preceding kernel of the stream has completed and its
// memory operations are visible (a no-op for a kernel launched without the attribute).
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float tanh_fast(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x));
  return t;
}
__device__ __forceinline__ float sigmoid_fast(float x) {
  // 0.5 tanh(x / 2) + 0.5: one MUFU op (tanh.approx, abs. error ~5e-4, below bf16 resolution of the
  // gated values) instead of ex2 + rcp
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  return fmaf(t, 0.5f, 0.5f);
}
// Packed fp32 pairs (sm_100 executes two fp32 FMAs / adds per instruction) and 3-input max.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ uint64_t f2_pack_bits(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// 16-byte asynchronous copy global -> shared (no registers in between); `valid` false writes zeros.
__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc, bool valid) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc),
               "r"(valid ? 16 : 0)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Four 8x8 matrices of 16-bit elements from shared memory, each transposed on the way: lanes 8m..8m+7
// give the addresses of the eight 16-byte rows of matrix m; lane T receives, in r[m], the elements
// [2 (T % 4)][T / 4] (low half) and [2 (T % 4) + 1][T / 4] (high half) of the stored matrix m.
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr)
               : "memory");
}
// The inverse direction: lane T holds, in r[m], the elements [T / 4][2 (T % 4)] and [T / 4][2 (T % 4) + 1]
// of a matrix whose TRANSPOSE is written to the eight 16-byte rows addressed by lanes 8m..8m+7.
__device__ __forceinline__ void stmatrix_x4_trans(uint32_t smem_addr, const uint32_t (&r)[4]) {
  asm volatile("stmatrix.sync.aligned.m8n8.x4.trans.shared.b16 [%0], {%1,%2,%3,%4};" ::"r"(smem_addr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3])
               : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

}  // namespace tpf

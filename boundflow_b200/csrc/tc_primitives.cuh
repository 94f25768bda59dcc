// PTX wrappers shared by the tcgen05 kernels: mbarriers with bounded waits, bulk asynchronous
// copies, shared-memory matrix descriptors (K-major, 128-byte swizzle), TF32 MMA issue / commit
// and tensor-memory loads.
#pragma once
#include <stdint.h>

#include "common.cuh"

namespace bf {
namespace tc {

constexpr long long WAIT_LIMIT = 4000000000LL;  // clock cycles (~2 s) before a wait gives up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
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
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when another thread aborted or the limit was reached.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > WAIT_LIMIT) {
      *abort_flag = 1;
      return false;
    }
  }
  return true;
}
// Warp-collective bounded wait: lane 0 polls the barrier, every lane receives the outcome.  The warp leaves
// converged (the instructions that follow a wait are often .sync.aligned: tcgen05.ld, shuffles) and only one
// thread per warp spends shared-memory bandwidth on polling.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
  ok = __shfl_sync(0xffffffffu, ok, 0);
  return ok != 0;
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
               "r"(bytes), "r"(bar)
               : "memory");
}
// Teardown after an abort: waits (clock-bounded) until the bulk copies this thread issued into a `stages`-deep ring
// have landed, so that the CTA does not release shared memory that a copy is still writing.  Copy number j used
// stage j % stages in barrier phase (j / stages) & 1; only the last `stages` copies can still be in flight.  The
// calling thread armed those phases itself (arrive.expect_tx), so a stage's barrier cannot move past the awaited
// phase while this runs and try_wait on that phase's parity answers "completed" exactly when the bytes are in.
__device__ __forceinline__ void drain_bulk_copies(unsigned long long* full_bars, int stages, int issued) {
  for (int j = (issued > stages ? issued - stages : 0); j < issued; ++j) {
    const uint32_t bar = smem_u32(&full_bars[j % stages]);
    const uint32_t parity = (uint32_t)(j / stages) & 1u;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity) && clock64() - t0 < 200000000LL) {
    }
  }
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  // K-major, 128-byte swizzle: rows of 128 B, 8-row groups 1024 B apart (SBO), LBO unused (= 1), descriptor version 1.
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  const uint32_t z = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(z), "r"(z), "r"(z), "r"(z)
      : "memory");
}
// The twelve MMAs of one 32-wide k-block of a 3xTF32 product D += A * B (four 8-wide k-slices x {a_lo*b_hi,
// a_hi*b_lo, a_hi*b_hi}) as ONE instruction sequence.  The issuing thread's chain of dependent instructions is what
// limits the MMA rate next to sixteen busy producer warps, so nothing is recomputed here: the caller passes the
// descriptors of the first slice (stage base, built once per stage with plain adds on a base descriptor) and each
// further slice is 32 bytes = 2 descriptor units on; one predicate says whether the very first MMA accumulates.
__device__ __forceinline__ void mma_kblock_3xtf32(uint32_t tmem_d, uint64_t a_hi, uint64_t a_lo, uint64_t b_hi, uint64_t b_lo,
                                                  uint32_t idesc, uint32_t accumulate_first) {
  const uint32_t z = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred pacc, pone;\n\t"
      ".reg .b64 ah, al, bh, bl;\n\t"
      "setp.ne.b32 pacc, %6, 0;\n\t"
      "setp.eq.b32 pone, %7, %7;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %2, %3, %5, {%7, %7, %7, %7}, pacc;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %4, %5, {%7, %7, %7, %7}, pone;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %3, %5, {%7, %7, %7, %7}, pone;\n\t"
      "add.u64 ah, %1, 2;\n\t"
      "add.u64 al, %2, 2;\n\t"
      "add.u64 bh, %3, 2;\n\t"
      "add.u64 bl, %4, 2;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], al, bh, %5, {%7, %7, %7, %7}, pone;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], ah, bl, %5, {%7, %7, %7, %7}, pone;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], ah, bh, %5, {%7, %7, %7, %7}, pone;\n\t"
      "add.u64 ah, %1, 4;\n\t"
      "add.u64 al, %2, 4;\n\t"
      "add.u64 bh, %3, 4;\n\t"
      "add.u64 bl, %4, 4;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], al, bh, %5, {%7, %7, %7, %7}, pone;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], ah, bl, %5, {%7, %7, %7, %7}, pone;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], ah, bh, %5, {%7, %7, %7, %7}, pone;\n\t"
      "add.u64 ah, %1, 6;\n\t"
      "add.u64 al, %2, 6;\n\t"
      "add.u64 bh, %3, 6;\n\t"
      "add.u64 bl, %4, 6;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], al, bh, %5, {%7, %7, %7, %7}, pone;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], ah, bl, %5, {%7, %7, %7, %7}, pone;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], ah, bh, %5, {%7, %7, %7, %7}, pone;\n\t"
      "}"
      ::"r"(tmem_d), "l"(a_hi), "l"(a_lo), "l"(b_hi), "l"(b_lo), "r"(idesc), "r"(accumulate_first), "r"(z)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// ---- CTA pairs (thread-block clusters of two, tcgen05 cta_group::2) ----
// The same twelve MMAs issued by the leader CTA of a pair: 256 accumulator rows (128 in each CTA's tensor memory), each
// CTA's tensor core reads its own A tile and its own half of the B rows from its own shared memory at the offsets the
// descriptors name, so every operand byte is read once per pair instead of once per CTA.
__device__ __forceinline__ void mma_kblock_3xtf32_pair(uint32_t tmem_d, uint64_t a_hi, uint64_t a_lo, uint64_t b_hi, uint64_t b_lo,
                                                  uint32_t idesc, uint32_t accumulate_first) {
  const uint32_t z = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred pacc, pone;\n\t"
      ".reg .b64 ah, al, bh, bl;\n\t"
      "setp.ne.b32 pacc, %6, 0;\n\t"
      "setp.eq.b32 pone, %7, %7;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %2, %3, %5, {%7, %7, %7, %7, %7, %7, %7, %7}, pacc;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %4, %5, {%7, %7, %7, %7, %7, %7, %7, %7}, pone;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %3, %5, {%7, %7, %7, %7, %7, %7, %7, %7}, pone;\n\t"
      "add.u64 ah, %1, 2;\n\t"
      "add.u64 al, %2, 2;\n\t"
      "add.u64 bh, %3, 2;\n\t"
      "add.u64 bl, %4, 2;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], al, bh, %5, {%7, %7, %7, %7, %7, %7, %7, %7}, pone;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], ah, bl, %5, {%7, %7, %7, %7, %7, %7, %7, %7}, pone;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], ah, bh, %5, {%7, %7, %7, %7, %7, %7, %7, %7}, pone;\n\t"
      "add.u64 ah, %1, 4;\n\t"
      "add.u64 al, %2, 4;\n\t"
      "add.u64 bh, %3, 4;\n\t"
      "add.u64 bl, %4, 4;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], al, bh, %5, {%7, %7, %7, %7, %7, %7, %7, %7}, pone;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], ah, bl, %5, {%7, %7, %7, %7, %7, %7, %7, %7}, pone;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], ah, bh, %5, {%7, %7, %7, %7, %7, %7, %7, %7}, pone;\n\t"
      "add.u64 ah, %1, 6;\n\t"
      "add.u64 al, %2, 6;\n\t"
      "add.u64 bh, %3, 6;\n\t"
      "add.u64 bl, %4, 6;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], al, bh, %5, {%7, %7, %7, %7, %7, %7, %7, %7}, pone;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], ah, bl, %5, {%7, %7, %7, %7, %7, %7, %7, %7}, pone;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], ah, bh, %5, {%7, %7, %7, %7, %7, %7, %7, %7}, pone;\n\t"
      "}"
      ::"r"(tmem_d), "l"(a_hi), "l"(a_lo), "l"(b_hi), "l"(b_lo), "r"(idesc), "r"(accumulate_first), "r"(z)
      : "memory");
}
// arrives on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void mma_commit_pair(uint32_t bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(both)
               : "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// all threads of both CTAs; also orders shared-memory writes (barrier initialisation) before the peer's accesses
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ float tf32_rna(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}
// x rounded to TF32 precision (10 explicit mantissa bits), to nearest with ties away from zero -- what
// cvt.rna.tf32.f32 computes for finite values -- by two integer operations; the producers need eight roundings
// per loaded float4 and the conversion instruction runs on a slower pipe than the integer ALU.
__device__ __forceinline__ float tf32_round(float x) { return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u); }
__device__ __forceinline__ float sgnf(float a) { return (a > 0.f) ? 1.f : ((a < 0.f) ? -1.f : 0.f); }

}  // namespace tc
}  // namespace bf

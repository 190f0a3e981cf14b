// Thin inline-PTX wrappers for the sm_100a features the tensor-core kernels use:
// mbarriers, TMA (cp.async.bulk.tensor, never multicast), tcgen05 (TMEM
// allocation, MMA, commit, load), and the shared-memory / instruction descriptors
// tcgen05.mma consumes.  Device code only.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace elman {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// ------------------------------ mbarrier -----------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count)
               : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Same, with a suspend-time hint: the hardware may park the thread until the phase
// completes or the hint (in ns) expires instead of returning at once, which keeps a
// waiting warp from competing for issue slots with the warps doing the work.
__device__ __forceinline__ bool mbar_try_wait_suspend(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(20000u)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
constexpr unsigned long long kWaitDeadlineNs = 2000000000ull;  // 2 s wall-clock cap per wait

// Bounded wait.  `abort_flag` is a shared-memory word any thread of the CTA may set;
// returns false when the iteration limit or the wall-clock cap ran out, or the flag
// was raised.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, long limit,
                                          volatile int* abort_flag) {
  long spins = 0;
  unsigned long long t0 = 0;
  while (!mbar_try_wait(bar, parity)) {
    if (++spins > limit || *abort_flag != 0) return false;
    if ((spins & 1023) == 0) {
      unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitDeadlineNs) return false;
    }
  }
  return true;
}

// ------------------------------ fences --------------------------------------
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ------------------------------ TMA -----------------------------------------
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
// 2D tile load global -> shared, completion on an mbarrier of this CTA.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, int c0, int c1,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(m), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

// ------------------------------ TMEM ----------------------------------------
// Warp-collective: allocate `ncols` (power of two >= 32) TMEM columns; the base
// address is written to *smem_slot.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_slot)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

// ------------------------------ descriptors ---------------------------------
// Shared-memory matrix descriptor for a K-major bf16 tile written by TMA with
// 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
// The tile base must be 1024-byte aligned; stepping 16 elements along K adds
// 32 bytes to the start address.
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);  // start address
  d |= (uint64_t)1 << 16;                      // leading byte offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;            // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                      // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                      // SWIZZLE_128B
  return d;
}

// Shared-memory matrix descriptor for an MN-major bf16 operand: the tile is stored as
// rows of K, each row holding 64 consecutive M (or N) elements = 128 bytes, written by
// TMA with 128-byte swizzle from a [K, MN] row-major matrix.  Groups of 8 K rows are
// 1024 bytes apart (stride byte offset); the next block of 64 MN elements starts
// `mn_block_bytes` further on (leading byte offset).  One K=16 MMA step covers two
// 8-row groups: stepping 16 along K adds 2048 bytes to the start address.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t mn_block_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((mn_block_bytes >> 4) & 0x3FFF) << 16;  // leading byte offset
  d |= (uint64_t)(1024 >> 4) << 32;                       // stride byte offset
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// K-major bf16 tile whose rows are 64 bytes (32 elements) with 64-byte swizzle: groups of 8
// rows are 512 bytes apart; within a row the 16-byte chunk index is XORed with bits 1..2 of
// the row index.  Used for operands assembled on chip from 32-column pieces.
__device__ __forceinline__ uint64_t umma_desc_k_sw64(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(512 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)4 << 61;                      // SWIZZLE_64B
  return d;
}

// Instruction descriptor: kind::f16, A and B bf16 K-major, fp32 accumulate.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) |
         ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier when all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// Load 32 consecutive fp32 columns of this thread's TMEM lane (warp-collective:
// the warp reads lanes [32*(warp%4), +32), thread i gets lane base+i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// Store 16 consecutive 32-bit columns of this thread's TMEM lane (warp-collective,
// same lane mapping as tmem_ld16).
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: the A operand (M=128 rows in the 128 lanes, K=16 bf16
// packed two per 32-bit column = 8 columns) is read from tensor memory.
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ------------------------------ CTA pairs (cta_group::2) --------------------
// Two CTAs of a cluster (ranks 2k, 2k+1) act as one MMA unit: M = 256 rows, each CTA holds
// its 128 rows of A, its half of B's N columns and its 128 rows of the accumulator (same
// TMEM columns in both).  One thread of the even CTA issues the MMAs and the commits.
// The allocation calls are made by the same warp of BOTH CTAs.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_slot)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
// 2D tile load into THIS CTA's shared memory whose byte count is credited to an mbarrier
// given as a shared::cluster address (the even CTA's barrier, for both CTAs of the pair).
// No multicast: each CTA fetches its own tile.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, int c0,
                                                 int c1, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(m), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One ring stage of the CTA-pair main loop as a single instruction sequence: test the NEXT
// stage's barrier first, issue this stage's four K=16 MMAs, commit them to this stage's
// "free" barrier in both CTAs, and only then read the test's result.  An MMA costs its issuing
// thread about as long as it runs, so whatever else that thread does between MMAs is time
// the tensor pipe idles; the barrier test's latency is spent under the MMAs this way.
__device__ __forceinline__ bool umma_stage_pair(uint32_t tmem_d, uint64_t da, uint64_t db,
                                                uint64_t a_step, uint64_t b_step, uint32_t idesc,
                                                uint32_t accumulate_first, uint64_t* free_bar,
                                                uint64_t* next_full_bar, uint32_t next_parity) {
  uint32_t ready;
  asm volatile(
      "{\n\t.reg .pred pw, pa, pt;\n\t"
      ".reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
      "tcgen05.fence::after_thread_sync;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 pw, [%9], %10;\n\t"
      "setp.ne.b32 pa, %6, 0;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "add.u64 a1, %2, %4;\n\t"
      "add.u64 b1, %3, %5;\n\t"
      "add.u64 a2, a1, %4;\n\t"
      "add.u64 b2, b1, %5;\n\t"
      "add.u64 a3, a2, %4;\n\t"
      "add.u64 b3, b2, %5;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%1], %2, %3, %7, pa;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%1], a1, b1, %7, pt;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%1], a2, b2, %7, pt;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%1], a3, b3, %7, pt;\n\t"
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%8], %11;\n\t"
      "selp.b32 %0, 1, 0, pw;\n\t}"
      : "=r"(ready)
      : "r"(tmem_d), "l"(da), "l"(db), "l"(a_step), "l"(b_step), "r"(accumulate_first),
        "r"(idesc), "r"(smem_u32(free_bar)), "r"(smem_u32(next_full_bar)), "r"(next_parity),
        "h"((uint16_t)3)
      : "memory");
  return ready != 0;
}
// Arrive on the mbarrier at the same shared-memory offset in every CTA of `cta_mask` when
// all MMAs issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(smem_u32(bar)), "h"(cta_mask)
      : "memory");
}
// Arrive on an mbarrier of another CTA of the cluster (address from mapa).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

}  // namespace ptx

// Host side: build a 2D bf16 tensor map with 128-byte swizzle over a row-major
// matrix [rows, cols] with row stride `ld` elements; box = box_rows x 64 columns.
int make_tmap_bf16_sw128(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                         uint64_t ld, uint32_t box_rows);

}  // namespace elman

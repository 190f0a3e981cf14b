// Device helpers shared by the cluster kernels: distributed-shared-memory stores
// with mbarrier byte credits, cluster-scope mbarrier operations, bulk tensor stores,
// bounded waits, and the fast activation math of the bf16 epilogues.
#pragma once

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace elman {
namespace tch {

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
// 16-byte store into a peer's shared memory that credits 16 bytes to an mbarrier of
// that peer when it lands (no fence, no separate arrive on the sender's side).
__device__ __forceinline__ void st_async_v4(uint32_t remote_addr, uint32_t a, uint32_t b, uint32_t c,
                                            uint32_t d, uint32_t remote_bar) {
  asm volatile(
      "st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
      ::"r"(remote_addr), "r"(a), "r"(b), "r"(c), "r"(d), "r"(remote_bar)
      : "memory");
}
__device__ __forceinline__ float4 lds_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds_u4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts_u16(uint32_t addr, unsigned short v) {
  asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr), "h"(v) : "memory");
}
__device__ __forceinline__ unsigned short lds_u16(uint32_t addr) {
  unsigned short v;
  asm volatile("ld.shared.b16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(ptx::smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ------------------------- bulk tensor (TMA) stores ------------------------
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, const void* smem_src, int c0,
                                             int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(m), "r"(ptx::smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int c0,
                                             int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(m), "r"(ptx::smem_u32(smem_src)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, int c0, int c1,
                                            int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(ptx::smem_u32(smem_dst)), "l"(m), "r"(ptx::smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// Bulk copy from this CTA's shared memory into a cluster peer's, crediting `bytes` to an
// mbarrier of that peer when the data has landed (16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void bulk_copy_to_peer(uint32_t dst_cluster_addr, uint32_t src_cta_addr,
                                                  uint32_t bytes, uint32_t peer_bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst_cluster_addr), "r"(src_cta_addr), "r"(bytes), "r"(peer_bar_cluster_addr)
      : "memory");
}
__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_read_all() {  // sources may be overwritten
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_all() {  // writes are complete
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// ------------------------------ bounded waits -------------------------------
struct Waiter {
  long limit;
  volatile int* local_abort;
  const int* global_abort;
  __device__ __forceinline__ bool give_up(long& spins, unsigned long long& t0) const {
    ++spins;
    if (spins > limit || *local_abort != 0) return true;
    if ((spins & 255) == 0) {
      if (ld_relaxed_gpu(global_abort) != 0) return true;
      unsigned long long now = ptx::globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > ptx::kWaitDeadlineNs) return true;
    }
    return false;
  }
  __device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity) const {
    long spins = 0;
    unsigned long long t0 = 0;
    while (!ptx::mbar_try_wait_suspend(bar, parity))
      if (give_up(spins, t0)) return false;
    return true;
  }
  __device__ __forceinline__ bool wait_cluster(uint64_t* bar, uint32_t parity) const {
    long spins = 0;
    unsigned long long t0 = 0;
    while (!mbar_try_wait_cluster(bar, parity))
      if (give_up(spins, t0)) return false;
    return true;
  }
};

// ------------------------------ epilogue math -------------------------------
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float sigmoid_fast(float z) { return __fdividef(1.f, 1.f + __expf(-z)); }
// 1 - tanh(v)^2 without cancellation: 4u/(1+u)^2 with u = exp(-2|v|)
__device__ __forceinline__ float dtanh_from_v(float v) {
  const float u = __expf(-2.f * fabsf(v));
  const float r = __fdividef(1.f, 1.f + u);
  return 4.f * u * r * r;
}
__device__ __forceinline__ float bf16_bits_to_f(unsigned short u) {
  return __uint_as_float(((uint32_t)u) << 16);
}
__device__ __forceinline__ unsigned short f_to_bf16_bits(float f) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}

}  // namespace tch
}  // namespace elman

// Two microbenchmarks behind the layout of the recurrence kernels (standalone program, not part of
// the library):
//  1. tcgen05.mma issue rate for small N (M=128, K=16) with the A operand in shared or in tensor
//     memory and 1, 2 or 4 issuing warps: what one CTA can issue per recurrence step.
//  2. a per-step all-gather of a [32 x d] bf16 state among the CTAs of ONE cluster, three ways:
//     (0) bulk copies shared -> peer shared memory, (1) 16-byte st.async stores, (2) global write,
//     remote mbarrier arrive, bulk load from global memory.  This is the exchange a single-cluster
//     dense recurrence would need every step; the shipped dense kernel exchanges through global
//     step counters across 10 clusters instead, the low-rank kernel uses form (0) for its rank vector.
// Every wait is bounded (400 000 polls, then a flag that ends all loops).
// Build and run:  python -m elman_b200.build --microbench  &&  elman_b200/lib/mma_issue_and_cluster_exchange
#include <cstdio>
#include <cstdlib>
#include <cuda_bf16.h>
#include "../sm100_ptx.cuh"

using namespace elman;

#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); exit(1);} } while (0)

__device__ __forceinline__ bool bwait(uint64_t* bar, uint32_t parity, int* bad) {
  long spins = 0;
  while (!ptx::mbar_try_wait(bar, parity)) {
    if (++spins > 400000 || *(volatile int*)bad) { *bad = 1; return false; }
  }
  return true;
}

// ---------------------------------------------------------------- 1. MMA
__global__ void __launch_bounds__(320) mma_bench(int N, int issuers, int a_tmem, int reps, long long* out) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t done_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int bad;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;                 // [128 x 64] bf16 swizzled tile (contents irrelevant)
  uint8_t* sB = smem + 16384;         // [N x 64]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < (16384 + 256 * 128) / 4; i += blockDim.x) ((uint32_t*)smem)[i] = 0x3c003c00u;
  if (tid == 0) { bad = 0; ptx::mbar_init(&done_bar, issuers); ptx::mbar_fence_init(); }
  if (warp == 0) { ptx::tmem_alloc(&tmem_slot, 512); ptx::tmem_relinquish(); }
  ptx::fence_proxy_async_smem();
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tb = tmem_slot;
  long long t0 = 0, t1 = 0, t2 = 0;
  if (warp >= 1 && warp <= issuers && lane == 0) {
    const int mw = warp - 1;
    const uint32_t idesc = ptx::umma_idesc_bf16(128, N);
    const uint32_t d_tmem = tb + 256 + mw * N;      // accumulators in columns [256, 512): issuers * N <= 256
    const uint64_t da0 = ptx::umma_desc_k_sw128(ptx::smem_u32(sA));
    const uint64_t db0 = ptx::umma_desc_k_sw128(ptx::smem_u32(sB));
    t0 = clock64();
    for (int m = mw; m < reps; m += issuers) {
      const int k = m & 3;
      if (a_tmem) ptx::umma_bf16_ts(d_tmem, tb + (uint32_t)((m & 31) * 8), db0 + 2 * k, idesc, m >= issuers);
      else ptx::umma_bf16(d_tmem, da0 + 2 * k, db0 + 2 * k, idesc, m >= issuers);
    }
    ptx::umma_commit(&done_bar);
    t1 = clock64();
    bwait(&done_bar, 0, &bad);
    t2 = clock64();
    out[mw * 2] = t1 - t0;
    out[mw * 2 + 1] = t2 - t0;
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 0) ptx::tmem_dealloc(tb, 512);
}

// ---------------------------------------------------------------- 2. exchange
__device__ __forceinline__ uint32_t mapa(uint32_t a, uint32_t r) {
  uint32_t o; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(o) : "r"(a), "r"(r)); return o;
}
__device__ __forceinline__ uint32_t ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void bulk_s2s(uint32_t dst_cluster, uint32_t src_cta, uint32_t bytes, uint32_t bar_cluster) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_cluster), "r"(src_cta), "r"(bytes), "r"(bar_cluster) : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst_cta, const void* src, uint32_t bytes, uint32_t bar_cta) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_cta), "l"(src), "r"(bytes), "r"(bar_cta) : "memory");
}
__device__ __forceinline__ void st_async_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
               ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d), "r"(bar) : "memory");
}
__device__ __forceinline__ void arrive_remote_release(uint32_t bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(ptx::smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool bwait_cluster(uint64_t* bar, uint32_t parity, int* bad) {
  long spins = 0;
  while (!try_wait_cluster(bar, parity)) {
    if (++spins > 400000 || *(volatile int*)bad) { *bad = 1; return false; }
  }
  return true;
}

// mode 0: bulk smem->peer smem; 1: st.async; 2: global + arrive + bulk load
// slice = bytes each CTA contributes per step (8 KB at d=1280: 128 features x 32 batch x 2 B)
__global__ void __launch_bounds__(160) xchg_bench(int mode, int NC, int slice, int iters, uint8_t* gbuf, long long* out) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full[2];
  __shared__ __align__(8) uint64_t ready[2];
  __shared__ int bad;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* mine = smem;                         // my slice (source)
  uint8_t* buf = smem + 16384;                  // 2 x [NC * slice] gathered state
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t c = ctarank();
  const int total = NC * slice;
  if (tid == 0) {
    bad = 0;
    ptx::mbar_init(&full[0], 1); ptx::mbar_init(&full[1], 1);
    ptx::mbar_init(&ready[0], NC * 4); ptx::mbar_init(&ready[1], NC * 4);
    ptx::mbar_fence_init();
  }
  for (int i = tid; i < slice / 4; i += blockDim.x) ((uint32_t*)mine)[i] = c * 1000 + i;
  __syncthreads();
  cluster_sync();
  long long t0 = clock64();
  // warps 0..3: "epilogue" threads (senders); warp 4: receiver/producer thread
  if (warp < 4) {
    for (int it = 0; it < iters; ++it) {
      const int b = it & 1;
      // everybody needs the whole state of iteration it-1 before producing iteration it
      if (it > 0 && !bwait_cluster(&full[(it - 1) & 1], ((it - 1) >> 1) & 1, &bad)) break;
      if (mode == 0) {
        ptx::fence_proxy_async_smem();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (tid < NC) {
          const uint32_t dst = mapa(ptx::smem_u32(buf + b * total + c * slice), tid);
          bulk_s2s(dst, ptx::smem_u32(mine), slice, mapa(ptx::smem_u32(&full[b]), tid));
        }
      } else if (mode == 1) {
        const uint4* src = (const uint4*)mine;
        for (int r = 0; r < NC; ++r) {
          const uint32_t dst = mapa(ptx::smem_u32(buf + b * total + c * slice), r);
          const uint32_t bar = mapa(ptx::smem_u32(&full[b]), r);
          for (int i = tid; i < slice / 16; i += 128) {
            const uint4 v = src[i];
            st_async_v4(dst + i * 16, v.x, v.y, v.z, v.w, bar);
          }
        }
      } else {
        uint4* g = (uint4*)(gbuf + (size_t)b * total + c * slice);
        const uint4* src = (const uint4*)mine;
        for (int i = tid; i < slice / 16; i += 128) g[i] = src[i];
        __syncwarp();
        if (lane == 0)
          for (int r = 0; r < NC; ++r) arrive_remote_release(mapa(ptx::smem_u32(&ready[b]), r));
      }
    }
  } else if (lane == 0) {
    for (int it = 0; it < iters; ++it) {
      const int b = it & 1;
      if (mode == 2) {
        // all writers' slices are in global memory (their release-arrives), then pull the state
        if (!bwait_cluster(&ready[b], (it >> 1) & 1, &bad)) break;
        asm volatile("fence.proxy.async.global;" ::: "memory");
        ptx::mbar_arrive_expect_tx(&full[b], (uint32_t)total);
        bulk_g2s(ptx::smem_u32(buf + b * total), gbuf + (size_t)b * total, (uint32_t)total, ptx::smem_u32(&full[b]));
      } else {
        ptx::mbar_arrive_expect_tx(&full[b], (uint32_t)total);
      }
      if (!bwait_cluster(&full[b], (it >> 1) & 1, &bad)) break;
    }
  }
  __syncthreads();
  long long t1 = clock64();
  cluster_sync();
  if (tid == 0) { out[c * 2] = t1 - t0; out[c * 2 + 1] = bad; }
}

int main(int argc, char** argv) {
  long long* out;
  CK(cudaMallocManaged(&out, 1024));
  CK(cudaFuncSetAttribute(mma_bench, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
  printf("== tcgen05.mma M=128 K=16, cycles for `reps` MMAs: issue-done / all-complete ==\n");
  const int Ns[] = {16, 32, 64, 128, 256};
  for (int a_tmem = 0; a_tmem <= 1; ++a_tmem)
    for (int ni = 0; ni < 5; ++ni)
      for (int issuers = 1; issuers <= 8; issuers *= 2) {
        const int reps = 80;
        if (issuers * Ns[ni] > 256) continue;   // the accumulators must stay inside tensor memory
        for (int rep = 0; rep < 2; ++rep) {
          mma_bench<<<1, 320, 64 * 1024>>>(Ns[ni], issuers, a_tmem, reps, out);
          CK(cudaDeviceSynchronize());
        }
        printf("A=%s N=%3d issuers=%d reps=%d: issue %lld  complete %lld cycles  (%.1f cyc/MMA)\n",
               a_tmem ? "tmem" : "smem", Ns[ni], issuers, reps, out[0], out[1], (double)out[1] / reps);
      }
  // exchange
  uint8_t* gbuf;
  CK(cudaMalloc(&gbuf, 4 << 20));
  CK(cudaFuncSetAttribute(xchg_bench, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  CK(cudaFuncSetAttribute(xchg_bench, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
  printf("== per-step all-gather inside one cluster, cycles per step ==\n");
  const int NCs[] = {4, 8, 10, 16};
  const int slices[] = {2048, 4096, 8192};
  for (int mode = 0; mode < 3; ++mode)
    for (int ci = 0; ci < 4; ++ci)
      for (int si = 0; si < 3; ++si) {
        const int NC = NCs[ci], slice = slices[si], iters = 400;
        if (2 * NC * slice + 16384 + 2048 > 200 * 1024) continue;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(NC); cfg.blockDim = dim3(160);
        cfg.dynamicSmemBytes = 200 * 1024;
        cudaLaunchAttribute attr; attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = NC; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr; cfg.numAttrs = 1;
        int maxc = 0;
        if (cudaOccupancyMaxActiveClusters(&maxc, xchg_bench, &cfg) != cudaSuccess || maxc < 1) {
          cudaGetLastError();
          printf("mode %d NC=%d: cluster not launchable\n", mode, NC);
          continue;
        }
        for (int rep = 0; rep < 2; ++rep) {
          CK(cudaLaunchKernelEx(&cfg, xchg_bench, mode, NC, slice, iters, gbuf, out));
          CK(cudaDeviceSynchronize());
        }
        printf("mode %d (%s) NC=%2d slice=%5d B (state %6d B): %.0f cycles/step, bad=%lld\n", mode,
               mode == 0 ? "bulk smem->smem" : mode == 1 ? "st.async" : "global+bulk load", NC, slice,
               NC * slice, (double)out[0] / iters, out[1]);
      }
  return 0;
}

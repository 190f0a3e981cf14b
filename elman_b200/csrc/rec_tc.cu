// Persistent tensor-core recurrence for the dense Elman cells (E1 / E0), bf16.
//
// Replaces the reference's per-step host loop — one cuBLAS GEMM plus one to three
// elementwise kernels per time step, W_h re-read from L2/HBM every step
// (elman/cuda/lib/mamba_gated_elman_gpu.cu.cc:451-473 forward, :527-558 backward;
// stock_elman_gpu.cu.cc:267-294, :372-405) — by ONE launch that runs all T steps.
//
// Work split.  The recurrent matrix W [d,d] is cut into tiles of 128 rows (output
// features) x Kc columns (Kc = d / S).  CTA (i, j) keeps tile (i, j) resident in
// shared memory for the whole sequence.  The S CTAs that share a row block form a
// thread-block cluster.  Per step and batch group a CTA
//   1. waits until the slice h[:, j*Kc : (j+1)*Kc] of the previous state is
//      complete (a counter in global memory that the producing CTAs bump),
//   2. pulls that slice with TMA (bf16, 128-byte swizzle) into a shared-memory ring,
//   3. issues Kc/16 tcgen05.mma  (M = 128 rows of W, N = batch, K = 16) into a
//      double-buffered accumulator in tensor memory,
//   4. drains the accumulator with tcgen05.ld and scatters the partial sums to the
//      cluster peer that owns each row (distributed shared memory),
//   5. as owner of 128/S rows, adds the S partials, applies the fused epilogue
//      (forward: + W_x x_t + b, tanh, h*silu(z); backward: the tanh / gate
//      derivatives and the running bias gradient) and writes the new state, then
//      bumps the counter.
// Roles are warp-specialised: warp 0 = TMA producer, warps 1..4 = MMA issuers (warp 1
// owns the TMEM allocation), warps 5..8 = drain (step 4), warps 9..12 = finalise
// (step 5), warp 13 = publisher of the step counter.  Independent batch groups are
// pipelined through the same rings, so one group's global round trip, its drain and
// its finalising each overlap another group's math.
//
// Every wait (global counters, mbarriers) is bounded; a wait that gives up raises
// an abort word all CTAs poll, records a status code and the kernel drains and
// returns with tensor memory freed.
#include <cooperative_groups.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace elman {

namespace {

constexpr int TILE_M = 128;
constexpr int NUM_EPI_THREADS = 128;
constexpr int NUM_MMA_WARPS = 4;
constexpr int NUM_DRAIN_THREADS = 128;  // four warps: one per quarter of the TMEM lanes
// FG = number of finalising warp groups: 1 everywhere except the throughput plan with four or
// more batch groups, where two groups alternate over the (step, group) items.
constexpr int threads_for(int fg) {
  return 32 + NUM_MMA_WARPS * 32 + NUM_DRAIN_THREADS + fg * NUM_EPI_THREADS + 32;  // + publisher warp
}
constexpr int NUM_THREADS = threads_for(1);
constexpr int MAX_S = 8;
constexpr int MAX_GROUPS = 16;
constexpr int MAX_QUADS = 2;       // batch quads (4 rows) per epilogue thread and step
constexpr int COUNTER_STRIDE = 32; // ints; one 128-byte line per counter
constexpr int TRACE_STEPS = 64;
constexpr int TRACE_SLOTS = 16;

struct RecTcParams {
  int T, B, d;
  int S;        // K split = cluster size
  int Kc;       // d / S
  int G;        // batch groups
  int Ng;       // batch rows per group
  int Npad;     // Ng rounded up to 16 (MMA N)
  int nstages;  // state ring depth
  int R;        // d / 128: producers per K slice and step
  int reps;     // batch replicas of the whole grid (independent: they never wait on each other)
  int Brep;     // batch rows per replica (= G * Ng)
  int direct_publish;  // 1: each epilogue warp releases the step counter itself
  int w_tmem;          // 1: the resident tile of W lives in tensor memory (A operand from TMEM)
  uint32_t w_col0;     // first TMEM column of that tile
  const bf16* Wg;      // W in global memory (row-major [d,d]) for the one-time load
  int nmw;      // MMA-issuing warps (independent accumulator chains)
  uint32_t tmem_cols;
  // forward
  const bf16* pre; const bf16* g; bf16* h; bf16* y; bf16* v;
  // backward
  const bf16* h_in; const bf16* v_in; const bf16* dy; bf16* dv; bf16* dg; float* db;
  int* ready;       // [G][S] counters, COUNTER_STRIDE ints apart
  int* abort_word;  // global abort flag
  int* status;
  long spin_limit;
  int self_gate;      // 1: no gate input, the new state gates itself (y = h silu(h))
  int stall_step;     // test hook: block 0 waits at this step for a count nobody publishes (-1 off)
  long long* trace;   // optional [TRACE_STEPS][TRACE_SLOTS] cycle stamps of CTA 0, or null
};

// ------------------------- cluster / DSMEM helpers -------------------------
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
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
// Store to a peer's shared memory that also credits `bytes` to an mbarrier in the
// same peer when the data has landed: data and signal travel together, so the
// sender needs neither a fence nor a separate arrive.
__device__ __forceinline__ void st_async_f32(uint32_t remote_addr, float v, uint32_t remote_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
               ::"r"(remote_addr), "r"(__float_as_uint(v)), "r"(remote_bar)
               : "memory");
}
__device__ __forceinline__ void st_async_v4(uint32_t remote_addr, uint32_t a, uint32_t b, uint32_t c,
                                            uint32_t d, uint32_t remote_bar) {
  asm volatile(
      "st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
      ::"r"(remote_addr), "r"(a), "r"(b), "r"(c), "r"(d), "r"(remote_bar)
      : "memory");
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ float4 lds_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(addr));
  return v;
}
__device__ __forceinline__ void mbar_arrive_remote_relaxed(uint32_t remote_bar_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar_addr)
               : "memory");
}
__device__ __forceinline__ float2 lds_f2(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ void fence_acq_rel_cluster() {
  asm volatile("fence.acq_rel.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t remote_bar_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar_addr)
               : "memory");
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
__device__ __forceinline__ void epi_bar_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(NUM_EPI_THREADS) : "memory");
}
// Barrier over the threads of one finalising group (named barrier 1 + group) that also
// ORs a predicate: every thread gets the same answer, so they can leave a loop together.
__device__ __forceinline__ bool epi_bar_or(bool pred, int group) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "bar.red.or.pred q, %3, %2, p;\n\t"
      "selp.b32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)pred), "n"(NUM_EPI_THREADS), "r"(1 + group)
      : "memory");
  return r != 0;
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, int c0, int c1,
                                            int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(ptx::smem_u32(smem_dst)), "l"(m), "r"(ptx::smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// Cycle stamps of CTA 0 for the first TRACE_STEPS virtual steps (diagnostics only).
__device__ __forceinline__ void stamp(long long* trace, int q, int slot) {
  if (trace != nullptr && blockIdx.x == 0 && q < TRACE_STEPS)
    trace[q * TRACE_SLOTS + slot] = clock64();
}

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* m, int c0, int c1,
                                            int c2, int c3, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(ptx::smem_u32(smem_dst)), "l"(m), "r"(ptx::smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
        "r"(c3)
      : "memory");
}
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}

struct Waiter {
  long limit;
  volatile int* local_abort;
  const int* global_abort;
  // Shared bookkeeping of the three wait flavours: iteration cap, wall-clock cap,
  // CTA-local abort flag and (less often) the grid-wide abort word.
  __device__ __forceinline__ bool give_up(long& spins, unsigned long long& t0, int gmask) const {
    ++spins;
    if (spins > limit || *local_abort != 0) return true;
    if ((spins & gmask) == 0) {
      if (ld_relaxed_gpu(global_abort) != 0) return true;
      unsigned long long now = ptx::globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > ptx::kWaitDeadlineNs) return true;
    }
    return false;
  }
  // mbarrier wait (CTA scope acquire)
  __device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity) const {
    long spins = 0;
    unsigned long long t0 = 0;
    while (!ptx::mbar_try_wait_suspend(bar, parity))
      if (give_up(spins, t0, 255)) return false;
    return true;
  }
  __device__ __forceinline__ bool wait_cluster(uint64_t* bar, uint32_t parity) const {
    long spins = 0;
    unsigned long long t0 = 0;
    while (!mbar_try_wait_cluster(bar, parity))
      if (give_up(spins, t0, 255)) return false;
    return true;
  }
  __device__ __forceinline__ bool wait_counter(const int* ctr, int target) const {
    long spins = 0;
    unsigned long long t0 = 0;
    while (ld_acquire_gpu(ctr) < target)
      if (give_up(spins, t0, 15)) return false;
    return true;
  }
};

__device__ __forceinline__ float bf16_bits_to_f(unsigned short u) {
  return __uint_as_float(((uint32_t)u) << 16);
}
__device__ __forceinline__ unsigned short ldg_bf16_bits(const bf16* p) {
  return __ldg(reinterpret_cast<const unsigned short*>(p));
}
__device__ __forceinline__ unsigned short f_to_bf16_bits(float f) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}

// ---------------------------------------------------------------------------
// the kernel
// ---------------------------------------------------------------------------
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
__device__ __forceinline__ float2 bf16x2_to_f2(uint32_t u) {
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u));
}
__device__ __forceinline__ uint32_t f2_to_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t ldg_u32(const bf16* p) {
  return __ldg(reinterpret_cast<const unsigned int*>(p));
}
__device__ __forceinline__ void stg_u32(bf16* p, uint32_t v) {
  *reinterpret_cast<unsigned int*>(p) = v;
}

template <bool BWD, int FG>
__global__ void __launch_bounds__(threads_for(FG), 1)
rec_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmState,
              const __grid_constant__ CUtensorMap tmI0, const __grid_constant__ CUtensorMap tmI1,
              const __grid_constant__ CUtensorMap tmI2, const __grid_constant__ CUtensorMap tmI3,
              RecTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t w_bar;
  __shared__ __align__(8) uint64_t full_bar[4];       // state ring: TMA -> MMA
  __shared__ __align__(8) uint64_t empty_bar[4];      // state ring: MMA -> TMA
  __shared__ __align__(8) uint64_t acc_full_bar[2];   // MMA -> epilogue
  __shared__ __align__(8) uint64_t acc_empty_bar[2];  // epilogue -> MMA
  __shared__ __align__(8) uint64_t red_full_bar[2];   // peers' partials landed (owner side)
  __shared__ __align__(8) uint64_t red_empty_bar[2];  // owners consumed my partials (source side)
  __shared__ __align__(8) uint64_t stored_bar[2];     // epilogue warps stored the new state
  __shared__ __align__(8) uint64_t in_full[2];        // epilogue inputs of a step landed (TMA)
  __shared__ __align__(8) uint64_t in_empty[2];       // ... and were consumed
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ float db_part[2][FG * NUM_EPI_THREADS];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = p.S, Kc = p.Kc, Npad = p.Npad, Ng = p.Ng, G = p.G, nmw = p.nmw;
  const int rows_own = TILE_M / S;
  const uint32_t j = cluster_ctarank();   // K slice index == rank in cluster
  // Batch replicas: the grid is `reps` copies of the (d/128) x S arrangement, copy r working
  // on batch rows [r * Brep, (r+1) * Brep) with step counters of its own.  Sequences are
  // independent, so the copies share nothing but the weights they each load once.
  const int per_rep = (p.d / TILE_M) * S;
  const int rep = blockIdx.x / per_rep;
  const int i = (blockIdx.x - rep * per_rep) / S;   // row block index
  const int b0 = rep * p.Brep;                      // first batch row of this replica
  int* const ready = p.ready + rep * G * MAX_S * COUNTER_STRIDE;
  const int nkt = Kc / 64;                // 64-column tiles per K slice
  const int total_q = p.T * G;

  // dynamic shared memory carve-up (1024-byte aligned for the swizzled tiles)
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sW = smem;                                    // nkt tiles of [128 x 64] bf16
  const int w_bytes = p.w_tmem ? 0 : TILE_M * Kc * 2;    // W in tensor memory needs no tile here
  uint8_t* sState = sW + w_bytes;                        // nstages x nkt tiles of [Npad x 64]
  const int state_tile_bytes = Npad * 64 * 2;
  const int state_stage_bytes = nkt * state_tile_bytes;
  // partial sums from the S cluster peers: [2 buffers][S sources][Npad batch][rows_own]
  float* sStage = (float*)(sState + p.nstages * state_stage_bytes);
  const int stg_src_floats = Npad * rows_own;
  const int stg_buf_floats = S * stg_src_floats;
  // epilogue inputs of my feature chunk for one (step, batch group), double buffered:
  // [2][NIN arrays][Npad batch rows][rows_own features] bf16, fetched by TMA one step ahead
  constexpr int NIN = BWD ? 4 : 2;
  uint8_t* sIn = (uint8_t*)(sStage + 2 * stg_buf_floats);
  const int in_tile_bytes = Npad * rows_own * 2;
  const uint32_t tmem_cols = p.tmem_cols;

  Waiter waiter{p.spin_limit, &abort_flag, p.abort_word};

  if (tid == 0) {
    abort_flag = 0;
    ptx::mbar_init(&w_bar, 1);
    for (int s = 0; s < 4; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], nmw);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&acc_full_bar[a], nmw);
      ptx::mbar_init(&acc_empty_bar[a], 4);
      ptx::mbar_init(&red_full_bar[a], 1);  // the owner's expect_tx arrive; data credits bytes
      ptx::mbar_init(&red_empty_bar[a], S);
      ptx::mbar_init(&stored_bar[a], NUM_EPI_THREADS / 32);
      ptx::mbar_init(&in_full[a], 1);
      ptx::mbar_init(&in_empty[a], NUM_EPI_THREADS / 32);
    }
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmW);
    ptx::prefetch_tmap(&tmState);
  }
  if (warp == 1) {
    ptx::tmem_alloc(&tmem_slot, tmem_cols);
    ptx::tmem_relinquish();
  }
  if (tid < FG * NUM_EPI_THREADS) { db_part[0][tid] = 0.f; db_part[1][tid] = 0.f; }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  // peers must have initialised their barriers before any remote arrive / store
  cluster_sync_all();
  const uint32_t tmem_base = tmem_slot;
  const int kid = BWD ? KID_REC_TC_BWD : KID_REC_TC_FWD;

  if (p.w_tmem) {
    // One-time load of my tile of W into tensor memory: row m of the tile goes to TMEM
    // lane m, its Kc bf16 values packed two per 32-bit column.  The four drain
    // warps cover the 128 lanes (warp w may touch lanes [32*(w%4), +32)).
    if (warp > NUM_MMA_WARPS && warp <= NUM_MMA_WARPS + NUM_DRAIN_THREADS / 32) {
      const int quarter = warp & 3;
      const int m = quarter * 32 + lane;
      const uint4* src = reinterpret_cast<const uint4*>(p.Wg + (long)(i * TILE_M + m) * p.d +
                                                        (long)j * Kc);
      const uint32_t tw = tmem_base + ((uint32_t)(quarter * 32) << 16) + p.w_col0;
      for (int c = 0; c < Kc / 2; c += 16) {
        uint32_t r[16];
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          const uint4 w4 = __ldg(src + (c >> 2) + v4);
          r[4 * v4] = w4.x; r[4 * v4 + 1] = w4.y; r[4 * v4 + 2] = w4.z; r[4 * v4 + 3] = w4.w;
        }
        ptx::tmem_st16(tw + (uint32_t)c, r);
      }
      ptx::tmem_st_wait();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
  }

  if (warp == 0) {
    // =========================== TMA producer ===============================
    if (lane == 0) {
      // resident tile of W (shared-memory variant)
      if (!p.w_tmem) {
        ptx::mbar_arrive_expect_tx(&w_bar, (uint32_t)w_bytes);
        for (int kk = 0; kk < nkt; ++kk)
          ptx::tma_load_2d(sW + kk * (TILE_M * 128), &tmW, (int)j * Kc + kk * 64, i * TILE_M,
                           &w_bar);
      }
      for (int q = 0; q < total_q; ++q) {
        const int step = q / G, grp = q - step * G;
        const int s = q % p.nstages;
        const uint32_t ph = (uint32_t)(q / p.nstages) & 1u;
        // the epilogue's inputs for this (step, group) do not depend on the recurrence:
        // fetch them now, a whole dependency chain before they are needed
        bool ok = waiter.wait(&in_empty[q & 1], ((uint32_t)(q >> 1) & 1u) ^ 1u);
        if (ok) {
          const int t = BWD ? (p.T - 1 - step) : step;
          const int f0 = i * TILE_M + (int)j * rows_own;
          uint8_t* dst = sIn + (q & 1) * NIN * in_tile_bytes;
          ptx::mbar_arrive_expect_tx(&in_full[q & 1], (uint32_t)(NIN * in_tile_bytes));
          tma_load_3d(dst, &tmI0, f0, b0 + grp * Ng, t, &in_full[q & 1]);
          tma_load_3d(dst + in_tile_bytes, &tmI1, f0, b0 + grp * Ng, t, &in_full[q & 1]);
          if (BWD) {
            tma_load_3d(dst + 2 * in_tile_bytes, &tmI2, f0, b0 + grp * Ng, t + 1, &in_full[q & 1]);
            tma_load_3d(dst + 3 * in_tile_bytes, &tmI3, f0, b0 + grp * Ng, t, &in_full[q & 1]);
          }
        }
        ok = ok && waiter.wait(&empty_bar[s], ph ^ 1u);
        if (ok && step > 0)
          ok = waiter.wait_counter(ready + (grp * MAX_S + (int)j) * COUNTER_STRIDE,
                                   step * p.R * (p.direct_publish ? NUM_EPI_THREADS / 32 : 1) +
                                       ((step == p.stall_step && blockIdx.x == 0) ? (1 << 28) : 0));
        if (!ok) {
          if (atomicExch(p.abort_word, 1) == 0) report_timeout(p.status, kid, step);
          abort_flag = 1;
          break;
        }
        stamp(p.trace, q, 0);  // dependency satisfied
        // data written by other SMs through the generic proxy -> read by TMA
        fence_proxy_async_global();
        stamp(p.trace, q, 11);  // proxy fence done
        const int slot = BWD ? (p.T - step) : step;  // time index of the input state
        ptx::mbar_arrive_expect_tx(&full_bar[s], (uint32_t)state_stage_bytes);
        // one 4-D box: all nkt 64-column tiles of my K slice for this batch group
        tma_load_4d(sState + s * state_stage_bytes, &tmState, 0, b0 + grp * Ng, (int)j * nkt, slot,
                    &full_bar[s]);
        stamp(p.trace, q, 1);  // loads issued
      }
    }
    __syncwarp();
  } else if (warp <= NUM_MMA_WARPS) {
    // ====================== MMA issuers (warps 1..nmw) =======================
    // MMA number m of a step (tile m/4, 16-wide K chunk m%4) is issued by MMA warp
    // m % nmw into that warp's own accumulator: nmw short dependent chains run
    // concurrently instead of one long one; the epilogue adds the nmw accumulators.
    const int mw = warp - 1;
    if (lane == 0 && mw < nmw) {
      const uint32_t idesc = ptx::umma_idesc_bf16(TILE_M, Npad);
      const int nmma = nkt * 4;
      bool ok = p.w_tmem ? true : waiter.wait(&w_bar, 0);
      for (int q = 0; q < total_q && ok; ++q) {
        const int s = q % p.nstages;
        const uint32_t ph = (uint32_t)(q / p.nstages) & 1u;
        const int a = q & 1;
        const uint32_t aph = (uint32_t)(q >> 1) & 1u;
        ok = waiter.wait(&acc_empty_bar[a], aph ^ 1u) && waiter.wait(&full_bar[s], ph);
        if (!ok) break;
        if (mw == 0) stamp(p.trace, q, 2);  // state tile landed
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)((a * nmw + mw) * Npad);
        const uint32_t w0 = ptx::smem_u32(sW);
        const uint32_t s0 = ptx::smem_u32(sState + s * state_stage_bytes);
        for (int m = mw; m < nmma; m += nmw) {
          const int kk = m >> 2, k = m & 3;
          const uint64_t db = ptx::umma_desc_k_sw128(s0 + kk * state_tile_bytes) + 2 * k;
          if (p.w_tmem) {  // 16 bf16 of K = 8 columns of the tile in tensor memory
            ptx::umma_bf16_ts(d_tmem, tmem_base + p.w_col0 + (uint32_t)(m * 8), db, idesc,
                              m >= nmw ? 1u : 0u);
          } else {
            const uint64_t da = ptx::umma_desc_k_sw128(w0 + kk * (TILE_M * 128)) + 2 * k;
            ptx::umma_bf16(d_tmem, da, db, idesc, m >= nmw ? 1u : 0u);
          }
        }
        ptx::umma_commit(&empty_bar[s]);
        ptx::umma_commit(&acc_full_bar[a]);
        if (mw == 0) stamp(p.trace, q, 3);  // MMAs issued
      }
      if (!ok) {
        if (abort_flag == 0 && atomicExch(p.abort_word, 1) == 0) report_timeout(p.status, kid, 0xFFFFF1);
        abort_flag = 1;
      }
    }
    __syncwarp();
  } else if (warp <= NUM_MMA_WARPS + NUM_DRAIN_THREADS / 32) {
    // ============================ drain ======================================
    // Reads the finished accumulators out of tensor memory, adds the nmw chains and
    // scatters each row to the shared memory of the CTA that finalises it.  A role of
    // its own so that, with several batch groups in flight, the scatter of one group
    // overlaps the finalising of the previous one.
    const int quarter = warp & 3;            // TMEM lane quarter this warp may read
    const int m = quarter * 32 + lane;       // accumulator row held by this thread
    const int owner = m / rows_own;          // cluster rank that finalises row m
    const int m_local = m - owner * rows_own;
    const bool tracer = (warp == NUM_MMA_WARPS + 1 && lane == 0);
    const uint32_t stage_local = ptx::smem_u32(sStage);
    for (int q = 0; q < total_q; ++q) {
      const int a = q & 1;
      const uint32_t aph = (uint32_t)(q >> 1) & 1u;
      bool good = waiter.wait(&acc_full_bar[a], aph) &&
                  waiter.wait_cluster(&red_empty_bar[a], aph ^ 1u);
      good = __all_sync(0xffffffffu, good);
      if (tracer) stamp(p.trace, q, 4);  // accumulator complete
      if (!good) {
        if (abort_flag == 0 && atomicExch(p.abort_word, 1) == 0)
          report_timeout(p.status, kid, 0xFFFFF2);
        abort_flag = 1;
        break;
      }
      ptx::tc_fence_after();
      // staging layout at the owner: [source][batch quad][row][4 batch values];
      // a warp's 16-byte stores for one quad cover 32 consecutive rows = 512 bytes
      const uint32_t remote =
          mapa(stage_local + (uint32_t)((a * S + (int)j) * stg_src_floats + m_local * 4) * 4u,
               (uint32_t)owner);
      const uint32_t remote_bar = mapa(ptx::smem_u32(&red_full_bar[a]), (uint32_t)owner);
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) +
                             (uint32_t)(a * nmw * Npad);
      for (int c = 0; c < Npad; c += 16) {
        // all accumulators of this column chunk in flight at once, one wait
        uint32_t r[16], rb[16], rc[16], rd[16];
        ptx::tmem_ld16(taddr + (uint32_t)c, r);
        if (nmw > 1) ptx::tmem_ld16(taddr + (uint32_t)(Npad + c), rb);
        if (nmw > 2) ptx::tmem_ld16(taddr + (uint32_t)(2 * Npad + c), rc);
        if (nmw > 3) ptx::tmem_ld16(taddr + (uint32_t)(3 * Npad + c), rd);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          float acc = __uint_as_float(r[k]);
          if (nmw > 1) acc += __uint_as_float(rb[k]);
          if (nmw > 2) acc += __uint_as_float(rc[k]);
          if (nmw > 3) acc += __uint_as_float(rd[k]);
          r[k] = __float_as_uint(acc);
        }
#pragma unroll
        for (int k = 0; k < 16; k += 4)
          if (c + k < Ng)
            st_async_v4(remote + (uint32_t)(((c + k) >> 2) * rows_own * 4) * 4u, r[k], r[k + 1],
                        r[k + 2], r[k + 3], remote_bar);
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&acc_empty_bar[a]);
      if (tracer) stamp(p.trace, q, 5);  // partials scattered
    }
    __syncwarp();
  } else if (warp <= NUM_MMA_WARPS + (NUM_DRAIN_THREADS + FG * NUM_EPI_THREADS) / 32) {
    // ============================ finalise ===================================
    // FG groups of four warps; group fg takes the items q with q % FG == fg.  With FG = 2 that
    // is also the index of the double-buffered staging area, input tiles and barriers, so the
    // groups share nothing and one finalises while the other prepares or stores.
    const int ft = tid - (1 + NUM_MMA_WARPS) * 32 - NUM_DRAIN_THREADS;
    const int fg = ft / NUM_EPI_THREADS;
    const int et = ft - fg * NUM_EPI_THREADS;   // 0..127 within the group
    // finalise mapping: this thread owns the feature pair fp of my chunk for the
    // batch quads qd0, qd0 + nbq, ... (a quad = 4 consecutive batch rows)
    const int pairs = rows_own / 2;
    const int nbq = NUM_EPI_THREADS / pairs;
    const int fp = et % pairs;
    const int qd0 = et / pairs;
    const int nquads = (Ng + 3) / 4;
    const int f = i * TILE_M + (int)j * rows_own + 2 * fp;  // first feature of the pair
    const int my_kslice = (i * TILE_M + (int)j * rows_own) / Kc;
    const uint32_t stage_local = ptx::smem_u32(sStage);
    const long BD = (long)p.B * p.d;
    float db0 = 0.f, db1 = 0.f;

    // raw prefetched inputs of the next step, and the values derived from them
    const uint32_t in_a = ptx::smem_u32(sIn);
    float2 e0[MAX_QUADS][4], e1[MAX_QUADS][4];
    uint32_t late0[MAX_QUADS][4], late1[MAX_QUADS][4];  // outputs nobody waits for
    // element offsets inside one (time step, batch group) block; -1 marks padding
    int eoff[MAX_QUADS][4];
#pragma unroll
    for (int e = 0; e < MAX_QUADS; ++e)
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int b = 4 * (qd0 + e * nbq) + u;
        eoff[e][u] = b < Ng ? b * p.d + f : -1;
      }
    auto block_base = [&](int q) -> long {
      const int step = q / G, grp = q - step * G;
      const int t = BWD ? (p.T - 1 - step) : step;
      return ((long)t * p.B + b0 + (long)grp * Ng) * p.d;
    };
    // everything that does not depend on the recurrent term
    auto premath = [&](int q) {
      const uint32_t tile0 = in_a + (uint32_t)((q & 1) * NIN * in_tile_bytes + 4 * fp);
#pragma unroll
      for (int e = 0; e < MAX_QUADS; ++e) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (eoff[e][u] >= 0) {
            const uint32_t ia = tile0 + (uint32_t)((4 * (qd0 + e * nbq) + u) * rows_own * 2);
            if (!BWD) {
              e0[e][u] = bf16x2_to_f2(lds_u32(ia));
              const float2 gz = bf16x2_to_f2(lds_u32(ia + in_tile_bytes));
              e1[e][u] = make_float2(gz.x * sigmoid_fast(gz.x), gz.y * sigmoid_fast(gz.y));
            } else {
              float2 gz = bf16x2_to_f2(lds_u32(ia));
              const float2 dy = bf16x2_to_f2(lds_u32(ia + in_tile_bytes));
              const float2 hv = bf16x2_to_f2(lds_u32(ia + 2 * in_tile_bytes));
              const float2 vv = bf16x2_to_f2(lds_u32(ia + 3 * in_tile_bytes));
              if (p.self_gate) gz = hv;
              const float sx = sigmoid_fast(gz.x), sy = sigmoid_fast(gz.y);
              const float gx = dy.x * hv.x * sx * (1.f + gz.x * (1.f - sx));
              const float gy = dy.y * hv.y * sy * (1.f + gz.y * (1.f - sy));
              late0[e][u] = f2_to_bf16x2(gx, gy);
              e0[e][u] = make_float2(dy.x * gz.x * sx, dy.y * gz.y * sy);
              if (p.self_gate) {   // d(h silu(h))/dh = silu(h) + h silu'(h)
                e0[e][u].x += gx;
                e0[e][u].y += gy;
              }
              e1[e][u] = make_float2(dtanh_from_v(vv.x), dtanh_from_v(vv.y));
            }
          }
        }
      }
    };

    for (int q = fg; q < total_q; q += FG) {
      const int step = q / G;
      const long base_q = block_base(q);
      const int a = q & 1;
      const uint32_t aph = (uint32_t)(q >> 1) & 1u;
      if (et == 0)  // arm this step's reduction barrier with the bytes all S sources will send me
        ptx::mbar_arrive_expect_tx(&red_full_bar[a], (uint32_t)(S * rows_own * nquads * 16));
      // everything that does not need the recurrent term, while the MMAs are in flight
      bool in_ok = waiter.wait(&in_full[q & 1], (uint32_t)(q >> 1) & 1u);
      in_ok = __all_sync(0xffffffffu, in_ok);
      if (in_ok) {
        premath(q);
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&in_empty[q & 1]);  // the buffer may be refilled
      }
      if (et == 0) stamp(p.trace, q, 12);  // step-local math done
      // A failed (timed-out / aborted) wait never skips the named barrier below:
      // the thread marks the CTA aborted, skips the data movement, and everybody
      // leaves the loop together after the barrier.
      // ---- owner: add the S partials, fused epilogue, write the new state ----
      bool good = in_ok;
      if (good) {
        good = waiter.wait_cluster(&red_full_bar[a], aph);
        good = __all_sync(0xffffffffu, good);
        if (et == 0) stamp(p.trace, q, 6);  // all partials landed
      }
      if (good) {
        const uint32_t stg = stage_local + (uint32_t)(a * stg_buf_floats + 2 * fp * 4) * 4u;
        float4 s0[MAX_QUADS], s1[MAX_QUADS];  // sums for feature 2fp and 2fp+1, 4 batch rows
#pragma unroll
        for (int e = 0; e < MAX_QUADS; ++e) {
          const int qd = qd0 + e * nbq;
          s0[e] = make_float4(0.f, 0.f, 0.f, 0.f);
          s1[e] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (qd < nquads) {
#pragma unroll
            for (int src = 0; src < MAX_S; ++src) {
              if (src >= S) break;
              const uint32_t ad = stg + (uint32_t)(src * stg_src_floats + qd * rows_own * 4) * 4u;
              const float4 x0 = lds_f4(ad), x1 = lds_f4(ad + 16);
              s0[e].x += x0.x; s0[e].y += x0.y; s0[e].z += x0.z; s0[e].w += x0.w;
              s1[e].x += x1.x; s1[e].y += x1.y; s1[e].z += x1.z; s1[e].w += x1.w;
            }
          }
        }
        if (et == 0) stamp(p.trace, q, 14);  // partial sums read
#pragma unroll
        for (int e = 0; e < MAX_QUADS; ++e) {
          const float a0[4] = {s0[e].x, s0[e].y, s0[e].z, s0[e].w};
          const float a1[4] = {s1[e].x, s1[e].y, s1[e].z, s1[e].w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (eoff[e][u] >= 0) {
              const long idx = base_q + eoff[e][u];
              if (!BWD) {
                const float v0 = a0[u] + e0[e][u].x, v1 = a1[u] + e0[e][u].y;
                const float h0 = tanh_fast(v0), h1 = tanh_fast(v1);
                stg_u32(p.h + idx + BD, f2_to_bf16x2(h0, h1));
                late0[e][u] = f2_to_bf16x2(v0, v1);
                if (p.self_gate) {   // the gate is the state as stored
                  const float2 hs = bf16x2_to_f2(f2_to_bf16x2(h0, h1));
                  late1[e][u] = f2_to_bf16x2(h0 * hs.x * sigmoid_fast(hs.x), h1 * hs.y * sigmoid_fast(hs.y));
                } else {
                  late1[e][u] = f2_to_bf16x2(h0 * e1[e][u].x, h1 * e1[e][u].y);
                }
              } else {
                const float d0 = (e0[e][u].x + a0[u]) * e1[e][u].x;
                const float d1 = (e0[e][u].y + a1[u]) * e1[e][u].y;
                stg_u32(p.dv + idx, f2_to_bf16x2(d0, d1));
                db0 += d0;
                db1 += d1;
              }
            }
          }
        }
      } else {
        if (abort_flag == 0 && atomicExch(p.abort_word, 1) == 0) report_timeout(p.status, kid, step);
        abort_flag = 1;
      }
      // hand the publication of this chunk to the publisher warp: its gpu-scope
      // release would otherwise stall this warp's next loads and stores
      __syncwarp();
      if (lane == 0 && good) {
        if (p.direct_publish)  // one gpu-scope release per epilogue warp, no hand-off
          red_release_gpu_add(ready + ((q - step * G) * MAX_S + my_kslice) * COUNTER_STRIDE, 1);
        else
          ptx::mbar_arrive(&stored_bar[a]);
      }
      if (et == 0) stamp(p.trace, q, 7);  // new state stored
      // all 128 epilogue threads meet here, whether their waits succeeded or not,
      // and agree on whether to stop
      if (epi_bar_or(!good || abort_flag != 0, fg)) {
        abort_flag = 1;
        break;
      }
      if (et == 0) stamp(p.trace, q, 8);  // epilogue threads met
      // tell every source that its slot in my staging buffer `a` is free again
      // (my reads of it completed before the barrier above; no data is published here)
      if (et < S) mbar_arrive_remote_relaxed(mapa(ptx::smem_u32(&red_empty_bar[a]), (uint32_t)et));
      // outputs that no other CTA waits for
#pragma unroll
      for (int e = 0; e < MAX_QUADS; ++e) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (eoff[e][u] >= 0) {
            const long idx = base_q + eoff[e][u];
            if (!BWD) {
              if (p.v != nullptr) stg_u32(p.v + idx, late0[e][u]);
              stg_u32(p.y + idx, late1[e][u]);
            } else {
              if (p.dg != nullptr) stg_u32(p.dg + idx, late0[e][u]);
            }
          }
        }
      }
      if (et == 0) stamp(p.trace, q, 15);  // late outputs stored
      if (et == 0) stamp(p.trace, q, 10);  // next step's inputs requested
    }
    if (BWD) { db_part[0][ft] = db0; db_part[1][ft] = db1; }
  } else {
    // =========================== publisher ==================================
    // Waits until the four epilogue warps have stored their part of the new state
    // (mbarrier, CTA scope), then bumps the step counter with a gpu-scope release:
    // the stores are ordered before the counter for every CTA that acquires it.
    if (lane == 0 && !p.direct_publish) {
      const int my_kslice = (i * TILE_M + (int)j * rows_own) / Kc;
      for (int q = 0; q < total_q; ++q) {
        const int step = q / G, grp = q - step * G;
        const int a = q & 1;
        const uint32_t aph = (uint32_t)(q >> 1) & 1u;
        if (!waiter.wait(&stored_bar[a], aph)) break;   // the failing role reports the abort
        red_release_gpu_add(ready + (grp * MAX_S + my_kslice) * COUNTER_STRIDE, 1);
        stamp(p.trace, q, 9);  // published
      }
    }
    __syncwarp();
  }

  // ------------------------------ teardown ---------------------------------
  ptx::tc_fence_before();
  __syncthreads();
  if (abort_flag != 0) {
    // let copies that may still be in flight land before memory is released
    for (int k = 0; k < 2000; ++k) __nanosleep(100);
  }
  if (BWD && abort_flag == 0 && tid < rows_own) {
    // feature tid of my chunk = pair tid/2, element tid%2, summed over the batch slots
    const int pairs = rows_own / 2;
    float ssum = 0.f;
    for (int k = tid / 2; k < FG * NUM_EPI_THREADS; k += pairs) ssum += db_part[tid & 1][k];
    p.db[(long)rep * p.d + i * TILE_M + (int)j * rows_own + tid] = ssum;   // one row of sums per replica
  }
  // no CTA may exit while a peer can still address its shared memory
  cluster_sync_all();
  if (warp == 1) ptx::tmem_dealloc(tmem_base, tmem_cols);
}

// db[j] += db[r * d + j] for r = 1 .. reps-1, in that order
__global__ void fold_rows_kernel(float* db, int d, int reps) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= d) return;
  float s = db[j];
  for (int r = 1; r < reps; ++r) s += db[(long)r * d + j];
  db[j] = s;
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_state_tmap(CUtensorMap* out, const void* base, int slots, int B, int d, int box_rows,
                    int box_tiles) {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) !=
            cudaSuccess || qres != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return set_error(ELMAN_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    }
    fn = (EncodeTiledFn)ptr;
  }
  // view [slots][B][d/64][64]: dim0 = 64 columns (one 128-byte swizzle row), dim1 = batch row,
  // dim2 = 64-column tile index, dim3 = time slot; a box covers box_tiles tiles at once
  cuuint64_t dims[4] = {64, (cuuint64_t)B, (cuuint64_t)(d / 64), (cuuint64_t)slots};
  cuuint64_t strides[3] = {(cuuint64_t)d * 2, 128, (cuuint64_t)B * d * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, (cuuint32_t)box_tiles, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult rc = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS)
    return set_error(ELMAN_ERR_CUDA, "cuTensorMapEncodeTiled (state) failed (%d)", (int)rc);
  return ELMAN_OK;
}

// [slots][B][d] bf16 seen as (d, B, slots), no swizzle: box = box_cols features x box_rows
// batch rows x 1 time slot.  Used for the epilogue's input tiles.
int make_io_tmap(CUtensorMap* out, const void* base, int slots, int B, int d, int box_cols,
                 int box_rows) {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) !=
            cudaSuccess || qres != cudaDriverEntryPointSuccess) {
      cudaGetLastError();
      return set_error(ELMAN_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    }
    fn = (EncodeTiledFn)ptr;
  }
  cuuint64_t dims[3] = {(cuuint64_t)d, (cuuint64_t)B, (cuuint64_t)slots};
  cuuint64_t strides[2] = {(cuuint64_t)d * 2, (cuuint64_t)B * d * 2};
  cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult rc = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS)
    return set_error(ELMAN_ERR_CUDA, "cuTensorMapEncodeTiled (epilogue inputs) failed (%d)", (int)rc);
  return ELMAN_OK;
}

struct RecPlan {
  int reps = 1;   // batch replicas of the grid; G then counts the groups of ONE replica
  int S, Kc, G, Ng, Npad, nstages, nmw, w_tmem;
  int fg;   // finalising warp groups (kernel instantiation)
  uint32_t tmem_cols;
  size_t smem;
  bool ok;
};

size_t plan_smem(int S, int Kc, int Npad, int nstages, bool w_tmem, int nin) {
  size_t w = w_tmem ? 0 : (size_t)TILE_M * Kc * 2;
  size_t st = (size_t)nstages * Npad * Kc * 2;
  size_t stg = (size_t)2 * TILE_M * Npad * 4;
  size_t in = (size_t)2 * nin * Npad * (TILE_M / S) * 2;  // epilogue input tiles, double buffered
  return w + st + stg + in + 1024 + 64;
}

// Full plan for one K split S and one cap on the batch-group size, or ok == false.
RecPlan plan_for(int B, int d, int S, int ng_cap, bool want_w_tmem, int nin) {
  RecPlan pl{};
  pl.ok = false;
  pl.w_tmem = 0;
  const size_t smem_cap = 225 * 1024;
  if (d % S != 0) return pl;
  const int Kc = d / S;
  if (Kc % 64 != 0 || (d / 128) * S > 148) return pl;
  const long want_G = options().rec_groups;
  int G = 0, Ng = 0;
  if (want_G > 0) {
    if (B % want_G != 0) return pl;
    G = (int)want_G;
    Ng = B / G;
  } else {
    int cap = 8 * MAX_QUADS * S < ng_cap ? 8 * MAX_QUADS * S : ng_cap;
    for (int g = 1; g <= MAX_GROUPS; ++g) {
      if (B % g != 0) continue;
      if (B / g <= cap) { G = g; Ng = B / g; break; }
    }
    if (G == 0) return pl;
  }
  if (G > MAX_GROUPS || Ng > 8 * MAX_QUADS * S || Ng > 256) return pl;
  const int Npad = (Ng + 15) / 16 * 16;
  int nmw = (int)options().rec_mma_warps;
  if (nmw <= 0) nmw = NUM_MMA_WARPS;
  if (nmw > NUM_MMA_WARPS) nmw = NUM_MMA_WARPS;
  if (nmw > Kc / 16) nmw = Kc / 16;
  while (nmw > 1 && 2 * nmw * Npad > 512) --nmw;
  if (2 * nmw * Npad > 512) return pl;
  if (want_w_tmem)  // fewer accumulator chains if that lets the W tile fit
    while (nmw > 2 && 2 * nmw * Npad + Kc / 2 > 512) --nmw;
  const bool w_tmem = want_w_tmem && 2 * nmw * Npad + Kc / 2 <= 512;
  uint32_t cols = 32;
  while (cols < (uint32_t)(2 * nmw * Npad + (w_tmem ? Kc / 2 : 0))) cols <<= 1;
  pl.w_tmem = w_tmem ? 1 : 0;
  // a single batch group runs strictly step after step: one ring stage is enough
  const int min_stages = G > 1 ? 2 : 1;
  int nstages = G > 1 ? 4 : 2;
  while (nstages > min_stages && plan_smem(S, Kc, Npad, nstages, w_tmem, nin) > smem_cap) --nstages;
  if (plan_smem(S, Kc, Npad, nstages, w_tmem, nin) > smem_cap) return pl;
  pl.S = S; pl.Kc = Kc; pl.G = G; pl.Ng = Ng; pl.Npad = Npad; pl.nstages = nstages;
  pl.nmw = nmw; pl.tmem_cols = cols;
  // with four or more batch groups in flight the finalising warps set the pace: two groups
  // of them alternate (a second kernel instantiation, so the other plans keep their registers)
  pl.fg = (G >= 4 && options().rec_fin_groups != 1) ? 2 : 1;
  pl.smem = plan_smem(S, Kc, Npad, nstages, w_tmem, nin);
  pl.ok = true;
  return pl;
}

// Every CTA waits on every other one, so the whole grid must be resident at once:
// ask the runtime how many clusters of this shape fit.
// One lock for everything that touches the kernels' per-device attributes: the planner's
// occupancy queries and the set-attribute + launch pair of a launch (a second host thread
// must not change the shared-memory attribute between the two).
std::mutex g_rec_mutex;

template <typename Kernel>
bool kernel_is_coresident(Kernel kern, const RecPlan& pl, int d);

bool plan_is_coresident(const RecPlan& pl, int d, bool bwd) {
  // the instantiation that will be launched: registers, and so occupancy, differ
  if (bwd)
    return pl.fg == 2 ? kernel_is_coresident(rec_tc_kernel<true, 2>, pl, d)
                      : kernel_is_coresident(rec_tc_kernel<true, 1>, pl, d);
  return pl.fg == 2 ? kernel_is_coresident(rec_tc_kernel<false, 2>, pl, d)
                    : kernel_is_coresident(rec_tc_kernel<false, 1>, pl, d);
}

// How many clusters of this plan's kernel fit on the device at once (0 on error).
template <typename Kernel>
int kernel_max_clusters(Kernel kern, const RecPlan& pl, int d);

int plan_max_clusters(const RecPlan& pl, int d, bool bwd) {
  if (bwd)
    return pl.fg == 2 ? kernel_max_clusters(rec_tc_kernel<true, 2>, pl, d)
                      : kernel_max_clusters(rec_tc_kernel<true, 1>, pl, d);
  return pl.fg == 2 ? kernel_max_clusters(rec_tc_kernel<false, 2>, pl, d)
                    : kernel_max_clusters(rec_tc_kernel<false, 1>, pl, d);
}

template <typename Kernel>
bool kernel_is_coresident(Kernel kern, const RecPlan& pl, int d) {
  return kernel_max_clusters(kern, pl, d) * pl.S >= (d / TILE_M) * pl.S * pl.reps;
}

template <typename Kernel>
int kernel_max_clusters(Kernel kern, const RecPlan& pl, int d) {
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem) !=
      cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((d / TILE_M) * pl.S);
  cfg.blockDim = dim3(threads_for(pl.fg));
  cfg.dynamicSmemBytes = pl.smem;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = pl.S;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  int max_clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return max_clusters;
}

// Largest K split first (most CTAs, smallest resident tile); a split whose clusters do
// not all fit on the device at once is skipped.  Results are cached per shape.
RecPlan make_plan(int T, int B, int d, int compact, bool bwd) {
  RecPlan none{};
  none.ok = false;
  if (T < 1 || B < 1 || d < 128 || (d % 128) != 0) return none;
  const int nin = bwd ? 4 : 2;  // arrays the epilogue reads per step
  compact = (compact ? 1 : 0) | (bwd ? 2 : 0);   // also carries the direction
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); dev = 0; }
  // co-residency depends on the device; callers may come from several host threads
  // (autograd's) and use several GPUs
  typedef std::tuple<int, int, int, int, long, long, long, long, long, long, long, long> Key;
  static std::map<Key, RecPlan> cache;
  std::lock_guard<std::mutex> lock(g_rec_mutex);
  const Key key(dev, B, d, compact, options().rec_ksplit, options().rec_groups,
                options().rec_mma_warps, options().rec_w_tmem, options().rec_large_batch,
                options().rec_fin_groups, options().rec_replicas, options().rec_group_cap);
  {
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
  }
  RecPlan found = none;
  const long want_S = options().rec_ksplit;
  if (compact & 1) {
    // smallest footprint: the smallest K split whose tile of W fits in shared memory
    // or, failing that, in tensor memory
    for (int S = 1; S <= MAX_S && !found.ok; S <<= 1) {
      if (want_S > 0 && S != want_S) continue;
      for (int wt = 0; wt <= 1 && !found.ok; ++wt) {
        if (wt == 1 && options().rec_w_tmem == 2) continue;
        RecPlan pl = plan_for(B, d, S, 32, wt != 0, nin);
        if (pl.ok && (wt == 0 || pl.w_tmem) && plan_is_coresident(pl, d, bwd)) found = pl;
      }
    }
  } else if (B <= 32 || options().rec_groups > 0 || options().rec_large_batch == 0) {
    // latency plan: the largest K split (shortest per-step chain); the weight tile in tensor
    // memory when it fits beside the accumulators (the MMAs issue faster with the A operand
    // there: 32 instead of 44 cycles per MMA with four issuing warps), else in shared memory
    for (int S = MAX_S; S >= 1 && !found.ok; S >>= 1) {
      if (want_S > 0 && S != want_S) continue;
      for (int ng_cap = 32; ng_cap >= 16 && !found.ok; ng_cap >>= 1)
        for (int wt = 1; wt >= 0 && !found.ok; --wt) {
          if (wt == 1 && options().rec_w_tmem == 2) continue;
          RecPlan pl = plan_for(B, d, S, ng_cap, wt != 0, nin);
          if (pl.ok && (wt == 0 || pl.w_tmem) && plan_is_coresident(pl, d, bwd)) found = pl;
        }
    }
  } else {
    // throughput plan for batches that need several groups anyway: the widest group
    // first (fixed per-group costs are paid fewer times per step), the weight tile in
    // tensor memory when shared memory cannot hold it beside the wider state tiles
    const int cap0 = options().rec_group_cap >= 16 && options().rec_group_cap <= 64
                         ? (int)options().rec_group_cap : 64;
    for (int ng_cap = cap0; ng_cap >= 16 && !found.ok; ng_cap >>= 1)
      for (int S = MAX_S; S >= 1 && !found.ok; S >>= 1) {
        if (want_S > 0 && S != want_S) continue;
        for (int wt = 0; wt <= 1 && !found.ok; ++wt) {
          if ((wt == 0 && options().rec_w_tmem == 1) || (wt == 1 && options().rec_w_tmem == 2)) continue;
          RecPlan pl = plan_for(B, d, S, ng_cap, wt != 0, nin);
          if (pl.ok && pl.Ng > ng_cap / 2 && (wt == 0 || pl.w_tmem) && plan_is_coresident(pl, d, bwd))
            found = pl;
        }
      }
    // Batch replicas: when the grid leaves most of the device idle, run several copies of it,
    // each on its own share of the batch groups (sequences are independent, the copies never
    // wait on each other).  Fewer groups pass through each block per step.
    if (found.ok && options().rec_replicas != 1) {
      const int clusters_one = d / TILE_M;
      const int fit = plan_max_clusters(found, d, bwd) / clusters_one;
      int want = (int)options().rec_replicas;          // 0 = as many as fit
      int reps = want > 0 ? want : REC_MAX_REPLICAS;
      if (reps > REC_MAX_REPLICAS) reps = REC_MAX_REPLICAS;
      if (reps > fit) reps = fit;
      while (reps > 1 && found.G % reps != 0) --reps;
      if (reps > 1) {
        RecPlan rp = plan_for(B / reps, d, found.S, found.Ng, found.w_tmem != 0, nin);
        if (rp.ok && rp.S == found.S && rp.Ng == found.Ng && rp.w_tmem == found.w_tmem) {
          rp.reps = reps;
          if (plan_is_coresident(rp, d, bwd)) found = rp;
        }
      }
    }
  }
  cache[key] = found;
  return found;
}

template <bool BWD, int FG>
int launch_rec_tc_fg(const RecPlan& pl, RecTcParams& p, const void* W, const void* state,
                     cudaStream_t stream) {
  auto kern = rec_tc_kernel<BWD, FG>;
  CUtensorMap tmW, tmState, tmI[4];
  ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmW, W, (uint64_t)p.d, (uint64_t)p.d, (uint64_t)p.d, TILE_M));
  ELMAN_RETURN_IF(make_state_tmap(&tmState, state, p.T + 1, p.B, p.d, pl.Npad, pl.Kc / 64));
  {
    // forward: pre, gate;  backward: gate, dy, h (T+1 slots), v
    const void* ins[4] = {BWD ? (const void*)p.g : (const void*)p.pre,
                          BWD ? (const void*)p.dy : (const void*)p.g,
                          BWD ? (const void*)p.h_in : (const void*)p.pre,
                          BWD ? (const void*)p.v_in : (const void*)p.g};
    const int slots[4] = {p.T, p.T, BWD ? p.T + 1 : p.T, p.T};
    for (int k = 0; k < 4; ++k)
      ELMAN_RETURN_IF(make_io_tmap(&tmI[k], ins[k], slots[k], p.B, p.d, TILE_M / pl.S, pl.Npad));
  }
  std::lock_guard<std::mutex> lock(g_rec_mutex);   // set-attribute and launch as one unit
  ELMAN_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)pl.smem));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((p.d / TILE_M) * pl.S * pl.reps);
  cfg.blockDim = dim3(threads_for(FG));
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = pl.S;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = 1;
  // every CTA waits on every other: the whole grid must be resident at once
  int max_clusters = 0;
  ELMAN_CUDA_CHECK(cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg));
  if (max_clusters * pl.S < (int)cfg.gridDim.x)
    return set_error(ELMAN_ERR_UNSUPPORTED, "recurrence grid of %d CTAs is not co-resident (%d clusters of %d fit)",
                     (int)cfg.gridDim.x, max_clusters, pl.S);
  ELMAN_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, tmW, tmState, tmI[0], tmI[1], tmI[2], tmI[3], p));
  count_launch(true);
  return ELMAN_OK;
}

template <bool BWD>
int launch_rec_tc(const RecPlan& pl, RecTcParams& p, const void* W, const void* state,
                  cudaStream_t stream) {
  if (pl.fg == 2) return launch_rec_tc_fg<BWD, 2>(pl, p, W, state, stream);
  return launch_rec_tc_fg<BWD, 1>(pl, p, W, state, stream);
}

void fill_plan(const RecPlan& pl, RecTcParams& p) {
  p.S = pl.S; p.Kc = pl.Kc; p.G = pl.G; p.Ng = pl.Ng; p.Npad = pl.Npad; p.nstages = pl.nstages;
  p.nmw = pl.nmw; p.tmem_cols = pl.tmem_cols;
  p.direct_publish = 0;  // set per direction by the callers
  p.w_tmem = pl.w_tmem;
  p.w_col0 = (uint32_t)(2 * pl.nmw * pl.Npad);
  p.R = p.d / TILE_M;
  p.reps = pl.reps;
  p.Brep = pl.G * pl.Ng;
  p.spin_limit = options().spin_limit;
  p.stall_step = (int)options().test_stall_step;
  p.status = device_status_ptr();
}

}  // namespace

bool rec_tc_supported(int T, int B, int d, int bwd) { return make_plan(T, B, d, 0, bwd != 0).ok; }

int rec_tc_blocks(int T, int B, int d, int compact) {
  // batch groups are pipelined through the same blocks, so they do not add any
  RecPlan f = make_plan(T, B, d, compact, false), b = make_plan(T, B, d, compact, true);
  if (!f.ok || !b.ok) return 0;
  const int nf = f.S * f.reps, nb = b.S * b.reps;
  return (d / TILE_M) * (nf > nb ? nf : nb);
}

size_t rec_tc_sync_bytes() {
  return (size_t)(MAX_GROUPS * MAX_S * COUNTER_STRIDE + 64) * sizeof(int) +
         (size_t)TRACE_STEPS * TRACE_SLOTS * sizeof(long long);
}

static long long* g_last_trace = nullptr;
static long long* trace_area(int* sync) {
  if (options().rec_trace == 0) return nullptr;
  g_last_trace = (long long*)(sync + MAX_GROUPS * MAX_S * COUNTER_STRIDE + 64);
  return g_last_trace;
}
void set_last_trace(long long* device_buffer) { g_last_trace = device_buffer; }
int rec_tc_copy_trace(long long* dst, int max_entries) {
  if (g_last_trace == nullptr) return set_error(ELMAN_ERR_ARG, "no trace was recorded");
  int n = TRACE_STEPS * TRACE_SLOTS;
  if (n > max_entries) n = max_entries;
  ELMAN_CUDA_CHECK(cudaMemcpy(dst, g_last_trace, (size_t)n * sizeof(long long),
                              cudaMemcpyDeviceToHost));
  return ELMAN_OK;
}

int rec_fwd_tc(const RecFwdArgs& a, cudaStream_t stream) {
  RecPlan pl = make_plan(a.T, a.B, a.d, a.compact, false);
  if (!pl.ok && a.compact) pl = make_plan(a.T, a.B, a.d, 0, false);  // no compact plan: the regular one
  if (!pl.ok) return set_error(ELMAN_ERR_UNSUPPORTED, "shape not supported by the tensor-core recurrence");
  RecTcParams p{};
  p.T = a.T; p.B = a.B; p.d = a.d;
  fill_plan(pl, p);
  p.pre = (const bf16*)a.pre; p.h = (bf16*)a.h; p.y = (bf16*)a.y;
  p.self_gate = a.g == nullptr ? 1 : 0;     // the gate tile is then fetched from `pre`, unused
  p.g = (const bf16*)(a.g != nullptr ? a.g : a.pre);
  p.v = (bf16*)a.v;
  ELMAN_CUDA_CHECK(cudaMemsetAsync(a.sync, 0, rec_tc_sync_bytes(), stream));
  p.ready = a.sync;
  p.abort_word = a.sync + MAX_GROUPS * MAX_S * COUNTER_STRIDE;
  p.trace = trace_area(a.sync);
  p.Wg = (const bf16*)a.W;
  // option rec_direct_publish: 0 = auto (measured best: forward direct, backward through the
  // publisher warp), 1 = direct in both, 2 = publisher warp in both
  // with several batch groups in flight the release's latency only stalls the epilogue
  // warps, which are the busiest role: hand it to the publisher warp then
  p.direct_publish = options().rec_direct_publish == 2 ? 0
                     : options().rec_direct_publish == 1 ? 1 : (pl.G == 1 ? 1 : 0);
  return launch_rec_tc<false>(pl, p, a.W, a.h, stream);
}

int rec_bwd_tc(const RecBwdArgs& a, cudaStream_t stream) {
  RecPlan pl = make_plan(a.T, a.B, a.d, a.compact, true);
  if (!pl.ok && a.compact) pl = make_plan(a.T, a.B, a.d, 0, true);  // no compact plan: the regular one
  if (!pl.ok) return set_error(ELMAN_ERR_UNSUPPORTED, "shape not supported by the tensor-core recurrence");
  RecTcParams p{};
  p.T = a.T; p.B = a.B; p.d = a.d;
  fill_plan(pl, p);
  p.h_in = (const bf16*)a.h; p.v_in = (const bf16*)a.v;
  p.self_gate = a.g == nullptr ? 1 : 0;
  p.g = (const bf16*)(a.g != nullptr ? a.g : a.dy);
  p.dy = (const bf16*)a.dy; p.dv = (bf16*)a.dv; p.dg = (bf16*)a.dg; p.db = a.db;
  ELMAN_CUDA_CHECK(cudaMemsetAsync(a.sync, 0, rec_tc_sync_bytes(), stream));
  // slot T of dv (the gradient carried in from later steps, or zeros) is filled by the caller
  p.ready = a.sync;
  p.abort_word = a.sync + MAX_GROUPS * MAX_S * COUNTER_STRIDE;
  p.trace = trace_area(a.sync);
  p.Wg = (const bf16*)a.Wt;
  p.direct_publish = options().rec_direct_publish == 1 ? 1 : 0;
  ELMAN_RETURN_IF(launch_rec_tc<true>(pl, p, a.Wt, a.dv, stream));
  if (pl.reps > 1) {   // fold the replicas' bias-gradient rows into the first
    fold_rows_kernel<<<(a.d + 255) / 256, 256, 0, stream>>>(a.db, a.d, pl.reps);
    count_launch(false);
    ELMAN_CUDA_CHECK(cudaGetLastError());
  }
  return ELMAN_OK;
}

}  // namespace elman

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
// Roles are warp-specialised: warp 0 = TMA producer, warp 1 = MMA issuer and TMEM
// owner, warps 2..5 = epilogue.  Independent batch groups are pipelined through
// the same rings, so one group's global round trip overlaps another's math.
//
// Every wait (global counters, mbarriers) is bounded; a wait that gives up raises
// an abort word all CTAs poll, records a status code and the kernel drains and
// returns with tensor memory freed.
#include <cooperative_groups.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace elman {

namespace {

constexpr int TILE_M = 128;
constexpr int NUM_EPI_THREADS = 128;
constexpr int NUM_THREADS = 64 + NUM_EPI_THREADS;
constexpr int MAX_S = 8;
constexpr int MAX_GROUPS = 16;
constexpr int MAX_E = 16;          // epilogue elements per thread and step
constexpr int COUNTER_STRIDE = 32; // ints; one 128-byte line per counter

struct RecTcParams {
  int T, B, d;
  int S;        // K split = cluster size
  int Kc;       // d / S
  int G;        // batch groups
  int Ng;       // batch rows per group
  int Npad;     // Ng rounded up to 16 (MMA N)
  int nstages;  // state ring depth
  int R;        // d / 128: producers per K slice and step
  // forward
  const bf16* pre; const bf16* g; bf16* h; bf16* y; bf16* v;
  // backward
  const bf16* h_in; const bf16* v_in; const bf16* dy; bf16* dv; bf16* dg; float* db;
  int* ready;       // [G][S] counters, COUNTER_STRIDE ints apart
  int* abort_word;  // global abort flag
  int* status;
  long spin_limit;
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
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, int c0, int c1,
                                            int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(ptx::smem_u32(smem_dst)), "l"(m), "r"(ptx::smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
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
    while (!ptx::mbar_try_wait(bar, parity))
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
template <bool BWD>
__global__ void __launch_bounds__(NUM_THREADS, 1)
rec_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmState,
              RecTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t w_bar;
  __shared__ __align__(8) uint64_t full_bar[4];       // state ring: TMA -> MMA
  __shared__ __align__(8) uint64_t empty_bar[4];      // state ring: MMA -> TMA
  __shared__ __align__(8) uint64_t acc_full_bar[2];   // MMA -> epilogue
  __shared__ __align__(8) uint64_t acc_empty_bar[2];  // epilogue -> MMA
  __shared__ __align__(8) uint64_t red_full_bar[2];   // peers' partials landed (owner side)
  __shared__ __align__(8) uint64_t red_empty_bar[2];  // owners consumed my partials (source side)
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ float db_part[NUM_EPI_THREADS];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = p.S, Kc = p.Kc, Npad = p.Npad, Ng = p.Ng, G = p.G;
  const int rows_own = TILE_M / S;
  const uint32_t j = cluster_ctarank();   // K slice index == rank in cluster
  const int i = blockIdx.x / S;           // row block index
  const int nkt = Kc / 64;                // 64-column tiles per K slice
  const int total_q = p.T * G;

  // dynamic shared memory carve-up (1024-byte aligned for the swizzled tiles)
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sW = smem;                                    // nkt tiles of [128 x 64] bf16
  const int w_bytes = TILE_M * Kc * 2;
  uint8_t* sState = sW + w_bytes;                        // nstages x nkt tiles of [Npad x 64]
  const int state_tile_bytes = Npad * 64 * 2;
  const int state_stage_bytes = nkt * state_tile_bytes;
  float* sStage = (float*)(sState + p.nstages * state_stage_bytes);  // [2][S][rows_own][Npad+1]
  const int stg_row = Npad + 1;
  const int stg_buf_floats = S * rows_own * stg_row;

  Waiter waiter{p.spin_limit, &abort_flag, p.abort_word};

  if (tid == 0) {
    abort_flag = 0;
    ptx::mbar_init(&w_bar, 1);
    for (int s = 0; s < 4; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    const int red_arrivals = S > 4 ? S : 4;
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(&acc_full_bar[a], 1);
      ptx::mbar_init(&acc_empty_bar[a], 4);
      ptx::mbar_init(&red_full_bar[a], red_arrivals);
      ptx::mbar_init(&red_empty_bar[a], S);
    }
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmW);
    ptx::prefetch_tmap(&tmState);
  }
  if (warp == 1) {
    uint32_t cols = 2 * Npad < 32 ? 32 : 2 * Npad;
    uint32_t pow2 = 32;
    while (pow2 < cols) pow2 <<= 1;
    ptx::tmem_alloc(&tmem_slot, pow2);
    ptx::tmem_relinquish();
  }
  if (tid >= 64) db_part[tid - 64] = 0.f;
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  // peers must have initialised their barriers before any remote arrive / store
  cluster_sync_all();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    // =========================== TMA producer ===============================
    if (lane == 0) {
      // resident tile of W
      ptx::mbar_arrive_expect_tx(&w_bar, (uint32_t)w_bytes);
      for (int kk = 0; kk < nkt; ++kk)
        ptx::tma_load_2d(sW + kk * (TILE_M * 128), &tmW, (int)j * Kc + kk * 64, i * TILE_M, &w_bar);
      for (int q = 0; q < total_q; ++q) {
        const int step = q / G, grp = q - step * G;
        const int s = q % p.nstages;
        const uint32_t ph = (uint32_t)(q / p.nstages) & 1u;
        bool ok = waiter.wait(&empty_bar[s], ph ^ 1u);
        if (ok && step > 0)
          ok = waiter.wait_counter(p.ready + (grp * MAX_S + (int)j) * COUNTER_STRIDE, step * p.R);
        if (!ok) {
          if (atomicExch(p.abort_word, 1) == 0) report_timeout(p.status, BWD ? KID_REC_TC_BWD : KID_REC_TC_FWD, step);
          abort_flag = 1;
          break;
        }
        // data written by other SMs through the generic proxy -> read by TMA
        ptx::fence_proxy_async();
        const int slot = BWD ? (p.T - step) : step;  // time index of the input state
        ptx::mbar_arrive_expect_tx(&full_bar[s], (uint32_t)state_stage_bytes);
        for (int kk = 0; kk < nkt; ++kk)
          tma_load_3d(sState + s * state_stage_bytes + kk * state_tile_bytes, &tmState,
                      (int)j * Kc + kk * 64, grp * Ng, slot, &full_bar[s]);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // =========================== MMA issuer =================================
    if (lane == 0) {
      const uint32_t idesc = ptx::umma_idesc_bf16(TILE_M, Npad);
      bool ok = waiter.wait(&w_bar, 0);
      for (int q = 0; q < total_q && ok; ++q) {
        const int s = q % p.nstages;
        const uint32_t ph = (uint32_t)(q / p.nstages) & 1u;
        const int a = q & 1;
        const uint32_t aph = (uint32_t)(q >> 1) & 1u;
        ok = waiter.wait(&acc_empty_bar[a], aph ^ 1u) && waiter.wait(&full_bar[s], ph);
        if (!ok) break;
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(a * Npad);
        for (int kk = 0; kk < nkt; ++kk) {
          const uint64_t da = ptx::umma_desc_k_sw128(ptx::smem_u32(sW + kk * (TILE_M * 128)));
          const uint64_t db = ptx::umma_desc_k_sw128(
              ptx::smem_u32(sState + s * state_stage_bytes + kk * state_tile_bytes));
#pragma unroll
          for (int k = 0; k < 4; ++k)
            ptx::umma_bf16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kk > 0 || k > 0) ? 1u : 0u);
        }
        ptx::umma_commit(&empty_bar[s]);
        ptx::umma_commit(&acc_full_bar[a]);
      }
      if (!ok) {
        if (abort_flag == 0 && atomicExch(p.abort_word, 1) == 0)
          report_timeout(p.status, BWD ? KID_REC_TC_BWD : KID_REC_TC_FWD, 0xFFFFF1);
        abort_flag = 1;
      }
    }
    __syncwarp();
  } else {
    // =========================== epilogue ===================================
    const int et = tid - 64;                 // 0..127
    const int quarter = warp & 3;            // TMEM lane quarter this warp may read
    const int m = quarter * 32 + lane;       // accumulator row held by this thread
    const int owner = m / rows_own;          // cluster rank that finalises row m
    const int m_local = m - owner * rows_own;
    const int rows_in_warp = rows_own < 32 ? rows_own : 32;
    // finalise mapping: feature fl of my chunk, batch rows bq, bq+S, ...
    const int fl = et % rows_own;
    const int bq = et / rows_own;
    const int f = i * TILE_M + (int)j * rows_own + fl;  // global feature index
    const int my_kslice = f / Kc;
    const uint32_t stage_local = ptx::smem_u32(sStage);
    const long BD = (long)p.B * p.d;
    float db_acc = 0.f;
    bool ok = true;

    // element registers: forward (pre, z) / backward (a = dy*silu(g), dtanh)
    float e0[MAX_E], e1[MAX_E];
    auto prefetch = [&](int q) {
      const int step = q / G, grp = q - step * G;
      const int t = BWD ? (p.T - 1 - step) : step;
#pragma unroll
      for (int e = 0; e < MAX_E; ++e) {
        const int b = bq + e * S;
        if (b < Ng) {
          const long idx = ((long)t * p.B + grp * Ng + b) * p.d + f;
          if (!BWD) {
            e0[e] = bf16_bits_to_f(ldg_bf16_bits(p.pre + idx));
            e1[e] = bf16_bits_to_f(ldg_bf16_bits(p.g + idx));
          } else {
            const float gz = bf16_bits_to_f(ldg_bf16_bits(p.g + idx));
            const float dyv = bf16_bits_to_f(ldg_bf16_bits(p.dy + idx));
            const float hv = bf16_bits_to_f(ldg_bf16_bits(p.h_in + idx + BD));
            const float th = tanhf(bf16_bits_to_f(ldg_bf16_bits(p.v_in + idx)));
            p.dg[idx] = __float2bfloat16_rn(dyv * hv * dsiluf_(gz));
            e0[e] = dyv * siluf_(gz);
            e1[e] = 1.f - th * th;
          }
        }
      }
    };
    if (total_q > 0) prefetch(0);

    for (int q = 0; q < total_q; ++q) {
      const int step = q / G, grp = q - step * G;
      const int t = BWD ? (p.T - 1 - step) : step;
      const int a = q & 1;
      const uint32_t aph = (uint32_t)(q >> 1) & 1u;
      // ---- drain my accumulator row and scatter it to the owning peer ----
      ok = waiter.wait(&acc_full_bar[a], aph) && waiter.wait_cluster(&red_empty_bar[a], aph ^ 1u);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tc_fence_after();
      {
        const uint32_t remote =
            mapa(stage_local + (uint32_t)(((a * S + (int)j) * rows_own + m_local) * stg_row) * 4u,
                 (uint32_t)owner);
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(a * Npad);
        for (int c = 0; c < Npad; c += 16) {
          uint32_t r[16];
          ptx::tmem_ld16(taddr + (uint32_t)c, r);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int k = 0; k < 16; ++k)
            if (c + k < Ng) st_cluster_f32(remote + (uint32_t)(c + k) * 4u, __uint_as_float(r[k]));
        }
        ptx::tc_fence_before();
        fence_acq_rel_cluster();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&acc_empty_bar[a]);
        if ((lane % rows_in_warp) == 0)
          mbar_arrive_remote(mapa(ptx::smem_u32(&red_full_bar[a]), (uint32_t)owner));
      }
      // ---- owner: add the S partials, fused epilogue, publish the new state ----
      ok = waiter.wait_cluster(&red_full_bar[a], aph);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const float* stg = sStage + a * stg_buf_floats + fl * stg_row;
#pragma unroll
      for (int e = 0; e < MAX_E; ++e) {
        const int b = bq + e * S;
        if (b < Ng) {
          float acc = 0.f;
          for (int src = 0; src < S; ++src) acc += stg[src * rows_own * stg_row + b];
          const long idx = ((long)t * p.B + grp * Ng + b) * p.d + f;
          if (!BWD) {
            const float val = acc + e0[e];
            const float hv = tanhf(val);
            p.h[idx + BD] = __float2bfloat16_rn(hv);
            if (p.v != nullptr) p.v[idx] = __float2bfloat16_rn(val);
            p.y[idx] = __float2bfloat16_rn(hv * siluf_(e1[e]));
          } else {
            const float dvv = (e0[e] + acc) * e1[e];
            p.dv[idx] = __float2bfloat16_rn(dvv);
            db_acc += dvv;
          }
        }
      }
      // all 128 epilogue threads have written their part of the chunk
      epi_bar_sync();
      if (et == 0) {
        __threadfence();
        red_release_gpu_add(p.ready + (grp * MAX_S + my_kslice) * COUNTER_STRIDE, 1);
      }
      // tell every source that its slot in my staging buffer `a` is free again
      if (et < S) mbar_arrive_remote(mapa(ptx::smem_u32(&red_empty_bar[a]), (uint32_t)et));
      if (q + 1 < total_q) prefetch(q + 1);
    }
    if (!ok) {
      if (abort_flag == 0 && atomicExch(p.abort_word, 1) == 0)
        report_timeout(p.status, BWD ? KID_REC_TC_BWD : KID_REC_TC_FWD, 0xFFFFF2);
      abort_flag = 1;
    }
    if (BWD) db_part[et] = db_acc;
  }

  // ------------------------------ teardown ---------------------------------
  ptx::tc_fence_before();
  __syncthreads();
  if (abort_flag != 0) {
    // let copies that may still be in flight land before memory is released
    for (int k = 0; k < 2000; ++k) __nanosleep(100);
  }
  if (BWD && abort_flag == 0 && tid >= 64) {
    const int et = tid - 64;
    if (et < rows_own) {
      float ssum = 0.f;
      for (int k = et; k < NUM_EPI_THREADS; k += rows_own) ssum += db_part[k];
      p.db[i * TILE_M + (int)j * rows_own + et] = ssum;
    }
  }
  // no CTA may exit while a peer can still address its shared memory
  cluster_sync_all();
  if (warp == 1) {
    uint32_t cols = 2 * Npad < 32 ? 32 : 2 * Npad;
    uint32_t pow2 = 32;
    while (pow2 < cols) pow2 <<= 1;
    ptx::tmem_dealloc(tmem_base, pow2);
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_state_tmap(CUtensorMap* out, const void* base, int slots, int B, int d, int box_rows) {
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
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult rc = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS)
    return set_error(ELMAN_ERR_CUDA, "cuTensorMapEncodeTiled (state) failed (%d)", (int)rc);
  return ELMAN_OK;
}

struct RecPlan {
  int S, Kc, G, Ng, Npad, nstages;
  size_t smem;
  bool ok;
};

size_t plan_smem(int S, int Kc, int Npad, int nstages) {
  size_t w = (size_t)TILE_M * Kc * 2;
  size_t st = (size_t)nstages * Npad * Kc * 2;
  size_t stg = (size_t)2 * TILE_M * (Npad + 1) * 4;
  (void)S;
  return w + st + stg + 1024 + 64;
}

RecPlan make_plan(int T, int B, int d) {
  RecPlan pl{};
  pl.ok = false;
  if (T < 1 || B < 1 || d < 128 || (d % 128) != 0) return pl;
  const size_t smem_cap = 200 * 1024;
  long want_S = options().rec_ksplit;
  long want_G = options().rec_groups;
  int best_S = 0;
  for (int S = MAX_S; S >= 1; S >>= 1) {
    if (want_S > 0 && S != want_S) continue;
    if (d % S != 0) continue;
    int Kc = d / S;
    if (Kc % 64 != 0) continue;
    if ((d / 128) * S > 148) continue;
    if (plan_smem(S, Kc, 16, 2) > smem_cap) continue;
    best_S = S;
    break;
  }
  if (best_S == 0) return pl;
  const int S = best_S, Kc = d / S;
  // batch groups: Ng <= MAX_E * S and Ng <= 32 by default; groups must tile B exactly
  int G = 0, Ng = 0;
  if (want_G > 0) {
    if (B % want_G != 0) return pl;
    G = (int)want_G;
    Ng = B / G;
  } else {
    int cap = MAX_E * S < 32 ? MAX_E * S : 32;
    for (int g = 1; g <= MAX_GROUPS; ++g) {
      if (B % g != 0) continue;
      if (B / g <= cap) { G = g; Ng = B / g; break; }
    }
    if (G == 0) return pl;
  }
  if (G > MAX_GROUPS || Ng > MAX_E * S || Ng > 256) return pl;
  int Npad = (Ng + 15) / 16 * 16;
  if (2 * Npad > 512) return pl;
  int nstages = 4;
  while (nstages > 2 && plan_smem(S, Kc, Npad, nstages) > smem_cap) --nstages;
  if (plan_smem(S, Kc, Npad, nstages) > smem_cap) return pl;
  pl.S = S; pl.Kc = Kc; pl.G = G; pl.Ng = Ng; pl.Npad = Npad; pl.nstages = nstages;
  pl.smem = plan_smem(S, Kc, Npad, nstages);
  pl.ok = true;
  return pl;
}

template <bool BWD>
int launch_rec_tc(const RecPlan& pl, RecTcParams& p, const void* W, const void* state,
                  cudaStream_t stream) {
  auto kern = rec_tc_kernel<BWD>;
  CUtensorMap tmW, tmState;
  ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmW, W, (uint64_t)p.d, (uint64_t)p.d, (uint64_t)p.d, TILE_M));
  ELMAN_RETURN_IF(make_state_tmap(&tmState, state, p.T + 1, p.B, p.d, pl.Npad));
  ELMAN_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)pl.smem));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((p.d / TILE_M) * pl.S);
  cfg.blockDim = dim3(NUM_THREADS);
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
  ELMAN_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, tmW, tmState, p));
  count_launch(true);
  return ELMAN_OK;
}

void fill_plan(const RecPlan& pl, RecTcParams& p) {
  p.S = pl.S; p.Kc = pl.Kc; p.G = pl.G; p.Ng = pl.Ng; p.Npad = pl.Npad; p.nstages = pl.nstages;
  p.R = p.d / TILE_M;
  p.spin_limit = options().spin_limit;
  p.status = device_status_ptr();
}

}  // namespace

bool rec_tc_supported(int T, int B, int d) { return make_plan(T, B, d).ok; }

size_t rec_tc_sync_bytes() {
  return (size_t)(MAX_GROUPS * MAX_S * COUNTER_STRIDE + 64) * sizeof(int);
}

int rec_fwd_tc(const RecFwdArgs& a, cudaStream_t stream) {
  RecPlan pl = make_plan(a.T, a.B, a.d);
  if (!pl.ok) return set_error(ELMAN_ERR_UNSUPPORTED, "shape not supported by the tensor-core recurrence");
  RecTcParams p{};
  p.T = a.T; p.B = a.B; p.d = a.d;
  fill_plan(pl, p);
  p.pre = (const bf16*)a.pre; p.g = (const bf16*)a.g; p.h = (bf16*)a.h; p.y = (bf16*)a.y;
  p.v = (bf16*)a.v;
  ELMAN_CUDA_CHECK(cudaMemsetAsync(a.sync, 0, rec_tc_sync_bytes(), stream));
  p.ready = a.sync;
  p.abort_word = a.sync + MAX_GROUPS * MAX_S * COUNTER_STRIDE;
  return launch_rec_tc<false>(pl, p, a.W, a.h, stream);
}

int rec_bwd_tc(const RecBwdArgs& a, cudaStream_t stream) {
  RecPlan pl = make_plan(a.T, a.B, a.d);
  if (!pl.ok) return set_error(ELMAN_ERR_UNSUPPORTED, "shape not supported by the tensor-core recurrence");
  RecTcParams p{};
  p.T = a.T; p.B = a.B; p.d = a.d;
  fill_plan(pl, p);
  p.h_in = (const bf16*)a.h; p.v_in = (const bf16*)a.v; p.g = (const bf16*)a.g;
  p.dy = (const bf16*)a.dy; p.dv = (bf16*)a.dv; p.dg = (bf16*)a.dg; p.db = a.db;
  ELMAN_CUDA_CHECK(cudaMemsetAsync(a.sync, 0, rec_tc_sync_bytes(), stream));
  // slot T of dv is the all-zero "gradient from the future" read by the first step
  ELMAN_CUDA_CHECK(cudaMemsetAsync((bf16*)a.dv + (size_t)a.T * a.B * a.d, 0,
                                   (size_t)a.B * a.d * sizeof(bf16), stream));
  p.ready = a.sync;
  p.abort_word = a.sync + MAX_GROUPS * MAX_S * COUNTER_STRIDE;
  return launch_rec_tc<true>(pl, p, a.Wt, a.dv, stream);
}

}  // namespace elman

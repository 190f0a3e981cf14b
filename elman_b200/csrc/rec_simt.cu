// CUDA-core persistent recurrence kernels (any shape, fp32 or bf16 storage, fp32 math).
//
// One cooperative launch runs all T steps.  Every CTA owns a contiguous block of
// output features.  Per step it stages the previous state (h_{t-1}, or dv_{t+1}
// in the backward sweep) from L2 into shared memory, computes its rows of the
// mat-vec product with one warp per row, applies the fused tanh / gate epilogue
// and meets the other CTAs at a bounded grid barrier.
//
// Forward (reference: MambaGatedElmanForward::Run time loop,
// elman/cuda/lib/mamba_gated_elman_gpu.cu.cc:451-473, and FusedTanhGateKernel :165-233):
//   v_t = pre_t + h_{t-1} W^T ; h_t = tanh(v_t) ; y_t = h_t * silu(g_t)
// Backward (reference: MambaGatedElmanBackward::Run loop :527-558 and kernels :240-372):
//   dh = dy_t*silu(g_t) + dv_{t+1} W ; dg_t = dy_t*h_t*silu'(g_t) ;
//   dv_t = dh*(1 - tanh(v_t)^2) ; db += sum_b dv_t
// The low-rank variants replace the single product by U (V state), with the rank-r
// intermediate exchanged through a small fp32 buffer and a second barrier
// (reference: pure_lowrank_elman_fused_gpu.cu.cc:244-270 and :355-501).
#include <cooperative_groups.h>

#include "common.cuh"

namespace elman {

namespace {

constexpr int NTHREADS = 256;
constexpr int NWARPS = NTHREADS / 32;
constexpr int BSUB = 8;  // batch elements accumulated in registers at a time

struct SyncState {
  int* counter;     // monotonically increasing arrival counter
  int* abort_flag;  // set when any CTA gives up
  int* status;      // host-visible status word
  long spin_limit;
  int target;       // arrivals expected at the next barrier
  int kernel_id;
};

// Returns false if the barrier was abandoned (timeout here or in another CTA).
__device__ __forceinline__ bool grid_barrier(SyncState& s, int step) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    red_release_gpu_add(s.counter, 1);
    bool ok = true;
    long spins = 0;
    while (ld_acquire_gpu(s.counter) < s.target) {
      if (++spins > s.spin_limit || ld_relaxed_gpu(s.abort_flag) != 0) { ok = false; break; }
    }
    if (!ok) {
      if (atomicExch(s.abort_flag, 1) == 0) report_timeout(s.status, s.kernel_id, step);
    }
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  s.target += gridDim.x;
  return s_ok != 0;
}

template <typename T> __device__ __forceinline__ T ld_cg(const T* p);
template <> __device__ __forceinline__ float ld_cg<float>(const float* p) { return __ldcg(p); }
template <> __device__ __forceinline__ bf16 ld_cg<bf16>(const bf16* p) {
  unsigned short u = __ldcg(reinterpret_cast<const unsigned short*>(p));
  return __ushort_as_bfloat16(u);
}

// Stage state[b0 .. b0+nb)[0..K) (global, written by other CTAs during this
// kernel, hence L2-only loads) into shared memory as floats, row stride K.
template <typename TS>
__device__ __forceinline__ void stage_state(const TS* __restrict__ state, long row_stride,
                                            int b0, int nb, int K, float* hs) {
  for (int i = threadIdx.x; i < nb * K; i += NTHREADS) {
    int b = i / K, k = i - b * K;
    hs[i] = to_f(ld_cg(state + (long)(b0 + b) * row_stride + k));
  }
}

// For the rows [r_lo, r_hi) owned by this CTA compute acc[b] = sum_k Wm[r,k]*hs[b,k]
// for the nb staged batch rows and hand (r, b, acc) to `emit` (called by one lane).
template <typename T, typename Emit>
__device__ __forceinline__ void rows_times_state(const T* __restrict__ Wm, long ldw, int K,
                                                 int r_lo, int r_hi, const float* hs, int b0,
                                                 int nb, Emit emit) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = r_lo + warp; r < r_hi; r += NWARPS) {
    const T* wrow = Wm + (long)r * ldw;
    for (int bs = 0; bs < nb; bs += BSUB) {
      float acc[BSUB];
#pragma unroll
      for (int j = 0; j < BSUB; ++j) acc[j] = 0.f;
      for (int k = lane; k < K; k += 32) {
        float w = to_f(wrow[k]);
#pragma unroll
        for (int j = 0; j < BSUB; ++j) {
          int b = bs + j < nb ? bs + j : nb - 1;  // clamp: duplicates are discarded below
          acc[j] = fmaf(w, hs[b * K + k], acc[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < BSUB; ++j) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
      }
      // lane j handles batch element bs+j
      float mine = 0.f;
#pragma unroll
      for (int j = 0; j < BSUB; ++j) if (lane == j) mine = acc[j];
      bool valid = lane < BSUB && bs + lane < nb;
      emit(r, b0 + bs + lane, mine, valid);
    }
  }
}

struct FwdEpilogue {
  int t, B, d;
  template <typename T>
  __device__ __forceinline__ void run(const T* pre, const T* g, T* h, T* y, T* v, int r, int b,
                                      float acc) const {
    long idx = ((long)t * B + b) * d + r;
    float val = acc + to_f(pre[idx]);
    float hv = tanhf(val);
    if (v != nullptr) v[idx] = from_f<T>(val);
    h[idx + (long)B * d] = from_f<T>(hv);
    // no gate input: the state gates itself, y = h silu(h), with h as stored
    const float gz = g != nullptr ? to_f(g[idx]) : to_f(from_f<T>(hv));
    y[idx] = from_f<T>(hv * siluf_(gz));
  }
};

// One backward element; returns dv (after rounding to T, as stored).
template <typename T>
__device__ __forceinline__ float bwd_element(const T* h, const T* v, const T* g, const T* dy,
                                             T* dv, T* dg, long idx, long BD, float acc) {
  float dyv = to_f(dy[idx]);
  float hv = to_f(h[idx + BD]);
  float dh;
  if (g != nullptr) {
    float gz = to_f(g[idx]);
    dh = dyv * siluf_(gz) + acc;
    dg[idx] = from_f<T>(dyv * hv * dsiluf_(gz));
  } else {   // self gate y = h silu(h): d y / d h = silu(h) + h silu'(h)
    dh = dyv * (siluf_(hv) + hv * dsiluf_(hv)) + acc;
  }
  float th = tanhf(to_f(v[idx]));
  float dvv = dh * (1.f - th * th);
  dv[idx] = from_f<T>(dvv);
  return dvv;
}

inline __device__ void cta_rows(int total, int& lo, int& hi) {
  int per = (total + gridDim.x - 1) / gridDim.x;
  lo = blockIdx.x * per;
  hi = lo + per < total ? lo + per : total;
  if (lo > total) lo = total;
}

struct DenseParams {
  int T, B, d, Bc;
  const void* W; const void* pre; const void* g; const void* h_in; const void* v_in;
  const void* dy;
  void* h; void* y; void* v; void* dv; void* dg; float* db;
  SyncState sync;
};

template <typename T>
__global__ void __launch_bounds__(NTHREADS) rec_fwd_simt_kernel(DenseParams p) {
  extern __shared__ float hs[];
  const T* W = (const T*)p.W;
  T* h = (T*)p.h;
  int r_lo, r_hi;
  cta_rows(p.d, r_lo, r_hi);
  SyncState sync = p.sync;
  const long BD = (long)p.B * p.d;
  for (int t = 0; t < p.T; ++t) {
    for (int b0 = 0; b0 < p.B; b0 += p.Bc) {
      int nb = p.B - b0 < p.Bc ? p.B - b0 : p.Bc;
      stage_state<T>(h + (long)t * BD, p.d, b0, nb, p.d, hs);
      __syncthreads();
      FwdEpilogue ep{t, p.B, p.d};
      rows_times_state<T>(W, p.d, p.d, r_lo, r_hi, hs, b0, nb,
                          [&](int r, int b, float acc, bool valid) {
                            if (valid)
                              ep.run<T>((const T*)p.pre, (const T*)p.g, h, (T*)p.y, (T*)p.v, r, b,
                                        acc);
                          });
      __syncthreads();
    }
    if (t + 1 < p.T) {
      if (!grid_barrier(sync, t)) return;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(NTHREADS) rec_bwd_simt_kernel(DenseParams p) {
  extern __shared__ float hs[];
  const T* Wt = (const T*)p.W;
  T* dv = (T*)p.dv;
  int r_lo, r_hi;
  cta_rows(p.d, r_lo, r_hi);
  SyncState sync = p.sync;
  const long BD = (long)p.B * p.d;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // db partial sums live in shared memory after the staged state.  Each entry is
  // only ever touched by lane 0 of the warp that owns the row, in a fixed order,
  // so the bias gradient is bit-reproducible (the reference uses float atomics).
  float* db_s = hs + (long)p.Bc * p.d;
  for (int i = threadIdx.x; i < r_hi - r_lo; i += NTHREADS) db_s[i] = 0.f;
  __syncthreads();

  for (int t = p.T - 1; t >= 0; --t) {
    // slot T of dv holds the gradient carried in from the steps after this call
    // (all zero when there are none), so the first step reads it like any other
    const bool has_rec = true;
    for (int b0 = 0; b0 < p.B; b0 += p.Bc) {
      int nb = p.B - b0 < p.Bc ? p.B - b0 : p.Bc;
      if (has_rec) {
        stage_state<T>(dv + (long)(t + 1) * BD, p.d, b0, nb, p.d, hs);
        __syncthreads();
      }
      auto emit = [&](int r, int b, float acc, bool valid) {
        float dvv = 0.f;
        if (valid) {
          long idx = ((long)t * p.B + b) * p.d + r;
          dvv = bwd_element<T>((const T*)p.h_in, (const T*)p.v_in, (const T*)p.g,
                               (const T*)p.dy, dv, (T*)p.dg, idx, BD, acc);
        }
        // fixed-order sum over the BSUB lanes that hold batch elements
#pragma unroll
        for (int o = BSUB / 2; o > 0; o >>= 1) dvv += __shfl_xor_sync(0xffffffffu, dvv, o);
        if (lane == 0) db_s[r - r_lo] += dvv;
      };
      if (has_rec) {
        rows_times_state<T>(Wt, p.d, p.d, r_lo, r_hi, hs, b0, nb, emit);
        __syncthreads();
      } else {
        for (int r = r_lo + warp; r < r_hi; r += NWARPS)
          for (int bs = 0; bs < nb; bs += BSUB)
            emit(r, b0 + bs + lane, 0.f, lane < BSUB && bs + lane < nb);
      }
    }
    if (t > 0) {
      if (!grid_barrier(sync, t)) return;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < r_hi - r_lo; i += NTHREADS) p.db[r_lo + i] = db_s[i];
}

struct LowRankParams {
  int T, B, d, r, Bc1, Bc2, db_off;
  const void* U; const void* V;  // forward: U[d,r], V[r,d]; backward: Vt[d,r] as "U", Ut[r,d] as "V"
  const void* pre; const void* g; const void* h_in; const void* v_in; const void* dy;
  void* h; void* y; void* v; void* dv; void* dg; float* db;
  float* tmp;  // [B,r] rank-r intermediate
  SyncState sync;
};

template <typename T, bool BWD>
__global__ void __launch_bounds__(NTHREADS) lowrank_simt_kernel(LowRankParams p) {
  extern __shared__ float hs[];
  const T* U = (const T*)p.U;
  const T* V = (const T*)p.V;
  int d_lo, d_hi, q_lo, q_hi;
  cta_rows(p.d, d_lo, d_hi);
  cta_rows(p.r, q_lo, q_hi);
  SyncState sync = p.sync;
  const long BD = (long)p.B * p.d;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* tmp = p.tmp;
  float* db_s = hs + p.db_off;
  if (BWD) {
    for (int i = threadIdx.x; i < d_hi - d_lo; i += NTHREADS) db_s[i] = 0.f;
    __syncthreads();
  }
  int step_no = 0;
  for (int s = 0; s < p.T; ++s) {
    const int t = BWD ? p.T - 1 - s : s;
    const bool has_rec = true;   // backward: slot T of dv holds the carried-in gradient (or zeros)
    const T* state = BWD ? (const T*)p.dv + (long)(t + 1) * BD : (const T*)p.h + (long)t * BD;
    if (has_rec) {
      // phase A: tmp[b, q] = sum_k V[q, k] state[b, k]
      for (int b0 = 0; b0 < p.B; b0 += p.Bc1) {
        int nb = p.B - b0 < p.Bc1 ? p.B - b0 : p.Bc1;
        stage_state<T>(state, p.d, b0, nb, p.d, hs);
        __syncthreads();
        rows_times_state<T>(V, p.d, p.d, q_lo, q_hi, hs, b0, nb,
                            [&](int q, int b, float acc, bool valid) {
                              if (valid) tmp[(long)b * p.r + q] = acc;
                            });
        __syncthreads();
      }
      if (!grid_barrier(sync, step_no++)) return;
    }
    // phase B: out[b, j] = sum_q U[j, q] tmp[b, q]  -> epilogue
    for (int b0 = 0; b0 < p.B; b0 += p.Bc2) {
      int nb = p.B - b0 < p.Bc2 ? p.B - b0 : p.Bc2;
      if (has_rec) {
        stage_state<float>(tmp, p.r, b0, nb, p.r, hs);
        __syncthreads();
      }
      auto emit = [&](int j, int b, float acc, bool valid) {
        if (!BWD) {
          if (valid) {
            FwdEpilogue ep{t, p.B, p.d};
            ep.run<T>((const T*)p.pre, (const T*)p.g, (T*)p.h, (T*)p.y, (T*)p.v, j, b, acc);
          }
        } else {
          float dvv = 0.f;
          if (valid) {
            long idx = ((long)t * p.B + b) * p.d + j;
            dvv = bwd_element<T>((const T*)p.h_in, (const T*)p.v_in, (const T*)p.g,
                                 (const T*)p.dy, (T*)p.dv, (T*)p.dg, idx, BD, acc);
          }
#pragma unroll
          for (int o = BSUB / 2; o > 0; o >>= 1) dvv += __shfl_xor_sync(0xffffffffu, dvv, o);
          if (lane == 0) db_s[j - d_lo] += dvv;  // one owner lane per feature: deterministic
        }
      };
      if (has_rec) {
        rows_times_state<T>(U, p.r, p.r, d_lo, d_hi, hs, b0, nb, emit);
        __syncthreads();
      } else {
        for (int j = d_lo + warp; j < d_hi; j += NWARPS)
          for (int bs = 0; bs < nb; bs += BSUB)
            emit(j, b0 + bs + lane, 0.f, lane < BSUB && bs + lane < nb);
      }
    }
    if (s + 1 < p.T) {
      if (!grid_barrier(sync, step_no++)) return;
    }
  }
  if (BWD) {
    __syncthreads();
    for (int i = threadIdx.x; i < d_hi - d_lo; i += NTHREADS) p.db[d_lo + i] = db_s[i];
  }
}

struct LaunchShape {
  int grid;
  int Bc;      // batch rows staged per pass (first product)
  int Bc2;     // batch rows staged per pass (second product, low-rank only)
  int db_off;  // float offset of the db partial sums in dynamic shared memory
  size_t smem;
};

int staged_rows(size_t budget, int B, int K, int* Bc) {
  size_t row_bytes = (size_t)K * sizeof(float);
  if (row_bytes == 0 || row_bytes > budget)
    return set_error(ELMAN_ERR_UNSUPPORTED, "state row of %d floats does not fit shared memory", K);
  int n = (int)(budget / row_bytes);
  if (n > B) n = B;
  if (n > BSUB) n -= n % BSUB;
  *Bc = n;
  return ELMAN_OK;
}

// Picks the batch chunks held in shared memory and a grid that is co-resident.
// K2 > 0 adds a second staged product (low-rank); with_db reserves one float per
// owned row behind the staged state.
template <typename Kern>
int plan_launch(Kern kern, int rows, int B, int K, int K2, bool with_db, LaunchShape* out) {
  int dev = 0;
  ELMAN_CUDA_CHECK(cudaGetDevice(&dev));
  int sms = 0, max_smem = 0;
  ELMAN_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  ELMAN_CUDA_CHECK(cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
  size_t budget = (size_t)max_smem > 65536 ? (size_t)max_smem - 32768 : 16384;
  if (budget > 160 * 1024) budget = 160 * 1024;
  int Bc = 0, Bc2 = 0;
  ELMAN_RETURN_IF(staged_rows(budget, B, K, &Bc));
  size_t floats = (size_t)Bc * K;
  if (K2 > 0) {
    ELMAN_RETURN_IF(staged_rows(budget, B, K2, &Bc2));
    size_t f2 = (size_t)Bc2 * K2;
    if (f2 > floats) floats = f2;
  }
  int grid = (rows + NWARPS - 1) / NWARPS;
  if (grid < 1) grid = 1;
  size_t smem = 0;
  for (int iter = 0; iter < 4; ++iter) {
    int per_cta = (rows + grid - 1) / grid;
    smem = (floats + (with_db ? (size_t)per_cta : 0)) * sizeof(float);
    ELMAN_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem));
    int per_sm = 0;
    ELMAN_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, NTHREADS, smem));
    if (per_sm < 1) return set_error(ELMAN_ERR_CUDA, "recurrence kernel does not fit on an SM");
    if (grid <= sms * per_sm) break;
    grid = sms * per_sm;
  }
  out->grid = grid;
  out->Bc = Bc;
  out->Bc2 = Bc2;
  out->db_off = (int)floats;
  out->smem = smem;
  return ELMAN_OK;
}

SyncState make_sync(int* sync_words, int grid, int kernel_id) {
  SyncState s;
  s.counter = sync_words;
  s.abort_flag = sync_words + 1;
  s.status = device_status_ptr();
  s.spin_limit = options().spin_limit;
  s.target = grid;
  s.kernel_id = kernel_id;
  return s;
}

template <typename Kern, typename P>
int launch_coop(Kern kern, P& params, int grid, size_t smem, cudaStream_t stream) {
  void* args[] = {&params};
  ELMAN_CUDA_CHECK(cudaLaunchCooperativeKernel((const void*)kern, dim3(grid), dim3(NTHREADS), args,
                                               smem, stream));
  count_launch(false);
  return ELMAN_OK;
}

template <typename T>
int launch_dense(bool bwd, DenseParams& p, int* sync_words, cudaStream_t stream) {
  LaunchShape ls;
  if (!bwd) {
    auto kern = rec_fwd_simt_kernel<T>;
    ELMAN_RETURN_IF(plan_launch(kern, p.d, p.B, p.d, 0, false, &ls));
    p.Bc = ls.Bc;
    p.sync = make_sync(sync_words, ls.grid, KID_REC_SIMT);
    return launch_coop(kern, p, ls.grid, ls.smem, stream);
  }
  auto kern = rec_bwd_simt_kernel<T>;
  ELMAN_RETURN_IF(plan_launch(kern, p.d, p.B, p.d, 0, true, &ls));
  p.Bc = ls.Bc;
  p.sync = make_sync(sync_words, ls.grid, KID_REC_SIMT);
  return launch_coop(kern, p, ls.grid, ls.smem, stream);
}

template <typename T, bool BWD>
int launch_lowrank(LowRankParams& p, int* sync_words, cudaStream_t stream) {
  auto kern = lowrank_simt_kernel<T, BWD>;
  LaunchShape ls;
  ELMAN_RETURN_IF(plan_launch(kern, p.d, p.B, p.d, p.r, BWD, &ls));
  p.Bc1 = ls.Bc;
  p.Bc2 = ls.Bc2;
  p.db_off = ls.db_off;
  p.sync = make_sync(sync_words, ls.grid, KID_LOWRANK_SIMT);
  return launch_coop(kern, p, ls.grid, ls.smem, stream);
}

}  // namespace

size_t rec_sync_bytes() { return 256; }

int rec_fwd_generic(int dtype, const RecFwdArgs& a, cudaStream_t stream) {
  if (a.T <= 0 || a.B <= 0 || a.d <= 0) return ELMAN_OK;
  DenseParams p{};
  p.T = a.T; p.B = a.B; p.d = a.d;
  p.W = a.W; p.pre = a.pre; p.g = a.g; p.h = a.h; p.y = a.y; p.v = a.v;
  ELMAN_CUDA_CHECK(cudaMemsetAsync(a.sync, 0, rec_sync_bytes(), stream));
  if (dtype == ELMAN_F32) return launch_dense<float>(false, p, a.sync, stream);
  return launch_dense<bf16>(false, p, a.sync, stream);
}

int rec_bwd_generic(int dtype, const RecBwdArgs& a, cudaStream_t stream) {
  if (a.d > 0) ELMAN_CUDA_CHECK(cudaMemsetAsync(a.db, 0, sizeof(float) * a.d, stream));
  if (a.T <= 0 || a.B <= 0 || a.d <= 0) return ELMAN_OK;
  DenseParams p{};
  p.T = a.T; p.B = a.B; p.d = a.d;
  p.W = a.Wt; p.h_in = a.h; p.v_in = a.v; p.g = a.g; p.dy = a.dy;
  p.dv = a.dv; p.dg = a.dg; p.db = a.db;
  ELMAN_CUDA_CHECK(cudaMemsetAsync(a.sync, 0, rec_sync_bytes(), stream));
  if (dtype == ELMAN_F32) return launch_dense<float>(true, p, a.sync, stream);
  return launch_dense<bf16>(true, p, a.sync, stream);
}

int lowrank_fwd_generic(int dtype, const LowRankFwdArgs& a, cudaStream_t stream) {
  if (a.T <= 0 || a.B <= 0 || a.d <= 0 || a.r <= 0) return ELMAN_OK;
  LowRankParams p{};
  p.T = a.T; p.B = a.B; p.d = a.d; p.r = a.r;
  p.U = a.U; p.V = a.V; p.pre = a.pre; p.g = a.g; p.h = a.h; p.y = a.y; p.v = a.v; p.tmp = a.tmp;
  ELMAN_CUDA_CHECK(cudaMemsetAsync(a.sync, 0, rec_sync_bytes(), stream));
  if (dtype == ELMAN_F32) return launch_lowrank<float, false>(p, a.sync, stream);
  return launch_lowrank<bf16, false>(p, a.sync, stream);
}

int lowrank_bwd_generic(int dtype, const LowRankBwdArgs& a, cudaStream_t stream) {
  if (a.d > 0) ELMAN_CUDA_CHECK(cudaMemsetAsync(a.db, 0, sizeof(float) * a.d, stream));
  if (a.T <= 0 || a.B <= 0 || a.d <= 0 || a.r <= 0) return ELMAN_OK;
  LowRankParams p{};
  p.T = a.T; p.B = a.B; p.d = a.d; p.r = a.r;
  // dh_rec = (dv U) V : first contract over d with U^T [r,d], then over r with V^T [d,r]
  p.V = a.Ut; p.U = a.Vt;
  p.h_in = a.h; p.v_in = a.v; p.g = a.g; p.dy = a.dy; p.dv = a.dv; p.dg = a.dg; p.db = a.db;
  p.tmp = a.tmp;
  ELMAN_CUDA_CHECK(cudaMemsetAsync(a.sync, 0, rec_sync_bytes(), stream));
  if (dtype == ELMAN_F32) return launch_lowrank<float, true>(p, a.sync, stream);
  return launch_lowrank<bf16, true>(p, a.sync, stream);
}

}  // namespace elman

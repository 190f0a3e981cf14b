// Shared declarations of the elman_b200 library: dtype helpers, error plumbing,
// the bounded-wait status word, and the internal kernel-launcher prototypes.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/elman_b200.h"

namespace elman {

typedef __nv_bfloat16 bf16;

// ---------------------------------------------------------------------------
// host-side error handling
// ---------------------------------------------------------------------------
int set_error(int code, const char* fmt, ...);

#define ELMAN_CUDA_CHECK(expr)                                                        \
  do {                                                                                \
    cudaError_t _e = (expr);                                                          \
    if (_e != cudaSuccess)                                                            \
      return ::elman::set_error(ELMAN_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,       \
                                cudaGetErrorString(_e), __FILE__, __LINE__);          \
  } while (0)

#define ELMAN_RETURN_IF(expr)        \
  do {                               \
    int _rc = (expr);                \
    if (_rc != ELMAN_OK) return _rc; \
  } while (0)

#define ELMAN_ARG_CHECK(cond, ...) \
  do {                             \
    if (!(cond)) return ::elman::set_error(ELMAN_ERR_ARG, __VA_ARGS__); \
  } while (0)

// ---------------------------------------------------------------------------
// options / counters (api.cu)
// ---------------------------------------------------------------------------
struct Options {
  long force_generic = 0;
  long spin_limit = 4000000;   // iterations of a device-side poll loop
  long rec_ksplit = 0;
  long rec_groups = 0;
  long time_kernels = 0;
  long rec_trace = 0;
  long rec_mma_warps = 0;
  long rec_direct_publish = 0;
  long rec_w_tmem = 0;
  long gemm_persistent = 0;    // 0 auto, 1 never, 2 always: the persistent 128x256 GEMM kernel
  long gemm_pair = 0;          // 0 auto, 1 never, 2 whenever possible: 256x256 tiles on CTA pairs
  long rec_fin_groups = 0;     // 0 auto (two finalising groups from four batch groups on), 1 = always one
  long rec_large_batch = 1;    // 1: batches over 32 take the wide-group throughput plan
  // Failure-detection test hook: >= 1 makes thread block 0 of the tensor-core kernels wait, at
  // that step (GEMM: K iteration), for something nothing will deliver, so that a real bounded
  // wait runs out and the give-up path of every role executes.  -1 = off.
  long rec_group_cap = 0;      // widest batch group of the throughput plan: 0 auto (64), 16 / 32 / 64
  long rec_replicas = 0;       // batch replicas of the throughput plan: 0 auto, 1 off, n = at most n
  long test_stall_step = -1;
};
Options& options();
void count_launch(bool tensor_core);

// Host-visible status word of the current device (mapped pinned memory).
// Device code writes a non-zero code there when a bounded wait gives up.
int* device_status_ptr();   // device-side alias, or nullptr if unavailable

// kernel ids recorded in the status word
enum KernelId { KID_REC_SIMT = 1, KID_REC_TC_FWD = 2, KID_REC_TC_BWD = 3, KID_GEMM_TC = 4,
                KID_LOWRANK_SIMT = 5, KID_WAIT_PROBE = 6, KID_LOWRANK_TC = 7 };

// ---------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + __expf(-z)); }
__device__ __forceinline__ float siluf_(float z) { return z * sigmoidf_(z); }
__device__ __forceinline__ float dsiluf_(float z) {
  float s = sigmoidf_(z);
  return s * (1.0f + z * (1.0f - s));
}

__device__ __forceinline__ void report_timeout(int* status, int kernel_id, int step) {
  if (status != nullptr) {
    atomicCAS(status, 0, (kernel_id << 24) | (step & 0xFFFFFF));
    __threadfence_system();
  }
}

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_relaxed_gpu(const int* p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// ---------------------------------------------------------------------------
// internal launchers (each returns ELMAN_OK or an error code)
// ---------------------------------------------------------------------------

// C[m,n] = sum_k A(m,k) * B(k,n) (+ bias[n]) (+ C[m,n]); arbitrary element strides.
int gemm_generic(int dtype, int M, int N, int K, const void* A, long sAm, long sAk,
                 const void* B, long sBk, long sBn, const void* bias, void* C, long ldc,
                 int accumulate, cudaStream_t stream);

// C[M,N] = A[M,K] * W[N,K]^T, bf16, TMA + tcgen05.  Returns ELMAN_ERR_UNSUPPORTED
// (without setting an error message) when the shape or alignment rules it out.
int gemm_tc_nt(int M, int N, int K, const bf16* A, int lda, const bf16* W, int ldw,
               const bf16* bias, void* C, int ldc, int c_is_f32, int accumulate,
               cudaStream_t stream);
// General form: a_mn / b_mn != 0 mean the operand is stored [K, M] resp. [K, N]
// (MN-major), which the tensor core reads directly — no transpose pass.
// `splitk`: optional scratch for fp32 partial sums (GEMM_MAX_KSPLIT * M * N floats cover every
// case); with it, shapes with few output tiles and a long K are cut along K.
constexpr int GEMM_MAX_KSPLIT = 4;
// Optional epilogue of the layer's input projection: the N = 2*split output columns are not
// stored as one matrix but as three dense [M, split] ones — columns [0, split) raw into C and
// silu-activated into C_act, columns [split, 2*split) into C_hi.  split % 32 == 0, bf16 out.
// mode 1 (the [h;x] gate of the E1 extension): N = split; the epilogue adds the matrix C_hi
// (the x-part of the gate pre-activation, dense [M, N]) to the product, stores the sum to C and
// aux * silu(sum) to C_act, with aux (the hidden states) dense [M, N].
struct GemmSplit {
  int split;
  void* C_act;
  void* C_hi;
  int mode = 0;
  const void* aux = nullptr;
};
int gemm_tc(int M, int N, int K, const bf16* A, int lda, int a_mn, const bf16* W, int ldw,
            int b_mn, const bf16* bias, void* C, int ldc, int c_is_f32, int accumulate,
            cudaStream_t stream, float* splitk = nullptr, size_t splitk_bytes = 0,
            const GemmSplit* split = nullptr);

// Elementwise layer kernels (layer_ops.cu).
size_t add_rmsnorm_bwd_scratch_bytes(int D);
int add_rmsnorm_fwd(int dtype, long M, int D, const void* x, const float* res_in, const void* w,
                    float eps, float* res_out, void* y, float* rstd, cudaStream_t st);
int add_rmsnorm_bwd(int dtype, long M, int D, const void* dy, const float* dres_out,
                    const float* res_out, const float* rstd, const void* w, float* dres_in,
                    void* dx, void* dw, float* scratch, cudaStream_t st);
int split_silu(int dtype, long M, int d, const void* xz, void* x_raw, void* x_act, void* z,
               cudaStream_t st);
int silu_bwd_concat(int dtype, long M, int d, const void* d_act, const void* x_raw, const void* dz,
                    void* dxz, cudaStream_t st);
// [h;x]-gate extension: y = h * silu(zg);  dzg = dy * h * silu'(zg), t = dy * silu(zg) * scale;
// dst = src * scale;  dst = value
int gate_apply(int dtype, long n, const void* h, const void* zg, void* y, cudaStream_t st);
int gate_backward_prep(int dtype, long n, const void* dy, const void* h, const void* zg, float scale,
                       void* dzg, void* t, cudaStream_t st);
int scale_copy(int dtype, long n, const void* src, float scale, void* dst, cudaStream_t st);
int fill_value(int dtype, long n, float value, void* dst, cudaStream_t st);
// AdamW over flat buffers (train_ops.cu); advances *step by one first.
int adamw_step(int dtype, long n, void* p, const void* g, void* m, void* v, float lr, float beta1,
               float beta2, float eps, float weight_decay, float* step, const float* grad_scale,
               cudaStream_t st);
bool gemm_tc_supported(int M, int N, int K, const void* A, int lda, const void* W, int ldw,
                       const void* C, int ldc, int c_is_f32);

// out[rows, cols] = in[cols, rows]^T for a dense row-major matrix.
int transpose2d(int dtype, int rows_in, int cols_in, const void* in, void* out,
                cudaStream_t stream);
// out[n] = sum_m in[m, n]  (deterministic two-pass; scratch holds 64*N floats).
int column_sum(int dtype, long M, int N, const void* in, void* out, float* scratch,
               cudaStream_t stream);
size_t column_sum_scratch_bytes(int N);
int copy_rows(int dtype, const void* src, void* dst, long n, cudaStream_t stream);
int float_to_dtype(int dtype, const float* src, void* dst, long n, cudaStream_t stream);
// dst[rows_dst, cols_dst] = src[rows, cols], cropped or zero-padded (dense row-major both).
int resize2d(int dtype, const void* src, int rows, int cols, void* dst, int rows_dst, int cols_dst,
             cudaStream_t stream);

// Dense recurrence, CUDA-core persistent kernel.
//   forward : h[t+1] = tanh(pre[t] + h[t] W^T);  y[t] = h[t+1] * silu(g[t])
//   backward: dv[t] = (dy[t]*silu(g[t]) + dv[t+1] Wt^T) * (1 - tanh(v[t])^2), dg[t] = dy*h*silu'(g)
struct RecFwdArgs {
  int T, B, d;
  const void* W;      // [d,d] recurrent matrix ([out,in])
  const void* pre;    // [T,B,d] W_x x_t + b
  const void* g;      // [T,B,d]; null: self gate (dg is then not written and may be null) gate pre-activation; null: the state gates itself, y = h silu(h)
  void* h;            // [T+1,B,d], h[0] already holds h0
  void* y;            // [T,B,d]
  void* v;            // [T,B,d] or null
  int* sync;          // zeroed ints (barrier / step counters)
  int compact = 0;    // tensor-core kernel: prefer the plan with the fewest resident blocks
};
struct RecBwdArgs {
  int T, B, d;
  const void* Wt;     // [d,d] transpose of the recurrent matrix ([in,out])
  const void* h;      // [T+1,B,d]
  const void* v;      // [T,B,d]
  const void* g;      // [T,B,d]
  const void* dy;     // [T,B,d]
  void* dv;           // [T,B,d]
  void* dg;           // [T,B,d]
  float* db;          // [d] fp32 sum over t,b of dv
  int* sync;
  int compact = 0;
};
size_t rec_sync_bytes();
int rec_fwd_generic(int dtype, const RecFwdArgs& a, cudaStream_t stream);
int rec_bwd_generic(int dtype, const RecBwdArgs& a, cudaStream_t stream);

// Low-rank (E5) recurrence, CUDA-core persistent kernel: the recurrent term is
// U (V state) with V:[r,d], U:[d,r]; tmp holds the rank-r intermediate [B,r] floats x2.
struct LowRankFwdArgs {
  int T, B, d, r;
  const void* U;      // [d,r]
  const void* V;      // [r,d]
  const void* pre; const void* g; void* h; void* y; void* v;
  float* tmp;         // 2*B*r floats
  int* sync;
};
struct LowRankBwdArgs {
  int T, B, d, r;
  const void* Ut;     // [r,d] = U^T
  const void* Vt;     // [d,r] = V^T
  const void* h; const void* v; const void* g; const void* dy;
  void* dv; void* dg; float* db;
  float* tmp;
  int* sync;
};
int lowrank_fwd_generic(int dtype, const LowRankFwdArgs& a, cudaStream_t stream);
int lowrank_bwd_generic(int dtype, const LowRankBwdArgs& a, cudaStream_t stream);

// Dense recurrence, bf16, tcgen05 + TMA persistent cluster kernel.
// Batch replicas of a recurrence grid (throughput plan); the backward kernel writes one row of
// bias-gradient sums per replica, so callers give its `db` REC_MAX_REPLICAS * d floats.
constexpr int REC_MAX_REPLICAS = 4;
bool rec_tc_supported(int T, int B, int d, int bwd);   // per direction: the plans differ
// resident thread blocks of one launch (compact: smallest-footprint plan), 0 if unsupported
int rec_tc_blocks(int T, int B, int d, int compact);
size_t rec_tc_sync_bytes();
int rec_fwd_tc(const RecFwdArgs& a, cudaStream_t stream);
int rec_bwd_tc(const RecBwdArgs& a, cudaStream_t stream);
// Copies the cycle stamps of the last traced launch (option rec_trace) to the host.
int rec_tc_copy_trace(long long* dst, int max_entries);
void set_last_trace(long long* device_buffer);   // the buffer the next copy reads
constexpr size_t kTraceBytes = 64 * 16 * sizeof(long long);

// Low-rank (E5) recurrence, bf16, tcgen05: one cluster of d/128 CTAs, the rank-r
// intermediate exchanged through distributed shared memory only.
//   forward : in0 = pre, in1 = gate, state = h [T+1,B,d] (h[0] filled), out0 = v (or null),
//             out1 = y
//   backward: in0 = gate, in1 = dy, in2 = h [T+1,B,d], in3 = v, state = dv [T+1,B,d],
//             out0 = dgate, db = fp32 [d]; Urole = V^T [d,r], Vrole = U^T [r,d]
struct LowRankTcArgs {
  int T, B, d, r, bwd;
  const void* Urole;   // [d, r]  second product
  const void* Vrole;   // [r, d]  first product
  const void* in0; const void* in1; const void* in2; const void* in3;
  void* state; void* out0; void* out1; float* db;
  void* UP; void* VP;  // scratch for the zero-padded factors (lowrank_tc_pad_bytes)
  int* sync;           // 256 bytes
  long long* trace = nullptr;   // optional 64 x 16 cycle stamps (option rec_trace)
};
bool lowrank_tc_supported(int T, int B, int d, int r, int bwd);
int lowrank_tc_blocks(int T, int B, int d, int r);   // resident blocks (one cluster), 0 if unsupported
void lowrank_tc_pad_bytes(int d, int r, size_t* up_bytes, size_t* vp_bytes);
int lowrank_tc(const LowRankTcArgs& a, cudaStream_t stream);

// C1 = A^T B1 and C2 = A^T B2 in one launch (csrc/gemm_tc.cu); ELMAN_ERR_UNSUPPORTED (without a
// recorded error message) when the shapes do not allow it.
int gemm_tc_dual_tn(int M, int N, int K, const bf16* A, const bf16* B1, const bf16* B2, void* C1,
                    void* C2, cudaStream_t stream);

// Spectral normalisation of a [d, d] matrix (csrc/spectral.cu): three power-iteration steps
// from u (advanced in place), v and sigma saved for the backward pass.
int spectral_norm_fwd(int dtype, int d, const void* W, void* u, float* v, float* sigma, void* W_eff,
                      float target, float eps, int iters, cudaStream_t st);
int spectral_norm_bwd(int dtype, int d, const void* W, const void* u, const float* v,
                      const float* sigma, const void* G, void* dW, int accumulate, float target,
                      float eps, cudaStream_t st);

}  // namespace elman

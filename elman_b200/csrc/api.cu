// C ABI of the library: argument checks, workspace carving and the sequence of
// kernels behind each entry point declared in include/elman_b200.h.
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "common.cuh"

namespace elman {

// ---------------------------------------------------------------------------
// errors, options, counters, status word
// ---------------------------------------------------------------------------
static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

Options& options() {
  static Options o;
  return o;
}

static std::atomic<long> g_launches{0};
static std::atomic<long> g_tc_launches{0};
void count_launch(bool tensor_core) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (tensor_core) g_tc_launches.fetch_add(1, std::memory_order_relaxed);
}

// One host-mapped status word per device, created on first use.
static constexpr int kMaxDevices = 64;
static int* g_status_host[kMaxDevices] = {nullptr};
static int* g_status_dev[kMaxDevices] = {nullptr};

static int ensure_status(int dev) {
  if (dev < 0 || dev >= kMaxDevices) return -1;
  if (g_status_host[dev] != nullptr) return 0;
  int* hp = nullptr;
  if (cudaHostAlloc((void**)&hp, 64, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  memset(hp, 0, 64);
  int* dp = nullptr;
  if (cudaHostGetDevicePointer((void**)&dp, hp, 0) != cudaSuccess) {
    cudaGetLastError();
    cudaFreeHost(hp);
    return -1;
  }
  g_status_host[dev] = hp;
  g_status_dev[dev] = dp;
  return 0;
}

// Set while an entry point that promises not to allocate is running on this thread.
static thread_local bool g_no_alloc = false;

int* device_status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  if (g_no_alloc) {  // use the status word only if an earlier call already created it
    return (dev >= 0 && dev < kMaxDevices) ? g_status_dev[dev] : nullptr;
  }
  if (ensure_status(dev) != 0) return nullptr;
  return g_status_dev[dev];
}

static int check_status_on_entry() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return ELMAN_OK;
  if (dev < 0 || dev >= kMaxDevices || g_status_host[dev] == nullptr) return ELMAN_OK;
  int code = *(volatile int*)g_status_host[dev];
  if (code != 0)
    return set_error(ELMAN_ERR_TIMEOUT,
                     "an earlier launch gave up a bounded device-side wait (kernel %d, step %d); "
                     "results of that launch are invalid",
                     (code >> 24) & 0xFF, code & 0xFFFFFF);
  return ELMAN_OK;
}

// ---------------------------------------------------------------------------
// workspace carving
// ---------------------------------------------------------------------------
struct Carver {
  char* base;
  size_t off = 0;
  explicit Carver(void* p) : base((char*)p) {}
  void* take(size_t bytes) {
    off = (off + 255) & ~(size_t)255;
    void* p = base ? base + off : nullptr;
    off += bytes;
    return p;
  }
  size_t total() const { return (off + 255) & ~(size_t)255; }
};

static inline size_t esize(int dtype) { return dtype == ELMAN_F32 ? 4 : 2; }

static int check_common(int dtype, int T, int B, int d) {
  ELMAN_ARG_CHECK(dtype == ELMAN_F32 || dtype == ELMAN_BF16, "unknown dtype %d", dtype);
  ELMAN_ARG_CHECK(T >= 0 && B >= 0 && d >= 0, "negative size (T=%d B=%d d=%d)", T, B, d);
  ELMAN_ARG_CHECK((long)T * B * d < (1L << 40), "tensor too large");
  return check_status_on_entry();
}

#define REQUIRE_PTR(p) ELMAN_ARG_CHECK((p) != nullptr, "argument %s is NULL", #p)

static bool use_tc(int dtype) { return dtype == ELMAN_BF16 && options().force_generic == 0; }

// C[M,N] = A[M,K] W[N,K]^T (+bias) (+C): tcgen05 when possible, CUDA cores otherwise.
static int proj_nt(int dtype, int M, int N, int K, const void* A, int lda, const void* W, int ldw,
                   const void* bias, void* C, int ldc, int accumulate, cudaStream_t st) {
  if (M == 0 || N == 0) return ELMAN_OK;
  if (use_tc(dtype) && gemm_tc_supported(M, N, K, A, lda, W, ldw, C, ldc, 0)) {
    return gemm_tc_nt(M, N, K, (const bf16*)A, lda, (const bf16*)W, ldw, (const bf16*)bias, C, ldc,
                      0, accumulate, st);
  }
  return gemm_generic(dtype, M, N, K, A, lda, 1, W, 1, ldw, bias, C, ldc, accumulate, st);
}

// C[M,N] = A[M,K] Bm[K,N] (+C).  Bt is scratch for Bm^T (K*N elements) used by the
// tensor-core path, or NULL to force the strided CUDA-core kernel.
static int gemm_nn(int dtype, int M, int N, int K, const void* A, int lda, const void* Bm, int ldb,
                   void* Bt, void* C, int ldc, int accumulate, cudaStream_t st) {
  if (M == 0 || N == 0) return ELMAN_OK;
  (void)Bt;
  if (use_tc(dtype) && (N & 7) == 0 && gemm_tc_supported(M, N, K, A, lda, Bm, ldb, C, ldc, 0)) {
    // Bm is [K, N] with N contiguous: an MN-major B operand, read in place
    return gemm_tc(M, N, K, (const bf16*)A, lda, 0, (const bf16*)Bm, ldb, 1, nullptr, C, ldc, 0,
                   accumulate, st);
  }
  return gemm_generic(dtype, M, N, K, A, lda, 1, Bm, ldb, 1, nullptr, C, ldc, accumulate, st);
}

// C[M,N] = Am^T Bm where the inputs are stored as Am[K,M] and Bm[K,N] (sum over the
// leading "row" index, K = T*B): both operands are MN-major for the tensor core and are
// read in place.  `splitk` is optional scratch for fp32 partial sums over K ranges.
// The two weight gradients that share dv: dW_a = dv^T a, dW_b = dv^T b, [d, d] each.
static int gemm_tn(int dtype, int M, int N, long K, const void* Am, const void* Bm, void* C,
                   cudaStream_t st, float* splitk = nullptr, size_t splitk_bytes = 0,
                   int accumulate = 0);
static int weight_grads_pair(int dtype, int d, long TB, const void* dv, const void* a, void* dW_a,
                             const void* b, void* dW_b, cudaStream_t st, float* splitk,
                             size_t splitk_bytes) {
  if (use_tc(dtype) && TB < (1L << 31)) {
    const int rc = gemm_tc_dual_tn(d, d, (int)TB, (const bf16*)dv, (const bf16*)a, (const bf16*)b,
                                   dW_a, dW_b, st);
    if (rc != ELMAN_ERR_UNSUPPORTED) return rc;
  }
  ELMAN_RETURN_IF(gemm_tn(dtype, d, d, TB, dv, a, dW_a, st, splitk, splitk_bytes, 0));
  return gemm_tn(dtype, d, d, TB, dv, b, dW_b, st, splitk, splitk_bytes, 0);
}

static size_t splitk_scratch_bytes(int dtype, int M, int N) {
  return dtype == ELMAN_BF16 ? (size_t)GEMM_MAX_KSPLIT * M * N * sizeof(float) : 0;
}
static int gemm_tn(int dtype, int M, int N, long K, const void* Am, const void* Bm, void* C,
                   cudaStream_t st, float* splitk, size_t splitk_bytes, int accumulate) {
  if (M == 0 || N == 0) return ELMAN_OK;
  if (use_tc(dtype) && K < (1L << 31) && (M & 7) == 0 && (N & 7) == 0 && (K & 7) == 0 &&
      gemm_tc_supported(M, N, (int)K, Am, M, Bm, N, C, N, 0)) {
    return gemm_tc(M, N, (int)K, (const bf16*)Am, M, 1, (const bf16*)Bm, N, 1, nullptr, C, N, 0,
                   accumulate, st, splitk, splitk_bytes);
  }
  return gemm_generic(dtype, M, N, (int)K, Am, 1, M, Bm, N, 1, nullptr, C, N, accumulate, st);
}

// Optional per-phase timing with CUDA events on the caller's stream (option
// "time_kernels"): phase 0 = forward recurrence, 1 = backward recurrence,
// 2 = forward projection GEMM(s), 3 = backward GEMMs and their transposes.
static constexpr int kPhases = 4;
static cudaEvent_t g_ev[kPhases][2];
static bool g_ev_ready = false;
static bool g_ev_recorded[kPhases] = {false, false, false, false};

struct PhaseTimer {
  int phase;
  cudaStream_t st;
  bool on;
  PhaseTimer(int ph, cudaStream_t s)
      : phase(ph), st(s), on(options().time_kernels != 0 && !g_no_alloc) {
    if (!on) return;
    if (!g_ev_ready) {
      for (int i = 0; i < kPhases; ++i)
        for (int j = 0; j < 2; ++j) cudaEventCreate(&g_ev[i][j]);
      g_ev_ready = true;
    }
    cudaEventRecord(g_ev[phase][0], st);
  }
  ~PhaseTimer() {
    if (!on) return;
    cudaEventRecord(g_ev[phase][1], st);
    g_ev_recorded[phase] = true;
  }
};

static bool dense_tc_ok(int dtype, int T, int B, int d, int bwd) {
  return use_tc(dtype) && rec_tc_supported(T, B, d, bwd);
}

// ---------------------------------------------------------------------------
// E1
// ---------------------------------------------------------------------------
struct E1FwdWs { void* pre; int* sync; };
static size_t carve_e1_fwd(int dtype, int T, int B, int d, void* ws, E1FwdWs* o) {
  Carver c(ws);
  o->pre = c.take((size_t)T * B * d * esize(dtype));
  size_t sb = rec_sync_bytes() > rec_tc_sync_bytes() ? rec_sync_bytes() : rec_tc_sync_bytes();
  o->sync = (int*)c.take(sb);
  return c.total();
}

struct E1BwdWs { void* Wt; void* dv; float* db; int* sync; void* WxT; float* splitk; size_t splitk_bytes; };
static size_t carve_e1_bwd(int dtype, int T, int B, int d, void* ws, E1BwdWs* o) {
  Carver c(ws);
  size_t es = esize(dtype);
  o->Wt = c.take((size_t)d * d * es);
  o->dv = c.take((size_t)(T + 1) * B * d * es);  // slot T: zero "gradient from the future"
  o->db = (float*)c.take((size_t)REC_MAX_REPLICAS * d * sizeof(float));
  size_t sb = rec_sync_bytes() > rec_tc_sync_bytes() ? rec_sync_bytes() : rec_tc_sync_bytes();
  o->sync = (int*)c.take(sb);
  o->WxT = nullptr;  // the GEMMs read transposed operands in place
  o->splitk_bytes = splitk_scratch_bytes(dtype, d, d);   // partial sums of the dW GEMMs
  o->splitk = o->splitk_bytes ? (float*)c.take(o->splitk_bytes) : nullptr;
  return c.total();
}

static int run_rec_fwd(int dtype, int T, int B, int d, const void* W, const void* pre,
                       const void* g, void* h, void* y, void* v, int* sync, cudaStream_t st,
                       int compact = 0) {
  PhaseTimer timer(0, st);
  RecFwdArgs a{T, B, d, W, pre, g, h, y, v, sync};
  a.compact = compact;
  if (dense_tc_ok(dtype, T, B, d, 0)) {
    // a plan that was co-resident when it was made may not be at launch time (another
    // context holds SMs): nothing was launched then, and the CUDA-core kernel takes over
    const int rc = rec_fwd_tc(a, st);
    if (rc != ELMAN_ERR_UNSUPPORTED) return rc;
  }
  return rec_fwd_generic(dtype, a, st);
}

// dv_in: [B,d] gradient of the pre-activation of the step after this call's last
// one (null = none); it becomes slot T of dv, the state the first reverse step reads.
static int run_rec_bwd(int dtype, int T, int B, int d, const void* Wt, const void* h,
                       const void* v, const void* g, const void* dy, void* dv, void* dg, float* db,
                       int* sync, const void* dv_in, cudaStream_t st, int compact = 0) {
  {
    const size_t slot = (size_t)B * d * esize(dtype);
    char* last = (char*)dv + (size_t)T * slot;
    if (dv_in != nullptr)
      ELMAN_CUDA_CHECK(cudaMemcpyAsync(last, dv_in, slot, cudaMemcpyDeviceToDevice, st));
    else
      ELMAN_CUDA_CHECK(cudaMemsetAsync(last, 0, slot, st));
  }
  PhaseTimer timer(1, st);
  RecBwdArgs a{T, B, d, Wt, h, v, g, dy, dv, dg, db, sync};
  a.compact = compact;
  if (dense_tc_ok(dtype, T, B, d, 1)) {
    const int rc = rec_bwd_tc(a, st);
    if (rc != ELMAN_ERR_UNSUPPORTED) return rc;   // see run_rec_fwd
  }
  return rec_bwd_generic(dtype, a, st);
}

}  // namespace elman

using namespace elman;

extern "C" {

int elman_b200_version(void) { return 100; }

const char* elman_b200_last_error(void) { return g_err; }

int elman_b200_device_status(int* detail, int clear) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return set_error(ELMAN_ERR_CUDA, "no current CUDA device");
  }
  if (detail) *detail = 0;
  if (dev < 0 || dev >= kMaxDevices || g_status_host[dev] == nullptr) return ELMAN_OK;
  int code = *(volatile int*)g_status_host[dev];
  if (detail) *detail = code;
  if (clear) *(volatile int*)g_status_host[dev] = 0;
  return code == 0 ? ELMAN_OK : ELMAN_ERR_TIMEOUT;
}

int elman_b200_set_option(const char* name, long value) {
  if (name == nullptr) return set_error(ELMAN_ERR_ARG, "option name is NULL");
  Options& o = options();
  if (!strcmp(name, "force_generic")) o.force_generic = value;
  else if (!strcmp(name, "spin_limit")) o.spin_limit = value < 1 ? 1 : value;
  else if (!strcmp(name, "rec_ksplit")) o.rec_ksplit = value;
  else if (!strcmp(name, "rec_groups")) o.rec_groups = value;
  else if (!strcmp(name, "time_kernels")) o.time_kernels = value;
  else if (!strcmp(name, "rec_trace")) o.rec_trace = value;
  else if (!strcmp(name, "rec_mma_warps")) o.rec_mma_warps = value;
  else if (!strcmp(name, "rec_direct_publish")) o.rec_direct_publish = value;
  else if (!strcmp(name, "rec_w_tmem")) o.rec_w_tmem = value;
  else if (!strcmp(name, "rec_large_batch")) o.rec_large_batch = value;
  else if (!strcmp(name, "rec_fin_groups")) o.rec_fin_groups = value;
  else if (!strcmp(name, "gemm_persistent")) o.gemm_persistent = value;
  else if (!strcmp(name, "gemm_pair")) o.gemm_pair = value;
  else if (!strcmp(name, "test_stall_step")) o.test_stall_step = value;
  else if (!strcmp(name, "rec_replicas")) o.rec_replicas = value;
  else if (!strcmp(name, "rec_group_cap")) o.rec_group_cap = value;
  else return set_error(ELMAN_ERR_ARG, "unknown option '%s'", name);
  return ELMAN_OK;
}

long elman_b200_get_option(const char* name) {
  if (name == nullptr) return -1;
  Options& o = options();
  if (!strcmp(name, "force_generic")) return o.force_generic;
  if (!strcmp(name, "spin_limit")) return o.spin_limit;
  if (!strcmp(name, "rec_ksplit")) return o.rec_ksplit;
  if (!strcmp(name, "rec_groups")) return o.rec_groups;
  if (!strcmp(name, "time_kernels")) return o.time_kernels;
  if (!strcmp(name, "rec_trace")) return o.rec_trace;
  if (!strcmp(name, "rec_mma_warps")) return o.rec_mma_warps;
  if (!strcmp(name, "rec_direct_publish")) return o.rec_direct_publish;
  if (!strcmp(name, "rec_w_tmem")) return o.rec_w_tmem;
  if (!strcmp(name, "rec_large_batch")) return o.rec_large_batch;
  if (!strcmp(name, "rec_fin_groups")) return o.rec_fin_groups;
  if (!strcmp(name, "gemm_persistent")) return o.gemm_persistent;
  if (!strcmp(name, "gemm_pair")) return o.gemm_pair;
  if (!strcmp(name, "test_stall_step")) return o.test_stall_step;
  if (!strcmp(name, "rec_replicas")) return o.rec_replicas;
  if (!strcmp(name, "rec_group_cap")) return o.rec_group_cap;
  return -1;
}

int elman_b200_last_timing(int phase, float* ms) {
  ELMAN_ARG_CHECK(phase >= 0 && phase < kPhases && ms != nullptr, "bad phase %d", phase);
  if (!g_ev_ready || !g_ev_recorded[phase])
    return set_error(ELMAN_ERR_ARG, "phase %d was not timed (set option time_kernels)", phase);
  ELMAN_CUDA_CHECK(cudaEventSynchronize(g_ev[phase][1]));
  ELMAN_CUDA_CHECK(cudaEventElapsedTime(ms, g_ev[phase][0], g_ev[phase][1]));
  return ELMAN_OK;
}

int elman_b200_recurrence_trace(long long* dst, int max_entries) {
  ELMAN_ARG_CHECK(dst != nullptr && max_entries > 0, "bad trace buffer");
  return rec_tc_copy_trace(dst, max_entries);
}

long elman_b200_launch_count(void) { return g_launches.load(); }
long elman_b200_tc_launch_count(void) { return g_tc_launches.load(); }

int elman_b200_recurrence_blocks(int dtype, int flags, int T, int B, int d) {
  if (T <= 0 || B <= 0 || d <= 0) return 0;
  return dense_tc_ok(dtype, T, B, d, 0) && dense_tc_ok(dtype, T, B, d, 1) ? rec_tc_blocks(T, B, d, (flags & ELMAN_FLAG_COMPACT) ? 1 : 0)
                                     : 0;
}

// ------------------------------- E1 ----------------------------------------

size_t elman_e1_forward_workspace(int dtype, int T, int B, int d) {
  E1FwdWs w;
  return carve_e1_fwd(dtype, T, B, d, nullptr, &w);
}

int elman_e1_forward(int dtype, int training, int T, int B, int d, const void* x, const void* z,
                     const void* h0, const void* W_x, const void* W_h, const void* b, void* h,
                     void* output, void* v, void* workspace, size_t workspace_bytes,
                     void* stream) {
  return elman_e1_forward_flags(dtype, 0, training, T, B, d, x, z, h0, W_x, W_h, b, h, output, v,
                                workspace, workspace_bytes, stream);
}

int elman_e1_forward_flags(int dtype, int flags, int training, int T, int B, int d, const void* x,
                           const void* z, const void* h0, const void* W_x, const void* W_h,
                           const void* b, void* h, void* output, void* v, void* workspace,
                           size_t workspace_bytes, void* stream) {
  ELMAN_ARG_CHECK((flags & ~ELMAN_FLAG_COMPACT) == 0, "unknown flags 0x%x", flags);
  ELMAN_RETURN_IF(check_common(dtype, T, B, d));
  if (B == 0 || d == 0) return ELMAN_OK;
  REQUIRE_PTR(h0); REQUIRE_PTR(h);
  cudaStream_t st = (cudaStream_t)stream;
  ELMAN_RETURN_IF(copy_rows(dtype, h0, h, (long)B * d, st));
  if (T == 0) return ELMAN_OK;
  REQUIRE_PTR(x); REQUIRE_PTR(z); REQUIRE_PTR(W_x); REQUIRE_PTR(W_h); REQUIRE_PTR(b);
  REQUIRE_PTR(output); REQUIRE_PTR(workspace);
  ELMAN_ARG_CHECK(!training || v != nullptr, "v must be provided when training");
  ELMAN_ARG_CHECK(((uintptr_t)workspace & 255) == 0, "workspace must be 256-byte aligned");
  E1FwdWs w;
  size_t need = carve_e1_fwd(dtype, T, B, d, workspace, &w);
  if (workspace_bytes < need)
    return set_error(ELMAN_ERR_WORKSPACE, "workspace %zu < required %zu", workspace_bytes, need);
  // time-parallel input projection with the bias fused into the epilogue
  {
    PhaseTimer timer(2, st);
    ELMAN_RETURN_IF(proj_nt(dtype, T * B, d, d, x, d, W_x, d, b, w.pre, d, 0, st));
  }
  return run_rec_fwd(dtype, T, B, d, W_h, w.pre, z, h, output, training ? v : nullptr, w.sync, st,
                     (flags & ELMAN_FLAG_COMPACT) ? 1 : 0);
}

size_t elman_e1_backward_workspace(int dtype, int T, int B, int d) {
  E1BwdWs w;
  return carve_e1_bwd(dtype, T, B, d, nullptr, &w);
}

int elman_e1_backward(int dtype, int T, int B, int d, const void* W_x, const void* W_h,
                      const void* x, const void* z, const void* h, const void* v,
                      const void* d_output, void* dx, void* dz, void* dW_x, void* dW_h, void* db,
                      void* workspace, size_t workspace_bytes, void* stream) {
  return elman_e1_backward_carry(dtype, 0, T, B, d, W_x, W_h, x, z, h, v, d_output, nullptr, dx,
                                 dz, dW_x, dW_h, db, nullptr, workspace, workspace_bytes, stream);
}

int elman_e1_backward_carry(int dtype, int flags, int T, int B, int d, const void* W_x,
                            const void* W_h,
                            const void* x, const void* z, const void* h, const void* v,
                            const void* d_output, const void* dv_in, void* dx, void* dz,
                            void* dW_x, void* dW_h, void* db, void* dv_out, void* workspace,
                            size_t workspace_bytes, void* stream) {
  ELMAN_ARG_CHECK((flags & ~ELMAN_FLAG_COMPACT) == 0, "unknown flags 0x%x", flags);
  ELMAN_RETURN_IF(check_common(dtype, T, B, d));
  if (d == 0) return ELMAN_OK;
  cudaStream_t st = (cudaStream_t)stream;
  REQUIRE_PTR(dW_x); REQUIRE_PTR(dW_h); REQUIRE_PTR(db);
  size_t es = esize(dtype);
  if (T == 0 || B == 0) {
    ELMAN_CUDA_CHECK(cudaMemsetAsync(dW_x, 0, (size_t)d * d * es, st));
    ELMAN_CUDA_CHECK(cudaMemsetAsync(dW_h, 0, (size_t)d * d * es, st));
    ELMAN_CUDA_CHECK(cudaMemsetAsync(db, 0, (size_t)d * es, st));
    // no steps: the carried gradient passes through unchanged
    if (dv_out != nullptr && B > 0) {
      if (dv_in != nullptr)
        ELMAN_CUDA_CHECK(cudaMemcpyAsync(dv_out, dv_in, (size_t)B * d * es,
                                         cudaMemcpyDeviceToDevice, st));
      else
        ELMAN_CUDA_CHECK(cudaMemsetAsync(dv_out, 0, (size_t)B * d * es, st));
    }
    return ELMAN_OK;
  }
  REQUIRE_PTR(W_x); REQUIRE_PTR(W_h); REQUIRE_PTR(x); REQUIRE_PTR(z); REQUIRE_PTR(h);
  REQUIRE_PTR(v); REQUIRE_PTR(d_output); REQUIRE_PTR(dx); REQUIRE_PTR(dz); REQUIRE_PTR(workspace);
  ELMAN_ARG_CHECK(((uintptr_t)workspace & 255) == 0, "workspace must be 256-byte aligned");
  E1BwdWs w;
  size_t need = carve_e1_bwd(dtype, T, B, d, workspace, &w);
  if (workspace_bytes < need)
    return set_error(ELMAN_ERR_WORKSPACE, "workspace %zu < required %zu", workspace_bytes, need);
  const int TB = T * B;
  ELMAN_RETURN_IF(transpose2d(dtype, d, d, W_h, w.Wt, st));
  ELMAN_RETURN_IF(run_rec_bwd(dtype, T, B, d, w.Wt, h, v, z, d_output, w.dv, dz, w.db, w.sync,
                              dv_in, st, (flags & ELMAN_FLAG_COMPACT) ? 1 : 0));
  if (dv_out != nullptr)
    ELMAN_CUDA_CHECK(cudaMemcpyAsync(dv_out, w.dv, (size_t)B * d * es, cudaMemcpyDeviceToDevice, st));
  ELMAN_RETURN_IF(float_to_dtype(dtype, w.db, db, d, st));
  // dx = dv W_x ; dW_x = dv^T x ; dW_h = dv^T h[0:T]
  PhaseTimer timer(3, st);
  ELMAN_RETURN_IF(gemm_nn(dtype, TB, d, d, w.dv, d, W_x, d, w.WxT, dx, d, 0, st));
  ELMAN_RETURN_IF(weight_grads_pair(dtype, d, TB, w.dv, x, dW_x, h, dW_h, st, w.splitk, w.splitk_bytes));
  return ELMAN_OK;
}

// ---------------- E1 forward for callers that cannot allocate ----------------
//
// The scratch the forward pass needs (the projected inputs W_x x_t + b for all t,
// plus the step counters) lives in this file-scope device array instead of a
// caller-provided workspace.  Every device that loads the library carries the
// array until the process exits.
static __device__ __align__(256) unsigned char g_e1_static_scratch[ELMAN_E1_STATIC_SCRATCH_BYTES];
// Device address of the array per device.  The symbol itself is only a host-side
// handle; kernels must be given the address cudaGetSymbolAddress returns.
static void* g_e1_static_scratch_ptr[kMaxDevices] = {nullptr};

size_t elman_e1_forward_static_scratch_bytes(void) { return ELMAN_E1_STATIC_SCRATCH_BYTES; }

int elman_e1_forward_static(int dtype, int training, int T, int B, int d, const void* x,
                            const void* z, const void* h0, const void* W_x, const void* W_h,
                            const void* b, void* h, void* output, void* v, void* stream) {
  ELMAN_RETURN_IF(check_common(dtype, T, B, d));
  if (B == 0 || d == 0) return ELMAN_OK;
  REQUIRE_PTR(h0); REQUIRE_PTR(h);
  E1FwdWs w;
  const size_t need = carve_e1_fwd(dtype, T, B, d, nullptr, &w);
  if (need > (size_t)ELMAN_E1_STATIC_SCRATCH_BYTES)
    return set_error(ELMAN_ERR_WORKSPACE,
                     "T=%d B=%d d=%d needs %zu bytes of scratch; the built-in array of "
                     "elman_e1_forward_static holds %zu (use elman_e1_forward with a workspace)",
                     T, B, d, need, (size_t)ELMAN_E1_STATIC_SCRATCH_BYTES);
  int dev = 0;
  ELMAN_CUDA_CHECK(cudaGetDevice(&dev));
  ELMAN_ARG_CHECK(dev >= 0 && dev < kMaxDevices, "device index %d out of range", dev);
  void* scratch = nullptr;
  {
    static std::mutex setup_mutex;
    std::lock_guard<std::mutex> lock(setup_mutex);
    if (g_e1_static_scratch_ptr[dev] == nullptr) {
      // set-up, once per device, with that device current
      void* ptr = nullptr;
      ELMAN_CUDA_CHECK(cudaGetSymbolAddress((void**)&ptr, g_e1_static_scratch));
      g_e1_static_scratch_ptr[dev] = ptr;
    }
    scratch = g_e1_static_scratch_ptr[dev];
  }
  cudaStream_t st = (cudaStream_t)stream;
  struct NoAllocScope {
    NoAllocScope() { g_no_alloc = true; }
    ~NoAllocScope() { g_no_alloc = false; }
  } scope;
  ELMAN_RETURN_IF(copy_rows(dtype, h0, h, (long)B * d, st));
  if (T == 0) return ELMAN_OK;
  REQUIRE_PTR(x); REQUIRE_PTR(z); REQUIRE_PTR(W_x); REQUIRE_PTR(W_h); REQUIRE_PTR(b);
  REQUIRE_PTR(output);
  ELMAN_ARG_CHECK(!training || v != nullptr, "v must be provided when training");
  carve_e1_fwd(dtype, T, B, d, scratch, &w);
  // the step counters inside the array are cleared by the recurrence launcher on
  // every call; the projected inputs are fully overwritten before they are read
  ELMAN_RETURN_IF(proj_nt(dtype, T * B, d, d, x, d, W_x, d, b, w.pre, d, 0, st));
  return run_rec_fwd(dtype, T, B, d, W_h, w.pre, z, h, output, training ? v : nullptr, w.sync, st);
}

// ------------------------------- E0 ----------------------------------------

struct E0FwdWs { void* pre; void* gate; int* sync; };
static size_t carve_e0_fwd(int dtype, int T, int B, int d, void* ws, E0FwdWs* o) {
  Carver c(ws);
  o->pre = c.take((size_t)T * B * d * esize(dtype));
  o->gate = c.take((size_t)T * B * d * esize(dtype));
  size_t sb = rec_sync_bytes() > rec_tc_sync_bytes() ? rec_sync_bytes() : rec_tc_sync_bytes();
  o->sync = (int*)c.take(sb);
  return c.total();
}

size_t elman_e0_forward_workspace(int dtype, int T, int B, int d) {
  E0FwdWs w;
  return carve_e0_fwd(dtype, T, B, d, nullptr, &w);
}

int elman_e0_forward(int dtype, int training, int T, int B, int d, const void* x, const void* h0,
                     const void* W_x, const void* W_h, const void* W_gate, const void* b,
                     const void* b_gate, void* h, void* output, void* v, void* gate_cache,
                     void* workspace, size_t workspace_bytes, void* stream) {
  ELMAN_RETURN_IF(check_common(dtype, T, B, d));
  if (B == 0 || d == 0) return ELMAN_OK;
  REQUIRE_PTR(h0); REQUIRE_PTR(h);
  cudaStream_t st = (cudaStream_t)stream;
  ELMAN_RETURN_IF(copy_rows(dtype, h0, h, (long)B * d, st));
  if (T == 0) return ELMAN_OK;
  REQUIRE_PTR(x); REQUIRE_PTR(W_x); REQUIRE_PTR(W_h); REQUIRE_PTR(W_gate); REQUIRE_PTR(b);
  REQUIRE_PTR(b_gate); REQUIRE_PTR(output); REQUIRE_PTR(workspace);
  ELMAN_ARG_CHECK(!training || (v != nullptr && gate_cache != nullptr),
                  "v and gate_cache must be provided when training");
  ELMAN_ARG_CHECK(((uintptr_t)workspace & 255) == 0, "workspace must be 256-byte aligned");
  E0FwdWs w;
  size_t need = carve_e0_fwd(dtype, T, B, d, workspace, &w);
  if (workspace_bytes < need)
    return set_error(ELMAN_ERR_WORKSPACE, "workspace %zu < required %zu", workspace_bytes, need);
  void* gate = (training && gate_cache != nullptr) ? gate_cache : w.gate;
  ELMAN_RETURN_IF(proj_nt(dtype, T * B, d, d, x, d, W_x, d, b, w.pre, d, 0, st));
  ELMAN_RETURN_IF(proj_nt(dtype, T * B, d, d, x, d, W_gate, d, b_gate, gate, d, 0, st));
  return run_rec_fwd(dtype, T, B, d, W_h, w.pre, gate, h, output, training ? v : nullptr, w.sync,
                     st);
}

struct E0BwdWs {
  void* Wt; void* dv; void* dg; float* db; float* cs; int* sync;
  void* WT2; float* splitk; size_t splitk_bytes;
};
static size_t carve_e0_bwd(int dtype, int T, int B, int d, void* ws, E0BwdWs* o) {
  Carver c(ws);
  size_t es = esize(dtype);
  o->Wt = c.take((size_t)d * d * es);
  o->dv = c.take((size_t)(T + 1) * B * d * es);  // slot T: zero "gradient from the future"
  o->dg = c.take((size_t)T * B * d * es);
  o->db = (float*)c.take((size_t)REC_MAX_REPLICAS * d * sizeof(float));
  o->cs = (float*)c.take(column_sum_scratch_bytes(d));
  size_t sb = rec_sync_bytes() > rec_tc_sync_bytes() ? rec_sync_bytes() : rec_tc_sync_bytes();
  o->sync = (int*)c.take(sb);
  o->WT2 = nullptr;  // the GEMMs read transposed operands in place
  o->splitk_bytes = splitk_scratch_bytes(dtype, d, d);
  o->splitk = o->splitk_bytes ? (float*)c.take(o->splitk_bytes) : nullptr;
  return c.total();
}

size_t elman_e0_backward_workspace(int dtype, int T, int B, int d) {
  E0BwdWs w;
  return carve_e0_bwd(dtype, T, B, d, nullptr, &w);
}

int elman_e0_backward(int dtype, int T, int B, int d, const void* W_x, const void* W_h,
                      const void* W_gate, const void* x, const void* h, const void* v,
                      const void* gate_cache, const void* d_output, void* dx, void* dW_x,
                      void* dW_h, void* dW_gate, void* db, void* db_gate, void* workspace,
                      size_t workspace_bytes, void* stream) {
  ELMAN_RETURN_IF(check_common(dtype, T, B, d));
  if (d == 0) return ELMAN_OK;
  cudaStream_t st = (cudaStream_t)stream;
  REQUIRE_PTR(dW_x); REQUIRE_PTR(dW_h); REQUIRE_PTR(dW_gate); REQUIRE_PTR(db); REQUIRE_PTR(db_gate);
  size_t es = esize(dtype);
  if (T == 0 || B == 0) {
    ELMAN_CUDA_CHECK(cudaMemsetAsync(dW_x, 0, (size_t)d * d * es, st));
    ELMAN_CUDA_CHECK(cudaMemsetAsync(dW_h, 0, (size_t)d * d * es, st));
    ELMAN_CUDA_CHECK(cudaMemsetAsync(dW_gate, 0, (size_t)d * d * es, st));
    ELMAN_CUDA_CHECK(cudaMemsetAsync(db, 0, (size_t)d * es, st));
    ELMAN_CUDA_CHECK(cudaMemsetAsync(db_gate, 0, (size_t)d * es, st));
    return ELMAN_OK;
  }
  REQUIRE_PTR(W_x); REQUIRE_PTR(W_h); REQUIRE_PTR(W_gate); REQUIRE_PTR(x); REQUIRE_PTR(h);
  REQUIRE_PTR(v); REQUIRE_PTR(gate_cache); REQUIRE_PTR(d_output); REQUIRE_PTR(dx);
  REQUIRE_PTR(workspace);
  ELMAN_ARG_CHECK(((uintptr_t)workspace & 255) == 0, "workspace must be 256-byte aligned");
  E0BwdWs w;
  size_t need = carve_e0_bwd(dtype, T, B, d, workspace, &w);
  if (workspace_bytes < need)
    return set_error(ELMAN_ERR_WORKSPACE, "workspace %zu < required %zu", workspace_bytes, need);
  const int TB = T * B;
  ELMAN_RETURN_IF(transpose2d(dtype, d, d, W_h, w.Wt, st));
  ELMAN_RETURN_IF(run_rec_bwd(dtype, T, B, d, w.Wt, h, v, gate_cache, d_output, w.dv, w.dg, w.db,
                              w.sync, nullptr, st));
  ELMAN_RETURN_IF(float_to_dtype(dtype, w.db, db, d, st));
  ELMAN_RETURN_IF(column_sum(dtype, TB, d, w.dg, db_gate, w.cs, st));
  // dx = dv W_x + dg W_gate
  ELMAN_RETURN_IF(gemm_nn(dtype, TB, d, d, w.dv, d, W_x, d, w.WT2, dx, d, 0, st));
  ELMAN_RETURN_IF(gemm_nn(dtype, TB, d, d, w.dg, d, W_gate, d, w.WT2, dx, d, 1, st));
  // dW_x = dv^T x ; dW_h = dv^T h[0:T] ; dW_gate = dg^T x
  ELMAN_RETURN_IF(weight_grads_pair(dtype, d, TB, w.dv, x, dW_x, h, dW_h, st, w.splitk, w.splitk_bytes));
  ELMAN_RETURN_IF(gemm_tn(dtype, d, d, TB, w.dg, x, dW_gate, st, w.splitk, w.splitk_bytes));
  return ELMAN_OK;
}

// ------------------------------- E5 ----------------------------------------

// In the bf16 tensor-core path every factor is used zero-padded to rp = rank rounded
// up to 64: the time-parallel GEMMs then meet the TMA alignment rules for any rank
// (e.g. 270) and the extra columns contribute exact zeros.
static inline int e5_rank_alloc(int dtype, int r) { return dtype == ELMAN_BF16 ? (r + 63) / 64 * 64 : r; }
static inline int e5_rank_run(int dtype, int r) { return use_tc(dtype) ? (r + 63) / 64 * 64 : r; }

struct E5FwdWs {
  long long* trace;
  void* Vx; void* pre; void* Vz; void* gate; float* tmp; int* sync; void* UP; void* VP;
  void* UxP; void* VxP; void* UzP; void* VzP;
};
static size_t carve_e5_fwd(int dtype, int T, int B, int d, int r, void* ws, E5FwdWs* o) {
  Carver c(ws);
  size_t es = esize(dtype);
  const int ra = e5_rank_alloc(dtype, r);
  o->Vx = c.take((size_t)T * B * ra * es);
  o->pre = c.take((size_t)T * B * d * es);
  o->Vz = c.take((size_t)T * B * ra * es);
  o->gate = c.take((size_t)T * B * d * es);
  o->tmp = (float*)c.take((size_t)2 * B * r * sizeof(float));
  o->sync = (int*)c.take(rec_sync_bytes());
  o->trace = (long long*)c.take(kTraceBytes);
  o->UP = o->VP = o->UxP = o->VxP = o->UzP = o->VzP = nullptr;
  if (dtype == ELMAN_BF16) {  // zero-padded factors
    size_t up = 0, vp = 0;
    lowrank_tc_pad_bytes(d, r, &up, &vp);
    o->UP = c.take(up);
    o->VP = c.take(vp);
    o->UxP = c.take((size_t)d * ra * es);
    o->VxP = c.take((size_t)d * ra * es);
    o->UzP = c.take((size_t)d * ra * es);
    o->VzP = c.take((size_t)d * ra * es);
  }
  return c.total();
}

size_t elman_e5_forward_workspace(int dtype, int T, int B, int d, int r) {
  E5FwdWs w;
  return carve_e5_fwd(dtype, T, B, d, r, nullptr, &w);
}

int elman_e5_forward(int dtype, int training, int T, int B, int d, int r, const void* x,
                     const void* h0, const void* U_h, const void* V_h, const void* U_x,
                     const void* V_x, const void* U_z, const void* V_z, const void* b, void* h,
                     void* output, void* v, void* workspace, size_t workspace_bytes,
                     void* stream) {
  ELMAN_RETURN_IF(check_common(dtype, T, B, d));
  ELMAN_ARG_CHECK(r >= 1, "rank must be positive (got %d)", r);
  if (B == 0 || d == 0) return ELMAN_OK;
  REQUIRE_PTR(h0); REQUIRE_PTR(h);
  cudaStream_t st = (cudaStream_t)stream;
  ELMAN_RETURN_IF(copy_rows(dtype, h0, h, (long)B * d, st));
  if (T == 0) return ELMAN_OK;
  REQUIRE_PTR(x); REQUIRE_PTR(U_h); REQUIRE_PTR(V_h); REQUIRE_PTR(U_x); REQUIRE_PTR(V_x);
  REQUIRE_PTR(U_z); REQUIRE_PTR(V_z); REQUIRE_PTR(b); REQUIRE_PTR(output); REQUIRE_PTR(workspace);
  ELMAN_ARG_CHECK(!training || v != nullptr, "v must be provided when training");
  ELMAN_ARG_CHECK(((uintptr_t)workspace & 255) == 0, "workspace must be 256-byte aligned");
  E5FwdWs w;
  size_t need = carve_e5_fwd(dtype, T, B, d, r, workspace, &w);
  if (workspace_bytes < need)
    return set_error(ELMAN_ERR_WORKSPACE, "workspace %zu < required %zu", workspace_bytes, need);
  const int TB = T * B;
  const int rp = e5_rank_run(dtype, r);
  const void *Ux = U_x, *Vx = V_x, *Uz = U_z, *Vz = V_z;
  if (rp != r) {
    ELMAN_RETURN_IF(resize2d(dtype, U_x, d, r, w.UxP, d, rp, st));
    ELMAN_RETURN_IF(resize2d(dtype, V_x, r, d, w.VxP, rp, d, st));
    ELMAN_RETURN_IF(resize2d(dtype, U_z, d, r, w.UzP, d, rp, st));
    ELMAN_RETURN_IF(resize2d(dtype, V_z, r, d, w.VzP, rp, d, st));
    Ux = w.UxP; Vx = w.VxP; Uz = w.UzP; Vz = w.VzP;
  }
  // pre = (x V_x^T) U_x^T + b ; gate = (x V_z^T) U_z^T
  ELMAN_RETURN_IF(proj_nt(dtype, TB, rp, d, x, d, Vx, d, nullptr, w.Vx, rp, 0, st));
  ELMAN_RETURN_IF(proj_nt(dtype, TB, d, rp, w.Vx, rp, Ux, rp, b, w.pre, d, 0, st));
  ELMAN_RETURN_IF(proj_nt(dtype, TB, rp, d, x, d, Vz, d, nullptr, w.Vz, rp, 0, st));
  ELMAN_RETURN_IF(proj_nt(dtype, TB, d, rp, w.Vz, rp, Uz, rp, nullptr, w.gate, d, 0, st));
  if (use_tc(dtype) && lowrank_tc_supported(T, B, d, r, 0)) {
    LowRankTcArgs ta{};
    ta.T = T; ta.B = B; ta.d = d; ta.r = r; ta.bwd = 0;
    ta.Urole = U_h; ta.Vrole = V_h;
    ta.in0 = w.pre; ta.in1 = w.gate;
    ta.state = h; ta.out0 = training ? v : nullptr; ta.out1 = output;
    ta.UP = w.UP; ta.VP = w.VP; ta.sync = w.sync; ta.trace = w.trace;
    return lowrank_tc(ta, st);
  }
  LowRankFwdArgs a{T, B, d, r, U_h, V_h, w.pre, w.gate, h, output, training ? v : nullptr, w.tmp,
                   w.sync};
  return lowrank_fwd_generic(dtype, a, st);
}

struct E5BwdWs {
  void* Vz; void* gate; void* Ut; void* Vt; void* dv; void* dg; float* db; float* tmp; int* sync;
  void* Vx; void* Vh; void* dVx; void* dVz; void* dVh;
  void* UP; void* VP;
  void* P[6];    // zero-padded U_h, V_h, U_x, V_x, U_z, V_z
  void* dUP; void* dVP;  // padded weight-gradient scratch
  long long* trace;
  float* splitk; size_t splitk_bytes;   // fp32 partial sums of the weight-gradient GEMMs
};
static size_t carve_e5_bwd(int dtype, int T, int B, int d, int r, void* ws, E5BwdWs* o) {
  Carver c(ws);
  size_t es = esize(dtype);
  const int ra = e5_rank_alloc(dtype, r);
  size_t TBr = (size_t)T * B * ra * es, TBd = (size_t)T * B * d * es;
  o->Vz = c.take(TBr);
  o->gate = c.take(TBd);
  o->Ut = c.take((size_t)d * r * es);
  o->Vt = c.take((size_t)d * r * es);
  o->dv = c.take(TBd + (size_t)B * d * es);  // one extra time slot: the zero gradient from the future
  o->dg = c.take(TBd);
  o->db = (float*)c.take((size_t)d * sizeof(float));
  o->tmp = (float*)c.take((size_t)2 * B * r * sizeof(float));
  o->sync = (int*)c.take(rec_sync_bytes());
  o->trace = (long long*)c.take(kTraceBytes);
  o->splitk_bytes = splitk_scratch_bytes(dtype, d, ra);
  o->splitk = o->splitk_bytes ? (float*)c.take(o->splitk_bytes) : nullptr;
  o->Vx = c.take(TBr);
  o->Vh = c.take(TBr);
  o->dVx = c.take(TBr);
  o->dVz = c.take(TBr);
  o->dVh = c.take(TBr);
  o->UP = o->VP = o->dUP = o->dVP = nullptr;
  for (int i = 0; i < 6; ++i) o->P[i] = nullptr;
  if (dtype == ELMAN_BF16) {
    size_t up = 0, vp = 0;
    lowrank_tc_pad_bytes(d, r, &up, &vp);
    o->UP = c.take(up);
    o->VP = c.take(vp);
    for (int i = 0; i < 6; ++i) o->P[i] = c.take((size_t)d * ra * es);
    o->dUP = c.take((size_t)d * ra * es);
    o->dVP = c.take((size_t)d * ra * es);
  }
  return c.total();
}

size_t elman_e5_backward_workspace(int dtype, int T, int B, int d, int r) {
  E5BwdWs w;
  return carve_e5_bwd(dtype, T, B, d, r, nullptr, &w);
}

int elman_e5_backward(int dtype, int T, int B, int d, int r, const void* U_h, const void* V_h,
                      const void* U_x, const void* V_x, const void* U_z, const void* V_z,
                      const void* x, const void* h, const void* v, const void* d_output, void* dx,
                      void* dU_h, void* dV_h, void* dU_x, void* dV_x, void* dU_z, void* dV_z,
                      void* db, void* workspace, size_t workspace_bytes, void* stream) {
  return elman_e5_backward_carry(dtype, T, B, d, r, U_h, V_h, U_x, V_x, U_z, V_z, x, h, v, d_output,
                                 nullptr, dx, dU_h, dV_h, dU_x, dV_x, dU_z, dV_z, db, nullptr,
                                 workspace, workspace_bytes, stream);
}

int elman_b200_lowrank_blocks(int dtype, int T, int B, int d, int r) {
  if (T <= 0 || B <= 0 || d <= 0 || r <= 0 || !use_tc(dtype)) return 0;
  return lowrank_tc_supported(T, B, d, r, 0) && lowrank_tc_supported(T, B, d, r, 1)
             ? lowrank_tc_blocks(T, B, d, r) : 0;
}

int elman_e5_backward_carry(int dtype, int T, int B, int d, int r, const void* U_h,
                            const void* V_h, const void* U_x, const void* V_x, const void* U_z,
                            const void* V_z, const void* x, const void* h, const void* v,
                            const void* d_output, const void* dv_in, void* dx, void* dU_h,
                            void* dV_h, void* dU_x, void* dV_x, void* dU_z, void* dV_z, void* db,
                            void* dv_out, void* workspace, size_t workspace_bytes, void* stream) {
  ELMAN_RETURN_IF(check_common(dtype, T, B, d));
  ELMAN_ARG_CHECK(r >= 1, "rank must be positive (got %d)", r);
  if (d == 0) return ELMAN_OK;
  cudaStream_t st = (cudaStream_t)stream;
  REQUIRE_PTR(dU_h); REQUIRE_PTR(dV_h); REQUIRE_PTR(dU_x); REQUIRE_PTR(dV_x); REQUIRE_PTR(dU_z);
  REQUIRE_PTR(dV_z); REQUIRE_PTR(db);
  size_t es = esize(dtype);
  if (T == 0 || B == 0) {
    void* outs[6] = {dU_h, dV_h, dU_x, dV_x, dU_z, dV_z};
    for (void* p : outs) ELMAN_CUDA_CHECK(cudaMemsetAsync(p, 0, (size_t)d * r * es, st));
    ELMAN_CUDA_CHECK(cudaMemsetAsync(db, 0, (size_t)d * es, st));
    if (dv_out != nullptr && B > 0) {   // no steps: the carried gradient passes through
      if (dv_in != nullptr)
        ELMAN_CUDA_CHECK(cudaMemcpyAsync(dv_out, dv_in, (size_t)B * d * es,
                                         cudaMemcpyDeviceToDevice, st));
      else
        ELMAN_CUDA_CHECK(cudaMemsetAsync(dv_out, 0, (size_t)B * d * es, st));
    }
    return ELMAN_OK;
  }
  REQUIRE_PTR(U_h); REQUIRE_PTR(V_h); REQUIRE_PTR(U_x); REQUIRE_PTR(V_x); REQUIRE_PTR(U_z);
  REQUIRE_PTR(V_z); REQUIRE_PTR(x); REQUIRE_PTR(h); REQUIRE_PTR(v); REQUIRE_PTR(d_output);
  REQUIRE_PTR(dx); REQUIRE_PTR(workspace);
  ELMAN_ARG_CHECK(((uintptr_t)workspace & 255) == 0, "workspace must be 256-byte aligned");
  E5BwdWs w;
  size_t need = carve_e5_bwd(dtype, T, B, d, r, workspace, &w);
  if (workspace_bytes < need)
    return set_error(ELMAN_ERR_WORKSPACE, "workspace %zu < required %zu", workspace_bytes, need);
  const int TB = T * B;
  const int rp = e5_rank_run(dtype, r);
  const bool padded = rp != r;
  // factors as the time-parallel GEMMs see them: U [d, rp], V [rp, d]
  const void* F[6] = {U_h, V_h, U_x, V_x, U_z, V_z};
  if (padded) {
    for (int i = 0; i < 6; ++i) {
      if (i % 2 == 0) ELMAN_RETURN_IF(resize2d(dtype, F[i], d, r, w.P[i], d, rp, st));
      else ELMAN_RETURN_IF(resize2d(dtype, F[i], r, d, w.P[i], rp, d, st));
      F[i] = w.P[i];
    }
  }
  const void *Uh = F[0], *Vh = F[1], *Ux = F[2], *Vx = F[3], *Uz = F[4], *Vz = F[5];
  // recompute the gate pre-activation (the reference does the same per step)
  ELMAN_RETURN_IF(proj_nt(dtype, TB, rp, d, x, d, Vz, d, nullptr, w.Vz, rp, 0, st));
  ELMAN_RETURN_IF(proj_nt(dtype, TB, d, rp, w.Vz, rp, Uz, rp, nullptr, w.gate, d, 0, st));
  ELMAN_RETURN_IF(transpose2d(dtype, d, r, U_h, w.Ut, st));  // [r,d]
  ELMAN_RETURN_IF(transpose2d(dtype, r, d, V_h, w.Vt, st));  // [d,r]
  {  // slot T of dv: the pre-activation gradient of the step after this call's last one
    const size_t slot = (size_t)B * d * es;
    char* last = (char*)w.dv + (size_t)T * slot;
    if (dv_in != nullptr)
      ELMAN_CUDA_CHECK(cudaMemcpyAsync(last, dv_in, slot, cudaMemcpyDeviceToDevice, st));
    else
      ELMAN_CUDA_CHECK(cudaMemsetAsync(last, 0, slot, st));
  }
  if (use_tc(dtype) && lowrank_tc_supported(T, B, d, r, 1)) {
    // dh_rec = (dv U) V: first product with U^T [r,d], second with V^T [d,r]
    LowRankTcArgs ta{};
    ta.T = T; ta.B = B; ta.d = d; ta.r = r; ta.bwd = 1;
    ta.Urole = w.Vt; ta.Vrole = w.Ut;
    ta.in0 = w.gate; ta.in1 = d_output; ta.in2 = h; ta.in3 = v;
    ta.state = w.dv; ta.out0 = w.dg; ta.out1 = nullptr; ta.db = w.db;
    ta.UP = w.UP; ta.VP = w.VP; ta.sync = w.sync; ta.trace = w.trace;
    ELMAN_RETURN_IF(lowrank_tc(ta, st));
  } else {
    LowRankBwdArgs a{T, B, d, r, w.Ut, w.Vt, h, v, w.gate, d_output, w.dv, w.dg, w.db, w.tmp,
                     w.sync};
    ELMAN_RETURN_IF(lowrank_bwd_generic(dtype, a, st));
  }
  if (dv_out != nullptr)
    ELMAN_CUDA_CHECK(cudaMemcpyAsync(dv_out, w.dv, (size_t)B * d * es, cudaMemcpyDeviceToDevice, st));
  ELMAN_RETURN_IF(float_to_dtype(dtype, w.db, db, d, st));
  // rank-r activations and their gradients, all time steps at once
  ELMAN_RETURN_IF(proj_nt(dtype, TB, rp, d, x, d, Vx, d, nullptr, w.Vx, rp, 0, st));
  ELMAN_RETURN_IF(proj_nt(dtype, TB, rp, d, h, d, Vh, d, nullptr, w.Vh, rp, 0, st));
  ELMAN_RETURN_IF(gemm_nn(dtype, TB, rp, d, w.dv, d, Ux, rp, nullptr, w.dVx, rp, 0, st));
  ELMAN_RETURN_IF(gemm_nn(dtype, TB, rp, d, w.dg, d, Uz, rp, nullptr, w.dVz, rp, 0, st));
  ELMAN_RETURN_IF(gemm_nn(dtype, TB, rp, d, w.dv, d, Uh, rp, nullptr, w.dVh, rp, 0, st));
  // dx = dVx V_x + dVz V_z
  ELMAN_RETURN_IF(gemm_nn(dtype, TB, d, rp, w.dVx, rp, Vx, d, nullptr, dx, d, 0, st));
  ELMAN_RETURN_IF(gemm_nn(dtype, TB, d, rp, w.dVz, rp, Vz, d, nullptr, dx, d, 1, st));
  // weight gradients: sums over all T*B rows (into padded scratch when the rank is padded)
  struct Job { const void* A; const void* Bm; void* dU_or_dV; bool is_u; };
  const Job jobs[6] = {{w.dv, w.Vh, dU_h, true},  {w.dVh, h, dV_h, false}, {w.dv, w.Vx, dU_x, true},
                       {w.dVx, x, dV_x, false},   {w.dg, w.Vz, dU_z, true}, {w.dVz, x, dV_z, false}};
  for (const Job& jb : jobs) {
    if (jb.is_u) {  // dU [d, r] = A^T [d, TB] * Bm [TB, rp]
      void* out = padded ? w.dUP : jb.dU_or_dV;
      ELMAN_RETURN_IF(gemm_tn(dtype, d, rp, TB, jb.A, jb.Bm, out, st, w.splitk, w.splitk_bytes));
      if (padded) ELMAN_RETURN_IF(resize2d(dtype, out, d, rp, jb.dU_or_dV, d, r, st));
    } else {        // dV [r, d] = A^T [rp, TB] * Bm [TB, d]
      void* out = padded ? w.dVP : jb.dU_or_dV;
      ELMAN_RETURN_IF(gemm_tn(dtype, rp, d, TB, jb.A, jb.Bm, out, st, w.splitk, w.splitk_bytes));
      if (padded) ELMAN_RETURN_IF(copy_rows(dtype, out, jb.dU_or_dV, (long)r * d, st));
    }
  }
  return ELMAN_OK;
}

// ------------------------------- E4 ----------------------------------------
// E1 whose recurrent matrix is the product U V of two rank-r factors
// (elman/models/lowrank_elman.py:16-46, :134-160 of the reference):
//   h_t = tanh(W_x x_t + U (V h_{t-1}) + b),  y_t = h_t * silu(z_t)
// The recurrence is the E5 one (the single-cluster low-rank kernel) fed with the dense
// projection of x and with z as the gate input; the time-parallel part is E1's.

struct E4FwdWs {
  void* pre; float* tmp; int* sync; long long* trace; void* UP; void* VP;
};
static size_t carve_e4_fwd(int dtype, int T, int B, int d, int r, void* ws, E4FwdWs* o) {
  Carver c(ws);
  size_t es = esize(dtype);
  o->pre = c.take((size_t)T * B * d * es);
  o->tmp = (float*)c.take((size_t)2 * B * r * sizeof(float));
  o->sync = (int*)c.take(rec_sync_bytes());
  o->trace = (long long*)c.take(kTraceBytes);
  o->UP = o->VP = nullptr;
  if (dtype == ELMAN_BF16) {
    size_t up = 0, vp = 0;
    lowrank_tc_pad_bytes(d, r, &up, &vp);
    o->UP = c.take(up);
    o->VP = c.take(vp);
  }
  return c.total();
}

size_t elman_e4_forward_workspace(int dtype, int T, int B, int d, int r) {
  E4FwdWs w;
  return carve_e4_fwd(dtype, T, B, d, r, nullptr, &w);
}

int elman_e4_forward(int dtype, int training, int T, int B, int d, int r, const void* x,
                     const void* z, const void* h0, const void* W_x, const void* U, const void* V,
                     const void* b, void* h, void* output, void* v, void* workspace,
                     size_t workspace_bytes, void* stream) {
  ELMAN_RETURN_IF(check_common(dtype, T, B, d));
  ELMAN_ARG_CHECK(r >= 1, "rank must be positive (got %d)", r);
  if (B == 0 || d == 0) return ELMAN_OK;
  REQUIRE_PTR(h0); REQUIRE_PTR(h);
  cudaStream_t st = (cudaStream_t)stream;
  ELMAN_RETURN_IF(copy_rows(dtype, h0, h, (long)B * d, st));
  if (T == 0) return ELMAN_OK;
  REQUIRE_PTR(x); REQUIRE_PTR(z); REQUIRE_PTR(W_x); REQUIRE_PTR(U); REQUIRE_PTR(V); REQUIRE_PTR(b);
  REQUIRE_PTR(output); REQUIRE_PTR(workspace);
  ELMAN_ARG_CHECK(!training || v != nullptr, "v must be provided when training");
  ELMAN_ARG_CHECK(((uintptr_t)workspace & 255) == 0, "workspace must be 256-byte aligned");
  E4FwdWs w;
  size_t need = carve_e4_fwd(dtype, T, B, d, r, workspace, &w);
  if (workspace_bytes < need)
    return set_error(ELMAN_ERR_WORKSPACE, "workspace %zu < required %zu", workspace_bytes, need);
  ELMAN_RETURN_IF(proj_nt(dtype, T * B, d, d, x, d, W_x, d, b, w.pre, d, 0, st));
  if (use_tc(dtype) && lowrank_tc_supported(T, B, d, r, 0)) {
    LowRankTcArgs ta{};
    ta.T = T; ta.B = B; ta.d = d; ta.r = r; ta.bwd = 0;
    ta.Urole = U; ta.Vrole = V;
    ta.in0 = w.pre; ta.in1 = z;
    ta.state = h; ta.out0 = training ? v : nullptr; ta.out1 = output;
    ta.UP = w.UP; ta.VP = w.VP; ta.sync = w.sync; ta.trace = w.trace;
    return lowrank_tc(ta, st);
  }
  LowRankFwdArgs a{T, B, d, r, U, V, w.pre, z, h, output, training ? v : nullptr, w.tmp, w.sync};
  return lowrank_fwd_generic(dtype, a, st);
}

struct E4BwdWs {
  void* Ut; void* Vt; void* dv; float* db; float* tmp; int* sync; long long* trace;
  void* Vh; void* dVh; void* UP; void* VP; void* UhP; void* VhP; void* dUP; void* dVP;
  float* splitk; size_t splitk_bytes;
};
static size_t carve_e4_bwd(int dtype, int T, int B, int d, int r, void* ws, E4BwdWs* o) {
  Carver c(ws);
  size_t es = esize(dtype);
  const int ra = e5_rank_alloc(dtype, r);
  size_t TBr = (size_t)T * B * ra * es, TBd = (size_t)T * B * d * es;
  o->Ut = c.take((size_t)d * r * es);
  o->Vt = c.take((size_t)d * r * es);
  o->dv = c.take(TBd + (size_t)B * d * es);  // one extra time slot: the zero gradient from the future
  o->db = (float*)c.take((size_t)d * sizeof(float));
  o->tmp = (float*)c.take((size_t)2 * B * r * sizeof(float));
  o->sync = (int*)c.take(rec_sync_bytes());
  o->trace = (long long*)c.take(kTraceBytes);
  o->splitk_bytes = splitk_scratch_bytes(dtype, d, d);
  o->splitk = o->splitk_bytes ? (float*)c.take(o->splitk_bytes) : nullptr;
  o->Vh = c.take(TBr);
  o->dVh = c.take(TBr);
  o->UP = o->VP = o->UhP = o->VhP = o->dUP = o->dVP = nullptr;
  if (dtype == ELMAN_BF16) {
    size_t up = 0, vp = 0;
    lowrank_tc_pad_bytes(d, r, &up, &vp);
    o->UP = c.take(up);
    o->VP = c.take(vp);
    o->UhP = c.take((size_t)d * ra * es);
    o->VhP = c.take((size_t)d * ra * es);
    o->dUP = c.take((size_t)d * ra * es);
    o->dVP = c.take((size_t)d * ra * es);
  }
  return c.total();
}

size_t elman_e4_backward_workspace(int dtype, int T, int B, int d, int r) {
  E4BwdWs w;
  return carve_e4_bwd(dtype, T, B, d, r, nullptr, &w);
}

int elman_e4_backward(int dtype, int T, int B, int d, int r, const void* W_x, const void* U,
                      const void* V, const void* x, const void* z, const void* h, const void* v,
                      const void* d_output, void* dx, void* dz, void* dW_x, void* dU, void* dV,
                      void* db, void* workspace, size_t workspace_bytes, void* stream) {
  ELMAN_RETURN_IF(check_common(dtype, T, B, d));
  ELMAN_ARG_CHECK(r >= 1, "rank must be positive (got %d)", r);
  if (d == 0) return ELMAN_OK;
  cudaStream_t st = (cudaStream_t)stream;
  REQUIRE_PTR(dW_x); REQUIRE_PTR(dU); REQUIRE_PTR(dV); REQUIRE_PTR(db);
  size_t es = esize(dtype);
  if (T == 0 || B == 0) {
    ELMAN_CUDA_CHECK(cudaMemsetAsync(dW_x, 0, (size_t)d * d * es, st));
    ELMAN_CUDA_CHECK(cudaMemsetAsync(dU, 0, (size_t)d * r * es, st));
    ELMAN_CUDA_CHECK(cudaMemsetAsync(dV, 0, (size_t)d * r * es, st));
    ELMAN_CUDA_CHECK(cudaMemsetAsync(db, 0, (size_t)d * es, st));
    return ELMAN_OK;
  }
  REQUIRE_PTR(W_x); REQUIRE_PTR(U); REQUIRE_PTR(V); REQUIRE_PTR(x); REQUIRE_PTR(z); REQUIRE_PTR(h);
  REQUIRE_PTR(v); REQUIRE_PTR(d_output); REQUIRE_PTR(dx); REQUIRE_PTR(dz); REQUIRE_PTR(workspace);
  ELMAN_ARG_CHECK(((uintptr_t)workspace & 255) == 0, "workspace must be 256-byte aligned");
  E4BwdWs w;
  size_t need = carve_e4_bwd(dtype, T, B, d, r, workspace, &w);
  if (workspace_bytes < need)
    return set_error(ELMAN_ERR_WORKSPACE, "workspace %zu < required %zu", workspace_bytes, need);
  const int TB = T * B;
  const int rp = e5_rank_run(dtype, r);
  const bool padded = rp != r;
  const void *Uh = U, *Vh = V;       // as the time-parallel GEMMs see them: U [d, rp], V [rp, d]
  if (padded) {
    ELMAN_RETURN_IF(resize2d(dtype, U, d, r, w.UhP, d, rp, st));
    ELMAN_RETURN_IF(resize2d(dtype, V, r, d, w.VhP, rp, d, st));
    Uh = w.UhP; Vh = w.VhP;
  }
  ELMAN_RETURN_IF(transpose2d(dtype, d, r, U, w.Ut, st));  // [r,d]
  ELMAN_RETURN_IF(transpose2d(dtype, r, d, V, w.Vt, st));  // [d,r]
  ELMAN_CUDA_CHECK(cudaMemsetAsync((char*)w.dv + (size_t)T * B * d * es, 0, (size_t)B * d * es, st));
  if (use_tc(dtype) && lowrank_tc_supported(T, B, d, r, 1)) {
    LowRankTcArgs ta{};
    ta.T = T; ta.B = B; ta.d = d; ta.r = r; ta.bwd = 1;
    ta.Urole = w.Vt; ta.Vrole = w.Ut;
    ta.in0 = z; ta.in1 = d_output; ta.in2 = h; ta.in3 = v;
    ta.state = w.dv; ta.out0 = dz; ta.out1 = nullptr; ta.db = w.db;
    ta.UP = w.UP; ta.VP = w.VP; ta.sync = w.sync; ta.trace = w.trace;
    ELMAN_RETURN_IF(lowrank_tc(ta, st));
  } else {
    LowRankBwdArgs a{T, B, d, r, w.Ut, w.Vt, h, v, z, d_output, w.dv, dz, w.db, w.tmp, w.sync};
    ELMAN_RETURN_IF(lowrank_bwd_generic(dtype, a, st));
  }
  ELMAN_RETURN_IF(float_to_dtype(dtype, w.db, db, d, st));
  // time-parallel part: dx = dv W_x, dW_x = dv^T x; rank activations Vh = h V^T, dVh = dv U
  ELMAN_RETURN_IF(gemm_nn(dtype, TB, d, d, w.dv, d, W_x, d, nullptr, dx, d, 0, st));
  ELMAN_RETURN_IF(gemm_tn(dtype, d, d, TB, w.dv, x, dW_x, st, w.splitk, w.splitk_bytes));
  ELMAN_RETURN_IF(proj_nt(dtype, TB, rp, d, h, d, Vh, d, nullptr, w.Vh, rp, 0, st));
  ELMAN_RETURN_IF(gemm_nn(dtype, TB, rp, d, w.dv, d, Uh, rp, nullptr, w.dVh, rp, 0, st));
  {  // dU [d, r] = dv^T [d, TB] * Vh [TB, rp]
    void* out = padded ? w.dUP : dU;
    ELMAN_RETURN_IF(gemm_tn(dtype, d, rp, TB, w.dv, w.Vh, out, st, w.splitk, w.splitk_bytes));
    if (padded) ELMAN_RETURN_IF(resize2d(dtype, out, d, rp, dU, d, r, st));
  }
  {  // dV [r, d] = dVh^T [rp, TB] * h[0:T] [TB, d]
    void* out = padded ? w.dVP : dV;
    ELMAN_RETURN_IF(gemm_tn(dtype, rp, d, TB, w.dVh, h, out, st, w.splitk, w.splitk_bytes));
    if (padded) ELMAN_RETURN_IF(copy_rows(dtype, out, dV, (long)r * d, st));
  }
  return ELMAN_OK;
}

// --------------------------- projection GEMM --------------------------------

int elman_projection(int dtype, int M, int N, int K, const void* A, int lda, const void* W,
                     int ldw, const void* bias, void* C, int ldc, int accumulate, void* stream) {
  ELMAN_ARG_CHECK(dtype == ELMAN_F32 || dtype == ELMAN_BF16, "unknown dtype %d", dtype);
  ELMAN_ARG_CHECK(M >= 0 && N >= 0 && K >= 0, "negative size");
  ELMAN_RETURN_IF(check_status_on_entry());
  if (M == 0 || N == 0) return ELMAN_OK;
  REQUIRE_PTR(A); REQUIRE_PTR(W); REQUIRE_PTR(C);
  ELMAN_ARG_CHECK(lda >= K && ldw >= K && ldc >= N, "row stride smaller than the row");
  return proj_nt(dtype, M, N, K, A, lda, W, ldw, bias, C, ldc, accumulate, (cudaStream_t)stream);
}

// ------------------- the phases of an E1 call, one by one --------------------

int elman_gemm(int dtype, int op, int M, int N, int K, const void* A, const void* B,
               const void* bias, void* C, int accumulate, void* stream) {
  ELMAN_ARG_CHECK(dtype == ELMAN_F32 || dtype == ELMAN_BF16, "unknown dtype %d", dtype);
  ELMAN_ARG_CHECK(M >= 0 && N >= 0 && K >= 0, "negative size");
  ELMAN_ARG_CHECK(op == ELMAN_GEMM_NT || op == ELMAN_GEMM_NN || op == ELMAN_GEMM_TN,
                  "unknown GEMM form %d", op);
  ELMAN_ARG_CHECK(bias == nullptr || op == ELMAN_GEMM_NT, "bias only with ELMAN_GEMM_NT");
  ELMAN_RETURN_IF(check_status_on_entry());
  if (M == 0 || N == 0) return ELMAN_OK;
  REQUIRE_PTR(C);
  cudaStream_t st = (cudaStream_t)stream;
  if (K == 0) {
    if (!accumulate)
      ELMAN_CUDA_CHECK(cudaMemsetAsync(C, 0, (size_t)M * N * esize(dtype), st));
    return ELMAN_OK;
  }
  REQUIRE_PTR(A); REQUIRE_PTR(B);
  if (op == ELMAN_GEMM_NT) return proj_nt(dtype, M, N, K, A, K, B, K, bias, C, N, accumulate, st);
  if (op == ELMAN_GEMM_NN) return gemm_nn(dtype, M, N, K, A, K, B, N, nullptr, C, N, accumulate, st);
  return gemm_tn(dtype, M, N, K, A, B, C, st, nullptr, 0, accumulate);
}

size_t elman_column_sum_workspace(int N) { return column_sum_scratch_bytes(N < 0 ? 0 : N); }

int elman_column_sum(int dtype, long M, int N, const void* in, void* out, void* workspace,
                     size_t workspace_bytes, void* stream) {
  ELMAN_ARG_CHECK(dtype == ELMAN_F32 || dtype == ELMAN_BF16, "unknown dtype %d", dtype);
  ELMAN_ARG_CHECK(M >= 0 && N >= 0, "negative size");
  ELMAN_RETURN_IF(check_status_on_entry());
  if (N == 0) return ELMAN_OK;
  REQUIRE_PTR(out); REQUIRE_PTR(workspace);
  ELMAN_ARG_CHECK(M == 0 || in != nullptr, "argument in is NULL");
  if (workspace_bytes < column_sum_scratch_bytes(N))
    return set_error(ELMAN_ERR_WORKSPACE, "workspace %zu < required %zu", workspace_bytes,
                     column_sum_scratch_bytes(N));
  return column_sum(dtype, M, N, in, out, (float*)workspace, (cudaStream_t)stream);
}

struct E1RecWs { void* Wt; float* db; int* sync; };
static size_t carve_e1_rec(int dtype, int d, void* ws, E1RecWs* o) {
  Carver c(ws);
  o->Wt = c.take((size_t)d * d * esize(dtype));
  o->db = (float*)c.take((size_t)REC_MAX_REPLICAS * d * sizeof(float));
  size_t sb = rec_sync_bytes() > rec_tc_sync_bytes() ? rec_sync_bytes() : rec_tc_sync_bytes();
  o->sync = (int*)c.take(sb);
  return c.total();
}

size_t elman_e1_recurrence_workspace(int dtype, int d) {
  E1RecWs w;
  return carve_e1_rec(dtype, d < 0 ? 0 : d, nullptr, &w);
}

int elman_e1_recurrence_forward(int dtype, int flags, int training, int T, int B, int d,
                                const void* pre, const void* z, const void* h0, const void* W_h,
                                void* h, void* output, void* v, void* workspace,
                                size_t workspace_bytes, void* stream) {
  ELMAN_ARG_CHECK((flags & ~ELMAN_FLAG_COMPACT) == 0, "unknown flags 0x%x", flags);
  ELMAN_RETURN_IF(check_common(dtype, T, B, d));
  if (B == 0 || d == 0) return ELMAN_OK;
  REQUIRE_PTR(h0); REQUIRE_PTR(h);
  cudaStream_t st = (cudaStream_t)stream;
  ELMAN_RETURN_IF(copy_rows(dtype, h0, h, (long)B * d, st));
  if (T == 0) return ELMAN_OK;
  REQUIRE_PTR(pre); REQUIRE_PTR(z); REQUIRE_PTR(W_h); REQUIRE_PTR(output); REQUIRE_PTR(workspace);
  ELMAN_ARG_CHECK(!training || v != nullptr, "v must be provided when training");
  ELMAN_ARG_CHECK(((uintptr_t)workspace & 255) == 0, "workspace must be 256-byte aligned");
  E1RecWs w;
  size_t need = carve_e1_rec(dtype, d, workspace, &w);
  if (workspace_bytes < need)
    return set_error(ELMAN_ERR_WORKSPACE, "workspace %zu < required %zu", workspace_bytes, need);
  return run_rec_fwd(dtype, T, B, d, W_h, pre, z, h, output, training ? v : nullptr, w.sync, st,
                     (flags & ELMAN_FLAG_COMPACT) ? 1 : 0);
}

int elman_e1_recurrence_backward(int dtype, int flags, int T, int B, int d, const void* W_h,
                                 const void* z, const void* h, const void* v,
                                 const void* d_output, const void* dv_in, const void* W_h_T,
                                 void* dv, void* dz, void* db, void* workspace,
                                 size_t workspace_bytes, void* stream) {
  ELMAN_ARG_CHECK((flags & ~ELMAN_FLAG_COMPACT) == 0, "unknown flags 0x%x", flags);
  ELMAN_RETURN_IF(check_common(dtype, T, B, d));
  if (d == 0 || B == 0) return ELMAN_OK;
  cudaStream_t st = (cudaStream_t)stream;
  REQUIRE_PTR(dv); REQUIRE_PTR(db);
  const size_t es = esize(dtype);
  if (T == 0) {  // no steps: the carried gradient passes through, nothing adds to the bias
    ELMAN_CUDA_CHECK(cudaMemsetAsync(db, 0, (size_t)d * es, st));
    if (dv_in != nullptr)
      ELMAN_CUDA_CHECK(cudaMemcpyAsync(dv, dv_in, (size_t)B * d * es, cudaMemcpyDeviceToDevice, st));
    else
      ELMAN_CUDA_CHECK(cudaMemsetAsync(dv, 0, (size_t)B * d * es, st));
    return ELMAN_OK;
  }
  ELMAN_ARG_CHECK(W_h != nullptr || W_h_T != nullptr, "W_h and W_h_T are both NULL");
  REQUIRE_PTR(z); REQUIRE_PTR(h); REQUIRE_PTR(v); REQUIRE_PTR(d_output);
  REQUIRE_PTR(dz); REQUIRE_PTR(workspace);
  ELMAN_ARG_CHECK(((uintptr_t)workspace & 255) == 0, "workspace must be 256-byte aligned");
  E1RecWs w;
  size_t need = carve_e1_rec(dtype, d, workspace, &w);
  if (workspace_bytes < need)
    return set_error(ELMAN_ERR_WORKSPACE, "workspace %zu < required %zu", workspace_bytes, need);
  const void* Wt = W_h_T;
  if (Wt == nullptr) {
    ELMAN_RETURN_IF(transpose2d(dtype, d, d, W_h, w.Wt, st));
    Wt = w.Wt;
  }
  ELMAN_RETURN_IF(run_rec_bwd(dtype, T, B, d, Wt, h, v, z, d_output, dv, dz, w.db, w.sync, dv_in,
                              st, (flags & ELMAN_FLAG_COMPACT) ? 1 : 0));
  return float_to_dtype(dtype, w.db, db, d, st);
}

// ---------------- E1 with the gate on [h; x] (extension of the reference's E1) ----------------
//   h_t = tanh(W_x x_t + W_h h_{t-1} + b),   y_t = h_t * silu(z_t + W_gh h_t)
// where z_t = W_gx x_t + b_g is the caller's time-parallel gate projection.  h never feeds
// back through the gate, so W_gh h_t is one more time-parallel GEMM over the stored states
// with the gate in its epilogue; backward adds dW_gh = dzg^T h and injects dzg W_gh into the
// gradient BPTT starts from.

// The BPTT kernels take the direct gradient of h_t as dy_t * silu(g_t).  Here it is
// dy_t silu(zg_t) + (dzg_t W_gh), which is handed to the same kernels as "dy" beside a
// constant gate g0 (silu(g0) is then a known scalar that is divided out beforehand).
static constexpr float kGateConst = 1.28125f;   // exact in bf16 and fp32
static float gate_const_inv_silu() {
  const double g = (double)kGateConst;
  return (float)(1.0 / (g / (1.0 + exp(-g))));
}

struct HxFwdWs { void* pre; void* y0; int* sync; };
static size_t carve_hx_fwd(int dtype, int T, int B, int d, void* ws, HxFwdWs* o) {
  Carver c(ws);
  o->pre = c.take((size_t)T * B * d * esize(dtype));
  o->y0 = c.take((size_t)T * B * d * esize(dtype));   // the recurrence's own (x-only) gate output
  size_t sb = rec_sync_bytes() > rec_tc_sync_bytes() ? rec_sync_bytes() : rec_tc_sync_bytes();
  o->sync = (int*)c.take(sb);
  return c.total();
}

size_t elman_e1_hx_forward_workspace(int dtype, int T, int B, int d) {
  HxFwdWs w;
  return carve_hx_fwd(dtype, T, B, d, nullptr, &w);
}

int elman_e1_hx_forward(int dtype, int training, int T, int B, int d, const void* x, const void* z,
                        const void* h0, const void* W_x, const void* W_h, const void* b,
                        const void* W_gh, void* h, void* output, void* v, void* z_gate,
                        void* workspace, size_t workspace_bytes, void* stream) {
  ELMAN_RETURN_IF(check_common(dtype, T, B, d));
  if (B == 0 || d == 0) return ELMAN_OK;
  REQUIRE_PTR(h0); REQUIRE_PTR(h);
  cudaStream_t st = (cudaStream_t)stream;
  ELMAN_RETURN_IF(copy_rows(dtype, h0, h, (long)B * d, st));
  if (T == 0) return ELMAN_OK;
  REQUIRE_PTR(x); REQUIRE_PTR(z); REQUIRE_PTR(W_x); REQUIRE_PTR(W_h); REQUIRE_PTR(b);
  REQUIRE_PTR(W_gh); REQUIRE_PTR(output); REQUIRE_PTR(z_gate); REQUIRE_PTR(workspace);
  ELMAN_ARG_CHECK(!training || v != nullptr, "v must be provided when training");
  ELMAN_ARG_CHECK(((uintptr_t)workspace & 255) == 0, "workspace must be 256-byte aligned");
  HxFwdWs w;
  size_t need = carve_hx_fwd(dtype, T, B, d, workspace, &w);
  if (workspace_bytes < need)
    return set_error(ELMAN_ERR_WORKSPACE, "workspace %zu < required %zu", workspace_bytes, need);
  const int TB = T * B;
  const size_t es = esize(dtype);
  ELMAN_RETURN_IF(proj_nt(dtype, TB, d, d, x, d, W_x, d, b, w.pre, d, 0, st));
  ELMAN_RETURN_IF(run_rec_fwd(dtype, T, B, d, W_h, w.pre, z, h, w.y0, training ? v : nullptr,
                              w.sync, st));
  const void* h1 = (const char*)h + (size_t)B * d * es;   // h_1 .. h_T
  if (use_tc(dtype) && (d & 31) == 0 && gemm_tc_supported(TB, d, d, h1, d, W_gh, d, z_gate, d, 0) &&
      ((((uintptr_t)z_gate | (uintptr_t)output | (uintptr_t)z | (uintptr_t)h1) & 15) == 0)) {
    GemmSplit ep{d, output, const_cast<void*>(z), 1, h1};   // sum with z, gate with h in the epilogue
    return gemm_tc(TB, d, d, (const bf16*)h1, d, 0, (const bf16*)W_gh, d, 0, nullptr, z_gate, d, 0,
                   0, st, nullptr, 0, &ep);
  }
  ELMAN_RETURN_IF(copy_rows(dtype, z, z_gate, (long)TB * d, st));
  ELMAN_RETURN_IF(proj_nt(dtype, TB, d, d, h1, d, W_gh, d, nullptr, z_gate, d, 1, st));
  return gate_apply(dtype, (long)TB * d, h1, z_gate, output, st);
}

struct HxBwdWs {
  void* Wt; void* dv; float* db; int* sync; float* splitk; size_t splitk_bytes;
  void* t; void* g0; void* dg0; void* Ws;
};
static size_t carve_hx_bwd(int dtype, int T, int B, int d, void* ws, HxBwdWs* o) {
  Carver c(ws);
  const size_t es = esize(dtype), TBd = (size_t)T * B * d * es;
  o->Wt = c.take((size_t)d * d * es);
  o->dv = c.take(TBd + (size_t)B * d * es);
  o->db = (float*)c.take((size_t)REC_MAX_REPLICAS * d * sizeof(float));
  size_t sb = rec_sync_bytes() > rec_tc_sync_bytes() ? rec_sync_bytes() : rec_tc_sync_bytes();
  o->sync = (int*)c.take(sb);
  o->splitk_bytes = splitk_scratch_bytes(dtype, d, d);
  o->splitk = o->splitk_bytes ? (float*)c.take(o->splitk_bytes) : nullptr;
  o->t = c.take(TBd);      // the gradient BPTT starts from, scaled for the constant gate
  o->g0 = c.take(TBd);     // the constant gate
  o->dg0 = c.take(TBd);    // the kernel's gate gradient for the constant gate (unused)
  o->Ws = c.take((size_t)d * d * es);   // W_gh / silu(g0)
  return c.total();
}

size_t elman_e1_hx_backward_workspace(int dtype, int T, int B, int d) {
  HxBwdWs w;
  return carve_hx_bwd(dtype, T, B, d, nullptr, &w);
}

int elman_e1_hx_backward(int dtype, int T, int B, int d, const void* W_x, const void* W_h,
                         const void* W_gh, const void* x, const void* z_gate, const void* h,
                         const void* v, const void* d_output, void* dx, void* dz, void* dW_x,
                         void* dW_h, void* db, void* dW_gh, void* workspace,
                         size_t workspace_bytes, void* stream) {
  ELMAN_RETURN_IF(check_common(dtype, T, B, d));
  if (d == 0) return ELMAN_OK;
  cudaStream_t st = (cudaStream_t)stream;
  REQUIRE_PTR(dW_x); REQUIRE_PTR(dW_h); REQUIRE_PTR(db); REQUIRE_PTR(dW_gh);
  const size_t es = esize(dtype);
  if (T == 0 || B == 0) {
    ELMAN_CUDA_CHECK(cudaMemsetAsync(dW_x, 0, (size_t)d * d * es, st));
    ELMAN_CUDA_CHECK(cudaMemsetAsync(dW_h, 0, (size_t)d * d * es, st));
    ELMAN_CUDA_CHECK(cudaMemsetAsync(dW_gh, 0, (size_t)d * d * es, st));
    ELMAN_CUDA_CHECK(cudaMemsetAsync(db, 0, (size_t)d * es, st));
    return ELMAN_OK;
  }
  REQUIRE_PTR(W_x); REQUIRE_PTR(W_h); REQUIRE_PTR(W_gh); REQUIRE_PTR(x); REQUIRE_PTR(z_gate);
  REQUIRE_PTR(h); REQUIRE_PTR(v); REQUIRE_PTR(d_output); REQUIRE_PTR(dx); REQUIRE_PTR(dz);
  REQUIRE_PTR(workspace);
  ELMAN_ARG_CHECK(((uintptr_t)workspace & 255) == 0, "workspace must be 256-byte aligned");
  HxBwdWs w;
  size_t need = carve_hx_bwd(dtype, T, B, d, workspace, &w);
  if (workspace_bytes < need)
    return set_error(ELMAN_ERR_WORKSPACE, "workspace %zu < required %zu", workspace_bytes, need);
  const int TB = T * B;
  const long n = (long)TB * d;
  const float inv_s = gate_const_inv_silu();
  const void* h1 = (const char*)h + (size_t)B * d * es;
  // dz = dy h silu'(zg);  t = dy silu(zg) / silu(g0);  t += dz (W_gh / silu(g0))
  ELMAN_RETURN_IF(gate_backward_prep(dtype, n, d_output, h1, z_gate, inv_s, dz, w.t, st));
  ELMAN_RETURN_IF(scale_copy(dtype, (long)d * d, W_gh, inv_s, w.Ws, st));
  ELMAN_RETURN_IF(gemm_nn(dtype, TB, d, d, dz, d, w.Ws, d, nullptr, w.t, d, 1, st));
  ELMAN_RETURN_IF(fill_value(dtype, n, kGateConst, w.g0, st));
  ELMAN_RETURN_IF(transpose2d(dtype, d, d, W_h, w.Wt, st));
  ELMAN_RETURN_IF(run_rec_bwd(dtype, T, B, d, w.Wt, h, v, w.g0, w.t, w.dv, w.dg0, w.db, w.sync,
                              nullptr, st));
  ELMAN_RETURN_IF(float_to_dtype(dtype, w.db, db, d, st));
  ELMAN_RETURN_IF(gemm_nn(dtype, TB, d, d, w.dv, d, W_x, d, nullptr, dx, d, 0, st));
  ELMAN_RETURN_IF(weight_grads_pair(dtype, d, TB, w.dv, x, dW_x, h, dW_h, st, w.splitk, w.splitk_bytes));
  ELMAN_RETURN_IF(gemm_tn(dtype, d, d, TB, dz, h1, dW_gh, st, w.splitk, w.splitk_bytes));
  return ELMAN_OK;
}

// ------------------------------- E33: self-gated E1 -------------------------------
//   h_t = tanh(W_x x_t + W_h h_{t-1} + b),   y_t = h_t * silu(h_t)
// The same recurrence kernels with no gate input (the state gates itself in the epilogue).

size_t elman_e33_forward_workspace(int dtype, int T, int B, int d) {
  return elman_e1_forward_workspace(dtype, T, B, d);
}

int elman_e33_forward(int dtype, int training, int T, int B, int d, const void* x, const void* h0,
                      const void* W_x, const void* W_h, const void* b, void* h, void* output,
                      void* v, void* workspace, size_t workspace_bytes, void* stream) {
  ELMAN_RETURN_IF(check_common(dtype, T, B, d));
  if (B == 0 || d == 0) return ELMAN_OK;
  REQUIRE_PTR(h0); REQUIRE_PTR(h);
  cudaStream_t st = (cudaStream_t)stream;
  ELMAN_RETURN_IF(copy_rows(dtype, h0, h, (long)B * d, st));
  if (T == 0) return ELMAN_OK;
  REQUIRE_PTR(x); REQUIRE_PTR(W_x); REQUIRE_PTR(W_h); REQUIRE_PTR(b); REQUIRE_PTR(output);
  REQUIRE_PTR(workspace);
  ELMAN_ARG_CHECK(!training || v != nullptr, "v must be provided when training");
  ELMAN_ARG_CHECK(((uintptr_t)workspace & 255) == 0, "workspace must be 256-byte aligned");
  E1FwdWs w;
  size_t need = carve_e1_fwd(dtype, T, B, d, workspace, &w);
  if (workspace_bytes < need)
    return set_error(ELMAN_ERR_WORKSPACE, "workspace %zu < required %zu", workspace_bytes, need);
  ELMAN_RETURN_IF(proj_nt(dtype, T * B, d, d, x, d, W_x, d, b, w.pre, d, 0, st));
  return run_rec_fwd(dtype, T, B, d, W_h, w.pre, nullptr, h, output, training ? v : nullptr, w.sync,
                     st);
}

size_t elman_e33_backward_workspace(int dtype, int T, int B, int d) {
  return elman_e1_backward_workspace(dtype, T, B, d);
}

int elman_e33_backward(int dtype, int T, int B, int d, const void* W_x, const void* W_h,
                       const void* x, const void* h, const void* v, const void* d_output, void* dx,
                       void* dW_x, void* dW_h, void* db, void* workspace, size_t workspace_bytes,
                       void* stream) {
  ELMAN_RETURN_IF(check_common(dtype, T, B, d));
  if (d == 0) return ELMAN_OK;
  cudaStream_t st = (cudaStream_t)stream;
  REQUIRE_PTR(dW_x); REQUIRE_PTR(dW_h); REQUIRE_PTR(db);
  const size_t es = esize(dtype);
  if (T == 0 || B == 0) {
    ELMAN_CUDA_CHECK(cudaMemsetAsync(dW_x, 0, (size_t)d * d * es, st));
    ELMAN_CUDA_CHECK(cudaMemsetAsync(dW_h, 0, (size_t)d * d * es, st));
    ELMAN_CUDA_CHECK(cudaMemsetAsync(db, 0, (size_t)d * es, st));
    return ELMAN_OK;
  }
  REQUIRE_PTR(W_x); REQUIRE_PTR(W_h); REQUIRE_PTR(x); REQUIRE_PTR(h); REQUIRE_PTR(v);
  REQUIRE_PTR(d_output); REQUIRE_PTR(dx); REQUIRE_PTR(workspace);
  ELMAN_ARG_CHECK(((uintptr_t)workspace & 255) == 0, "workspace must be 256-byte aligned");
  E1BwdWs w;
  size_t need = carve_e1_bwd(dtype, T, B, d, workspace, &w);
  if (workspace_bytes < need)
    return set_error(ELMAN_ERR_WORKSPACE, "workspace %zu < required %zu", workspace_bytes, need);
  const int TB = T * B;
  ELMAN_RETURN_IF(transpose2d(dtype, d, d, W_h, w.Wt, st));
  ELMAN_RETURN_IF(run_rec_bwd(dtype, T, B, d, w.Wt, h, v, nullptr, d_output, w.dv, nullptr, w.db,
                              w.sync, nullptr, st));
  ELMAN_RETURN_IF(float_to_dtype(dtype, w.db, db, d, st));
  ELMAN_RETURN_IF(gemm_nn(dtype, TB, d, d, w.dv, d, W_x, d, w.WxT, dx, d, 0, st));
  ELMAN_RETURN_IF(weight_grads_pair(dtype, d, TB, w.dv, x, dW_x, h, dW_h, st, w.splitk, w.splitk_bytes));
  return ELMAN_OK;
}

// ------------------ the layer's time-parallel ops around the cell ------------------

size_t elman_add_rmsnorm_backward_workspace(int D) {
  return add_rmsnorm_bwd_scratch_bytes(D < 0 ? 0 : D);
}

int elman_spectral_norm_forward(int dtype, int d, const void* W, void* u, float* v, float* sigma,
                                void* W_eff, float target_radius, float eps, int iterations,
                                void* stream) {
  ELMAN_ARG_CHECK(dtype == ELMAN_F32 || dtype == ELMAN_BF16, "unknown dtype %d", dtype);
  ELMAN_ARG_CHECK(d >= 0 && iterations >= 1, "bad size or iteration count");
  ELMAN_RETURN_IF(check_status_on_entry());
  if (d == 0) return ELMAN_OK;
  REQUIRE_PTR(W); REQUIRE_PTR(u); REQUIRE_PTR(v); REQUIRE_PTR(sigma); REQUIRE_PTR(W_eff);
  return spectral_norm_fwd(dtype, d, W, u, v, sigma, W_eff, target_radius, eps, iterations,
                           (cudaStream_t)stream);
}

int elman_spectral_norm_backward(int dtype, int d, const void* W, const void* u, const float* v,
                                 const float* sigma, const void* dW_eff, void* dW, int accumulate,
                                 float target_radius, float eps, void* stream) {
  ELMAN_ARG_CHECK(dtype == ELMAN_F32 || dtype == ELMAN_BF16, "unknown dtype %d", dtype);
  ELMAN_ARG_CHECK(d >= 0, "negative size");
  ELMAN_RETURN_IF(check_status_on_entry());
  if (d == 0) return ELMAN_OK;
  REQUIRE_PTR(W); REQUIRE_PTR(u); REQUIRE_PTR(v); REQUIRE_PTR(sigma); REQUIRE_PTR(dW_eff);
  REQUIRE_PTR(dW);
  return spectral_norm_bwd(dtype, d, W, u, v, sigma, dW_eff, dW, accumulate, target_radius, eps,
                           (cudaStream_t)stream);
}

int elman_add_rmsnorm_forward(int dtype, long M, int D, const void* x, const float* residual_in,
                              const void* weight, float eps, float* residual_out, void* y,
                              float* rstd, void* stream) {
  ELMAN_ARG_CHECK(dtype == ELMAN_F32 || dtype == ELMAN_BF16, "unknown dtype %d", dtype);
  ELMAN_ARG_CHECK(M >= 0 && D >= 0, "negative size");
  ELMAN_RETURN_IF(check_status_on_entry());
  if (M == 0 || D == 0) return ELMAN_OK;
  REQUIRE_PTR(x); REQUIRE_PTR(weight); REQUIRE_PTR(residual_out); REQUIRE_PTR(y); REQUIRE_PTR(rstd);
  return add_rmsnorm_fwd(dtype, M, D, x, residual_in, weight, eps, residual_out, y, rstd,
                         (cudaStream_t)stream);
}

int elman_add_rmsnorm_backward(int dtype, long M, int D, const void* dy,
                               const float* dresidual_out, const float* residual_out,
                               const float* rstd, const void* weight, float* dresidual_in,
                               void* dx, void* dweight, void* workspace, size_t workspace_bytes,
                               void* stream) {
  ELMAN_ARG_CHECK(dtype == ELMAN_F32 || dtype == ELMAN_BF16, "unknown dtype %d", dtype);
  ELMAN_ARG_CHECK(M >= 0 && D >= 0, "negative size");
  ELMAN_RETURN_IF(check_status_on_entry());
  if (D == 0) return ELMAN_OK;
  REQUIRE_PTR(dweight);
  if (M > 0) {
    REQUIRE_PTR(dy); REQUIRE_PTR(residual_out); REQUIRE_PTR(rstd); REQUIRE_PTR(weight);
    REQUIRE_PTR(workspace);
    ELMAN_ARG_CHECK(dresidual_in != nullptr || dx != nullptr, "neither dresidual_in nor dx given");
    if (workspace_bytes < add_rmsnorm_bwd_scratch_bytes(D))
      return set_error(ELMAN_ERR_WORKSPACE, "workspace %zu < required %zu", workspace_bytes,
                       add_rmsnorm_bwd_scratch_bytes(D));
  }
  return add_rmsnorm_bwd(dtype, M, D, dy, dresidual_out, residual_out, rstd, weight, dresidual_in,
                         dx, dweight, (float*)workspace, (cudaStream_t)stream);
}

size_t elman_in_proj_workspace(int dtype, long M, int d_inner) {
  if (M <= 0 || d_inner <= 0) return 0;
  return ((size_t)M * 2 * d_inner * esize(dtype) + 255) & ~(size_t)255;
}

int elman_in_proj_split_silu(int dtype, long M, int d_inner, int K, const void* u, const void* W_in,
                             void* x_raw, void* x_act, void* z, void* workspace,
                             size_t workspace_bytes, void* stream) {
  ELMAN_ARG_CHECK(dtype == ELMAN_F32 || dtype == ELMAN_BF16, "unknown dtype %d", dtype);
  ELMAN_ARG_CHECK(M >= 0 && d_inner >= 0 && K >= 0 && M < (1L << 31), "bad size");
  ELMAN_RETURN_IF(check_status_on_entry());
  if (M == 0 || d_inner == 0) return ELMAN_OK;
  REQUIRE_PTR(u); REQUIRE_PTR(W_in); REQUIRE_PTR(x_raw); REQUIRE_PTR(x_act); REQUIRE_PTR(z);
  cudaStream_t st = (cudaStream_t)stream;
  const int N = 2 * d_inner;
  if (use_tc(dtype) && (d_inner & 31) == 0 && K > 0 &&
      gemm_tc_supported((int)M, N, K, u, K, W_in, K, x_raw, d_inner, 0) &&
      ((((uintptr_t)x_raw | (uintptr_t)x_act | (uintptr_t)z) & 15) == 0)) {
    // split and silu inside the GEMM's epilogue: xz never exists in memory
    GemmSplit sp{d_inner, x_act, z};
    return gemm_tc((int)M, N, K, (const bf16*)u, K, 0, (const bf16*)W_in, K, 0, nullptr, x_raw,
                   d_inner, 0, 0, st, nullptr, 0, &sp);
  }
  REQUIRE_PTR(workspace);
  if (workspace_bytes < elman_in_proj_workspace(dtype, M, d_inner))
    return set_error(ELMAN_ERR_WORKSPACE, "workspace %zu < required %zu", workspace_bytes,
                     elman_in_proj_workspace(dtype, M, d_inner));
  if (K == 0) ELMAN_CUDA_CHECK(cudaMemsetAsync(workspace, 0, (size_t)M * N * esize(dtype), st));
  else ELMAN_RETURN_IF(proj_nt(dtype, (int)M, N, K, u, K, W_in, K, nullptr, workspace, N, 0, st));
  return split_silu(dtype, M, d_inner, workspace, x_raw, x_act, z, st);
}

int elman_silu_backward_concat(int dtype, long M, int d_inner, const void* d_act, const void* x_raw,
                               const void* dz, void* dxz, void* stream) {
  ELMAN_ARG_CHECK(dtype == ELMAN_F32 || dtype == ELMAN_BF16, "unknown dtype %d", dtype);
  ELMAN_ARG_CHECK(M >= 0 && d_inner >= 0, "negative size");
  ELMAN_RETURN_IF(check_status_on_entry());
  if (M == 0 || d_inner == 0) return ELMAN_OK;
  REQUIRE_PTR(d_act); REQUIRE_PTR(x_raw); REQUIRE_PTR(dz); REQUIRE_PTR(dxz);
  return silu_bwd_concat(dtype, M, d_inner, d_act, x_raw, dz, dxz, (cudaStream_t)stream);
}

int elman_adamw_step(int dtype, long n, void* params, const void* grads, void* exp_avg,
                     void* exp_avg_sq, float lr, float beta1, float beta2, float eps,
                     float weight_decay, float* step, const float* grad_scale, void* stream) {
  ELMAN_ARG_CHECK(dtype == ELMAN_F32 || dtype == ELMAN_BF16, "unknown dtype %d", dtype);
  ELMAN_ARG_CHECK(n >= 0, "negative size");
  ELMAN_RETURN_IF(check_status_on_entry());
  REQUIRE_PTR(step);
  if (n > 0) { REQUIRE_PTR(params); REQUIRE_PTR(grads); REQUIRE_PTR(exp_avg); REQUIRE_PTR(exp_avg_sq); }
  return adamw_step(dtype, n, params, grads, exp_avg, exp_avg_sq, lr, beta1, beta2, eps, weight_decay,
                    step, grad_scale, (cudaStream_t)stream);
}

}  // extern "C"

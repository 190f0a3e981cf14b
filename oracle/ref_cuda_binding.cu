// TEST INFRASTRUCTURE ONLY — C wrappers around the REFERENCE's own CUDA classes.
//
// This file is compiled together with the reference's unmodified kernel sources
// (elman/cuda/lib/{mamba_gated_elman,stock_elman,pure_lowrank_elman_fused}_gpu.cu.cc,
// taken from a checkout of the reference at build time; nothing of them is copied
// here) into oracle/_ref/libelman_ref_cuda.so.  It plays the part of the reference's
// pybind11 layer (elman/cuda/pytorch/elman_ladder.cc:22-281, :2956-3103): construct
// the XForward / XBackward struct with a cuBLAS handle and a stream and call Run().
// Buffers, including the workspace, are allocated by the caller.
#include <cublas_v2.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "hasty/elman_ladder.h"

using namespace hasty::v0::elman_ladder;
typedef __nv_bfloat16 bf16;

static cublasHandle_t g_handle = nullptr;
static cublasHandle_t handle(cudaStream_t st) {
  if (g_handle == nullptr) cublasCreate(&g_handle);
  cublasSetStream(g_handle, st);
  return g_handle;
}

#define DISPATCH(dtype, CALL)                 \
  do {                                        \
    if ((dtype) == 0) { typedef float T; CALL; } \
    else { typedef bf16 T; CALL; }            \
  } while (0)

extern "C" {

int ref_cuda_version(void) { return 1; }

void ref_e1_forward(int dtype, int training, int T_, int B, int d, const void* W_x,
                    const void* W_h, const void* b, const void* x, const void* z, void* h,
                    void* out, void* v, void* ws, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  DISPATCH(dtype, {
    MambaGatedElmanForward<T> f(training != 0, B, d, handle(st), st);
    f.Run(T_, (const T*)W_x, (const T*)W_h, (const T*)b, (const T*)x, (const T*)z, (T*)h, (T*)out,
          (T*)v, (T*)ws);
  });
}

void ref_e1_backward(int dtype, int T_, int B, int d, const void* W_x, const void* W_h,
                     const void* x, const void* z, const void* h, const void* v, const void* dy,
                     void* dx, void* dz, void* dW_x, void* dW_h, void* db, void* ws,
                     void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  DISPATCH(dtype, {
    MambaGatedElmanBackward<T> f(B, d, handle(st), st);
    f.Run(T_, (const T*)W_x, (const T*)W_h, (const T*)x, (const T*)z, (const T*)h, (const T*)v,
          (const T*)dy, (T*)dx, (T*)dz, (T*)dW_x, (T*)dW_h, (T*)db, (T*)ws);
  });
}

void ref_e0_forward(int dtype, int training, int T_, int B, int d, const void* W_x,
                    const void* W_h, const void* W_gate, const void* b, const void* b_gate,
                    const void* x, void* h, void* out, void* v, void* gate_cache, void* ws,
                    void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  DISPATCH(dtype, {
    StockElmanForward<T> f(training != 0, B, d, handle(st), st);
    f.Run(T_, (const T*)W_x, (const T*)W_h, (const T*)W_gate, (const T*)b, (const T*)b_gate,
          (const T*)x, (T*)h, (T*)out, (T*)v, (T*)gate_cache, (T*)ws);
  });
}

void ref_e0_backward(int dtype, int T_, int B, int d, const void* W_x, const void* W_h,
                     const void* W_gate, const void* x, const void* h, const void* v,
                     const void* gate_cache, const void* dy, void* dx, void* dW_x, void* dW_h,
                     void* dW_gate, void* db, void* db_gate, void* ws, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  DISPATCH(dtype, {
    StockElmanBackward<T> f(B, d, handle(st), st);
    f.Run(T_, (const T*)W_x, (const T*)W_h, (const T*)W_gate, (const T*)x, (const T*)h,
          (const T*)v, (const T*)gate_cache, (const T*)dy, (T*)dx, (T*)dW_x, (T*)dW_h,
          (T*)dW_gate, (T*)db, (T*)db_gate, (T*)ws);
  });
}

void ref_e5_forward(int dtype, int training, int T_, int B, int d, int r, const void* U_h,
                    const void* V_h, const void* U_x, const void* V_x, const void* U_z,
                    const void* V_z, const void* b, const void* x, void* h, void* out, void* v,
                    void* ws, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  DISPATCH(dtype, {
    PureLowRankElmanForwardFused<T> f(training != 0, B, d, r, handle(st), st);
    f.Run(T_, (const T*)U_h, (const T*)V_h, (const T*)U_x, (const T*)V_x, (const T*)U_z,
          (const T*)V_z, (const T*)b, (const T*)x, (T*)h, (T*)out, (T*)v, (T*)ws);
  });
}

void ref_e5_backward(int dtype, int T_, int B, int d, int r, const void* U_h, const void* V_h,
                     const void* U_x, const void* V_x, const void* U_z, const void* V_z,
                     const void* x, const void* h, const void* v, const void* dy, void* dx,
                     void* dU_h, void* dV_h, void* dU_x, void* dV_x, void* dU_z, void* dV_z,
                     void* db, void* ws, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  DISPATCH(dtype, {
    PureLowRankElmanBackwardFused<T> f(B, d, r, handle(st), st);
    f.Run(T_, (const T*)U_h, (const T*)V_h, (const T*)U_x, (const T*)V_x, (const T*)U_z,
          (const T*)V_z, (const T*)x, (const T*)h, (const T*)v, (const T*)dy, (T*)dx, (T*)dU_h,
          (T*)dV_h, (T*)dU_x, (T*)dV_x, (T*)dU_z, (T*)dV_z, (T*)db, (T*)ws);
  });
}

}  // extern "C"

// Time-parallel elementwise work around the cell, one kernel per pass instead of the
// reference's chains of framework ops:
//
//  * residual add + RMSNorm with an fp32 residual stream, forward and backward
//    (elman/models/ladder_lm.py:986-1003 and :1013-1026 of the reference: the Triton
//    rms_norm_fn of mamba_ssm when present, else add, cast, nn.RMSNorm, cast);
//  * the tail of the layer's input projection: split xz = in_proj(u) into its halves and
//    apply silu to the first (elman/models/mamba_gated_elman.py:283-297: chunk, silu, two
//    permute().contiguous() copies), and the matching backward (silu' and re-joining the two
//    gradient halves for the projection's backward GEMMs).  On the bf16 tensor-core path the
//    split and the silu run inside the GEMM's epilogue (gemm_tc.cu); these kernels are the
//    fp32 / irregular-shape path and the backward.
//
// All kernels are HBM-bound streaming passes: rows are handled by whole thread blocks with
// 16-byte accesses where the row length allows, no atomics (weight-gradient partial sums go
// through a [blocks, D] scratch and a fixed-order reduction).
#include "common.cuh"

namespace elman {

namespace {

constexpr int NT = 256;           // threads per block
constexpr int MAX_BLOCKS = 592;   // 4 per SM on a 148-SM part
constexpr int BWD_BLOCKS = 296;   // blocks (= partial-sum rows) of the norm's backward pass

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();                 // red may still be read from the previous use
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < NT / 32; ++w) t += red[w];   // same order in every thread: deterministic
  return t;
}

// res_out = x + res_in (fp32);  y = T(round_T(res_out) * rstd * w),  rstd = rsqrt(mean(.^2) + eps)
template <typename T>
__global__ void __launch_bounds__(NT)
add_rmsnorm_fwd_kernel(long M, int D, const T* __restrict__ x, const float* __restrict__ res_in,
                       const T* __restrict__ w, float eps, float* __restrict__ res_out,
                       T* __restrict__ y, float* __restrict__ rstd_out) {
  __shared__ float red[NT / 32];
  for (long row = blockIdx.x; row < M; row += gridDim.x) {
    const T* xr = x + row * D;
    const float* ri = res_in ? res_in + row * D : nullptr;
    float* ro = res_out + row * D;
    float ss = 0.f;
    for (int j = threadIdx.x; j < D; j += NT) {
      float r = to_f(xr[j]);
      if (ri) r += ri[j];
      ro[j] = r;
      const float v = to_f(from_f<T>(r));     // the norm sees the residual in the layer's dtype
      ss += v * v;
    }
    const float tot = block_sum(ss, red);
    const float rs = rsqrtf(tot / (float)D + eps);
    if (threadIdx.x == 0) rstd_out[row] = rs;
    T* yr = y + row * D;
    for (int j = threadIdx.x; j < D; j += NT) {
      const float v = to_f(from_f<T>(ro[j]));   // own write, same thread: visible
      yr[j] = from_f<T>(v * rs * to_f(w[j]));
    }
  }
}

// Backward of the above for one row:
//   xh = round_T(res_out) * rstd,  g = dy * w,  c = mean(g * xh)
//   dres_in = dres_out + rstd * (g - xh * c)      (fp32),  dx = T(dres_in)
//   dw_partial[block, j] += dy * xh
template <typename T>
__global__ void __launch_bounds__(NT)
add_rmsnorm_bwd_kernel(long M, int D, const T* __restrict__ dy, const float* __restrict__ dres_out,
                       const float* __restrict__ res_out, const float* __restrict__ rstd,
                       const T* __restrict__ w, float* __restrict__ dres_in, T* __restrict__ dx,
                       float* __restrict__ dw_partial) {
  __shared__ float red[NT / 32];
  // this thread's columns are the same for every row: keep their weight-gradient sums in
  // registers (up to 8 columns per thread, i.e. D <= 2048; wider rows go through memory)
  constexpr int KEEP = 8;
  float dwacc[KEEP];
#pragma unroll
  for (int k = 0; k < KEEP; ++k) dwacc[k] = 0.f;
  const bool in_regs = D <= KEEP * NT;
  float* dwp = dw_partial + (long)blockIdx.x * D;
  if (!in_regs)
    for (int j = threadIdx.x; j < D; j += NT) dwp[j] = 0.f;
  for (long row = blockIdx.x; row < M; row += gridDim.x) {
    const T* dyr = dy + row * D;
    const float* ro = res_out + row * D;
    const float rs = rstd[row];
    float dot = 0.f;
    for (int j = threadIdx.x; j < D; j += NT) {
      const float xh = to_f(from_f<T>(ro[j])) * rs;
      dot += to_f(dyr[j]) * to_f(w[j]) * xh;
    }
    const float c = block_sum(dot, red) / (float)D;
    int k = 0;
    for (int j = threadIdx.x; j < D; j += NT, ++k) {
      const float xh = to_f(from_f<T>(ro[j])) * rs;
      const float dyv = to_f(dyr[j]);
      float g = rs * (dyv * to_f(w[j]) - xh * c);
      if (dres_out) g += dres_out[row * D + j];
      if (dres_in) dres_in[row * D + j] = g;
      if (dx) dx[row * D + j] = from_f<T>(g);
      if (in_regs) {
#pragma unroll
        for (int q = 0; q < KEEP; ++q)
          if (q == k) dwacc[q] += dyv * xh;
      } else {
        dwp[j] += dyv * xh;
      }
    }
  }
  if (in_regs) {
    int k = 0;
    for (int j = threadIdx.x; j < D; j += NT, ++k) {
#pragma unroll
      for (int q = 0; q < KEEP; ++q)
        if (q == k) dwp[j] = dwacc[q];
    }
  }
}

// ---- bf16 rows whose length is a multiple of 8: 16-byte accesses, each row read once ----
constexpr int VCH = 2;   // 8-element chunks a thread keeps in registers: rows up to VCH*NT*8 wide

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float2 t = __bfloat1622float2(h[q]);
    f[2 * q] = t.x;
    f[2 * q + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int q = 0; q < 4; ++q) h[q] = __floats2bfloat162_rn(f[2 * q], f[2 * q + 1]);
  return u;
}

__global__ void __launch_bounds__(NT)
add_rmsnorm_fwd_bf16x8_kernel(long M, int D, const uint4* __restrict__ x, const float4* __restrict__ res_in,
                              const uint4* __restrict__ w, float eps, float4* __restrict__ res_out,
                              uint4* __restrict__ y, float* __restrict__ rstd_out) {
  __shared__ float red[NT / 32];
  const int nch = D / 8;
  for (long row = blockIdx.x; row < M; row += gridDim.x) {
    float v[VCH][8];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < VCH; ++k) {
      const int c = threadIdx.x + k * NT;
      if (c < nch) {
        float r[8];
        unpack8(x[row * nch + c], r);
        if (res_in != nullptr) {
          const float4 a = res_in[(row * nch + c) * 2], b = res_in[(row * nch + c) * 2 + 1];
          r[0] += a.x; r[1] += a.y; r[2] += a.z; r[3] += a.w;
          r[4] += b.x; r[5] += b.y; r[6] += b.z; r[7] += b.w;
        }
        res_out[(row * nch + c) * 2] = make_float4(r[0], r[1], r[2], r[3]);
        res_out[(row * nch + c) * 2 + 1] = make_float4(r[4], r[5], r[6], r[7]);
        unpack8(pack8(r), v[k]);          // the norm sees the residual rounded to bf16
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += v[k][e] * v[k][e];
      }
    }
    const float rs = rsqrtf(block_sum(ss, red) / (float)D + eps);
    if (threadIdx.x == 0) rstd_out[row] = rs;
#pragma unroll
    for (int k = 0; k < VCH; ++k) {
      const int c = threadIdx.x + k * NT;
      if (c < nch) {
        float wf[8], o[8];
        unpack8(w[c], wf);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = v[k][e] * rs * wf[e];
        y[row * nch + c] = pack8(o);
      }
    }
  }
}

__global__ void __launch_bounds__(NT)
add_rmsnorm_bwd_bf16x8_kernel(long M, int D, const uint4* __restrict__ dy, const float4* __restrict__ dres_out,
                              const float4* __restrict__ res_out, const float* __restrict__ rstd,
                              const uint4* __restrict__ w, float4* __restrict__ dres_in,
                              uint4* __restrict__ dx, float* __restrict__ dw_partial) {
  __shared__ float red[NT / 32];
  const int nch = D / 8;
  float dwacc[VCH][8];
  float wf[VCH][8];
#pragma unroll
  for (int k = 0; k < VCH; ++k) {
    const int c = threadIdx.x + k * NT;
#pragma unroll
    for (int e = 0; e < 8; ++e) { dwacc[k][e] = 0.f; wf[k][e] = 0.f; }
    if (c < nch) unpack8(w[c], wf[k]);
  }
  for (long row = blockIdx.x; row < M; row += gridDim.x) {
    const float rs = rstd[row];
    float dyv[VCH][8], xh[VCH][8];
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < VCH; ++k) {
      const int c = threadIdx.x + k * NT;
      if (c < nch) {
        unpack8(dy[row * nch + c], dyv[k]);
        const float4 a = res_out[(row * nch + c) * 2], b = res_out[(row * nch + c) * 2 + 1];
        const float r[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        unpack8(pack8(r), xh[k]);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xh[k][e] *= rs;
          dot += dyv[k][e] * wf[k][e] * xh[k][e];
        }
      }
    }
    const float cmean = block_sum(dot, red) / (float)D;
#pragma unroll
    for (int k = 0; k < VCH; ++k) {
      const int c = threadIdx.x + k * NT;
      if (c < nch) {
        float g[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          g[e] = rs * (dyv[k][e] * wf[k][e] - xh[k][e] * cmean);
          dwacc[k][e] += dyv[k][e] * xh[k][e];
        }
        if (dres_out != nullptr) {
          const float4 a = dres_out[(row * nch + c) * 2], b = dres_out[(row * nch + c) * 2 + 1];
          g[0] += a.x; g[1] += a.y; g[2] += a.z; g[3] += a.w;
          g[4] += b.x; g[5] += b.y; g[6] += b.z; g[7] += b.w;
        }
        if (dres_in != nullptr) {
          dres_in[(row * nch + c) * 2] = make_float4(g[0], g[1], g[2], g[3]);
          dres_in[(row * nch + c) * 2 + 1] = make_float4(g[4], g[5], g[6], g[7]);
        }
        if (dx != nullptr) dx[row * nch + c] = pack8(g);
      }
    }
  }
  float4* dwp = reinterpret_cast<float4*>(dw_partial + (long)blockIdx.x * D);
#pragma unroll
  for (int k = 0; k < VCH; ++k) {
    const int c = threadIdx.x + k * NT;
    if (c < nch) {
      dwp[c * 2] = make_float4(dwacc[k][0], dwacc[k][1], dwacc[k][2], dwacc[k][3]);
      dwp[c * 2 + 1] = make_float4(dwacc[k][4], dwacc[k][5], dwacc[k][6], dwacc[k][7]);
    }
  }
}

bool rows_vectorisable(int dtype, int D, const void* a, const void* b, const void* c, const void* d,
                       const void* e, const void* f) {
  if (dtype != ELMAN_BF16 || (D & 7) != 0 || D > VCH * NT * 8) return false;
  const uintptr_t bits = (uintptr_t)a | (uintptr_t)b | (uintptr_t)c | (uintptr_t)d | (uintptr_t)e |
                         (uintptr_t)f;
  return (bits & 15) == 0;
}

// out[j] = sum over the rows of partial[rows, D]: 32 columns per block, 8 row lanes that are
// combined in a fixed order (deterministic)
template <typename T>
__global__ void __launch_bounds__(256)
rows_sum_kernel(int rows, int D, const float* __restrict__ partial, T* __restrict__ out) {
  __shared__ float acc[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int j = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (j < D)
    for (int r = ty; r < rows; r += 8) s += partial[(long)r * D + j];
  acc[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && j < D) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += acc[k][tx];
    out[j] = from_f<T>(t);
  }
}

// xz [M, 2d] -> x_raw [M, d] (first half), x_act = silu(first half), z [M, d] (second half)
template <typename T>
__global__ void split_silu_kernel(long M, int d, const T* __restrict__ xz, T* __restrict__ x_raw,
                                  T* __restrict__ x_act, T* __restrict__ z) {
  const long n = M * d;
  for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long)gridDim.x * blockDim.x) {
    const long m = e / d;
    const int j = (int)(e - m * d);
    const T xr = xz[m * 2 * d + j];
    const float xf = to_f(xr);
    x_raw[e] = xr;
    x_act[e] = from_f<T>(siluf_(xf));
    z[e] = xz[m * 2 * d + d + j];
  }
}

// dxz [M, 2d] = [ d_act * silu'(x_raw) | dz ]
template <typename T>
__global__ void silu_bwd_concat_kernel(long M, int d, const T* __restrict__ d_act,
                                       const T* __restrict__ x_raw, const T* __restrict__ dz,
                                       T* __restrict__ dxz) {
  const long n = M * d;
  for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long)gridDim.x * blockDim.x) {
    const long m = e / d;
    const int j = (int)(e - m * d);
    dxz[m * 2 * d + j] = from_f<T>(to_f(d_act[e]) * dsiluf_(to_f(x_raw[e])));
    dxz[m * 2 * d + d + j] = dz[e];
  }
}

// 8 bf16 per thread and access: the streaming forms used when d is a multiple of 8
__global__ void silu_bwd_concat_bf16x8_kernel(long M, int d, const uint4* __restrict__ d_act,
                                              const uint4* __restrict__ x_raw,
                                              const uint4* __restrict__ dz, uint4* __restrict__ dxz) {
  const int dv = d / 8;
  const long n = M * dv;
  for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long)gridDim.x * blockDim.x) {
    const long m = e / dv;
    const int j = (int)(e - m * dv);
    const uint4 a = d_act[e], x = x_raw[e];
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&x);
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 af = __bfloat1622float2(a2[q]), xf = __bfloat1622float2(x2[q]);
      o2[q] = __floats2bfloat162_rn(af.x * dsiluf_(xf.x), af.y * dsiluf_(xf.y));
    }
    dxz[m * 2 * dv + j] = o;
    dxz[m * 2 * dv + dv + j] = dz[e];
  }
}

template <typename T>
__global__ void gate_apply_kernel(long n, const T* __restrict__ h, const T* __restrict__ zg, T* __restrict__ y) {
  for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long)gridDim.x * blockDim.x)
    y[e] = from_f<T>(to_f(h[e]) * siluf_(to_f(zg[e])));
}
template <typename T>
__global__ void gate_backward_prep_kernel(long n, const T* __restrict__ dy, const T* __restrict__ h,
                                          const T* __restrict__ zg, float scale, T* __restrict__ dzg,
                                          T* __restrict__ t) {
  for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long)gridDim.x * blockDim.x) {
    const float g = to_f(zg[e]), d = to_f(dy[e]);
    dzg[e] = from_f<T>(d * to_f(h[e]) * dsiluf_(g));
    t[e] = from_f<T>(d * siluf_(g) * scale);
  }
}
template <typename T>
__global__ void scale_copy_kernel(long n, const T* __restrict__ src, float scale, T* __restrict__ dst) {
  for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long)gridDim.x * blockDim.x)
    dst[e] = from_f<T>(to_f(src[e]) * scale);
}
template <typename T>
__global__ void fill_value_kernel(long n, float value, T* __restrict__ dst) {
  const T v = from_f<T>(value);
  for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long)gridDim.x * blockDim.x)
    dst[e] = v;
}

int grid_for(long n_items) {
  long g = (n_items + NT - 1) / NT;
  if (g < 1) g = 1;
  return (int)(g < MAX_BLOCKS ? g : MAX_BLOCKS);
}

}  // namespace

size_t add_rmsnorm_bwd_scratch_bytes(int D) { return (size_t)BWD_BLOCKS * D * sizeof(float); }

int add_rmsnorm_fwd(int dtype, long M, int D, const void* x, const float* res_in, const void* w,
                    float eps, float* res_out, void* y, float* rstd, cudaStream_t st) {
  if (M == 0 || D == 0) return ELMAN_OK;
  const int grid = (int)(M < MAX_BLOCKS ? M : MAX_BLOCKS);
  if (rows_vectorisable(dtype, D, x, res_in, w, res_out, y, nullptr))
    add_rmsnorm_fwd_bf16x8_kernel<<<grid, NT, 0, st>>>(M, D, (const uint4*)x, (const float4*)res_in,
                                                      (const uint4*)w, eps, (float4*)res_out,
                                                      (uint4*)y, rstd);
  else if (dtype == ELMAN_F32)
    add_rmsnorm_fwd_kernel<float><<<grid, NT, 0, st>>>(M, D, (const float*)x, res_in, (const float*)w,
                                                      eps, res_out, (float*)y, rstd);
  else
    add_rmsnorm_fwd_kernel<bf16><<<grid, NT, 0, st>>>(M, D, (const bf16*)x, res_in, (const bf16*)w,
                                                     eps, res_out, (bf16*)y, rstd);
  count_launch(false);
  ELMAN_CUDA_CHECK(cudaGetLastError());
  return ELMAN_OK;
}

int add_rmsnorm_bwd(int dtype, long M, int D, const void* dy, const float* dres_out,
                    const float* res_out, const float* rstd, const void* w, float* dres_in,
                    void* dx, void* dw, float* scratch, cudaStream_t st) {
  if (D == 0) return ELMAN_OK;
  if (M == 0) {
    ELMAN_CUDA_CHECK(cudaMemsetAsync(dw, 0, (size_t)D * (dtype == ELMAN_F32 ? 4 : 2), st));
    return ELMAN_OK;
  }
  const int grid = (int)(M < BWD_BLOCKS ? M : BWD_BLOCKS);
  if (rows_vectorisable(dtype, D, dy, dres_out, res_out, w, dres_in, dx) &&
      ((uintptr_t)scratch & 15) == 0) {
    add_rmsnorm_bwd_bf16x8_kernel<<<grid, NT, 0, st>>>(
        M, D, (const uint4*)dy, (const float4*)dres_out, (const float4*)res_out, rstd, (const uint4*)w,
        (float4*)dres_in, (uint4*)dx, scratch);
    rows_sum_kernel<bf16><<<(D + 31) / 32, 256, 0, st>>>(grid, D, scratch, (bf16*)dw);
  } else if (dtype == ELMAN_F32) {
    add_rmsnorm_bwd_kernel<float><<<grid, NT, 0, st>>>(M, D, (const float*)dy, dres_out, res_out, rstd,
                                                      (const float*)w, dres_in, (float*)dx, scratch);
    rows_sum_kernel<float><<<(D + 31) / 32, 256, 0, st>>>(grid, D, scratch, (float*)dw);
  } else {
    add_rmsnorm_bwd_kernel<bf16><<<grid, NT, 0, st>>>(M, D, (const bf16*)dy, dres_out, res_out, rstd,
                                                     (const bf16*)w, dres_in, (bf16*)dx, scratch);
    rows_sum_kernel<bf16><<<(D + 31) / 32, 256, 0, st>>>(grid, D, scratch, (bf16*)dw);
  }
  count_launch(false);
  count_launch(false);
  ELMAN_CUDA_CHECK(cudaGetLastError());
  return ELMAN_OK;
}

int split_silu(int dtype, long M, int d, const void* xz, void* x_raw, void* x_act, void* z,
               cudaStream_t st) {
  if (M == 0 || d == 0) return ELMAN_OK;
  const int grid = grid_for(M * d);
  if (dtype == ELMAN_F32)
    split_silu_kernel<float><<<grid, NT, 0, st>>>(M, d, (const float*)xz, (float*)x_raw, (float*)x_act,
                                                 (float*)z);
  else
    split_silu_kernel<bf16><<<grid, NT, 0, st>>>(M, d, (const bf16*)xz, (bf16*)x_raw, (bf16*)x_act,
                                                (bf16*)z);
  count_launch(false);
  ELMAN_CUDA_CHECK(cudaGetLastError());
  return ELMAN_OK;
}

int gate_apply(int dtype, long n, const void* h, const void* zg, void* y, cudaStream_t st) {
  if (dtype == ELMAN_F32) {
    if (n > 0) gate_apply_kernel<float><<<grid_for(n), NT, 0, st>>>(n, (const float*)h, (const float*)zg, (float*)y);
  } else {
    if (n > 0) gate_apply_kernel<bf16><<<grid_for(n), NT, 0, st>>>(n, (const bf16*)h, (const bf16*)zg, (bf16*)y);
  }
  if (n > 0) count_launch(false);
  ELMAN_CUDA_CHECK(cudaGetLastError());
  return ELMAN_OK;
}

int gate_backward_prep(int dtype, long n, const void* dy, const void* h, const void* zg, float scale,
                       void* dzg, void* t, cudaStream_t st) {
  if (n <= 0) return ELMAN_OK;
  if (dtype == ELMAN_F32)
    gate_backward_prep_kernel<float><<<grid_for(n), NT, 0, st>>>(
        n, (const float*)dy, (const float*)h, (const float*)zg, scale, (float*)dzg, (float*)t);
  else
    gate_backward_prep_kernel<bf16><<<grid_for(n), NT, 0, st>>>(
        n, (const bf16*)dy, (const bf16*)h, (const bf16*)zg, scale, (bf16*)dzg, (bf16*)t);
  count_launch(false);
  ELMAN_CUDA_CHECK(cudaGetLastError());
  return ELMAN_OK;
}

int scale_copy(int dtype, long n, const void* src, float scale, void* dst, cudaStream_t st) {
  if (n <= 0) return ELMAN_OK;
  if (dtype == ELMAN_F32)
    scale_copy_kernel<float><<<grid_for(n), NT, 0, st>>>(n, (const float*)src, scale, (float*)dst);
  else
    scale_copy_kernel<bf16><<<grid_for(n), NT, 0, st>>>(n, (const bf16*)src, scale, (bf16*)dst);
  count_launch(false);
  ELMAN_CUDA_CHECK(cudaGetLastError());
  return ELMAN_OK;
}

int fill_value(int dtype, long n, float value, void* dst, cudaStream_t st) {
  if (n <= 0) return ELMAN_OK;
  if (dtype == ELMAN_F32) fill_value_kernel<float><<<grid_for(n), NT, 0, st>>>(n, value, (float*)dst);
  else fill_value_kernel<bf16><<<grid_for(n), NT, 0, st>>>(n, value, (bf16*)dst);
  count_launch(false);
  ELMAN_CUDA_CHECK(cudaGetLastError());
  return ELMAN_OK;
}

int silu_bwd_concat(int dtype, long M, int d, const void* d_act, const void* x_raw, const void* dz,
                    void* dxz, cudaStream_t st) {
  if (M == 0 || d == 0) return ELMAN_OK;
  if (dtype == ELMAN_F32) {
    silu_bwd_concat_kernel<float><<<grid_for(M * d), NT, 0, st>>>(
        M, d, (const float*)d_act, (const float*)x_raw, (const float*)dz, (float*)dxz);
  } else if ((d & 7) == 0 && (((uintptr_t)d_act | (uintptr_t)x_raw | (uintptr_t)dz | (uintptr_t)dxz) & 15) == 0) {
    silu_bwd_concat_bf16x8_kernel<<<grid_for(M * (d / 8)), NT, 0, st>>>(
        M, d, (const uint4*)d_act, (const uint4*)x_raw, (const uint4*)dz, (uint4*)dxz);
  } else {
    silu_bwd_concat_kernel<bf16><<<grid_for(M * d), NT, 0, st>>>(
        M, d, (const bf16*)d_act, (const bf16*)x_raw, (const bf16*)dz, (bf16*)dxz);
  }
  count_launch(false);
  ELMAN_CUDA_CHECK(cudaGetLastError());
  return ELMAN_OK;
}

}  // namespace elman

// CUDA-core GEMM with arbitrary element strides, plus the small data-movement
// kernels (transpose, column sums, casts).  This is the fp32 path of the library
// and the path bf16 takes when a shape does not fit the tcgen05 kernels.
#include "common.cuh"

namespace elman {

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(int M, int N, int K, const T* __restrict__ A, long sAm, long sAk,
                 const T* __restrict__ B, long sBk, long sBn, const T* __restrict__ bias,
                 T* __restrict__ C, long ldc, int accumulate) {
  __shared__ float As[TK][TM + 4];
  __shared__ float Bs[TK][TN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  const int tx = tid % 16, ty = tid / 16;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const bool a_kfast = (sAk == 1);
  const bool b_kfast = (sBk == 1);
  for (int k0 = 0; k0 < K; k0 += TK) {
    for (int i = tid; i < TM * TK; i += 256) {
      int k, m;
      if (a_kfast) { k = i % TK; m = i / TK; } else { m = i % TM; k = i / TM; }
      int gm = m0 + m, gk = k0 + k;
      As[k][m] = (gm < M && gk < K) ? to_f(A[gm * sAm + gk * sAk]) : 0.f;
    }
    for (int i = tid; i < TN * TK; i += 256) {
      int k, n;
      if (b_kfast) { k = i % TK; n = i / TK; } else { n = i % TN; k = i / TN; }
      int gn = n0 + n, gk = k0 + k;
      Bs[k][n] = (gn < N && gk < K) ? to_f(B[gk * sBk + gn * sBn]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < TK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float r = acc[i][j];
      if (bias != nullptr) r += to_f(bias[gn]);
      if (accumulate) r += to_f(C[gm * ldc + gn]);
      C[gm * ldc + gn] = from_f<T>(r);
    }
  }
}

template <typename T>
__global__ void transpose_kernel(int rows, int cols, const T* __restrict__ in,
                                 T* __restrict__ out) {
  __shared__ T tile[32][33];
  int c = blockIdx.x * 32 + threadIdx.x;
  for (int j = threadIdx.y; j < 32; j += 8) {
    int r = blockIdx.y * 32 + j;
    if (r < rows && c < cols) tile[j][threadIdx.x] = in[(long)r * cols + c];
  }
  __syncthreads();
  int r2 = blockIdx.y * 32 + threadIdx.x;  // row index of `in`, column index of `out`
  for (int j = threadIdx.y; j < 32; j += 8) {
    int c2 = blockIdx.x * 32 + j;
    if (r2 < rows && c2 < cols) out[(long)c2 * rows + r2] = tile[threadIdx.x][j];
  }
}

constexpr int CS_SLICES = 64;

// pass 1: slice s sums rows s, s+S, ... into partial[s][n]
template <typename T>
__global__ void colsum_partial_kernel(long M, int N, const T* __restrict__ in,
                                      float* __restrict__ partial) {
  int n = blockIdx.x * blockDim.x + threadIdx.x;
  int s = blockIdx.y;
  if (n >= N) return;
  long per = (M + CS_SLICES - 1) / CS_SLICES;
  long m_lo = s * per, m_hi = m_lo + per < M ? m_lo + per : M;
  float acc = 0.f;
  for (long m = m_lo; m < m_hi; ++m) acc += to_f(in[m * N + n]);
  partial[(long)s * N + n] = acc;
}
template <typename T>
__global__ void colsum_final_kernel(int N, const float* __restrict__ partial,
                                    T* __restrict__ out) {
  int n = blockIdx.x * blockDim.x + threadIdx.x;
  if (n >= N) return;
  float acc = 0.f;
  for (int s = 0; s < CS_SLICES; ++s) acc += partial[(long)s * N + n];
  out[n] = from_f<T>(acc);
}

template <typename T>
__global__ void copy_kernel(const T* __restrict__ src, T* __restrict__ dst, long n) {
  long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  long stride = (long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) dst[i] = src[i];
}
template <typename T>
__global__ void cast_kernel(const float* __restrict__ src, T* __restrict__ dst, long n) {
  long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  long stride = (long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) dst[i] = from_f<T>(src[i]);
}

inline int grid_for(long n, int block) {
  long g = (n + block - 1) / block;
  return (int)(g < 1 ? 1 : (g > 148L * 16 ? 148L * 16 : g));
}

}  // namespace

int gemm_generic(int dtype, int M, int N, int K, const void* A, long sAm, long sAk,
                 const void* B, long sBk, long sBn, const void* bias, void* C, long ldc,
                 int accumulate, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return ELMAN_OK;
  dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
  if (dtype == ELMAN_F32) {
    gemm_simt_kernel<float><<<grid, 256, 0, stream>>>(
        M, N, K, (const float*)A, sAm, sAk, (const float*)B, sBk, sBn, (const float*)bias,
        (float*)C, ldc, accumulate);
  } else {
    gemm_simt_kernel<bf16><<<grid, 256, 0, stream>>>(
        M, N, K, (const bf16*)A, sAm, sAk, (const bf16*)B, sBk, sBn, (const bf16*)bias,
        (bf16*)C, ldc, accumulate);
  }
  count_launch(false);
  ELMAN_CUDA_CHECK(cudaGetLastError());
  return ELMAN_OK;
}

int transpose2d(int dtype, int rows_in, int cols_in, const void* in, void* out,
                cudaStream_t stream) {
  if (rows_in <= 0 || cols_in <= 0) return ELMAN_OK;
  dim3 grid((cols_in + 31) / 32, (rows_in + 31) / 32), block(32, 8);
  if (dtype == ELMAN_F32)
    transpose_kernel<float><<<grid, block, 0, stream>>>(rows_in, cols_in, (const float*)in,
                                                        (float*)out);
  else
    transpose_kernel<bf16><<<grid, block, 0, stream>>>(rows_in, cols_in, (const bf16*)in,
                                                       (bf16*)out);
  count_launch(false);
  ELMAN_CUDA_CHECK(cudaGetLastError());
  return ELMAN_OK;
}

size_t column_sum_scratch_bytes(int N) { return (size_t)CS_SLICES * N * sizeof(float); }

int column_sum(int dtype, long M, int N, const void* in, void* out, float* scratch,
               cudaStream_t stream) {
  if (N <= 0) return ELMAN_OK;
  dim3 grid((N + 127) / 128, CS_SLICES);
  if (dtype == ELMAN_F32) {
    colsum_partial_kernel<float><<<grid, 128, 0, stream>>>(M, N, (const float*)in, scratch);
    colsum_final_kernel<float><<<(N + 127) / 128, 128, 0, stream>>>(N, scratch, (float*)out);
  } else {
    colsum_partial_kernel<bf16><<<grid, 128, 0, stream>>>(M, N, (const bf16*)in, scratch);
    colsum_final_kernel<bf16><<<(N + 127) / 128, 128, 0, stream>>>(N, scratch, (bf16*)out);
  }
  count_launch(false);
  count_launch(false);
  ELMAN_CUDA_CHECK(cudaGetLastError());
  return ELMAN_OK;
}

int copy_rows(int dtype, const void* src, void* dst, long n, cudaStream_t stream) {
  if (n <= 0) return ELMAN_OK;
  size_t bytes = (size_t)n * (dtype == ELMAN_F32 ? 4 : 2);
  ELMAN_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, stream));
  return ELMAN_OK;
}

namespace {
// dst[rows_dst, cols_dst] = src[rows, cols] cropped or zero-padded to the new extents
template <typename T>
__global__ void resize2d_kernel(const T* __restrict__ src, int rows, int cols, T* __restrict__ dst,
                                int rows_dst, int cols_dst) {
  const long n = (long)rows_dst * cols_dst;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long)gridDim.x * blockDim.x) {
    const int r = (int)(i / cols_dst), c = (int)(i - (long)r * cols_dst);
    dst[i] = (r < rows && c < cols) ? src[(long)r * cols + c] : from_f<T>(0.f);
  }
}
}  // namespace

int resize2d(int dtype, const void* src, int rows, int cols, void* dst, int rows_dst, int cols_dst,
             cudaStream_t stream) {
  const long n = (long)rows_dst * cols_dst;
  if (n <= 0) return ELMAN_OK;
  if (dtype == ELMAN_F32)
    resize2d_kernel<float><<<grid_for(n, 256), 256, 0, stream>>>((const float*)src, rows, cols,
                                                                 (float*)dst, rows_dst, cols_dst);
  else
    resize2d_kernel<bf16><<<grid_for(n, 256), 256, 0, stream>>>((const bf16*)src, rows, cols,
                                                                (bf16*)dst, rows_dst, cols_dst);
  count_launch(false);
  ELMAN_CUDA_CHECK(cudaGetLastError());
  return ELMAN_OK;
}

int float_to_dtype(int dtype, const float* src, void* dst, long n, cudaStream_t stream) {
  if (n <= 0) return ELMAN_OK;
  if (dtype == ELMAN_F32)
    cast_kernel<float><<<grid_for(n, 256), 256, 0, stream>>>(src, (float*)dst, n);
  else
    cast_kernel<bf16><<<grid_for(n, 256), 256, 0, stream>>>(src, (bf16*)dst, n);
  count_launch(false);
  ELMAN_CUDA_CHECK(cudaGetLastError());
  return ELMAN_OK;
}

}  // namespace elman

// Spectral normalisation of a recurrent matrix as ONE kernel per direction:
//   forward   three power-iteration steps from a persistent vector u
//               v = W^T u / (|W^T u| + eps),  u = W v / (|W v| + eps)
//             sigma = |u^T W v|,  W_eff = W * target / (sigma + eps)
//   backward  dW += s G - <G, W> target / (sigma + eps)^2 * u v^T,   s = target / (sigma + eps)
//             (sigma depends on W through u^T W v with u, v held constant)
// This is what the reference cells' get_W_h does with a dozen framework ops per layer and
// step (elman/models/mamba_gated_elman.py:123-146, elman/models/stock_elman.py:104-125).
//
// One thread-block cluster works on one matrix: CTA k owns d/NC rows of W (for W v and for the
// partial sums of W^T u) and d/NC columns of v.  Partial vectors, column slices and norms are
// pushed into the peers' shared memory (distributed shared memory stores) between hardware
// cluster barriers — no global synchronisation, no spin-wait.  All arithmetic is fp32; a CTA's
// rows of W are read once into shared memory when they fit (d = 1280 in bf16: 200 KB), else
// from L2 in every pass.
#include "tc_helpers.cuh"

namespace elman {

namespace {

using namespace tch;

constexpr int SN_THREADS = 256;
constexpr int SN_MAX_NC = 16;

struct SpectralParams {
  int d, NC, R;            // R = d / NC rows (and columns of v) per CTA
  int iters;
  int cache;               // forward: my rows of W are copied into shared memory once
  float target, eps;
  const void* W;           // [d, d]
  void* u;                 // [d] in W's dtype, advanced in place
  float* v;                // [d] fp32 out (saved for the backward pass)
  float* sigma;            // [1] fp32 out
  void* W_eff;             // [d, d] out
  const void* G;           // backward: gradient of W_eff [d, d]
  void* dW;                // backward: gradient of W [d, d], accumulated into
  int accumulate;          // backward: dW += (1) or dW = (0)
};

__device__ __forceinline__ float ld_elem(const float* p, long i) { return p[i]; }
__device__ __forceinline__ float ld_elem(const bf16* p, long i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void st_elem(float* p, long i, float v) { p[i] = v; }
__device__ __forceinline__ void st_elem(bf16* p, long i, float v) { p[i] = __float2bfloat16_rn(v); }

// eight consecutive elements (the caller guarantees 8-element alignment of the index and row)
__device__ __forceinline__ void ld8(const float* p, long i, float (&o)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p + i), b = *reinterpret_cast<const float4*>(p + i + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void ld8(const bf16* p, long i, float (&o)[8]) {
  const uint4 a = *reinterpret_cast<const uint4*>(p + i);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = __bfloat1622float2(h[k]);
    o[2 * k] = f.x; o[2 * k + 1] = f.y;
  }
}

__device__ __forceinline__ void st8(float* p, long i, const float (&o)[8]) {
  *reinterpret_cast<float4*>(p + i) = make_float4(o[0], o[1], o[2], o[3]);
  *reinterpret_cast<float4*>(p + i + 4) = make_float4(o[4], o[5], o[6], o[7]);
}
__device__ __forceinline__ void st8(bf16* p, long i, const float (&o)[8]) {
  uint4 a;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&a);
#pragma unroll
  for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(o[2 * k], o[2 * k + 1]);
  *reinterpret_cast<uint4*>(p + i) = a;
}

__device__ __forceinline__ float ld_peer_f32(const float* local, uint32_t rank) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(mapa(ptx::smem_u32(local), rank)));
  return v;
}

__device__ __forceinline__ float block_sum(float x, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = x;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < SN_THREADS / 32; ++w) t += scratch[w];
  return t;
}

// sum over the cluster of one value per CTA (slot: a float in shared memory every CTA writes)
__device__ __forceinline__ float cluster_sum(const float* slot, int NC) {
  float t = 0.f;
  for (int p = 0; p < NC; ++p) t += ld_peer_f32(slot, (uint32_t)p);
  return t;
}

__device__ __forceinline__ void st_peer_f32(float* local, uint32_t rank, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(mapa(ptx::smem_u32(local), rank)), "f"(v)
               : "memory");
}

// Exchanges are PUSHES: a CTA stores what a peer needs straight into that peer's shared memory
// (fire and forget) before a cluster barrier, and everybody reads only its own shared memory
// after it; pulling the same values with remote loads costs a round trip per value.
template <typename T>
__global__ void __launch_bounds__(SN_THREADS, 1) spectral_fwd_kernel(SpectralParams p) {
  extern __shared__ __align__(16) float sn_smem[];
  __shared__ float s_red[SN_THREADS / 32];
  __shared__ float s_vsq[SN_MAX_NC], s_usq[SN_MAX_NC];   // every CTA's share of the two squared norms
  const int d = p.d, NC = p.NC, R = p.R;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = NC > 1 ? (int)cluster_ctarank() : 0;
  const int r0 = c * R;                   // my rows of W, my columns of v
  float* vpart = sn_smem;                 // [d]      my rows' contribution to W^T u
  float* vfull = vpart + d;               // [d]      W^T u, not yet normalised (slices pushed by their owners)
  float* inbox = vfull + d;               // [NC][R]  every CTA's partial of my columns
  float* u_loc = inbox + NC * R;          // [R]      my rows of u
  float* wv = u_loc + R;                  // [R]      my rows of W v
  const T* Wg = (const T*)p.W + (long)r0 * d;      // my rows in global memory
  T* u = (T*)p.u;
  const bool vec8 = (d & 7) == 0 && (((uintptr_t)p.W & 15) == 0);
  // my rows of W: read once into shared memory when they fit (every pass below then runs out
  // of shared memory), else streamed from L2 in every pass
  const T* W = Wg;
  if (p.cache) {
    T* Wc = reinterpret_cast<T*>(sn_smem + 2 * d + 4 * ((NC * R + 2 * R + 3) / 4));
    const long n8 = (long)R * d / 8;
#pragma unroll 4
    for (long e = tid; e < n8; e += SN_THREADS) {
      float w[8];
      ld8(Wg, 8 * e, w);
      st8(Wc, 8 * e, w);
    }
    W = Wc;
  }
  for (int r = tid; r < R; r += SN_THREADS) u_loc[r] = ld_elem(u, r0 + r);
  __syncthreads();
  if (NC > 1) cluster_sync_all();   // every CTA of the cluster is running before the first push
  float norm_u = 0.f, inv_v = 0.f;
  for (int it = 0; it < p.iters; ++it) {
    // A. vpart[col] = sum over my rows of W[row, col] u[row]   (threads over columns: coalesced)
    if (vec8) {
      for (int col = tid * 8; col < d; col += SN_THREADS * 8) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
        for (int r = 0; r < R; ++r) {
          float w[8];
          ld8(W, (long)r * d + col, w);
          const float ur = u_loc[r];
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[k] += w[k] * ur;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) vpart[col + k] = acc[k];
      }
    } else {
      for (int col = tid; col < d; col += SN_THREADS) {
        float acc = 0.f;
        for (int r = 0; r < R; ++r) acc += ld_elem(W, (long)r * d + col) * u_loc[r];
        vpart[col] = acc;
      }
    }
    __syncthreads();
    // ... each column's partial goes to the inbox of the CTA that owns the column
    for (int col = tid; col < d; col += SN_THREADS) {
      const int owner = col / R, k = col - owner * R;
      if (NC > 1) st_peer_f32(inbox + c * R + k, (uint32_t)owner, vpart[col]);
      else inbox[k] = vpart[col];
    }
    if (NC > 1) cluster_sync_all(); else __syncthreads();
    // B. my columns: sum the NC partials; push the sums (and my share of the squared norm) to all
    float sq = 0.f;
    for (int k = tid; k < R; k += SN_THREADS) {
      float acc = 0.f;
      for (int q = 0; q < NC; ++q) acc += inbox[q * R + k];
      sq += acc * acc;
      if (NC > 1) {
        for (int q = 0; q < NC; ++q) st_peer_f32(vfull + r0 + k, (uint32_t)q, acc);
      } else {
        vfull[k] = acc;
      }
    }
    sq = block_sum(sq, s_red);
    if (NC > 1) { if (tid < NC) st_peer_f32(&s_vsq[c], (uint32_t)tid, sq); }
    else if (tid == 0) s_vsq[0] = sq;
    if (NC > 1) cluster_sync_all(); else __syncthreads();
    // C. the norm of v (applied as a factor where v is used)
    float nv = 0.f;
    for (int q = 0; q < NC; ++q) nv += s_vsq[q];
    inv_v = 1.f / (sqrtf(nv) + p.eps);
    // D. my rows of W v (a warp per row: coalesced), and my share of its squared norm
    sq = 0.f;
    for (int r = warp; r < R; r += SN_THREADS / 32) {
      float acc = 0.f;
      if (vec8) {
        for (int col = lane * 8; col < d; col += 256) {
          float w[8];
          ld8(W, (long)r * d + col, w);
#pragma unroll
          for (int k = 0; k < 8; ++k) acc += w[k] * vfull[col + k];
        }
      } else {
        for (int col = lane; col < d; col += 32) acc += ld_elem(W, (long)r * d + col) * vfull[col];
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      acc *= inv_v;
      if (lane == 0) wv[r] = acc;
      sq += acc * acc;               // identical in every lane: count it once below
    }
    sq = block_sum(lane == 0 ? sq : 0.f, s_red);
    if (NC > 1) { if (tid < NC) st_peer_f32(&s_usq[c], (uint32_t)tid, sq); }
    else if (tid == 0) s_usq[0] = sq;
    if (NC > 1) cluster_sync_all(); else __syncthreads();
    // E. normalise my rows of u
    float nu = 0.f;
    for (int q = 0; q < NC; ++q) nu += s_usq[q];
    norm_u = sqrtf(nu);
    const float inv_u = 1.f / (norm_u + p.eps);
    for (int r = tid; r < R; r += SN_THREADS) u_loc[r] = wv[r] * inv_u;
    __syncthreads();
    // (what peers push into my inbox, vfull and norm slots for the next iteration arrives only
    // after they passed the barrier above, i.e. after my reads of this iteration's values that
    // precede my own arrival at it; vfull is read in D, before that barrier)
  }
  // sigma = |u^T W v| with u = W v / (|W v| + eps):  |W v|^2 / (|W v| + eps)
  const float sigma = fabsf(norm_u * norm_u / (norm_u + p.eps));
  const float scale = p.target / (sigma + p.eps);
  T* We = (T*)p.W_eff + (long)r0 * d;
  if (vec8 && (((uintptr_t)p.W_eff & 15) == 0)) {
#pragma unroll 4
    for (long e = tid; e < (long)R * d / 8; e += SN_THREADS) {
      float w[8];
      ld8(W, 8 * e, w);
#pragma unroll
      for (int k = 0; k < 8; ++k) w[k] *= scale;
      st8(We, 8 * e, w);
    }
  } else {
    for (long e = tid; e < (long)R * d; e += SN_THREADS) st_elem(We, e, ld_elem(W, e) * scale);
  }
  for (int r = tid; r < R; r += SN_THREADS) {
    st_elem(u, r0 + r, u_loc[r]);
    p.v[r0 + r] = vfull[r0 + r] * inv_v;
  }
  if (c == 0 && tid == 0) *p.sigma = sigma;
  if (NC > 1) cluster_sync_all();   // no CTA leaves while a peer may still write into its shared memory
}

template <typename T>
__global__ void __launch_bounds__(SN_THREADS, 1) spectral_bwd_kernel(SpectralParams p) {
  __shared__ float s_red[SN_THREADS / 32];
  __shared__ float s_dot;
  const int d = p.d, NC = p.NC, R = p.R;
  const int tid = threadIdx.x;
  const int c = NC > 1 ? (int)cluster_ctarank() : 0;
  const long e0 = (long)c * R * d, n = (long)R * d;
  const T* W = (const T*)p.W;
  const T* G = (const T*)p.G;
  const T* u = (const T*)p.u;
  T* dW = (T*)p.dW;
  const bool vec8 = (d & 7) == 0 && ((((uintptr_t)p.W | (uintptr_t)p.G | (uintptr_t)p.dW) & 15) == 0);
  float dot = 0.f;
  if (vec8) {
#pragma unroll 4
    for (long e = tid; e < n / 8; e += SN_THREADS) {
      float g[8], w[8];
      ld8(G, e0 + 8 * e, g);
      ld8(W, e0 + 8 * e, w);
#pragma unroll
      for (int k = 0; k < 8; ++k) dot += g[k] * w[k];
    }
  } else {
    for (long e = tid; e < n; e += SN_THREADS) dot += ld_elem(G, e0 + e) * ld_elem(W, e0 + e);
  }
  dot = block_sum(dot, s_red);
  if (tid == 0) s_dot = dot;
  if (NC > 1) cluster_sync_all(); else __syncthreads();
  const float gw = NC > 1 ? cluster_sum(&s_dot, NC) : s_dot;
  const float sigma = *p.sigma;
  const float s = p.target / (sigma + p.eps);
  const float k = gw * p.target / ((sigma + p.eps) * (sigma + p.eps));
  if (vec8) {
#pragma unroll 2
    for (long e = tid; e < n / 8; e += SN_THREADS) {
      const int r = (int)(8 * e / d), col = (int)(8 * e - (long)r * d);
      const float ku = k * ld_elem(u, c * R + r);
      float g[8];
      ld8(G, e0 + 8 * e, g);
#pragma unroll
      for (int q = 0; q < 8; ++q) g[q] = s * g[q] - ku * p.v[col + q];
      if (p.accumulate) {
        float o[8];
        ld8(dW, e0 + 8 * e, o);
#pragma unroll
        for (int q = 0; q < 8; ++q) g[q] += o[q];
      }
      st8(dW, e0 + 8 * e, g);
    }
  } else {
    for (long e = tid; e < n; e += SN_THREADS) {
      const int r = (int)(e / d), col = (int)(e - (long)r * d);
      float g = s * ld_elem(G, e0 + e) - k * ld_elem(u, c * R + r) * p.v[col];
      if (p.accumulate) g += ld_elem(dW, e0 + e);
      st_elem(dW, e0 + e, g);
    }
  }
  if (NC > 1) cluster_sync_all();
}

int cluster_size_for(int d) {
  for (int nc = SN_MAX_NC; nc > 1; nc >>= 1)
    if (d % nc == 0 && d / nc >= 8) return nc;
  return 1;
}

template <typename Kernel>
int launch_cluster(Kernel kern, const SpectralParams& p, size_t smem, cudaStream_t st) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.NC);
  cfg.blockDim = dim3(SN_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = p.NC; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = p.NC > 1 ? 1 : 0;
  if (p.NC > 8)
    ELMAN_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
  if (smem > 48 * 1024)
    ELMAN_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  ELMAN_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, p));
  count_launch(false);
  return ELMAN_OK;
}

}  // namespace

int spectral_norm_fwd(int dtype, int d, const void* W, void* u, float* v, float* sigma, void* W_eff,
                      float target, float eps, int iters, cudaStream_t st) {
  SpectralParams p{};
  p.d = d; p.NC = cluster_size_for(d); p.R = d / p.NC; p.iters = iters;
  p.target = target; p.eps = eps;
  p.W = W; p.u = u; p.v = v; p.sigma = sigma; p.W_eff = W_eff;
  size_t smem = ((size_t)2 * d + 4 * ((p.NC * p.R + 2 * p.R + 3) / 4)) * sizeof(float);
  if (smem > 200 * 1024)
    return set_error(ELMAN_ERR_UNSUPPORTED, "spectral norm: dim %d too large for the fused kernel", d);
  const size_t rows_bytes = (size_t)p.R * d * (dtype == ELMAN_BF16 ? 2 : 4);
  p.cache = ((d & 7) == 0 && (((uintptr_t)W & 15) == 0) && smem + rows_bytes <= 220 * 1024) ? 1 : 0;
  if (p.cache) smem += rows_bytes;
  if (dtype == ELMAN_BF16) return launch_cluster(spectral_fwd_kernel<bf16>, p, smem, st);
  return launch_cluster(spectral_fwd_kernel<float>, p, smem, st);
}

int spectral_norm_bwd(int dtype, int d, const void* W, const void* u, const float* v,
                      const float* sigma, const void* G, void* dW, int accumulate, float target,
                      float eps, cudaStream_t st) {
  SpectralParams p{};
  p.d = d; p.NC = cluster_size_for(d); p.R = d / p.NC;
  p.target = target; p.eps = eps;
  p.W = W; p.u = const_cast<void*>(u); p.v = const_cast<float*>(v);
  p.sigma = const_cast<float*>(sigma); p.G = G; p.dW = dW; p.accumulate = accumulate;
  if (dtype == ELMAN_BF16) return launch_cluster(spectral_bwd_kernel<bf16>, p, 0, st);
  return launch_cluster(spectral_bwd_kernel<float>, p, 0, st);
}

}  // namespace elman

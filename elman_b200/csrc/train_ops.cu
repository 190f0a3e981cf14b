// The optimizer tail of the training step on flat buffers: decoupled-weight-decay Adam
// (AdamW) over ALL parameters in one launch, with the gradient-clipping factor applied on
// load.  The reference's step is torch.nn.utils.clip_grad_norm_ + torch.optim.AdamW
// (train_ladder.py:360-365, :542-545), which run as dozens of per-tensor launches; here the
// parameters, gradients and both moment estimates each live in one contiguous buffer.
//
// The step counter and the clipping factor are read from device memory, so the launch can
// sit inside a captured CUDA graph and still advance every replay.  HBM-bound: per element
// it reads p, g, m, v and writes p, m, v (14 bytes for bf16 storage).
#include "common.cuh"

namespace elman {

namespace {

struct AdamParams {
  long n;
  float lr, beta1, beta2, eps, weight_decay;
  const float* step;        // device: number of this update (1, 2, ...), already advanced
  const float* grad_scale;  // device, or null: gradients are multiplied by it on load
};

__device__ __forceinline__ void adam_update(float& p, float g, float& m, float& v, float gs,
                                            const AdamParams& a, float bc1, float bc2_rsqrt) {
  g *= gs;
  p *= 1.f - a.lr * a.weight_decay;
  m = a.beta1 * m + (1.f - a.beta1) * g;
  v = a.beta2 * v + (1.f - a.beta2) * g * g;
  const float denom = sqrtf(v) * bc2_rsqrt + a.eps;
  p -= (a.lr / bc1) * (m / denom);
}

__global__ void adamw_bf16x8_kernel(AdamParams a, uint4* __restrict__ p, const uint4* __restrict__ g,
                                    uint4* __restrict__ m, uint4* __restrict__ v) {
  const float t = *a.step;
  const float bc1 = 1.f - powf(a.beta1, t);
  const float bc2_rsqrt = rsqrtf(1.f - powf(a.beta2, t));
  const float gs = a.grad_scale ? *a.grad_scale : 1.f;
  const long nv = a.n / 8;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += (long)gridDim.x * blockDim.x) {
    uint4 P = p[i], M = m[i], V = v[i];
    const uint4 G = g[i];
    __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&P);
    __nv_bfloat162* m2 = reinterpret_cast<__nv_bfloat162*>(&M);
    __nv_bfloat162* v2 = reinterpret_cast<__nv_bfloat162*>(&V);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&G);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float2 pf = __bfloat1622float2(p2[q]), mf = __bfloat1622float2(m2[q]);
      float2 vf = __bfloat1622float2(v2[q]);
      const float2 gf = __bfloat1622float2(g2[q]);
      adam_update(pf.x, gf.x, mf.x, vf.x, gs, a, bc1, bc2_rsqrt);
      adam_update(pf.y, gf.y, mf.y, vf.y, gs, a, bc1, bc2_rsqrt);
      p2[q] = __floats2bfloat162_rn(pf.x, pf.y);
      m2[q] = __floats2bfloat162_rn(mf.x, mf.y);
      v2[q] = __floats2bfloat162_rn(vf.x, vf.y);
    }
    p[i] = P; m[i] = M; v[i] = V;
  }
}

template <typename T>
__global__ void adamw_scalar_kernel(AdamParams a, long first, T* __restrict__ p, const T* __restrict__ g,
                                    T* __restrict__ m, T* __restrict__ v) {
  const float t = *a.step;
  const float bc1 = 1.f - powf(a.beta1, t);
  const float bc2_rsqrt = rsqrtf(1.f - powf(a.beta2, t));
  const float gs = a.grad_scale ? *a.grad_scale : 1.f;
  for (long i = first + (long)blockIdx.x * blockDim.x + threadIdx.x; i < a.n;
       i += (long)gridDim.x * blockDim.x) {
    float pf = to_f(p[i]), mf = to_f(m[i]), vf = to_f(v[i]);
    adam_update(pf, to_f(g[i]), mf, vf, gs, a, bc1, bc2_rsqrt);
    p[i] = from_f<T>(pf); m[i] = from_f<T>(mf); v[i] = from_f<T>(vf);
  }
}

__global__ void advance_step_kernel(float* step) { *step += 1.f; }

}  // namespace

int adamw_step(int dtype, long n, void* p, const void* g, void* m, void* v, float lr, float beta1,
               float beta2, float eps, float weight_decay, float* step, const float* grad_scale,
               cudaStream_t st) {
  advance_step_kernel<<<1, 1, 0, st>>>(step);
  count_launch(false);
  if (n > 0) {
    AdamParams a{n, lr, beta1, beta2, eps, weight_decay, step, grad_scale};
    const bool vec = dtype == ELMAN_BF16 &&
                     ((((uintptr_t)p | (uintptr_t)g | (uintptr_t)m | (uintptr_t)v) & 15) == 0);
    long done = 0;
    if (vec && n >= 8) {
      const long nv = n / 8;
      const int grid = (int)((nv + 255) / 256 < 148L * 8 ? (nv + 255) / 256 : 148L * 8);
      adamw_bf16x8_kernel<<<grid, 256, 0, st>>>(a, (uint4*)p, (const uint4*)g, (uint4*)m, (uint4*)v);
      count_launch(false);
      done = nv * 8;
    }
    if (done < n) {
      const long rest = n - done;
      const int grid = (int)((rest + 255) / 256 < 148L * 8 ? (rest + 255) / 256 : 148L * 8);
      if (dtype == ELMAN_F32)
        adamw_scalar_kernel<float><<<grid, 256, 0, st>>>(a, done, (float*)p, (const float*)g, (float*)m,
                                                        (float*)v);
      else
        adamw_scalar_kernel<bf16><<<grid, 256, 0, st>>>(a, done, (bf16*)p, (const bf16*)g, (bf16*)m,
                                                       (bf16*)v);
      count_launch(false);
    }
  }
  ELMAN_CUDA_CHECK(cudaGetLastError());
  return ELMAN_OK;
}

}  // namespace elman

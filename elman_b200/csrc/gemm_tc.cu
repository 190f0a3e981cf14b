// Time-parallel projection GEMM on the sm_100a tensor cores:
//   C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]) (+ C)
// bf16 operands, fp32 accumulation in tensor memory, bias / accumulate / down-cast
// fused into the epilogue.  This replaces the cuBLAS calls the reference makes for
// W_x x_t over all t, the gate projection, dx, dW_x and dW_h
// (elman/cuda/lib/mamba_gated_elman_gpu.cu.cc:440-448, :561-589; blas.h:51-72).
//
// One CTA computes one 128x128 tile.  Thread 0 of warp 0 streams 128x64 operand
// tiles with TMA (128-byte swizzle) through a 3-stage mbarrier ring, thread 0 of
// warp 1 issues tcgen05.mma (M=128, N=128, K=16) into a 128-column TMEM
// accumulator, and all four warps drain it with tcgen05.ld.  Two CTAs fit on an
// SM, so one tile's epilogue overlaps the other's main loop.  No multicast is used.
#include <mutex>

#include "common.cuh"
#include "sm100_ptx.cuh"
#include "tc_helpers.cuh"

namespace elman {

namespace {

// Per-device host state.  A kernel's opt-in shared-memory size is a per-device (per
// context) attribute, and callers may use several GPUs and several host threads in one
// process: remember per device what has been set, under a lock.
constexpr int kMaxDev = 64;
std::mutex g_dev_mutex;
int current_device_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return 0; }
  return (dev >= 0 && dev < kMaxDev) ? dev : 0;
}
template <typename Kernel>
int ensure_dynamic_smem(Kernel kern, int bytes, bool* done_per_device) {
  const int dev = current_device_slot();
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (!done_per_device[dev]) {
    ELMAN_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    done_per_device[dev] = true;
  }
  return ELMAN_OK;
}

constexpr int BM = 128, BN = 128, BK = 64;
constexpr int STAGES = 3;
constexpr int A_TILE_BYTES = BM * BK * 2;
constexpr int B_TILE_BYTES = BN * BK * 2;
constexpr int GEMM_SMEM = STAGES * (A_TILE_BYTES + B_TILE_BYTES) + 1024;  // + alignment slack
constexpr uint32_t TMEM_COLS = 128;

struct GemmParams {
  int M, N, K;
  const bf16* bias;
  void* C;
  long ldc;
  int c_is_f32;
  int accumulate;
  long spin_limit;
  int* status;
  int a_mn;  // A is given as [K, M] (M contiguous): MN-major operand, no transpose pass
  int b_mn;  // W is given as [K, N] (N contiguous)
  int split = 0;              // > 0: the input projection's three-output epilogue (GemmSplit)
  void* C_act = nullptr;
  void* C_hi = nullptr;
  int split_mode = 0;         // 1: the [h;x]-gate epilogue (sum with C_hi, gate with aux)
  const void* aux = nullptr;
  int stall_step = -1;        // test hook: block 0 arms a stage at this K iteration but loads nothing
  int ksplit = 1;             // persistent kernel: K range cut into this many work items per tile
  int c_tma = 0;              // pair kernel: plain bf16 output leaves through shared memory and
                              // bulk tensor stores (a third tensor map describes C)
  int dual = 0;               // pair kernel: two products that share A in one launch (second W and
                              // C in the tensor maps tmB2 / tmC2); c_tma only, no K split
  float* partial = nullptr;   // [ksplit][M][N] fp32 partial sums when ksplit > 1
};

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// One 32-column chunk of one output row, as it comes out of tensor memory: bias, optional
// accumulate into C, conversion and store.  `gm` is the row, `gn0` the chunk's first column.
__device__ __forceinline__ void store_chunk(const GemmParams& p, int gm, int gn0,
                                            const uint32_t (&r)[32], bool vec_ok,
                                            const bf16* bias32) {
  if (p.split > 0 && p.split_mode == 1) {
    // [h;x] gate: zg = product + z (dense [M, N] in C_hi) -> C;  y = h * silu(zg) -> C_act,
    // h dense [M, N] in aux.  N % 32 == 0: whole chunks only.
    if (gm < p.M && gn0 < p.N) {
      const long off = (long)gm * p.split + gn0;
      const bf16* zin = (const bf16*)p.C_hi + off;
      const bf16* hin = (const bf16*)p.aux + off;
      bf16* zout = (bf16*)p.C + off;
      bf16* yout = (bf16*)p.C_act + off;
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        const uint4 zv = *reinterpret_cast<const uint4*>(zin + j);
        const uint4 hv = *reinterpret_cast<const uint4*>(hin + j);
        const __nv_bfloat162* z2 = reinterpret_cast<const __nv_bfloat162*>(&zv);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&hv);
        uint4 o, y;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
        uint32_t* yw = reinterpret_cast<uint32_t*>(&y);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 zf = __bfloat1622float2(z2[q]), hf = __bfloat1622float2(h2[q]);
          ow[q] = pack_bf16(__uint_as_float(r[j + 2 * q]) + zf.x, __uint_as_float(r[j + 2 * q + 1]) + zf.y);
          const float2 gf = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&ow[q]));
          yw[q] = pack_bf16(hf.x * siluf_(gf.x), hf.y * siluf_(gf.y));
        }
        *reinterpret_cast<uint4*>(zout + j) = o;
        *reinterpret_cast<uint4*>(yout + j) = y;
      }
    }
    return;
  }
  if (p.split > 0) {
    // input projection of the layer: columns left of `split` are the recurrence's input —
    // stored raw (for the backward pass) and silu-activated — the others the gate input.
    // split % 32 == 0, so a chunk never straddles; all three outputs are dense [M, split].
    if (gm < p.M && gn0 < p.N) {
      const bool hi = gn0 >= p.split;
      const long off = (long)gm * p.split + (hi ? gn0 - p.split : gn0);
      bf16* raw = (hi ? (bf16*)p.C_hi : (bf16*)p.C) + off;
      bf16* act = (bf16*)p.C_act + off;
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 o, a;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
        uint32_t* aw = reinterpret_cast<uint32_t*>(&a);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float f0 = __uint_as_float(r[j + 2 * q]), f1 = __uint_as_float(r[j + 2 * q + 1]);
          ow[q] = pack_bf16(f0, f1);
          // silu of the value as stored (rounded to bf16), as a separate pass would see it
          const float2 rf = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&ow[q]));
          aw[q] = pack_bf16(siluf_(rf.x), siluf_(rf.y));
        }
        *reinterpret_cast<uint4*>(raw + j) = o;
        if (!hi) *reinterpret_cast<uint4*>(act + j) = a;
      }
    }
    return;
  }
  if (gm < p.M && gn0 < p.N) {
    float f[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(r[j]);
    const bool full = gn0 + 32 <= p.N;
    if (bias32 != nullptr) {   // the 32 bias values of this chunk (global or shared memory)
#pragma unroll
      for (int j = 0; j < 32; j += 2)
        if (full || gn0 + j + 1 < p.N) {
          const float2 b2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(bias32 + j));
          f[j] += b2.x;
          f[j + 1] += b2.y;
        } else if (gn0 + j < p.N) {
          f[j] += __bfloat162float(bias32[j]);
        }
    }
    if (p.c_is_f32) {
      float* crow = (float*)p.C + (long)gm * p.ldc + gn0;
      if (full && ((p.ldc & 3) == 0) && (((uintptr_t)p.C & 15) == 0)) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          float4 o = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
          if (p.accumulate) {
            float4 old = *reinterpret_cast<float4*>(crow + j);
            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
          }
          *reinterpret_cast<float4*>(crow + j) = o;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (gn0 + j < p.N) crow[j] = p.accumulate ? crow[j] + f[j] : f[j];
      }
    } else {
      bf16* crow = (bf16*)p.C + (long)gm * p.ldc + gn0;
      if (full && vec_ok) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          if (p.accumulate) {
            uint4 old = *reinterpret_cast<uint4*>(crow + j);
            const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              float2 of = __bfloat1622float2(o2[q]);
              f[j + 2 * q] += of.x;
              f[j + 2 * q + 1] += of.y;
            }
          }
          uint4 o;
          o.x = pack_bf16(f[j], f[j + 1]);
          o.y = pack_bf16(f[j + 2], f[j + 3]);
          o.z = pack_bf16(f[j + 4], f[j + 5]);
          o.w = pack_bf16(f[j + 6], f[j + 7]);
          *reinterpret_cast<uint4*>(crow + j) = o;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (gn0 + j < p.N) {
            float val = p.accumulate ? f[j] + __bfloat162float(crow[j]) : f[j];
            crow[j] = __float2bfloat16_rn(val);
          }
      }
    }
  }
}

__global__ void __launch_bounds__(128)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmAct,
               const __grid_constant__ CUtensorMap tmHi, GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_TILE_BYTES;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int nk = (p.K + BK - 1) / BK;

  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    ptx::mbar_init(&acc_bar, 1);
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmA);
    ptx::prefetch_tmap(&tmB);
  }
  if (warp == 0) {
    ptx::tmem_alloc(&tmem_slot, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      for (int i = 0; i < nk; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
        if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1u, p.spin_limit, abortp)) {
          abort_flag = 1;
          report_timeout(p.status, KID_GEMM_TC, i);
          break;
        }
        ptx::mbar_arrive_expect_tx(&full_bar[s], A_TILE_BYTES + B_TILE_BYTES);
        if (i == p.stall_step && blockIdx.x == 0 && blockIdx.y == 0) continue;
        if (p.a_mn) {  // two boxes of [64 K rows x 64 M elements]
          ptx::tma_load_2d(sA + s * A_TILE_BYTES, &tmA, m0, i * BK, &full_bar[s]);
          ptx::tma_load_2d(sA + s * A_TILE_BYTES + A_TILE_BYTES / 2, &tmA, m0 + 64, i * BK,
                           &full_bar[s]);
        } else {
          ptx::tma_load_2d(sA + s * A_TILE_BYTES, &tmA, i * BK, m0, &full_bar[s]);
        }
        if (p.b_mn) {
          ptx::tma_load_2d(sB + s * B_TILE_BYTES, &tmB, n0, i * BK, &full_bar[s]);
          ptx::tma_load_2d(sB + s * B_TILE_BYTES + B_TILE_BYTES / 2, &tmB, n0 + 64, i * BK,
                           &full_bar[s]);
        } else {
          ptx::tma_load_2d(sB + s * B_TILE_BYTES, &tmB, i * BK, n0, &full_bar[s]);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = ptx::umma_idesc_bf16(BM, BN) | (p.a_mn ? (1u << 15) : 0u) |
                             (p.b_mn ? (1u << 16) : 0u);
      bool ok = true;
      for (int i = 0; i < nk && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (uint32_t)(i / STAGES) & 1u;
        if (!ptx::mbar_wait(&full_bar[s], ph, p.spin_limit, abortp)) {
          abort_flag = 1;
          report_timeout(p.status, KID_GEMM_TC, i);
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t a_addr = ptx::smem_u32(sA + s * A_TILE_BYTES);
        const uint32_t b_addr = ptx::smem_u32(sB + s * B_TILE_BYTES);
        const uint64_t da = p.a_mn ? ptx::umma_desc_mn_sw128(a_addr, A_TILE_BYTES / 2)
                                   : ptx::umma_desc_k_sw128(a_addr);
        const uint64_t db = p.b_mn ? ptx::umma_desc_mn_sw128(b_addr, B_TILE_BYTES / 2)
                                   : ptx::umma_desc_k_sw128(b_addr);
        // one K=16 step: 32 bytes along a K-major row (2 address units), or two 8-row
        // groups = 2048 bytes of an MN-major tile (128 address units)
        const uint64_t a_step = p.a_mn ? 128 : 2, b_step = p.b_mn ? 128 : 2;
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          ptx::umma_bf16(tmem_base, da + a_step * k, db + b_step * k, idesc,
                         (i > 0 || k > 0) ? 1u : 0u);
        ptx::umma_commit(&empty_bar[s]);  // frees the stage when these MMAs retire
      }
      if (ok) ptx::umma_commit(&acc_bar);
    }
    __syncwarp();
  }

  // ----- epilogue: all four warps, warp w owns TMEM lanes [32w, 32w+32) -----
  bool ok = ptx::mbar_wait(&acc_bar, 0, p.spin_limit * 8, abortp);
  if (!ok && abort_flag == 0) {
    abort_flag = 1;
    report_timeout(p.status, KID_GEMM_TC, 0xFFFF);
  }
  ok = __all_sync(0xffffffffu, ok);
  ptx::tc_fence_after();
  if (ok) {
    const int gm = m0 + warp * 32 + lane;
    const bool vec_ok = ((p.ldc & 7) == 0) && (((uintptr_t)p.C & 15) == 0);
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t r[32];
      ptx::tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(c * 32), r);
      ptx::tmem_ld_wait();
      if (p.c_tma) {
        // plain bf16 output: through shared memory (the operand ring is idle now that every MMA
        // has retired: one 4 KB box per warp and column pair of chunks) and bulk tensor stores
        // (the input projection's three-output form, c_tma == 2: a tile left of `split` stores
        // the raw values and, through a second box, their silu; a tile right of it stores the
        // gate input; all three outputs are dense [M, split], split a multiple of the tile width)
        uint8_t* buf = smem + (warp * 2 + (c >> 1)) * 4096;
        uint8_t* buf_act = buf + 32768;
        const uint32_t row_a = ptx::smem_u32(buf) + (uint32_t)(lane * 128);
        const bool split_lo = p.c_tma == 2 && n0 < p.split;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float f[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) f[q] = __uint_as_float(r[8 * j + q]);
          if (p.bias != nullptr) {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const int n = n0 + c * 32 + 8 * j + q;
              if (n < p.N) f[q] += __bfloat162float(p.bias[n]);
            }
          }
          const uint32_t piece = (uint32_t)((c & 1) * 4 + j) ^ (uint32_t)(lane & 7);
          uint32_t w[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) w[q] = pack_bf16(f[2 * q], f[2 * q + 1]);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_a + (piece << 4)),
                       "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                       : "memory");
          if (split_lo) {   // silu of the value as stored (rounded to bf16)
            uint32_t a[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 rf = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w[q]));
              a[q] = pack_bf16(siluf_(rf.x), siluf_(rf.y));
            }
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_a + 32768u + (piece << 4)),
                         "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3])
                         : "memory");
          }
        }
        if (c & 1) {
          ptx::fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int col = n0 + (c - 1) * 32, row = m0 + warp * 32;
            if (p.c_tma == 1) {
              tch::tma_store_2d(&tmC, buf, col, row);
            } else if (split_lo) {
              tch::tma_store_2d(&tmC, buf, col, row);
              tch::tma_store_2d(&tmAct, buf_act, col, row);
            } else {
              tch::tma_store_2d(&tmHi, buf, col - p.split, row);
            }
            tch::bulk_commit();
          }
        }
      } else {
        store_chunk(p, gm, n0 + c * 32, r, vec_ok,
                    p.bias != nullptr ? p.bias + n0 + c * 32 : nullptr);
      }
    }
    if (p.c_tma && lane == 0) tch::bulk_wait_read_all();   // before the shared memory goes away
  } else {
    // Give copies that may still be in flight time to land before the CTA's
    // shared memory and tensor memory are released.
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 0) ptx::tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------
// Persistent variant for large shapes: 128 x 256 output tiles, one CTA per SM looping
// over tiles, four 48 KB stages, and the accumulator double-buffered in tensor memory
// (2 x 256 columns) so that the epilogue of one tile (four dedicated warps) runs under
// the main loop of the next.  Warp 0 = TMA producer, warp 1 = MMA issuer, warps 2..9 =
// epilogue.  Same arithmetic and K order per output element as gemm_tc_kernel.
// ---------------------------------------------------------------------------
constexpr int P_BM = 128, P_BN = 256, P_STAGES = 4;
constexpr int P_A_BYTES = P_BM * BK * 2, P_B_BYTES = P_BN * BK * 2;
constexpr int P_SMEM = P_STAGES * (P_A_BYTES + P_B_BYTES) + 1024;
constexpr int P_EPI_WARPS = 8;   // two per quarter of the TMEM lanes, each takes half of the columns
constexpr int P_THREADS = 64 + 32 * P_EPI_WARPS;
constexpr int P_BLOCK_BYTES = 64 * BK * 2;   // one [64 K rows x 64 MN elements] box

__global__ void __launch_bounds__(P_THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap tmA,
                          const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[P_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[P_STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ __align__(16) bf16 s_bias[2][P_BN];   // bias of the tile in accumulator buffer b

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + P_STAGES * P_A_BYTES;
  const int nk = (p.K + BK - 1) / BK;
  const int tiles_n = (p.N + P_BN - 1) / P_BN;
  const int tiles = ((p.M + P_BM - 1) / P_BM) * tiles_n;
  const int items = tiles * p.ksplit;   // work items: (tile, K range) pairs, the K range fastest

  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < P_STAGES; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&acc_full[b], 1);
      ptx::mbar_init(&acc_empty[b], P_EPI_WARPS);
    }
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmA);
    ptx::prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    ptx::tmem_alloc(&tmem_slot, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;   // running K-iteration index over all my tiles
      bool ok = true;
      for (int w = blockIdx.x; w < items && ok; w += gridDim.x) {
        const int t = w / p.ksplit, sp = w - t * p.ksplit;
        const int m0 = (t / tiles_n) * P_BM, n0 = (t % tiles_n) * P_BN;
        const int k_lo = (int)((long)sp * nk / p.ksplit), k_hi = (int)((long)(sp + 1) * nk / p.ksplit);
        for (int i = k_lo; i < k_hi; ++i, ++it) {
          const int s = it % P_STAGES;
          const uint32_t ph = (uint32_t)(it / P_STAGES) & 1u;
          if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1u, p.spin_limit, abortp)) {
            abort_flag = 1;
            report_timeout(p.status, KID_GEMM_TC, i);
            ok = false;
            break;
          }
          ptx::mbar_arrive_expect_tx(&full_bar[s], P_A_BYTES + P_B_BYTES);
          if (it == p.stall_step && blockIdx.x == 0) continue;
          if (p.a_mn) {
#pragma unroll
            for (int blk = 0; blk < P_BM / 64; ++blk)
              ptx::tma_load_2d(sA + s * P_A_BYTES + blk * P_BLOCK_BYTES, &tmA, m0 + 64 * blk,
                               i * BK, &full_bar[s]);
          } else {
            ptx::tma_load_2d(sA + s * P_A_BYTES, &tmA, i * BK, m0, &full_bar[s]);
          }
          if (p.b_mn) {
#pragma unroll
            for (int blk = 0; blk < P_BN / 64; ++blk)
              ptx::tma_load_2d(sB + s * P_B_BYTES + blk * P_BLOCK_BYTES, &tmB, n0 + 64 * blk,
                               i * BK, &full_bar[s]);
          } else {
            ptx::tma_load_2d(sB + s * P_B_BYTES, &tmB, i * BK, n0, &full_bar[s]);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = ptx::umma_idesc_bf16(P_BM, P_BN) | (p.a_mn ? (1u << 15) : 0u) |
                             (p.b_mn ? (1u << 16) : 0u);
      const uint64_t a_step = p.a_mn ? 128 : 2, b_step = p.b_mn ? 128 : 2;
      int it = 0, lt = 0;   // K-iteration and tile counters of this CTA
      bool ok = true;
      for (int w = blockIdx.x; w < items && ok; w += gridDim.x, ++lt) {
        const int sp = w % p.ksplit;
        const int k_lo = (int)((long)sp * nk / p.ksplit), k_hi = (int)((long)(sp + 1) * nk / p.ksplit);
        const int b = lt & 1;
        // the epilogue must have drained this accumulator buffer (two tiles ago)
        if (!ptx::mbar_wait(&acc_empty[b], (((uint32_t)(lt >> 1)) & 1u) ^ 1u, p.spin_limit * 8,
                            abortp)) {
          abort_flag = 1;
          report_timeout(p.status, KID_GEMM_TC, 0xFFFE);
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(b * P_BN);
        for (int i = k_lo; i < k_hi; ++i, ++it) {
          const int s = it % P_STAGES;
          const uint32_t ph = (uint32_t)(it / P_STAGES) & 1u;
          if (!ptx::mbar_wait(&full_bar[s], ph, p.spin_limit, abortp)) {
            abort_flag = 1;
            report_timeout(p.status, KID_GEMM_TC, i);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t a_addr = ptx::smem_u32(sA + s * P_A_BYTES);
          const uint32_t b_addr = ptx::smem_u32(sB + s * P_B_BYTES);
          const uint64_t da = p.a_mn ? ptx::umma_desc_mn_sw128(a_addr, P_BLOCK_BYTES)
                                     : ptx::umma_desc_k_sw128(a_addr);
          const uint64_t db = p.b_mn ? ptx::umma_desc_mn_sw128(b_addr, P_BLOCK_BYTES)
                                     : ptx::umma_desc_k_sw128(b_addr);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            ptx::umma_bf16(d_tmem, da + a_step * k, db + b_step * k, idesc,
                           (i > k_lo || k > 0) ? 1u : 0u);
          ptx::umma_commit(&empty_bar[s]);   // frees the stage when these MMAs retire
        }
        if (ok) ptx::umma_commit(&acc_full[b]);
      }
    }
    __syncwarp();
  } else {
    // ----- epilogue warps 2..9: warp w may read TMEM lanes [32 (w % 4), +32); the two warps
    // of a quarter split the tile's columns -----
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int et = tid - 64;                   // 0..255 among the epilogue threads
    constexpr int CH = P_BN / 32 / 2;          // 32-column chunks per warp
    const bool vec_ok = ((p.ldc & 7) == 0) && (((uintptr_t)p.C & 15) == 0);
    int lt = 0;
    for (int w = blockIdx.x; w < items; w += gridDim.x, ++lt) {
      const int t = w / p.ksplit, sp = w - t * p.ksplit;
      const int b = lt & 1;
      const int m0 = (t / tiles_n) * P_BM, n0 = (t % tiles_n) * P_BN;
      if (p.bias != nullptr) {   // one bias value per epilogue thread, while the MMAs still run
        const int n = n0 + et;
        s_bias[b][et] = n < p.N ? p.bias[n] : __float2bfloat16_rn(0.f);
      }
      bool ok = ptx::mbar_wait(&acc_full[b], ((uint32_t)(lt >> 1)) & 1u, p.spin_limit * 8, abortp);
      if (!ok && abort_flag == 0) {
        abort_flag = 1;
        report_timeout(p.status, KID_GEMM_TC, 0xFFFF);
      }
      // all epilogue threads: one shared verdict, and the bias values become visible
      uint32_t stop;
      asm volatile(
          "{\n\t.reg .pred pp, qq;\n\t"
          "setp.ne.b32 pp, %1, 0;\n\t"
          "bar.red.or.pred qq, 1, %2, pp;\n\t"
          "selp.b32 %0, 1, 0, qq;\n\t}"
          : "=r"(stop)
          : "r"((uint32_t)(!ok || abort_flag != 0)), "n"(32 * P_EPI_WARPS)
          : "memory");
      if (stop) break;
      ptx::tc_fence_after();
      const int gm = m0 + quarter * 32 + lane;
      const uint32_t tsrc = tmem_base + ((uint32_t)(quarter * 32) << 16) +
                            (uint32_t)(b * P_BN + half * (P_BN / 2));
      uint32_t r[2][32];
      ptx::tmem_ld32(tsrc, r[0]);
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        ptx::tmem_ld_wait();
        if (c + 1 < CH) ptx::tmem_ld32(tsrc + (uint32_t)((c + 1) * 32), r[(c + 1) & 1]);
        const int col = half * (P_BN / 2) + c * 32;
        if (p.ksplit == 1) {
          store_chunk(p, gm, n0 + col, r[c & 1], vec_ok,
                      p.bias != nullptr ? &s_bias[b][col] : nullptr);
        } else if (gm < p.M) {   // raw partial sums; splitk_reduce_kernel finishes the job
          float* dst = p.partial + ((long)sp * p.M + gm) * p.N + n0 + col;
          if (n0 + col + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<uint4*>(dst + j) =
                  make_uint4(r[c & 1][j], r[c & 1][j + 1], r[c & 1][j + 2], r[c & 1][j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + col + j < p.N) dst[j] = __uint_as_float(r[c & 1][j]);
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&acc_empty[b]);
    }
  }
  if (abort_flag != 0) {
    // let copies that may still be in flight land before shared and tensor memory go
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) ptx::tmem_dealloc(tmem_base, 512);
}

// ---------------------------------------------------------------------------
// CTA-pair variant: a cluster of two CTAs computes one 256 x 256 output tile with
// tcgen05.mma.cta_group::2 (M = 256).  CTA r of the pair loads its own 128 rows of A and
// its own 128 of the 256 columns' worth of W per K step (32 KB per stage and CTA instead
// of 48 KB for the same flops per SM: a deeper ring in the same shared memory, a third
// less L2 traffic), holds rows [128 r, 128 r + 128) of the accumulator in its tensor
// memory and runs the epilogue for them.  The even CTA's MMA thread issues for both;
// every load credits the even CTA's stage barrier; commits arrive on both CTAs' barriers
// (tcgen05.commit multicast); no load is multicast.  Roles, epilogue and K order per
// output element are those of the persistent kernel above.
// Persistent over the work items, one CTA per SM, six 32 KB stages, two accumulator
// buffers.  (A three-stage, one-tile-per-pair instantiation with two CTAs per SM was
// measured slower on every shape and is not built.)
// ---------------------------------------------------------------------------
constexpr int Q_BM = 256, Q_BN = 256;             // tile of the pair
constexpr int Q_A_BYTES = 128 * BK * 2, Q_B_BYTES = 128 * BK * 2;   // per CTA and stage
constexpr int Q_STAGE_BYTES = Q_A_BYTES + Q_B_BYTES;
constexpr int Q_STORE_BYTES = 32 * 128;           // per epilogue warp: 32 rows x 64 bf16, swizzled
template <int STAGES> constexpr int pair_smem_bytes() {
  return STAGES * Q_STAGE_BYTES + P_EPI_WARPS * Q_STORE_BYTES + 1024;
}

template <int STAGES, int ACC_BUFS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmA,
                    const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC,
                    const __grid_constant__ CUtensorMap tmB2,
                    const __grid_constant__ CUtensorMap tmC2, GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[STAGES];    // used in the even CTA only
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_full[ACC_BUFS];
  __shared__ __align__(8) uint64_t acc_empty[ACC_BUFS]; // used in the even CTA only
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ __align__(16) bf16 s_bias[ACC_BUFS][Q_BN];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = tch::cluster_ctarank();          // 0 = even CTA (issues the MMAs)
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * Q_A_BYTES;
  uint8_t* sStore = smem + STAGES * Q_STAGE_BYTES;   // one staging buffer per epilogue warp
  const int nk = (p.K + BK - 1) / BK;
  const int tiles_n = (p.N + Q_BN - 1) / Q_BN;
  const int tiles = ((p.M + Q_BM - 1) / Q_BM) * tiles_n;
  const int items = tiles * p.ksplit * (p.dual ? 2 : 1);   // dual: the second product's tiles follow
  constexpr uint32_t TCOLS = ACC_BUFS * Q_BN;

  if (tid == 0) {
    abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < ACC_BUFS; ++b) {
      ptx::mbar_init(&acc_full[b], 1);
      ptx::mbar_init(&acc_empty[b], 2 * P_EPI_WARPS);   // the epilogue warps of both CTAs
    }
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmA);
    ptx::prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(&tmem_slot, TCOLS);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  tch::cluster_sync_all();   // the peer's barriers exist before anything arrives on them
  ptx::tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  volatile int* abortp = &abort_flag;
  const uint32_t peer_abort = tch::mapa(ptx::smem_u32(&abort_flag), rank ^ 1u);
  // a CTA that gives up tells its peer, so that the pair ends together
  auto give_up = [&](int where) {
    abort_flag = 1;
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(peer_abort), "r"(1) : "memory");
    report_timeout(p.status, KID_GEMM_TC, where);
  };

  if (warp == 0) {
    if (lane == 0) {
      struct Cursor { int w, i, k_hi, m0, n0, second; };
      auto open_item = [&](Cursor& cu) {
        if (cu.w >= items) return;
        cu.second = (p.dual && cu.w >= tiles) ? 1 : 0;
        const int w1 = cu.w - cu.second * tiles;
        const int t = w1 / p.ksplit, sp = w1 - t * p.ksplit;
        cu.m0 = (t / tiles_n) * Q_BM + 128 * (int)rank;
        cu.n0 = (t % tiles_n) * Q_BN + 128 * (int)rank;
        cu.i = (int)((long)sp * nk / p.ksplit);
        cu.k_hi = (int)((long)(sp + 1) * nk / p.ksplit);
      };
      auto advance = [&](Cursor& cu) {
        if (++cu.i >= cu.k_hi) { cu.w += npairs; open_item(cu); }
      };
      Cursor ld{pair, 0, 0, 0, 0, 0};
      open_item(ld);
      for (int it = 0; ld.w < items; ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
        if (!ptx::mbar_wait(&empty_bar[s], ph ^ 1u, p.spin_limit, abortp)) {
          give_up(ld.i);
          break;
        }
        const uint32_t bar = tch::mapa(ptx::smem_u32(&full_bar[s]), 0);
        if (rank == 0) ptx::mbar_arrive_expect_tx(&full_bar[s], 2 * Q_STAGE_BYTES);
        if (!(it == p.stall_step && blockIdx.x == 0)) {
          const int i = ld.i, m0 = ld.m0, n0 = ld.n0;
          const CUtensorMap* tmW = ld.second ? &tmB2 : &tmB;
          if (p.a_mn) {
#pragma unroll
            for (int blk = 0; blk < 2; ++blk)
              ptx::tma_load_2d_pair(sA + s * Q_A_BYTES + blk * P_BLOCK_BYTES, &tmA, m0 + 64 * blk,
                                    i * BK, bar);
          } else {
            ptx::tma_load_2d_pair(sA + s * Q_A_BYTES, &tmA, i * BK, m0, bar);
          }
          if (p.b_mn) {
#pragma unroll
            for (int blk = 0; blk < 2; ++blk)
              ptx::tma_load_2d_pair(sB + s * Q_B_BYTES + blk * P_BLOCK_BYTES, tmW, n0 + 64 * blk,
                                    i * BK, bar);
          } else {
            ptx::tma_load_2d_pair(sB + s * Q_B_BYTES, tmW, i * BK, n0, bar);
          }
        }
        advance(ld);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = ptx::umma_idesc_bf16(Q_BM, Q_BN) | (p.a_mn ? (1u << 15) : 0u) |
                             (p.b_mn ? (1u << 16) : 0u);
      const uint64_t a_step = p.a_mn ? 128 : 2, b_step = p.b_mn ? 128 : 2;
      // descriptors of ring slot 0; slot s adds its byte offset / 16 to the address field
      const uint64_t da0 = p.a_mn ? ptx::umma_desc_mn_sw128(ptx::smem_u32(sA), P_BLOCK_BYTES)
                                  : ptx::umma_desc_k_sw128(ptx::smem_u32(sA));
      const uint64_t db0 = p.b_mn ? ptx::umma_desc_mn_sw128(ptx::smem_u32(sB), P_BLOCK_BYTES)
                                  : ptx::umma_desc_k_sw128(ptx::smem_u32(sB));
      int lt = 0;
      uint32_t s = 0, ph = 0;            // ring slot and phase of the next stage to consume
      bool ready = false;                // its barrier already seen complete
      bool ok = true;
      for (int w = pair; w < items && ok; w += npairs, ++lt) {
        const int sp = w % p.ksplit;
        const int k_lo = (int)((long)sp * nk / p.ksplit), k_hi = (int)((long)(sp + 1) * nk / p.ksplit);
        const int b = lt % ACC_BUFS;
        const uint32_t use = (uint32_t)(lt / ACC_BUFS);
        if (!ptx::mbar_wait(&acc_empty[b], (use & 1u) ^ 1u, p.spin_limit * 8, abortp)) {
          give_up(0xFFFE);
          ok = false;
          break;
        }
        const uint32_t d_tmem = tmem_base + (uint32_t)(b * Q_BN);
        for (int i = k_lo; i < k_hi; ++i) {
          if (!ready && !ptx::mbar_wait(&full_bar[s], ph, p.spin_limit, abortp)) {
            give_up(i);
            ok = false;
            break;
          }
          uint32_t s_next = s + 1, ph_next = ph;
          if (s_next == STAGES) { s_next = 0; ph_next ^= 1u; }
          ready = ptx::umma_stage_pair(d_tmem, da0 + (uint64_t)(s * (Q_A_BYTES / 16)),
                                       db0 + (uint64_t)(s * (Q_B_BYTES / 16)), a_step, b_step, idesc,
                                       i > k_lo ? 1u : 0u, &empty_bar[s], &full_bar[s_next], ph_next);
          s = s_next;
          ph = ph_next;
        }
        if (ok) ptx::umma_commit_pair(&acc_full[b], 3);
      }
    }
    __syncwarp();
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int et = tid - 64;
    constexpr int CH = Q_BN / 32 / 2;
    const bool vec_ok = ((p.ldc & 7) == 0) && (((uintptr_t)p.C & 15) == 0);
    int lt = 0;
    for (int w = pair; w < items; w += npairs, ++lt) {
      const int second = (p.dual && w >= tiles) ? 1 : 0;
      const int w1 = w - second * tiles;
      const int t = w1 / p.ksplit, sp = w1 - t * p.ksplit;
      const int b = lt % ACC_BUFS;
      const uint32_t use = (uint32_t)(lt / ACC_BUFS);
      const int m0 = (t / tiles_n) * Q_BM + 128 * (int)rank, n0 = (t % tiles_n) * Q_BN;
      if (p.bias != nullptr) {
        const int n = n0 + et;
        s_bias[b][et] = n < p.N ? p.bias[n] : __float2bfloat16_rn(0.f);
      }
      bool ok = ptx::mbar_wait(&acc_full[b], use & 1u, p.spin_limit * 8, abortp);
      if (!ok && abort_flag == 0) give_up(0xFFFF);
      uint32_t stop;
      asm volatile(
          "{\n\t.reg .pred pp, qq;\n\t"
          "setp.ne.b32 pp, %1, 0;\n\t"
          "bar.red.or.pred qq, 1, %2, pp;\n\t"
          "selp.b32 %0, 1, 0, qq;\n\t}"
          : "=r"(stop)
          : "r"((uint32_t)(!ok || abort_flag != 0)), "n"(32 * P_EPI_WARPS)
          : "memory");
      if (stop) break;
      ptx::tc_fence_after();
      const int gm = m0 + quarter * 32 + lane;
      const uint32_t tsrc = tmem_base + ((uint32_t)(quarter * 32) << 16) +
                            (uint32_t)(b * Q_BN + half * (Q_BN / 2));
      uint32_t r[2][32];
      ptx::tmem_ld32(tsrc, r[0]);
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        ptx::tmem_ld_wait();
        if (c + 1 < CH) ptx::tmem_ld32(tsrc + (uint32_t)((c + 1) * 32), r[(c + 1) & 1]);
        const int col = half * (Q_BN / 2) + c * 32;
        if (p.c_tma) {
          // bias, rounding, then this thread's 64 bytes of the row into the warp's staging
          // buffer in the 128-byte-swizzled layout of a [32 rows x 64 columns] box; every second
          // chunk completes a box, which one lane hands to a bulk tensor store (clipped at the
          // edges of C by the hardware).  The global writes are whole 128-byte rows this way.
          uint8_t* buf = sStore + (warp - 2) * Q_STORE_BYTES;
          if ((c & 1) == 0) {   // the previous box must have been read out of the buffer
            if (lane == 0) tch::bulk_wait_read_all();
            __syncwarp();
          }
          const uint32_t row_a = ptx::smem_u32(buf) + (uint32_t)(lane * 128);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float f[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) f[q] = __uint_as_float(r[c & 1][8 * j + q]);
            if (p.bias != nullptr) {
#pragma unroll
              for (int q = 0; q < 8; q += 2) {
                const float2 b2 = __bfloat1622float2(
                    *reinterpret_cast<const __nv_bfloat162*>(&s_bias[b][col + 8 * j + q]));
                f[q] += b2.x;
                f[q + 1] += b2.y;
              }
            }
            const uint32_t piece = (uint32_t)((c & 1) * 4 + j) ^ (uint32_t)(lane & 7);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_a + (piece << 4)),
                         "r"(pack_bf16(f[0], f[1])), "r"(pack_bf16(f[2], f[3])),
                         "r"(pack_bf16(f[4], f[5])), "r"(pack_bf16(f[6], f[7]))
                         : "memory");
          }
          if (c & 1) {
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tch::tma_store_2d(second ? &tmC2 : &tmC, buf, n0 + col - 32, m0 + quarter * 32);
              tch::bulk_commit();
            }
          }
        } else if (p.ksplit == 1) {
          store_chunk(p, gm, n0 + col, r[c & 1], vec_ok,
                      p.bias != nullptr ? &s_bias[b][col] : nullptr);
        } else if (gm < p.M) {
          float* dst = p.partial + ((long)sp * p.M + gm) * p.N + n0 + col;
          if (n0 + col + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
              *reinterpret_cast<uint4*>(dst + j) =
                  make_uint4(r[c & 1][j], r[c & 1][j + 1], r[c & 1][j + 2], r[c & 1][j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + col + j < p.N) dst[j] = __uint_as_float(r[c & 1][j]);
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(tch::mapa(ptx::smem_u32(&acc_empty[b]), 0));
    }
  }
  if (abort_flag != 0) {
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
  }
  if (p.c_tma && warp >= 2 && lane == 0) tch::bulk_wait_read_all();   // my last box has left
  ptx::tc_fence_before();
  __syncthreads();
  // neither CTA may leave while the other can still read its shared memory (the MMAs read
  // both CTAs' operand tiles) or arrive on its barriers
  tch::cluster_sync_all();
  if (warp == 1) ptx::tmem_dealloc_pair(tmem_base, TCOLS);
}

// C = sum over the K ranges of the partial sums (+ bias) (+ C), in a fixed order.
__global__ void splitk_reduce_kernel(GemmParams p) {
  const long total = (long)p.M * p.N;
  for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (long)gridDim.x * blockDim.x) {
    const long m = e / p.N;
    const int n = (int)(e - m * p.N);
    float acc = 0.f;
    for (int sp = 0; sp < p.ksplit; ++sp) acc += p.partial[(long)sp * total + e];
    if (p.bias != nullptr) acc += __bfloat162float(p.bias[n]);
    if (p.c_is_f32) {
      float* c = (float*)p.C + m * p.ldc + n;
      *c = p.accumulate ? *c + acc : acc;
    } else {
      bf16* c = (bf16*)p.C + m * p.ldc + n;
      *c = __float2bfloat16_rn(p.accumulate ? acc + __bfloat162float(*c) : acc);
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = (EncodeTiledFn)ptr;
    } else {
      cudaGetLastError();
    }
  }
  return fn;
}

}  // namespace

int make_tmap_bf16_sw128(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                         uint64_t ld, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr)
    return set_error(ELMAN_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult rc = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                   strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS)
    return set_error(ELMAN_ERR_CUDA,
                     "cuTensorMapEncodeTiled failed (%d) for [%llu x %llu] ld=%llu box_rows=%u",
                     (int)rc, (unsigned long long)rows, (unsigned long long)cols,
                     (unsigned long long)ld, box_rows);
  return ELMAN_OK;
}

bool gemm_tc_supported(int M, int N, int K, const void* A, int lda, const void* W, int ldw,
                       const void* C, int ldc, int c_is_f32) {
  (void)C; (void)ldc; (void)c_is_f32;
  if (M < 1 || N < 1 || K < 8) return false;
  // (for an MN-major operand the contiguous extent is M or N instead of K; the callers
  // of that form pass matrices whose both extents are multiples of 8)
  if ((K & 7) != 0 || (lda & 7) != 0 || (ldw & 7) != 0) return false;
  if (((uintptr_t)A & 15) != 0 || ((uintptr_t)W & 15) != 0) return false;
  return get_encode_fn() != nullptr;
}

int gemm_tc_nt(int M, int N, int K, const bf16* A, int lda, const bf16* W, int ldw,
               const bf16* bias, void* C, int ldc, int c_is_f32, int accumulate,
               cudaStream_t stream) {
  return gemm_tc(M, N, K, A, lda, 0, W, ldw, 0, bias, C, ldc, c_is_f32, accumulate, stream);
}

int gemm_tc_persistent(int M, int N, int K, const bf16* A, int lda, int a_mn, const bf16* W, int ldw,
                       int b_mn, const GemmParams& p, cudaStream_t stream);
int gemm_tc_pair(int M, int N, int K, const bf16* A, int lda, int a_mn, const bf16* W, int ldw,
                 int b_mn, GemmParams p, float* splitk, size_t splitk_bytes, cudaStream_t stream,
                 const bf16* W2 = nullptr, void* C2 = nullptr);
namespace { int sm_count(); }

int gemm_tc(int M, int N, int K, const bf16* A, int lda, int a_mn, const bf16* W, int ldw,
            int b_mn, const bf16* bias, void* C, int ldc, int c_is_f32, int accumulate,
            cudaStream_t stream, float* splitk, size_t splitk_bytes, const GemmSplit* split) {
  if (split != nullptr) {
    const int want_n = split->mode == 1 ? split->split : 2 * split->split;
    if (split->split <= 0 || (split->split & 31) != 0 || N != want_n || c_is_f32 ||
        accumulate || bias != nullptr || (split->mode == 1 && split->aux == nullptr) ||
        (((uintptr_t)C | (uintptr_t)split->C_act | (uintptr_t)split->C_hi |
          (uintptr_t)split->aux) & 15) != 0)
      return set_error(ELMAN_ERR_UNSUPPORTED, "split epilogue: shape or alignment not supported");
    splitk = nullptr;   // the three-output epilogue has no partial-sum form
  }
  {
    // option gemm_pair: 0 = CTA pairs (256x256 tiles) for shapes they tile well and fill the
    // device with (at least two tiles per SM pair, or a K split over the pairs) — a launch
    // that shares the SMs with others, like the per-chunk GEMMs of the layer pipeline, is
    // better served by the small one-tile CTAs; 1 = never; 2 = whenever the shape allows
    const long pair = options().gemm_pair;
    const long tiles256 = (long)((M + Q_BM - 1) / Q_BM) * ((N + Q_BN - 1) / Q_BN);
    const bool tiles_well = M >= Q_BM && N >= Q_BN && (N % Q_BN == 0 || N >= 4 * Q_BN) &&
                            (tiles256 >= sm_count() ||
                             (splitk != nullptr && split == nullptr && tiles256 * 4 <= sm_count()));
    if (pair != 1 && M >= 128 && N >= 128 && (pair == 2 || tiles_well)) {
      GemmParams q;
      q.M = M; q.N = N; q.K = K;
      q.bias = bias; q.C = C; q.ldc = ldc; q.c_is_f32 = c_is_f32; q.accumulate = accumulate;
      q.spin_limit = options().spin_limit;
      q.stall_step = (int)options().test_stall_step;
      q.status = device_status_ptr();
      q.a_mn = a_mn; q.b_mn = b_mn;
      if (split != nullptr) {
        q.split = split->split; q.C_act = split->C_act; q.C_hi = split->C_hi;
        q.split_mode = split->mode; q.aux = split->aux;
      }
      return gemm_tc_pair(M, N, K, A, lda, a_mn, W, ldw, b_mn, q, splitk, splitk_bytes, stream);
    }
  }
  {
    // option gemm_persistent: 0 = the persistent 128x256 kernel once its tiles fill the SMs,
    // 1 = never, 2 = always
    const long want = options().gemm_persistent;
    const long tiles = (long)((M + P_BM - 1) / P_BM) * ((N + P_BN - 1) / P_BN);
    // few output tiles but a long K (weight gradients summed over all time steps): cut K so
    // that the work items fill the SMs, if the caller gave room for the partial sums
    int ksplit = 1;
    if (splitk != nullptr && want != 1 && tiles * 2 <= sm_count()) {
      const int nk = (K + BK - 1) / BK;
      ksplit = (int)(sm_count() / tiles);
      if (ksplit > GEMM_MAX_KSPLIT) ksplit = GEMM_MAX_KSPLIT;
      while (ksplit > 1 && (nk / ksplit < 8 ||
                            (size_t)ksplit * M * N * sizeof(float) > splitk_bytes))
        --ksplit;
    }
    if (want == 2 || ksplit > 1 || (want == 0 && tiles >= sm_count())) {
      GemmParams q;
      q.ksplit = ksplit;
      q.partial = splitk;
      q.M = M; q.N = N; q.K = K;
      q.bias = bias; q.C = C; q.ldc = ldc; q.c_is_f32 = c_is_f32; q.accumulate = accumulate;
      q.spin_limit = options().spin_limit;
      q.stall_step = (int)options().test_stall_step;
      q.status = device_status_ptr();
      q.a_mn = a_mn; q.b_mn = b_mn;
      if (split != nullptr) {
        q.split = split->split; q.C_act = split->C_act; q.C_hi = split->C_hi;
        q.split_mode = split->mode; q.aux = split->aux;
      }
      return gemm_tc_persistent(M, N, K, A, lda, a_mn, W, ldw, b_mn, q, stream);
    }
  }
  static bool attr_set[kMaxDev] = {false};
  ELMAN_RETURN_IF(ensure_dynamic_smem(gemm_tc_kernel, GEMM_SMEM, attr_set));
  CUtensorMap tmA, tmB;
  if (a_mn)
    ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmA, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK));
  else
    ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM));
  if (b_mn)
    ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmB, W, (uint64_t)K, (uint64_t)N, (uint64_t)ldw, BK));
  else
    ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmB, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, BN));
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.bias = bias; p.C = C; p.ldc = ldc; p.c_is_f32 = c_is_f32; p.accumulate = accumulate;
  p.spin_limit = options().spin_limit;
  p.stall_step = (int)options().test_stall_step;
  p.status = device_status_ptr();
  p.a_mn = a_mn; p.b_mn = b_mn;
  if (split != nullptr) {
    p.split = split->split; p.C_act = split->C_act; p.C_hi = split->C_hi;
    p.split_mode = split->mode; p.aux = split->aux;
  }
  CUtensorMap tmC = tmA, tmAct = tmA, tmHi = tmA;
  p.c_tma = (!c_is_f32 && !accumulate && split == nullptr && (ldc & 7) == 0 &&
             ((uintptr_t)C & 15) == 0) ? 1 : 0;
  if (p.c_tma)
    ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmC, C, (uint64_t)M, (uint64_t)N, (uint64_t)ldc, 32));
  if (split != nullptr && split->mode == 0 && split->split % BN == 0) {
    // three dense [M, split] outputs, each through its own tensor map
    const uint64_t sp = (uint64_t)split->split;
    ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmC, C, (uint64_t)M, sp, sp, 32));
    ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmAct, split->C_act, (uint64_t)M, sp, sp, 32));
    ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmHi, split->C_hi, (uint64_t)M, sp, sp, 32));
    p.c_tma = 2;
  }
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  gemm_tc_kernel<<<grid, 128, GEMM_SMEM, stream>>>(tmA, tmB, tmC, tmAct, tmHi, p);
  count_launch(true);
  ELMAN_CUDA_CHECK(cudaGetLastError());
  return ELMAN_OK;
}

namespace {
int sm_count() {   // of the current device
  static int cached[kMaxDev] = {0};
  const int dev = current_device_slot();
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = 148;
    }
    cached[dev] = n;
  }
  return cached[dev];
}
}  // namespace

// The persistent 128x256 kernel: worth it once there is at least about one tile per SM.
int gemm_tc_persistent(int M, int N, int K, const bf16* A, int lda, int a_mn, const bf16* W, int ldw,
                       int b_mn, const GemmParams& p, cudaStream_t stream) {
  static bool attr_set[kMaxDev] = {false};
  ELMAN_RETURN_IF(ensure_dynamic_smem(gemm_tc_persistent_kernel, P_SMEM, attr_set));
  CUtensorMap tmA, tmB;
  if (a_mn)
    ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmA, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK));
  else
    ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, P_BM));
  if (b_mn)
    ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmB, W, (uint64_t)K, (uint64_t)N, (uint64_t)ldw, BK));
  else
    ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmB, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, P_BN));
  const int tiles = ((M + P_BM - 1) / P_BM) * ((N + P_BN - 1) / P_BN);
  const int items = tiles * p.ksplit;
  const int grid = items < sm_count() ? items : sm_count();
  gemm_tc_persistent_kernel<<<grid, P_THREADS, P_SMEM, stream>>>(tmA, tmB, p);
  count_launch(true);
  ELMAN_CUDA_CHECK(cudaGetLastError());
  if (p.ksplit > 1) {
    const long total = (long)M * N;
    const int rgrid = (int)((total + 255) / 256 < 148L * 8 ? (total + 255) / 256 : 148L * 8);
    splitk_reduce_kernel<<<rgrid, 256, 0, stream>>>(p);
    count_launch(false);
    ELMAN_CUDA_CHECK(cudaGetLastError());
  }
  return ELMAN_OK;
}

// The CTA-pair kernel; K is cut into ranges when the tiles alone would leave SM pairs idle.
int gemm_tc_pair(int M, int N, int K, const bf16* A, int lda, int a_mn, const bf16* W, int ldw,
                 int b_mn, GemmParams p, float* splitk, size_t splitk_bytes, cudaStream_t stream,
                 const bf16* W2, void* C2) {
  constexpr int PAIR_STAGES = 6;
  static bool attr_set[kMaxDev] = {false};
  const int pairs = sm_count() / 2;
  const int tiles = ((M + Q_BM - 1) / Q_BM) * ((N + Q_BN - 1) / Q_BN);
  int ksplit = 1;
  if (W2 == nullptr && splitk != nullptr && tiles * 2 <= pairs) {
    const int nk = (K + BK - 1) / BK;
    ksplit = pairs / tiles;
    if (ksplit > GEMM_MAX_KSPLIT) ksplit = GEMM_MAX_KSPLIT;
    while (ksplit > 1 && (nk / ksplit < 8 || (size_t)ksplit * M * N * sizeof(float) > splitk_bytes))
      --ksplit;
  }
  p.ksplit = ksplit;
  p.partial = splitk;
  CUtensorMap tmA, tmB;
  if (a_mn)
    ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmA, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, BK));
  else
    ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmA, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 128));
  if (b_mn)
    ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmB, W, (uint64_t)K, (uint64_t)N, (uint64_t)ldw, BK));
  else
    ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmB, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, 128));
  const int items = tiles * ksplit * (W2 != nullptr ? 2 : 1);
  // plain bf16 output (no accumulate, no K split, no multi-output epilogue) leaves by bulk
  // tensor stores; everything else by the epilogue threads' own stores
  CUtensorMap tmC = tmA;
  p.c_tma = (!p.c_is_f32 && !p.accumulate && ksplit == 1 && p.split == 0 && (p.ldc & 7) == 0 &&
             ((uintptr_t)p.C & 15) == 0) ? 1 : 0;
  if (p.c_tma)
    ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmC, p.C, (uint64_t)M, (uint64_t)N, (uint64_t)p.ldc, 32));
  CUtensorMap tmB2 = tmB, tmC2 = tmC;
  if (W2 != nullptr) {   // second product sharing A: same shapes and layouts, own W and C
    if (!p.c_tma || C2 == nullptr || ((uintptr_t)C2 & 15) != 0 || ((uintptr_t)W2 & 15) != 0)
      return set_error(ELMAN_ERR_UNSUPPORTED, "dual GEMM: output form or alignment not supported");
    if (b_mn)
      ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmB2, W2, (uint64_t)K, (uint64_t)N, (uint64_t)ldw, BK));
    else
      ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmB2, W2, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, 128));
    ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmC2, C2, (uint64_t)M, (uint64_t)N, (uint64_t)p.ldc, 32));
    p.dual = 1;
  }
  auto kern = gemm_tc_pair_kernel<PAIR_STAGES, 2>;
  ELMAN_RETURN_IF(ensure_dynamic_smem(kern, pair_smem_bytes<PAIR_STAGES>(), attr_set));
  const int grid = 2 * (items < pairs ? items : pairs);
  kern<<<grid, P_THREADS, pair_smem_bytes<PAIR_STAGES>(), stream>>>(tmA, tmB, tmC, tmB2, tmC2, p);
  count_launch(true);
  ELMAN_CUDA_CHECK(cudaGetLastError());
  if (ksplit > 1) {
    const long total = (long)M * N;
    const int rgrid = (int)((total + 255) / 256 < 148L * 8 ? (total + 255) / 256 : 148L * 8);
    splitk_reduce_kernel<<<rgrid, 256, 0, stream>>>(p);
    count_launch(false);
    ELMAN_CUDA_CHECK(cudaGetLastError());
  }
  return ELMAN_OK;
}

// Two products that share their first operand, C1 = A^T B1 and C2 = A^T B2 (A [K, M], B [K, N],
// all MN-major, bf16 out): the two weight gradients of a cell, dv^T x and dv^T h, in ONE launch
// of the CTA-pair kernel.  Each has too few output tiles to fill the device and would otherwise
// be cut along K with fp32 partial sums and a reduce pass; together their tiles occupy most of
// the SM pairs without a K split.  Returns ELMAN_ERR_UNSUPPORTED when the shapes do not allow it
// (the caller then runs them one by one).
int gemm_tc_dual_tn(int M, int N, int K, const bf16* A, const bf16* B1, const bf16* B2, void* C1,
                    void* C2, cudaStream_t stream) {
  if (options().gemm_pair == 1 || M < Q_BM || N < Q_BN || (M & 7) != 0 || (N & 7) != 0 ||
      (K & 7) != 0 || !gemm_tc_supported(M, N, K, A, M, B1, N, C1, N, 0))
    return ELMAN_ERR_UNSUPPORTED;
  GemmParams q;
  q.M = M; q.N = N; q.K = K;
  q.bias = nullptr; q.C = C1; q.ldc = N; q.c_is_f32 = 0; q.accumulate = 0;
  q.spin_limit = options().spin_limit;
  q.stall_step = (int)options().test_stall_step;
  q.status = device_status_ptr();
  q.a_mn = 1; q.b_mn = 1;
  return gemm_tc_pair(M, N, K, A, M, 1, B1, N, 1, q, nullptr, 0, stream, B2, C2);
}

}  // namespace elman

// Persistent tensor-core recurrence for the pure low-rank Elman cell (E5), bf16:
//   forward   h_t  = tanh(U (V h_{t-1}) + pre_t),   y_t = h_t * silu(g_t)
//   backward  dv_t = (dy_t*silu(g_t) + Vt' (Ut' dv_{t+1})) * (1 - tanh(v_t)^2)
// with U [d,r], V [r,d] (backward: the transposed pair).  The reference runs two
// dependent skinny cuBLAS GEMMs and an elementwise kernel per time step (17 launches
// per step in its backward; elman/cuda/lib/pure_lowrank_elman_fused_gpu.cu.cc:244-270,
// :355-501) and never got its fused back-to-back attempt to run
// (b2b_lowrank_elman_gpu.cu.cc is a stub).  Here ONE launch runs all T steps and the
// rank-r intermediate never leaves the chip.
//
// The d features are cut into NC = d/128 blocks; CTA c owns block c for the whole
// sequence and all NC CTAs form ONE thread-block cluster, so every exchange goes
// through distributed shared memory — there is no global-memory synchronisation:
//   phase 1  partial[r, B] = V[:, block c] * h[block c]     (A = V tile resident in
//            TENSOR MEMORY, B = my own slice of the state in shared memory)
//   reduce   the r rows are split into chunks of 32; chunk k is summed by CTA k from
//            the NC partials it receives (st.async with mbarrier byte credits), turned
//            into bf16 and all-gathered into every CTA's shared-memory operand tile
//   phase 2  out[block c, B] = U[block c, :] * Vh            (A = U tile in shared memory)
//   epilogue tanh / gate math in registers; the new state slice is written straight
//            into the swizzled shared-memory tile phase 1 of the next step reads, and
//            leaves for HBM by a bulk tensor store off the critical path.
// The only thing a CTA ever needs from another CTA per step is its share of the
// rank-r vector: the low-rank bottleneck is also the communication-minimal cut.
//
// All waits are bounded; named barriers are only ever reached by all of their threads
// (a reducing barrier carries the stop decision).  No TMA multicast.
#include <mutex>
#include "tc_helpers.cuh"

namespace elman {

namespace {

using namespace tch;

constexpr int LR_MMA_WARPS = 6;
constexpr int LR_EPI_THREADS = 256;   // two warps per quarter of the TMEM lanes, each takes half of the batch columns
constexpr int LR_THREADS = 32 * (1 + LR_MMA_WARPS) + LR_EPI_THREADS;  // loader + MMA + epilogue
constexpr int LR_MAX_NC = 16;
constexpr int LR_MAX_MT = 4;   // 128-row tiles of the padded rank (r_pad <= 512)

struct LowRankTcParams {
  int T, B, d, r;
  int NC;        // d / 128 = cluster size
  int Npad;      // batch rounded up to 16 (MMA N), <= 32
  int r_pad;     // rank rounded up to 64
  int Mr;        // 128-row tiles covering r_pad
  int n_own;     // r_pad / 32 chunks of the rank dimension, chunk k reduced by CTA k
  uint32_t tmem_cols;
  const bf16* VP;   // V role, zero padded to [Mr*128, d]
  float* db;        // backward: [d] fp32 bias gradient
  int* abort_word;
  int* status;
  long spin_limit;
  long long* trace;   // optional cycle stamps of CTA 0 ([64 steps][16 slots]), or null
  int stall_step;   // test hook: block 0 withholds its share of the rank vector at this step (-1 off)
};

// Barrier over the epilogue threads that also ORs a predicate.
__device__ __forceinline__ bool lr_bar_or(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "bar.red.or.pred q, 1, %2, p;\n\t"
      "selp.b32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)pred), "n"(LR_EPI_THREADS)
      : "memory");
  return r != 0;
}

// Cycle stamps of CTA 0 for its first 64 steps (diagnostics, option rec_trace): 0 state ready,
// 1 phase-1 MMAs issued, 2 phase-1 accumulators complete, 3 partials sent, 4 partials of my
// chunk landed, 5 chunk summed, 6 chunk gathered out, 7 rank vector landed, 8 phase-2 MMAs
// issued, 9 phase-2 accumulators complete, 10 new state written
__device__ __forceinline__ void lr_stamp(long long* trace, int c, int s, int slot) {
  if (trace != nullptr && c == 0 && s < 64) trace[s * 16 + slot] = clock64();
}

// byte offset of element (row b, column k) in a K-major bf16 operand made of
// [rows x 64] tiles with 128-byte swizzle (the layout TMA and tcgen05 agree on)
__device__ __forceinline__ uint32_t swz_off(int b, int k, int tile_bytes) {
  const int kk = k >> 6, col = k & 63;
  return (uint32_t)(kk * tile_bytes + b * 128 + ((((col >> 3) ^ (b & 7))) << 4) + ((col & 7) << 1));
}

template <bool BWD>
__global__ void __launch_bounds__(LR_THREADS, 1)
lowrank_tc_kernel(const __grid_constant__ CUtensorMap tmU, const __grid_constant__ CUtensorMap tmState,
                  const __grid_constant__ CUtensorMap tmIn0, const __grid_constant__ CUtensorMap tmIn1,
                  const __grid_constant__ CUtensorMap tmIn2, const __grid_constant__ CUtensorMap tmIn3,
                  const __grid_constant__ CUtensorMap tmOut0, const __grid_constant__ CUtensorMap tmOut1,
                  int has_out0, LowRankTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t u_bar;        // U tile landed (once)
  __shared__ __align__(8) uint64_t h0_bar;       // initial state tile landed (once)
  __shared__ __align__(8) uint64_t h_ready;      // epilogue wrote the next state tile
  __shared__ __align__(8) uint64_t acc1_full;    // phase-1 MMAs retired
  __shared__ __align__(8) uint64_t acc2_full;    // phase-2 MMAs retired
  __shared__ __align__(8) uint64_t part_full;    // all NC partials of my rank chunk landed
  __shared__ __align__(8) uint64_t vh_full;      // the whole rank-r vector landed
  __shared__ __align__(8) uint64_t in_full;      // this step's epilogue inputs landed
  __shared__ __align__(8) uint64_t in_empty;     // ... and were consumed
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  __shared__ float s_db[128];                    // backward: bias-gradient sums of the upper column half

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NC = p.NC, Npad = p.Npad, B = p.B, T = p.T, Mr = p.Mr;
  const int c = (int)cluster_ctarank();          // my feature block
  const int nku = p.r_pad / 64;                  // 64-column tiles along the rank
  constexpr int NIN = BWD ? 4 : 2;
  constexpr int NOUT = BWD ? 1 : 2;

  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sU = smem;                                   // nku tiles [128 x 64] (A of phase 2)
  const int h_tile = Npad * 128;                        // bytes of one [Npad x 64] tile
  uint8_t* sH = sU + nku * 16384;                       // 2 tiles: my slice of the state
  // the rank-r vector as phase 2 reads it: one [Npad x 32 columns] tile per owner chunk, rows of
  // 64 bytes with 64-byte swizzle, so that each owner's piece is one contiguous block
  uint8_t* sVh = sH + 2 * h_tile;
  const int vh_tile = Npad * 64;
  uint8_t* sStage = sVh + nku * h_tile;                 // [NC][Npad/4][32 rows][4] fp32 partials
  const int stage_src_bytes = 32 * Npad * 4;
  uint8_t* sGather = sStage + NC * stage_src_bytes;     // [Npad][32 rank columns] bf16
  uint8_t* sIn = sGather + Npad * 64;                   // NIN tiles [Npad x 128] bf16
  const int io_tile = Npad * 256;
  uint8_t* sOut = sIn + NIN * io_tile;                  // NOUT tiles [Npad x 128] bf16

  Waiter waiter{p.spin_limit, &abort_flag, p.abort_word};
  const int kid = KID_LOWRANK_TC;
  // TMEM columns: [0, Mr*64) the V tile (A of phase 1); then the accumulators
  const uint32_t acc_col0 = (uint32_t)(Mr * 64);
  const int nch1 = Mr * 2;                              // phase-1 chains: (row tile, K half)
  const int nmw2 = p.r_pad / 16 < LR_MMA_WARPS ? p.r_pad / 16 : LR_MMA_WARPS;

  if (tid == 0) {
    abort_flag = 0;
    ptx::mbar_init(&u_bar, 1);
    ptx::mbar_init(&h0_bar, 1);
    ptx::mbar_init(&h_ready, LR_EPI_THREADS / 32);
    ptx::mbar_init(&acc1_full, nch1 < LR_MMA_WARPS ? nch1 : LR_MMA_WARPS);
    ptx::mbar_init(&acc2_full, nmw2);
    ptx::mbar_init(&part_full, 1);
    ptx::mbar_init(&vh_full, 1);
    ptx::mbar_init(&in_full, 1);
    ptx::mbar_init(&in_empty, LR_EPI_THREADS / 32);
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&tmU);
    ptx::prefetch_tmap(&tmState);
  }
  if (warp == 1) {
    ptx::tmem_alloc(&tmem_slot, p.tmem_cols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  // One-time load of my tile of V into tensor memory: padded rank row rho goes to lane
  // rho % 128 of row tile rho / 128, its 128 bf16 (my feature block) into 64 columns.
  if (warp > LR_MMA_WARPS && warp <= LR_MMA_WARPS + 4) {
    const int quarter = warp & 3;
    const int m = quarter * 32 + lane;
    for (int mt = 0; mt < Mr; ++mt) {
      const uint4* src = reinterpret_cast<const uint4*>(p.VP + (long)(mt * 128 + m) * p.d + c * 128);
      const uint32_t tw = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(mt * 64);
      for (int cc = 0; cc < 64; cc += 16) {
        uint32_t r[16];
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          const uint4 w4 = __ldg(src + (cc >> 2) + v4);
          r[4 * v4] = w4.x; r[4 * v4 + 1] = w4.y; r[4 * v4 + 2] = w4.z; r[4 * v4 + 3] = w4.w;
        }
        ptx::tmem_st16(tw + (uint32_t)cc, r);
      }
    }
    ptx::tmem_st_wait();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  // peers must have initialised their barriers before any remote store reaches them
  cluster_sync_all();

  if (warp == 0) {
    // ============================== loader ===================================
    if (lane == 0) {
      ptx::mbar_arrive_expect_tx(&u_bar, (uint32_t)(nku * 16384));
      for (int kk = 0; kk < nku; ++kk)
        ptx::tma_load_2d(sU + kk * 16384, &tmU, kk * 64, c * 128, &u_bar);
      // initial state: forward h[0] = h0, backward the all-zero slot T of dv
      ptx::mbar_arrive_expect_tx(&h0_bar, (uint32_t)(2 * h_tile));
      for (int kk = 0; kk < 2; ++kk)
        tma_load_3d(sH + kk * h_tile, &tmState, c * 128 + kk * 64, 0, BWD ? T : 0, &h0_bar);
      for (int s = 0; s < T; ++s) {
        const int t = BWD ? T - 1 - s : s;
        if (s > 0 && !waiter.wait(&in_empty, (uint32_t)(s - 1) & 1u)) {
          abort_flag = 1;
          break;
        }
        ptx::mbar_arrive_expect_tx(&in_full, (uint32_t)(NIN * io_tile));
        tma_load_3d(sIn, &tmIn0, c * 128, 0, t, &in_full);
        tma_load_3d(sIn + io_tile, &tmIn1, c * 128, 0, t, &in_full);
        if (BWD) {
          tma_load_3d(sIn + 2 * io_tile, &tmIn2, c * 128, 0, t + 1, &in_full);  // h_t = slot t+1
          tma_load_3d(sIn + 3 * io_tile, &tmIn3, c * 128, 0, t, &in_full);
        }
      }
    }
    __syncwarp();
  } else if (warp <= LR_MMA_WARPS) {
    // ============================ MMA issuers =================================
    const int mw = warp - 1;
    if (lane == 0) {
      const uint32_t idesc = ptx::umma_idesc_bf16(128, Npad);
      const uint32_t sH_a = ptx::smem_u32(sH), sU_a = ptx::smem_u32(sU), sVh_a = ptx::smem_u32(sVh);
      bool ok = waiter.wait(&u_bar, 0);
      for (int s = 0; s < T && ok; ++s) {
        // ---- phase 1: partial[rank, batch] = V[:, my block] * state[my block] ----
        ok = (s == 0) ? waiter.wait(&h0_bar, 0) : waiter.wait(&h_ready, (uint32_t)(s - 1) & 1u);
        if (!ok) break;
        if (mw == 0) lr_stamp(p.trace, c, s, 0);
        ptx::tc_fence_after();
        for (int ch = mw; ch < nch1; ch += LR_MMA_WARPS) {
          const int mt = ch >> 1, half = ch & 1;
          const uint32_t d_tmem = tmem_base + acc_col0 + (uint32_t)(ch * Npad);
          const uint64_t db0 = ptx::umma_desc_k_sw128(sH_a + half * h_tile);
#pragma unroll
          for (int k = 0; k < 4; ++k)  // K = 64 per half: 4 steps of 16, 8 TMEM columns each
            ptx::umma_bf16_ts(d_tmem, tmem_base + (uint32_t)(mt * 64 + (half * 4 + k) * 8),
                              db0 + 2 * k, idesc, k > 0 ? 1u : 0u);
        }
        if (mw < nch1) ptx::umma_commit(&acc1_full);
        if (mw == 0) lr_stamp(p.trace, c, s, 1);
        // ---- phase 2: out[my block, batch] = U[my block, :] * Vh ----
        ok = waiter.wait_cluster(&vh_full, (uint32_t)s & 1u);
        if (!ok) break;
        if (mw == 0) lr_stamp(p.trace, c, s, 7);
        ptx::tc_fence_after();
        if (mw < nmw2) {
          const uint32_t d_tmem = tmem_base + acc_col0 + (uint32_t)(mw * Npad);
          for (int m = mw; m < p.r_pad / 16; m += nmw2) {
            const int kk = m >> 2, k = m & 3;
            const uint64_t da = ptx::umma_desc_k_sw128(sU_a + kk * 16384) + 2 * k;
            // 16 rank columns = half of owner chunk m/2's tile
            const uint64_t db = ptx::umma_desc_k_sw64(sVh_a + (m >> 1) * vh_tile) + 2 * (m & 1);
            ptx::umma_bf16(d_tmem, da, db, idesc, m >= nmw2 ? 1u : 0u);
          }
          ptx::umma_commit(&acc2_full);
        }
        if (mw == 0) lr_stamp(p.trace, c, s, 8);
      }
      if (!ok) {
        if (abort_flag == 0 && atomicExch(p.abort_word, 1) == 0) report_timeout(p.status, kid, 0xFFFFF1);
        abort_flag = 1;
      }
    }
    __syncwarp();
  } else {
    // ============================== epilogue ==================================
    const int et = tid - 32 * (1 + LR_MMA_WARPS);   // 0..255
    const int quarter = warp & 3;                    // TMEM lane quarter of this warp
    const int half = et >> 7;                        // which 16 batch columns of every 32 this warp takes
    const int m = quarter * 32 + lane;               // accumulator row / my feature in the block
    const bool is_owner = c < p.n_own;
    const uint32_t stage_a = ptx::smem_u32(sStage), gather_a = ptx::smem_u32(sGather);
    const uint32_t sH_a = ptx::smem_u32(sH), sVh_a = ptx::smem_u32(sVh);
    const uint32_t sIn_a = ptx::smem_u32(sIn), sOut_a = ptx::smem_u32(sOut);
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    float db_acc = 0.f;

    for (int s = 0; s < T; ++s) {
      const int t = BWD ? T - 1 - s : s;
      const uint32_t par = (uint32_t)s & 1u;
      if (et == 0) {  // arm this step's byte-counting barriers
        if (is_owner) ptx::mbar_arrive_expect_tx(&part_full, (uint32_t)(NC * stage_src_bytes));
        ptx::mbar_arrive_expect_tx(&vh_full, (uint32_t)(p.n_own * Npad * 64));
      }
      // ---- drain phase 1 and send every 32-row chunk of the partial to its owner ----
      bool good = waiter.wait(&acc1_full, par);
      good = __all_sync(0xffffffffu, good);
      if (et == 0) lr_stamp(p.trace, c, s, 2);
      if (good) {
        ptx::tc_fence_after();
        for (int mt = 0; mt < Mr; ++mt) {
          const int k = 4 * mt + quarter;            // chunk of the rank dimension (warp-uniform)
          if (k >= p.n_own) continue;
          const uint32_t remote = mapa(stage_a + (uint32_t)(c * stage_src_bytes + lane * 16), (uint32_t)k);
          const uint32_t remote_bar = mapa(ptx::smem_u32(&part_full), (uint32_t)k);
          const uint32_t ta = tmem_base + lane_base + acc_col0 + (uint32_t)(2 * mt * Npad);
          for (int cb = 16 * half; cb < Npad; cb += 32) {
            uint32_t r0[16], r1[16];
            ptx::tmem_ld16(ta + (uint32_t)cb, r0);
            ptx::tmem_ld16(ta + (uint32_t)(Npad + cb), r1);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int q4 = 0; q4 < 16; q4 += 4) {
              uint32_t o[4];
#pragma unroll
              for (int u = 0; u < 4; ++u)
                o[u] = __float_as_uint(__uint_as_float(r0[q4 + u]) + __uint_as_float(r1[q4 + u]));
              st_async_v4(remote + (uint32_t)(((cb + q4) >> 2) * 32 * 16), o[0], o[1], o[2], o[3],
                          remote_bar);
            }
          }
        }
        ptx::tc_fence_before();
        if (et == 0) lr_stamp(p.trace, c, s, 3);
        // ---- owner: add the NC partials of my chunk, round to bf16 ----
        if (is_owner) {
          good = waiter.wait_cluster(&part_full, par);
          good = __all_sync(0xffffffffu, good);
          if (et == 0) lr_stamp(p.trace, c, s, 4);
          if (good) {
            const int rl = et & 31, bgrp = et >> 5;
            for (int q4 = bgrp; q4 < Npad / 4; q4 += LR_EPI_THREADS / 32) {
              float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
              for (int src = 0; src < NC; ++src) {
                const float4 x = lds_f4(stage_a + (uint32_t)(src * stage_src_bytes + (q4 * 32 + rl) * 16));
                acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
              }
              // batch rows 4 q4 .. 4 q4 + 3, rank column rl of my chunk, in the 64-byte-swizzled
              // tile layout phase 2 reads: chunk (rl / 8) ^ ((row / 2) % 4) of the 64-byte row
              const float vals[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int b = 4 * q4 + u;
                sts_u16(gather_a + (uint32_t)(b * 64 + ((((rl >> 3) ^ ((b >> 1) & 3))) << 4) +
                                              ((rl & 7) << 1)),
                        f_to_bf16_bits(vals[u]));
              }
            }
            ptx::fence_proxy_async_smem();   // these writes are read by the bulk copies below
          }
        }
      }
      if (et == 0) lr_stamp(p.trace, c, s, 5);
      if (!good) {
        if (abort_flag == 0 && atomicExch(p.abort_word, 1) == 0) report_timeout(p.status, kid, s);
        abort_flag = 1;
      }
      // all epilogue threads meet (owners and non-owners) and agree whether to stop; this
      // barrier also orders last step's bulk-store reads before this step's tile writes
      if (lr_bar_or(!good || abort_flag != 0)) { abort_flag = 1; break; }
      // ---- owner: all-gather my bf16 chunk into every CTA's phase-2 operand tile ----
      // one bulk copy of the whole [Npad x 32] tile per destination CTA (slot c of its operand)
      if (is_owner && et < NC && !(s == p.stall_step && c == 0))
        bulk_copy_to_peer(mapa(sVh_a + (uint32_t)(c * vh_tile), (uint32_t)et), gather_a,
                          (uint32_t)vh_tile, mapa(ptx::smem_u32(&vh_full), (uint32_t)et));
      if (et == 0) lr_stamp(p.trace, c, s, 6);
      // ---- drain phase 2, fused tanh / gate epilogue for my feature, all batch rows ----
      good = waiter.wait(&acc2_full, par) && waiter.wait(&in_full, par);
      good = __all_sync(0xffffffffu, good);
      if (et == 0) lr_stamp(p.trace, c, s, 9);
      if (good) {
        ptx::tc_fence_after();
        for (int cb = 16 * half; cb < Npad; cb += 32) {
          float acc[16];
#pragma unroll
          for (int u = 0; u < 16; ++u) acc[u] = 0.f;
          for (int g0 = 0; g0 < nmw2; g0 += 3) {
            uint32_t r0[16], r1[16], r2[16];
            const uint32_t ta = tmem_base + lane_base + acc_col0 + (uint32_t)(g0 * Npad + cb);
            ptx::tmem_ld16(ta, r0);
            if (g0 + 1 < nmw2) ptx::tmem_ld16(ta + (uint32_t)Npad, r1);
            if (g0 + 2 < nmw2) ptx::tmem_ld16(ta + (uint32_t)(2 * Npad), r2);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int u = 0; u < 16; ++u) {
              acc[u] += __uint_as_float(r0[u]);
              if (g0 + 1 < nmw2) acc[u] += __uint_as_float(r1[u]);
              if (g0 + 2 < nmw2) acc[u] += __uint_as_float(r2[u]);
            }
          }
#pragma unroll
          for (int u = 0; u < 16; ++u) {
            const int b = cb + u;
            const uint32_t io = (uint32_t)(b * 256 + m * 2);
            float state = 0.f;
            if (b < B) {
              if (!BWD) {
                const float pre = bf16_bits_to_f(lds_u16(sIn_a + io));
                const float gz = bf16_bits_to_f(lds_u16(sIn_a + io_tile + io));
                const float val = acc[u] + pre;
                state = tanh_fast(val);
                if (has_out0) sts_u16(sOut_a + io, f_to_bf16_bits(val));
                sts_u16(sOut_a + io_tile + io, f_to_bf16_bits(state * gz * sigmoid_fast(gz)));
              } else {
                const float gz = bf16_bits_to_f(lds_u16(sIn_a + io));
                const float dy = bf16_bits_to_f(lds_u16(sIn_a + io_tile + io));
                const float hv = bf16_bits_to_f(lds_u16(sIn_a + 2 * io_tile + io));
                const float vv = bf16_bits_to_f(lds_u16(sIn_a + 3 * io_tile + io));
                const float sg = sigmoid_fast(gz);
                state = (dy * gz * sg + acc[u]) * dtanh_from_v(vv);
                sts_u16(sOut_a + io, f_to_bf16_bits(dy * hv * sg * (1.f + gz * (1.f - sg))));
                db_acc += state;
              }
            }
            // new state straight into the swizzled operand tile of the next step's phase 1
            sts_u16(sH_a + swz_off(b, m, h_tile), f_to_bf16_bits(state));
          }
        }
        ptx::tc_fence_before();
        ptx::fence_proxy_async_smem();   // generic writes -> tensor core / bulk-store reads
        __syncwarp();
        if (lane == 0) {
          ptx::mbar_arrive(&h_ready);
          ptx::mbar_arrive(&in_empty);
        }
        if (et == 0) lr_stamp(p.trace, c, s, 10);
      } else {
        if (abort_flag == 0 && atomicExch(p.abort_word, 1) == 0) report_timeout(p.status, kid, s);
        abort_flag = 1;
      }
      if (lr_bar_or(!good || abort_flag != 0)) { abort_flag = 1; break; }
      // ---- outputs leave by bulk tensor stores, off the critical path ----
      if (et == 0) {
        const int slot = BWD ? t : t + 1;
        tma_store_3d(&tmState, sH, c * 128, 0, slot);
        tma_store_3d(&tmState, sH + h_tile, c * 128 + 64, 0, slot);
        if (has_out0) tma_store_3d(&tmOut0, sOut, c * 128, 0, t);
        if (!BWD) tma_store_3d(&tmOut1, sOut + io_tile, c * 128, 0, t);
        bulk_commit();
        bulk_wait_read_all();
      }
    }
    if (et == 0) bulk_wait_all();
    if (BWD) {   // the two column halves of a feature, summed in a fixed order
      if (half == 1) s_db[m] = db_acc;
      lr_bar_or(false);
      if (half == 0 && abort_flag == 0) p.db[c * 128 + m] = db_acc + s_db[m];
    }
  }

  // ------------------------------ teardown ---------------------------------
  ptx::tc_fence_before();
  __syncthreads();
  if (abort_flag != 0) {
    for (int k = 0; k < 2000; ++k) __nanosleep(100);
  }
  cluster_sync_all();   // no CTA may exit while a peer can still address its shared memory
  if (warp == 1) ptx::tmem_dealloc(tmem_base, p.tmem_cols);
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn lr_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) ==
            cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
    else
      cudaGetLastError();
  }
  return fn;
}

// [slots][B][d] bf16 tensor seen as (d, B, slots); box = box_cols x box_rows x 1
int lr_tmap3d(CUtensorMap* out, const void* base, int d, int B, int slots, int box_cols,
              int box_rows, bool swizzle128) {
  EncodeTiledFn fn = lr_encode_fn();
  if (fn == nullptr) return set_error(ELMAN_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  cuuint64_t dims[3] = {(cuuint64_t)d, (cuuint64_t)B, (cuuint64_t)slots};
  cuuint64_t strides[2] = {(cuuint64_t)d * 2, (cuuint64_t)B * d * 2};
  cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult rc = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS)
    return set_error(ELMAN_ERR_CUDA, "cuTensorMapEncodeTiled (low-rank, 3-D) failed (%d)", (int)rc);
  return ELMAN_OK;
}

__global__ void lr_pad_kernel(const bf16* __restrict__ src, int rows, int cols, bf16* __restrict__ dst,
                              int rows_dst, int cols_dst) {
  long n = (long)rows_dst * cols_dst;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    int rr = (int)(i / cols_dst), cc = (int)(i - (long)rr * cols_dst);
    dst[i] = (rr < rows && cc < cols) ? src[(long)rr * cols + cc] : __float2bfloat16_rn(0.f);
  }
}

struct LrPlan {
  int NC, Npad, r_pad, Mr, n_own;
  uint32_t tmem_cols;
  size_t smem;
  bool ok;
};

LrPlan lr_plan(int T, int B, int d, int r, bool bwd) {
  LrPlan pl{};
  pl.ok = false;
  if (T < 1 || B < 1 || B > 32 || d < 128 || (d % 128) != 0 || r < 1) return pl;
  pl.NC = d / 128;
  if (pl.NC > LR_MAX_NC) return pl;
  pl.Npad = (B + 15) / 16 * 16;
  pl.r_pad = (r + 63) / 64 * 64;
  pl.Mr = (pl.r_pad + 127) / 128;
  if (pl.Mr > LR_MAX_MT) return pl;
  pl.n_own = pl.r_pad / 32;
  if (pl.n_own > pl.NC) return pl;
  const int nch1 = pl.Mr * 2;
  const int nmw2 = pl.r_pad / 16 < LR_MMA_WARPS ? pl.r_pad / 16 : LR_MMA_WARPS;
  const int acc_cols = (nch1 > nmw2 ? nch1 : nmw2) * pl.Npad;
  if (pl.Mr * 64 + acc_cols > 512) return pl;
  uint32_t cols = 32;
  while (cols < (uint32_t)(pl.Mr * 64 + acc_cols)) cols <<= 1;
  pl.tmem_cols = cols;
  const int nku = pl.r_pad / 64, h_tile = pl.Npad * 128, io_tile = pl.Npad * 256;
  pl.smem = (size_t)nku * 16384 + 2 * h_tile + (size_t)nku * h_tile +
            (size_t)pl.NC * 32 * pl.Npad * 4 + (size_t)pl.Npad * 64 +
            (size_t)(bwd ? 4 : 2) * io_tile + (size_t)(bwd ? 1 : 2) * io_tile + 1024 + 64;
  if (pl.smem > 225 * 1024) return pl;
  pl.ok = true;
  return pl;
}

template <bool BWD>
int lr_configure(const LrPlan& pl, cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr,
                 cudaStream_t stream) {
  auto kern = lowrank_tc_kernel<BWD>;
  ELMAN_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        (int)pl.smem));
  if (pl.NC > 8)
    ELMAN_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
  *cfg = cudaLaunchConfig_t{};
  cfg->gridDim = dim3(pl.NC);
  cfg->blockDim = dim3(LR_THREADS);
  cfg->dynamicSmemBytes = pl.smem;
  cfg->stream = stream;
  attr->id = cudaLaunchAttributeClusterDimension;
  attr->val.clusterDim.x = pl.NC;
  attr->val.clusterDim.y = 1;
  attr->val.clusterDim.z = 1;
  cfg->attrs = attr;
  cfg->numAttrs = 1;
  return ELMAN_OK;
}

// Can one cluster of NC CTAs of this kernel be resident?  (cached per shape)
template <bool BWD>
bool lr_launchable(const LrPlan& pl) {
  static int cache_nc[8], cache_smem[8], cache_ok[8], ncache = 0;
  static std::mutex cache_mutex;
  std::lock_guard<std::mutex> lock(cache_mutex);
  for (int i = 0; i < ncache; ++i)
    if (cache_nc[i] == pl.NC && cache_smem[i] == (int)pl.smem) return cache_ok[i] != 0;
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr;
  int ok = 0;
  if (lr_configure<BWD>(pl, &cfg, &attr, nullptr) == ELMAN_OK) {
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, lowrank_tc_kernel<BWD>, &cfg) == cudaSuccess)
      ok = n >= 1;
    else
      cudaGetLastError();
  } else {
    cudaGetLastError();
  }
  if (ncache < 8) { cache_nc[ncache] = pl.NC; cache_smem[ncache] = (int)pl.smem; cache_ok[ncache++] = ok; }
  return ok != 0;
}

}  // namespace

int lowrank_tc_blocks(int T, int B, int d, int r) {
  LrPlan f = lr_plan(T, B, d, r, false), b = lr_plan(T, B, d, r, true);
  return (f.ok && b.ok) ? f.NC : 0;
}

bool lowrank_tc_supported(int T, int B, int d, int r, int bwd) {
  if (options().force_generic != 0 || lr_encode_fn() == nullptr) return false;
  LrPlan pl = lr_plan(T, B, d, r, bwd != 0);
  if (!pl.ok) return false;
  return bwd ? lr_launchable<true>(pl) : lr_launchable<false>(pl);
}

void lowrank_tc_pad_bytes(int d, int r, size_t* up_bytes, size_t* vp_bytes) {
  const int r_pad = (r + 63) / 64 * 64;
  const int Mr = (r_pad + 127) / 128;
  *up_bytes = (size_t)d * r_pad * 2;
  *vp_bytes = (size_t)Mr * 128 * d * 2;
}

int lowrank_tc(const LowRankTcArgs& a, cudaStream_t stream) {
  const bool bwd = a.bwd != 0;
  LrPlan pl = lr_plan(a.T, a.B, a.d, a.r, bwd);
  if (!pl.ok) return set_error(ELMAN_ERR_UNSUPPORTED, "shape not supported by the low-rank tensor-core kernel");
  // zero-padded copies of the two factors: U role [d, r_pad], V role [Mr*128, d]
  lr_pad_kernel<<<148, 256, 0, stream>>>((const bf16*)a.Urole, a.d, a.r, (bf16*)a.UP, a.d, pl.r_pad);
  lr_pad_kernel<<<148, 256, 0, stream>>>((const bf16*)a.Vrole, a.r, a.d, (bf16*)a.VP, pl.Mr * 128, a.d);
  count_launch(false);
  count_launch(false);
  ELMAN_CUDA_CHECK(cudaGetLastError());
  ELMAN_CUDA_CHECK(cudaMemsetAsync(a.sync, 0, 256, stream));
  // (backward: slot T of the gradient state — the gradient carried in from later steps, or
  // zeros — is filled by the caller)
  CUtensorMap tmU, tmState, tmIn[4], tmOut[2];
  ELMAN_RETURN_IF(make_tmap_bf16_sw128(&tmU, a.UP, (uint64_t)a.d, (uint64_t)pl.r_pad,
                                       (uint64_t)pl.r_pad, 128));
  ELMAN_RETURN_IF(lr_tmap3d(&tmState, a.state, a.d, a.B, a.T + 1, 64, pl.Npad, true));
  const void* ins[4] = {a.in0, a.in1, bwd ? a.in2 : a.in0, bwd ? a.in3 : a.in1};
  const int in_slots[4] = {a.T, a.T, bwd ? a.T + 1 : a.T, a.T};
  for (int i = 0; i < 4; ++i)
    ELMAN_RETURN_IF(lr_tmap3d(&tmIn[i], ins[i], a.d, a.B, in_slots[i], 128, pl.Npad, false));
  const int has_out0 = a.out0 != nullptr ? 1 : 0;
  const void* o0 = has_out0 ? a.out0 : (bwd ? a.state : a.out1);
  const void* o1 = bwd ? o0 : a.out1;
  ELMAN_RETURN_IF(lr_tmap3d(&tmOut[0], o0, a.d, a.B, a.T, 128, pl.Npad, false));
  ELMAN_RETURN_IF(lr_tmap3d(&tmOut[1], o1, a.d, a.B, a.T, 128, pl.Npad, false));

  LowRankTcParams p{};
  p.T = a.T; p.B = a.B; p.d = a.d; p.r = a.r;
  p.NC = pl.NC; p.Npad = pl.Npad; p.r_pad = pl.r_pad; p.Mr = pl.Mr; p.n_own = pl.n_own;
  p.tmem_cols = pl.tmem_cols;
  p.VP = (const bf16*)a.VP;
  p.db = a.db;
  p.abort_word = a.sync;
  p.status = device_status_ptr();
  p.spin_limit = options().spin_limit;
  p.stall_step = (int)options().test_stall_step;
  p.trace = nullptr;
  if (options().rec_trace != 0 && a.trace != nullptr) {
    ELMAN_CUDA_CHECK(cudaMemsetAsync(a.trace, 0, 64 * 16 * sizeof(long long), stream));
    p.trace = a.trace;
    set_last_trace(a.trace);
  }
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr;
  if (bwd) {
    ELMAN_RETURN_IF(lr_configure<true>(pl, &cfg, &attr, stream));
    ELMAN_CUDA_CHECK(cudaLaunchKernelEx(&cfg, lowrank_tc_kernel<true>, tmU, tmState, tmIn[0], tmIn[1],
                                        tmIn[2], tmIn[3], tmOut[0], tmOut[1], has_out0, p));
  } else {
    ELMAN_RETURN_IF(lr_configure<false>(pl, &cfg, &attr, stream));
    ELMAN_CUDA_CHECK(cudaLaunchKernelEx(&cfg, lowrank_tc_kernel<false>, tmU, tmState, tmIn[0],
                                        tmIn[1], tmIn[2], tmIn[3], tmOut[0], tmOut[1], has_out0, p));
  }
  count_launch(true);
  return ELMAN_OK;
}

}  // namespace elman

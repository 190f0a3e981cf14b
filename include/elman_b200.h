/*
 * elman_b200 — C ABI of the B200 (sm_100a) Elman-layer recurrence library.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (passed as void*, a cudaStream_t).  All tensors are dense, row-major and
 * time-major: x[T,B,d] means element (t,b,i) lives at ((t*B)+b)*d+i.
 * `dtype` selects the storage type of every tensor of a call:
 *   ELMAN_F32  : float storage, float arithmetic (CUDA cores)
 *   ELMAN_BF16 : __nv_bfloat16 storage, float accumulation (tcgen05 tensor
 *                cores where the shape allows it, CUDA cores otherwise)
 * The library never allocates device memory inside a compute call: the caller
 * provides `workspace` of at least the size the matching *_workspace()
 * function returns, 256-byte aligned.  Work is enqueued on `stream` and the
 * call returns without synchronising.  Return value: ELMAN_OK or an error code;
 * elman_b200_last_error() gives the message of the calling thread's last error.
 *
 * Each function names the entry point of the reference (ekg/elman) it
 * replaces; the reference binds those through pybind11 in
 * elman/cuda/pytorch/elman_ladder.cc and implements them in elman/cuda/lib/.
 */
#ifndef ELMAN_B200_H_
#define ELMAN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ELMAN_OK 0
#define ELMAN_ERR_ARG 1        /* bad shape, null pointer, misaligned buffer, unknown dtype */
#define ELMAN_ERR_CUDA 2       /* a CUDA runtime/driver call failed */
#define ELMAN_ERR_TIMEOUT 3    /* a bounded device-side wait gave up in an earlier launch */
#define ELMAN_ERR_WORKSPACE 4  /* workspace too small */
#define ELMAN_ERR_UNSUPPORTED 5

#define ELMAN_F32 0
#define ELMAN_BF16 1

/* Library version (major*100 + minor). */
int elman_b200_version(void);

/* Message of the last error raised on the calling thread ("" if none). */
const char* elman_b200_last_error(void);

/*
 * Device-side waits (grid barrier, mbarrier polls, step flags) are bounded.  A
 * wait that gives up records a code in a host-visible status word and makes the
 * kernel return early.  This call reads that word for the current device
 * without synchronising: returns ELMAN_OK, or ELMAN_ERR_TIMEOUT with the
 * recorded detail (kernel id << 24 | step) in *detail.  `clear` != 0 resets it.
 * The compute entry points also check it on entry.
 */
int elman_b200_device_status(int* detail, int clear);

/*
 * Tuning and test knobs (process-wide):
 *   "force_generic"  1 = always take the CUDA-core kernels, 0 = default
 *   "spin_limit"     iteration cap of every device-side wait
 *   "rec_ksplit"     K-split (cluster size) of the tensor-core recurrence, 0 = auto
 *   "rec_groups"     independent batch groups pipelined by the recurrence, 0 = auto
 *   "time_kernels"   1 = bracket the phases of E1/E0 calls with CUDA events
 *   "rec_trace"      1 = the tensor-core recurrence records per-step cycle stamps
 *   "rec_mma_warps"  MMA-issuing warps (independent accumulator chains) of the
 *                    tensor-core recurrence, 1..4, 0 = auto
 *   "rec_direct_publish"  who advances the step counter of the tensor-core
 *                    recurrence: 0 = auto (forward: each epilogue warp after its own
 *                    stores; backward: a dedicated publisher warp), 1 = epilogue
 *                    warps in both directions, 2 = publisher warp in both.  All
 *                    modes give bit-identical results.
 *   "rec_w_tmem"     where the recurrent weight tile lives: 0 (default) = in tensor memory
 *                    (A operand read from TMEM) where the plan prefers it and it fits, 1 = in
 *                    tensor memory whenever it fits, 2 = always in shared memory; bit-identical
 *   "rec_fin_groups" 0 (default) = launches with four or more batch groups use the kernel
 *                    instantiation with two finalising warp groups, 1 = always one group
 *   "gemm_persistent" 0 (default) = the persistent 128x256 GEMM kernel once its tiles fill the
 *                    SMs (and for the split-K weight gradients), 1 = never, 2 = always
 *   "gemm_pair"      0 (default) = GEMMs whose 256x256 tiles fill the device (two per SM
 *                    pair, or a K split over the pairs) run on CTA pairs
 *                    (tcgen05.mma.cta_group::2), 1 = never, 2 = whenever the shape allows.
 *                    All GEMM kernels give bit-identical results.
 *   "rec_large_batch" 1 (default) = batches over 32 rows take the throughput plan of
 *                    the tensor-core recurrence (widest batch group first), 0 = the
 *                    latency plan for every batch size
 *   "rec_replicas"   batch replicas of the tensor-core recurrence's grid for batches over 32:
 *                    0 (default) = as many copies of the grid as fit on the device, each on
 *                    its own share of the batch (they never wait on each other), 1 = one
 *                    copy, n = at most n.  Results do not depend on it.
 *   "rec_group_cap"  widest batch group (16, 32 or 64 rows) the large-batch plan may form;
 *                    0 (default) = 64
 *   "test_stall_step" failure-detection test hook, -1 (default) = off.  With a value k >= 1
 *                    thread block 0 of the next tensor-core launches (recurrences: at time
 *                    step k; projection GEMMs: at K iteration k) waits for something that
 *                    nothing delivers.  The wait runs out after "spin_limit" polls, the
 *                    kernel records ELMAN_ERR_TIMEOUT in the status word, every block gives
 *                    up and the launch returns; its results are invalid.  Nothing faults.
 * Returns ELMAN_OK or ELMAN_ERR_ARG for an unknown name.
 */
int elman_b200_set_option(const char* name, long value);
long elman_b200_get_option(const char* name);

/*
 * Failure-detection test hook (no counterpart in the reference): launches one
 * tiny kernel that waits, for at most `spin_limit` polls, on a flag nothing
 * sets, then records ELMAN_ERR_TIMEOUT in the status word and returns.
 * `scratch` is 8 bytes of device memory; scratch[1] is set to 1 when the wait
 * gave up.  The device and context stay usable.
 */
int elman_b200_wait_probe(long spin_limit, void* scratch, void* stream);

/*
 * Measurement hook (no counterpart in the reference).  With option
 * "time_kernels" set, the dense-cell entry points record CUDA events on the
 * caller's stream around their phases: 0 forward recurrence kernel, 1 backward
 * recurrence kernel, 2 forward projection GEMM, 3 backward GEMMs.  This call
 * waits for the phase's stop event and returns the elapsed milliseconds of the
 * most recent call.
 */
int elman_b200_last_timing(int phase, float* ms);

/*
 * Diagnostics hook (no counterpart in the reference).  With option "rec_trace"
 * set, CTA 0 of the tensor-core recurrence kernels stores SM cycle stamps for its
 * first 64 steps, 16 slots per step.  Dense kernel (E0/E1/E33): 0 dependency
 * satisfied, 11 proxy fence done, 1 TMA issued, 2 state tile landed, 3 MMAs
 * issued, 4 accumulator complete, 5 partials scattered, 6 all partials landed,
 * 14 partial sums read, 7 new state stored, 8 epilogue threads met, 9 step
 * published, 10 next inputs requested.  Low-rank kernel (E5): 0 state ready,
 * 1 phase-1 MMAs issued, 2 rank accumulator complete, 3 partials sent, 4 partials
 * landed, 5 summed, 6 rank vector sent, 7 rank vector landed, 8 phase-2 MMAs
 * issued, 9 state accumulator complete, 10 state written.  This call
 * synchronises and copies up to max_entries stamps of the most recent traced
 * launch into dst (host).  The buffer lives in that call's workspace, which must
 * still be allocated.  `python -m elman_b200.step_trace` prints them as a table.
 */
int elman_b200_recurrence_trace(long long* dst, int max_entries);

/* Number of this library's kernel launches since load (for launch accounting). */
long elman_b200_launch_count(void);
/* Of those, launches that took a tcgen05 tensor-core kernel. */
long elman_b200_tc_launch_count(void);

/* ---------------------------------------------------------------------------
 * E1 — gated Elman cell.
 *   h_t = tanh(W_x x_t + W_h h_{t-1} + b),  y_t = h_t * silu(z_t)
 * Replaces mamba_gated_elman_forward / mamba_gated_elman_backward
 * (elman/cuda/pytorch/elman_ladder.cc:161-217, :219-281), i.e.
 * MambaGatedElmanForward<T>::Run / MambaGatedElmanBackward<T>::Run
 * (elman/cuda/lib/mamba_gated_elman_gpu.cu.cc:417-474, :492-593).
 *   x,z,output,v : [T,B,d]   h : [T+1,B,d] (h[0] is written from h0)
 *   W_x,W_h : [d,d] ([out,in])   b : [d]   h0 : [B,d]
 * `v` (pre-activations) may be NULL when training == 0.
 * Backward ignores the gradient of h, as the reference does, and returns
 * dx,dz : [T,B,d], dW_x,dW_h : [d,d], db : [d] (all overwritten).
 * ------------------------------------------------------------------------- */
size_t elman_e1_forward_workspace(int dtype, int T, int B, int d);
int elman_e1_forward(int dtype, int training, int T, int B, int d,
                     const void* x, const void* z, const void* h0,
                     const void* W_x, const void* W_h, const void* b,
                     void* h, void* output, void* v,
                     void* workspace, size_t workspace_bytes, void* stream);
size_t elman_e1_backward_workspace(int dtype, int T, int B, int d);
int elman_e1_backward(int dtype, int T, int B, int d,
                      const void* W_x, const void* W_h, const void* x, const void* z,
                      const void* h, const void* v, const void* d_output,
                      void* dx, void* dz, void* dW_x, void* dW_h, void* db,
                      void* workspace, size_t workspace_bytes, void* stream);

/*
 * elman_e1_forward with launch flags (an extension; elman_e1_forward is flags 0).
 *   ELMAN_FLAG_COMPACT  run the recurrence with the plan that keeps the fewest thread
 *                       blocks resident (a smaller split of the reduction dimension, the
 *                       weight tile in tensor memory where shared memory cannot hold it)
 *                       instead of the plan with the shortest step.  For callers that
 *                       overlap several recurrence launches on different streams: a step
 *                       gets somewhat slower, the launch leaves more of the GPU to others.
 * Results differ from flags 0 only by the summation order of the split reduction.
 */
#define ELMAN_FLAG_COMPACT 1
int elman_e1_forward_flags(int dtype, int flags, int training, int T, int B, int d,
                           const void* x, const void* z, const void* h0,
                           const void* W_x, const void* W_h, const void* b,
                           void* h, void* output, void* v,
                           void* workspace, size_t workspace_bytes, void* stream);

/*
 * E1 backward over one time chunk of a longer sequence (an extension: the
 * reference's backward, elman/cuda/pytorch/elman_ladder.cc:219-281, always sees
 * the whole sequence and has no such arguments).  A caller that splits a sequence
 * into chunks — running elman_e1_forward per chunk with h0 = the previous chunk's
 * last state — calls this once per chunk in reverse order:
 *   dv_in  : [B,d] or NULL.  Gradient of the pre-activation of the first step of
 *            the FOLLOWING chunk, i.e. that chunk's dv_out; NULL for the last chunk.
 *   dv_out : [B,d] or NULL.  Receives the gradient of this chunk's first
 *            pre-activation, to be handed to the preceding chunk.
 * Chained this way the chunks give bit-for-bit the dx, dz of one whole-sequence
 * call, and dW_x, dW_h, db that sum (over chunks) to its weight gradients.
 * elman_e1_backward is this function with both pointers NULL and flags 0; the
 * workspace size is the same.  `flags` as for elman_e1_forward_flags.
 */
int elman_e1_backward_carry(int dtype, int flags, int T, int B, int d,
                            const void* W_x, const void* W_h, const void* x, const void* z,
                            const void* h, const void* v, const void* d_output,
                            const void* dv_in,
                            void* dx, void* dz, void* dW_x, void* dW_h, void* db,
                            void* dv_out,
                            void* workspace, size_t workspace_bytes, void* stream);

/*
 * Number of thread blocks the recurrence kernel of an E1/E0 call of this shape
 * keeps resident for the whole launch (each occupies one SM), or 0 when the shape
 * takes a cooperative-launch kernel, which the driver only starts when it fits.
 * The blocks of one launch wait for one another, so a caller that overlaps
 * several recurrence launches on different streams must keep the sum of their
 * resident blocks within the device's SM count (no counterpart in the reference).
 */
int elman_b200_recurrence_blocks(int dtype, int flags, int T, int B, int d);

/* ---------------------------------------------------------------------------
 * E1 forward for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference.  It exists for callers
 * that hold no allocator they may call at this point: code running inside a
 * stream capture or a real-time section where cudaMalloc (which may synchronise
 * the device) is forbidden, plugins of a host application that owns all device
 * memory and hands out only tensors, or a C caller that simply has no workspace
 * to give.  It computes exactly what elman_e1_forward computes and takes the same
 * inputs and outputs, but no workspace: the scratch of the pass (the projected
 * inputs for all time steps and the step counters) lives in a device array built
 * into the library, ELMAN_E1_STATIC_SCRATCH_BYTES large.  Every GPU that loads
 * the library holds that array until the process exits.
 *
 * Limits and rules:
 *  - the pass must fit: elman_e1_forward_workspace(dtype,T,B,d) <=
 *    ELMAN_E1_STATIC_SCRATCH_BYTES, otherwise ELMAN_ERR_WORKSPACE is returned and
 *    nothing is launched (bf16: roughly T*B*d <= 8.3 million elements);
 *  - the first call on a device looks up the array's device address
 *    (cudaGetSymbolAddress); make that first call outside any stream capture;
 *  - the call itself performs no cudaMalloc/cudaFree/cudaHostAlloc and calls no
 *    allocating library routine;
 *  - all calls on a device share the one array, which keeps the previous call's
 *    contents: the parts that must start at zero are cleared on the stream by
 *    each call, and two calls whose GPU work may overlap (different streams, or
 *    different host threads on the same device) race on it — serialise them;
 *  - bounded-wait failures are reported through the status word only if an
 *    earlier (allocating) call already created it for this device.
 * ------------------------------------------------------------------------- */
#define ELMAN_E1_STATIC_SCRATCH_BYTES (16u * 1024u * 1024u)
size_t elman_e1_forward_static_scratch_bytes(void);
int elman_e1_forward_static(int dtype, int training, int T, int B, int d,
                            const void* x, const void* z, const void* h0,
                            const void* W_x, const void* W_h, const void* b,
                            void* h, void* output, void* v, void* stream);

/* ---------------------------------------------------------------------------
 * E1 with the output gate on [h_t ; x_t] — an EXTENSION: no class or kernel of the reference
 * implements it; its only specification is the formula in the reference's README.md:25-29,
 *     h_t = tanh(W_x x_t + W_h h_{t-1} + b),   y_t = h_t * silu(W_g [h_t ; x_t] + b_g).
 * With W_g = [W_gh | W_gx] the x-part z_t = W_gx x_t + b_g is the caller's time-parallel gate
 * projection (the same input `z` as the reference's E1 takes); this entry point adds
 * W_gh h_t: one more time-parallel GEMM over the stored states with the gate in its epilogue.
 *   z_gate [T,B,d] receives z_t + W_gh h_t (the backward pass needs it).
 * Backward returns dx (through W_x only; the caller adds dz W_gx for its projection),
 * dz (= gradient of z and of z_gate), dW_x, dW_h, db and dW_gh; the gradient of h is
 * dropped as in elman_e1_backward.  Parity of this pair is checked against a restatement of
 * the README formula, not against reference code.
 * ------------------------------------------------------------------------- */
size_t elman_e1_hx_forward_workspace(int dtype, int T, int B, int d);
int elman_e1_hx_forward(int dtype, int training, int T, int B, int d, const void* x, const void* z,
                        const void* h0, const void* W_x, const void* W_h, const void* b,
                        const void* W_gh, void* h, void* output, void* v, void* z_gate,
                        void* workspace, size_t workspace_bytes, void* stream);
size_t elman_e1_hx_backward_workspace(int dtype, int T, int B, int d);
int elman_e1_hx_backward(int dtype, int T, int B, int d, const void* W_x, const void* W_h,
                         const void* W_gh, const void* x, const void* z_gate, const void* h,
                         const void* v, const void* d_output, void* dx, void* dz, void* dW_x,
                         void* dW_h, void* db, void* dW_gh, void* workspace,
                         size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------
 * E4 — E1 with a low-rank recurrent matrix:
 *   h_t = tanh(W_x x_t + U (V h_{t-1}) + b),  y_t = h_t * silu(z_t),  U [d, r], V [r, d].
 * Replaces lowrank_elman_forward / lowrank_elman_backward
 * (elman/cuda/pytorch/elman_ladder.cc:2665-2726, :2728-2800; module
 * elman/models/lowrank_elman.py:28-46, :134-160).  The recurrence runs on the E5 kernels
 * (rank-r intermediate on chip) with the dense projection of x as its input and z as
 * the gate input; backward returns dx, dz, dW_x, dU, dV, db.
 * ------------------------------------------------------------------------- */
size_t elman_e4_forward_workspace(int dtype, int T, int B, int d, int r);
int elman_e4_forward(int dtype, int training, int T, int B, int d, int r, const void* x,
                     const void* z, const void* h0, const void* W_x, const void* U, const void* V,
                     const void* b, void* h, void* output, void* v, void* workspace,
                     size_t workspace_bytes, void* stream);
size_t elman_e4_backward_workspace(int dtype, int T, int B, int d, int r);
int elman_e4_backward(int dtype, int T, int B, int d, int r, const void* W_x, const void* U,
                      const void* V, const void* x, const void* z, const void* h, const void* v,
                      const void* d_output, void* dx, void* dz, void* dW_x, void* dU, void* dV,
                      void* db, void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------
 * E33 — E1 with a self gate:  h_t as E1,  y_t = h_t * silu(h_t)  (no gate input).
 * Replaces e33_self_gate_forward / e33_self_gate_backward
 * (elman/cuda/pytorch/elman_ladder.cc:444-497, :499-557; module
 * elman/models/e33_self_gate.py:30-50).  Same recurrence kernels as E1; the gate is taken
 * from the new state in their epilogue.  Backward returns dx, dW_x, dW_h, db.
 * (E32 and E57 of the reference call the E1 entry points directly and need nothing else.)
 * ------------------------------------------------------------------------- */
size_t elman_e33_forward_workspace(int dtype, int T, int B, int d);
int elman_e33_forward(int dtype, int training, int T, int B, int d, const void* x, const void* h0,
                      const void* W_x, const void* W_h, const void* b, void* h, void* output,
                      void* v, void* workspace, size_t workspace_bytes, void* stream);
size_t elman_e33_backward_workspace(int dtype, int T, int B, int d);
int elman_e33_backward(int dtype, int T, int B, int d, const void* W_x, const void* W_h,
                       const void* x, const void* h, const void* v, const void* d_output, void* dx,
                       void* dW_x, void* dW_h, void* db, void* workspace, size_t workspace_bytes,
                       void* stream);

/* ---------------------------------------------------------------------------
 * E0 — stock Elman cell with a learned, x-only output gate.
 *   h_t as E1,  y_t = h_t * silu(W_gate x_t + b_gate)
 * Replaces stock_elman_forward / stock_elman_backward
 * (elman/cuda/pytorch/elman_ladder.cc:22-84, :86-155), i.e.
 * StockElmanForward<T>::Run / StockElmanBackward<T>::Run
 * (elman/cuda/lib/stock_elman_gpu.cu.cc:214-296, :322-472).
 * gate_cache[T,B,d] holds W_gate x_t + b_gate; it and v are required when
 * training != 0 and may be NULL otherwise.
 * ------------------------------------------------------------------------- */
size_t elman_e0_forward_workspace(int dtype, int T, int B, int d);
int elman_e0_forward(int dtype, int training, int T, int B, int d,
                     const void* x, const void* h0,
                     const void* W_x, const void* W_h, const void* W_gate,
                     const void* b, const void* b_gate,
                     void* h, void* output, void* v, void* gate_cache,
                     void* workspace, size_t workspace_bytes, void* stream);
size_t elman_e0_backward_workspace(int dtype, int T, int B, int d);
int elman_e0_backward(int dtype, int T, int B, int d,
                      const void* W_x, const void* W_h, const void* W_gate,
                      const void* x, const void* h, const void* v,
                      const void* gate_cache, const void* d_output,
                      void* dx, void* dW_x, void* dW_h, void* dW_gate,
                      void* db, void* db_gate,
                      void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------
 * E5 — pure low-rank Elman cell (no dense matrix anywhere).
 *   h_t = tanh(U_h (V_h h_{t-1}) + U_x (V_x x_t) + b),  y_t = h_t * silu(U_z (V_z x_t))
 * Replaces pure_lowrank_elman_forward[_fused] / pure_lowrank_elman_backward[_fused]
 * (elman/cuda/pytorch/elman_ladder.cc:2802-2948, :2956-3103), i.e.
 * PureLowRankElmanForwardFused<T>::Run / PureLowRankElmanBackwardFused<T>::Run
 * (elman/cuda/lib/pure_lowrank_elman_fused_gpu.cu.cc:170-271, :295-505).
 *   U_* : [d,r]   V_* : [r,d]
 * ------------------------------------------------------------------------- */
size_t elman_e5_forward_workspace(int dtype, int T, int B, int d, int r);
int elman_e5_forward(int dtype, int training, int T, int B, int d, int r,
                     const void* x, const void* h0,
                     const void* U_h, const void* V_h, const void* U_x, const void* V_x,
                     const void* U_z, const void* V_z, const void* b,
                     void* h, void* output, void* v,
                     void* workspace, size_t workspace_bytes, void* stream);
size_t elman_e5_backward_workspace(int dtype, int T, int B, int d, int r);
int elman_e5_backward(int dtype, int T, int B, int d, int r,
                      const void* U_h, const void* V_h, const void* U_x, const void* V_x,
                      const void* U_z, const void* V_z,
                      const void* x, const void* h, const void* v, const void* d_output,
                      void* dx, void* dU_h, void* dV_h, void* dU_x, void* dV_x,
                      void* dU_z, void* dV_z, void* db,
                      void* workspace, size_t workspace_bytes, void* stream);

/*
 * E5 backward over one time chunk of a longer sequence (an extension, as
 * elman_e1_backward_carry): dv_in [B,d] or NULL is the following chunk's dv_out, dv_out
 * [B,d] or NULL receives the gradient of this chunk's first pre-activation.
 * elman_e5_backward is this function with both NULL; same workspace size.
 */
int elman_e5_backward_carry(int dtype, int T, int B, int d, int r,
                            const void* U_h, const void* V_h, const void* U_x, const void* V_x,
                            const void* U_z, const void* V_z,
                            const void* x, const void* h, const void* v, const void* d_output,
                            const void* dv_in,
                            void* dx, void* dU_h, void* dV_h, void* dU_x, void* dV_x,
                            void* dU_z, void* dV_z, void* db,
                            void* dv_out,
                            void* workspace, size_t workspace_bytes, void* stream);
/* Thread blocks an E5 recurrence launch of this shape keeps resident (one cluster), or 0
 * when the shape takes the cooperative-launch kernel; see elman_b200_recurrence_blocks. */
int elman_b200_lowrank_blocks(int dtype, int T, int B, int d, int r);

/* ---------------------------------------------------------------------------
 * Time-parallel projection  C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]) (+ C).
 * This is the GEMM the reference issues through cuBLAS for W_x x_t over all t
 * and for the gate projection (blas<T>::gemm, elman/cuda/lib/blas.h:20-173;
 * call sites mamba_gated_elman_gpu.cu.cc:440-448, stock_elman_gpu.cu.cc:245-264).
 * Row strides lda/ldw/ldc are in elements.  bias may be NULL.  accumulate != 0
 * adds into the existing C.  bf16 calls take the TMA + tcgen05 kernel when
 * K % 64 == 0 and the pointers/strides are 16-byte aligned.
 * ------------------------------------------------------------------------- */
int elman_projection(int dtype, int M, int N, int K,
                     const void* A, int lda, const void* W, int ldw,
                     const void* bias, void* C, int ldc, int accumulate, void* stream);

/* ---------------------------------------------------------------------------
 * The phases of an E1 call as separate entry points (an extension; the reference
 * only has the whole-call functions above).  elman_e1_forward is
 *   elman_gemm(NT: pre = x W_x^T + b)  ->  elman_e1_recurrence_forward
 * and elman_e1_backward(_carry) is
 *   elman_e1_recurrence_backward  ->  elman_gemm(NN: dx = dv W_x),
 *   elman_gemm(TN: dW_x = dv^T x), elman_gemm(TN: dW_h = dv^T h[0:T]).
 * A caller that overlaps work on several streams can keep the latency-bound
 * recurrence launches back to back on one stream and run the time-parallel GEMMs
 * of other chunks or layers beside them on another.
 *
 * elman_gemm: dense row-major operands, C[M,N] overwritten unless accumulate (then the
 *   product is added to C: a weight gradient summed over several calls).
 *   ELMAN_GEMM_NT  C = A[M,K] B[N,K]^T (+ bias[N])     (blas<T>::gemm call sites of the
 *   ELMAN_GEMM_NN  C = A[M,K] B[K,N]                     reference: elman/cuda/lib/
 *   ELMAN_GEMM_TN  C = A[K,M]^T B[K,N]                   mamba_gated_elman_gpu.cu.cc:440-448,
 *                                                        :560-592)
 * elman_column_sum: out[N] = sum over the M rows of in[M,N], deterministic (the bias
 *   gradient; the reference accumulates it with float atomics, :318-322).
 * elman_e1_recurrence_forward: h_t = tanh(pre_t + W_h h_{t-1}), y_t = h_t silu(z_t);
 *   pre,z,output,v : [T,B,d], h : [T+1,B,d], h0 : [B,d].
 * elman_e1_recurrence_backward: dv : [T+1,B,d] — slots 0..T-1 receive the gradient of
 *   pre (= of the pre-activations), slot T is scratch for the carried-in gradient;
 *   dv_in as for elman_e1_backward_carry (dv[0:1] of this call is the next dv_in);
 *   dz : [T,B,d]; db : [d] = sum over t,b of dv.  W_h_T, if not NULL, is W_h transposed
 *   ([in,out], dense): a caller that runs many chunks with the same weights passes it to
 *   save the transpose each call would otherwise do (W_h may then be NULL).
 * ------------------------------------------------------------------------- */
#define ELMAN_GEMM_NT 0
#define ELMAN_GEMM_NN 1
#define ELMAN_GEMM_TN 2
int elman_gemm(int dtype, int op, int M, int N, int K, const void* A, const void* B,
               const void* bias, void* C, int accumulate, void* stream);
size_t elman_column_sum_workspace(int N);
int elman_column_sum(int dtype, long M, int N, const void* in, void* out,
                     void* workspace, size_t workspace_bytes, void* stream);
size_t elman_e1_recurrence_workspace(int dtype, int d);
int elman_e1_recurrence_forward(int dtype, int flags, int training, int T, int B, int d,
                                const void* pre, const void* z, const void* h0, const void* W_h,
                                void* h, void* output, void* v,
                                void* workspace, size_t workspace_bytes, void* stream);
int elman_e1_recurrence_backward(int dtype, int flags, int T, int B, int d,
                                 const void* W_h, const void* z, const void* h, const void* v,
                                 const void* d_output, const void* dv_in, const void* W_h_T,
                                 void* dv, void* dz, void* db,
                                 void* workspace, size_t workspace_bytes, void* stream);

/*
 * Spectral normalisation of a recurrent matrix, one kernel per direction (replaces the
 * reference cells' get_W_h, elman/models/mamba_gated_elman.py:123-146 and
 * elman/models/stock_elman.py:104-125, a dozen framework ops per layer and step):
 * `iterations` power-iteration steps from u [d] (same dtype as W, advanced in place),
 *   v = W^T u / (|W^T u| + eps),  u = W v / (|W v| + eps),
 * sigma = |u^T W v|, W_eff = W * target_radius / (sigma + eps).  v [d] and sigma [1] (fp32) are
 * kept for the backward pass:  dW (+)= s dW_eff - <dW_eff, W> target_radius / (sigma + eps)^2 u v^T
 * with s = target_radius / (sigma + eps)  (u and v held constant, as in the reference, which
 * runs the iteration under no_grad).  One thread-block cluster per matrix; fp32 arithmetic.
 */
int elman_spectral_norm_forward(int dtype, int d, const void* W, void* u, float* v, float* sigma,
                                void* W_eff, float target_radius, float eps, int iterations,
                                void* stream);
int elman_spectral_norm_backward(int dtype, int d, const void* W, const void* u, const float* v,
                                 const float* sigma, const void* dW_eff, void* dW, int accumulate,
                                 float target_radius, float eps, void* stream);

/* ---------------------------------------------------------------------------
 * The time-parallel ops of the layer and the model around the cell (the callers of the
 * hot path), one kernel per pass.
 *
 * elman_add_rmsnorm_forward / _backward: residual add + RMSNorm with an fp32 residual
 *   stream — LadderLM's per-layer "residual = x + residual; x = norm(residual)"
 *   (elman/models/ladder_lm.py:986-1003, :1013-1026: the fused rms_norm_fn of mamba_ssm
 *   when that package is present, else add, cast, nn.RMSNorm, cast as separate passes).
 *     x [M,D] (dtype), residual_in [M,D] fp32 or NULL (first layer)
 *     residual_out [M,D] fp32 = x + residual_in
 *     y [M,D] (dtype) = round(residual_out) * rstd * weight,
 *     rstd [M] fp32 = 1/sqrt(mean(round(residual_out)^2) + eps)
 *   Backward takes dy (gradient of y) and dresidual_out (gradient that reaches residual_out
 *   from later layers, fp32, or NULL) and returns dresidual_in (fp32, or NULL) and/or dx
 *   (dtype, or NULL) — the same values, residual_in and x being summed — and dweight [D].
 *
 * elman_in_proj_split_silu: the layer's input projection with its tail
 *   (elman/models/mamba_gated_elman.py:283-297: in_proj, chunk, silu, and the two
 *   contiguous copies): xz = u W_in^T with u [M,K], W_in [2*d_inner, K];
 *     x_raw = xz[:, :d_inner], x_act = silu(x_raw), z = xz[:, d_inner:], each dense
 *     [M, d_inner].  For bf16 with d_inner % 32 == 0 the split and the silu run in the
 *   epilogue of the tcgen05 GEMM and xz is never written; otherwise `workspace`
 *   (elman_in_proj_workspace bytes) holds xz for a separate pass.
 * elman_silu_backward_concat: dxz [M, 2*d_inner] = [ d_act * silu'(x_raw) | dz ], the
 *   operand of the projection's backward GEMMs.
 * ------------------------------------------------------------------------- */
size_t elman_add_rmsnorm_backward_workspace(int D);
int elman_add_rmsnorm_forward(int dtype, long M, int D, const void* x, const float* residual_in,
                              const void* weight, float eps, float* residual_out, void* y,
                              float* rstd, void* stream);
int elman_add_rmsnorm_backward(int dtype, long M, int D, const void* dy,
                               const float* dresidual_out, const float* residual_out,
                               const float* rstd, const void* weight, float* dresidual_in,
                               void* dx, void* dweight, void* workspace, size_t workspace_bytes,
                               void* stream);
size_t elman_in_proj_workspace(int dtype, long M, int d_inner);
int elman_in_proj_split_silu(int dtype, long M, int d_inner, int K, const void* u, const void* W_in,
                             void* x_raw, void* x_act, void* z, void* workspace,
                             size_t workspace_bytes, void* stream);
int elman_silu_backward_concat(int dtype, long M, int d_inner, const void* d_act, const void* x_raw,
                               const void* dz, void* dxz, void* stream);

/*
 * elman_adamw_step: one AdamW update (decoupled weight decay) of ALL parameters, which the
 * caller keeps in one flat buffer, as are the gradients and both moment estimates — the
 * optimizer step of the reference's training loop (torch.optim.AdamW + clip_grad_norm_,
 * train_ladder.py:360-365, :542-545) as a single launch:
 *     g = grads * (*grad_scale)          (grad_scale: device pointer or NULL = 1; the
 *                                          clipping factor min(1, max_norm / |g|))
 *     p *= 1 - lr * weight_decay
 *     m = beta1 m + (1 - beta1) g;  v = beta2 v + (1 - beta2) g^2
 *     p -= lr / (1 - beta1^t) * m / (sqrt(v) / sqrt(1 - beta2^t) + eps)
 * `step` is a device float holding the number of updates done so far; the call advances it
 * by one first (t is the advanced value), so a captured CUDA graph advances it on every
 * replay.  Arithmetic in fp32, storage in `dtype`.
 */
int elman_adamw_step(int dtype, long n, void* params, const void* grads, void* exp_avg,
                     void* exp_avg_sq, float lr, float beta1, float beta2, float eps,
                     float weight_decay, float* step, const float* grad_scale, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ELMAN_B200_H_ */

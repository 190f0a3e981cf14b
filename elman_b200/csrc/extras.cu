// Small extra entry points: the bounded-wait probe used by the failure-detection
// tests.  The probe waits on a flag that nothing sets, with the caller's iteration
// limit, so that the give-up path (status word, early return, usable context) can
// be exercised without faulting or hanging the device.
#include "common.cuh"

namespace elman {
namespace {

__global__ void wait_probe_kernel(int* flag, long limit, int* status, int* gave_up) {
  if (threadIdx.x != 0) return;
  long spins = 0;
  bool ok = true;
  while (ld_acquire_gpu(flag) == 0) {
    if (++spins > limit) { ok = false; break; }
  }
  if (!ok) {
    report_timeout(status, KID_WAIT_PROBE, (int)(spins & 0xFFFFFF));
    *gave_up = 1;
  }
}

}  // namespace
}  // namespace elman

using namespace elman;

extern "C" int elman_b200_wait_probe(long spin_limit, void* scratch, void* stream) {
  ELMAN_ARG_CHECK(scratch != nullptr, "scratch is NULL");
  ELMAN_ARG_CHECK(spin_limit >= 1 && spin_limit <= 100000000L, "spin_limit out of range");
  cudaStream_t st = (cudaStream_t)stream;
  ELMAN_CUDA_CHECK(cudaMemsetAsync(scratch, 0, 8, st));
  int* words = (int*)scratch;
  wait_probe_kernel<<<1, 32, 0, st>>>(words, spin_limit, device_status_ptr(), words + 1);
  count_launch(false);
  ELMAN_CUDA_CHECK(cudaGetLastError());
  return ELMAN_OK;
}

// A self-test of the bounded wait the tensor-core kernels rest on (tcgen05.cuh): one warp waits, with a limit of a
// few hundred polls, on an mbarrier that nobody arrives at.  The wait must come back false, raise the CTA's abort
// flag and record who gave up in the status word it was given.  That word is this file's own: the status words of
// the product kernels are not touched, no copy and no tensor-core instruction is in flight, and the kernel returns
// by itself within microseconds.  The host reads the word and clears it.
#include "tcgen05.cuh"

namespace {

__device__ int g_selftest_status = 0;

__global__ void bounded_wait_selftest_kernel(uint32_t limit, int who, int* __restrict__ out) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    tc::mbar_init(&bar, 1);
    abort_flag = 0;
  }
  __syncthreads();
  bool completed = true;
  if (threadIdx.x == 0) completed = tc::mbar_wait_limited(&bar, 0, &abort_flag, who, limit, &g_selftest_status);
  __syncthreads();
  if (threadIdx.x == 0) {
    out[0] = completed ? 1 : 0;
    out[1] = (int)abort_flag;
    out[2] = g_selftest_status;
    g_selftest_status = 0;  // cleared for the next call
  }
}

}  // namespace

// out: int32[3] on the device: {1 if the wait claimed completion, the abort flag, the status word before clearing}.
PSB_API int psb_selftest_bounded_wait(int limit, int who, void* out, cudaStream_t stream) {
  if (limit < 1 || limit > 4096) PSB_REFUSE("selftest: the limit must be in [1, 4096] polls, not %d", limit);
  if (!out || who == 0) PSB_REFUSE("selftest: an output array and a non-zero code are needed");
  bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>((uint32_t)limit, who, (int*)out);
  PSB_LAUNCH_CHECK("selftest_bounded_wait");
  return 0;
}

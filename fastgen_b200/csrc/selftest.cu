// Self-tests of device-side helpers that no ordinary run exercises.
//
// fg_selftest_wait_timeout runs the bounded wait of the attention kernels (mbar_wait)
// against a barrier at which nothing ever arrives, with a short limit, so that the
// path "a wait ran out" is seen to end, to set the status bit and to release the
// other waits of the block.  It hangs nothing: every loop in it is counted.
#include "attention_mma.cuh"

namespace {

__global__ void wait_timeout_kernel(int limit, int* status, long long* out) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int gave_up;
  const int tid = threadIdx.x;
  if (tid == 0) {
    gave_up = 0;
    fg_mma::mbar_init(&bar, 1);
    fg_mma::mbar_fence_init();
  }
  __syncthreads();
  if (tid == 0) {
    // nobody arrives at `bar`: this wait runs to its limit
    const long long t0 = clock64();
    const bool ok = fg_mma::mbar_wait(&bar, 0, status, &gave_up, limit);
    out[0] = ok ? 1 : 0;
    out[2] = clock64() - t0;
  }
  __syncthreads();
  if (tid == 32) {
    // a second wait of the same block, with the full limit: the flag ends it at once
    const long long t0 = clock64();
    const bool ok = fg_mma::mbar_wait(&bar, 0, status, &gave_up);
    out[1] = ok ? 1 : 0;
    out[3] = clock64() - t0;
  }
  if (tid == 64) {
    // a wait on a completed phase is unaffected by the flag
    out[4] = fg_mma::mbar_wait(&bar, 1, status, &gave_up) ? 1 : 0;
  }
}

}  // namespace

// out: 5 long long on the device: [first wait returned, second wait returned, cycles of the
// first, cycles of the second, a wait on a completed phase returned].
extern "C" int fg_selftest_wait_timeout(int limit, int* status, long long* out, cudaStream_t stream) {
  FG_CHECK_ARG(limit > 0 && limit <= (1 << 16), "fg_selftest_wait_timeout: the limit must be in 1..65536 polls");
  FG_CHECK_ARG(status != nullptr && out != nullptr, "fg_selftest_wait_timeout: null pointer");
  wait_timeout_kernel<<<1, 96, 0, stream>>>(limit, status, out);
  FG_CHECK_LAUNCH("fg_selftest_wait_timeout");
  return 0;
}

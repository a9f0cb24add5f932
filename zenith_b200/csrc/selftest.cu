// Self-test of the bounded device-side wait that every kernel of this library relies on.
//
// zen_selftest_wait_limit launches ONE CTA of 64 threads in which warp 0 waits on an mbarrier that nobody
// ever arrives on and warp 1 waits on a second such barrier.  This translation unit is compiled with a
// wait limit of one millisecond, so the first wait gives up after that time: it records ZEN_ERR_TIMEOUT in
// the device status word and raises the CTA's abort flag, the second wait sees the flag and returns at
// once, and the kernel ends normally.  Nothing traps, faults or spins without a limit; the context stays
// usable.  The host then finds ZEN_ERR_TIMEOUT with zen_device_status_read and resets it with
// zen_device_status_clear — the path a timed-out production kernel would take.
#define ZEN_WAIT_LIMIT_NS 1000000ull
#include "zen_common.cuh"

namespace zen {

// out[0]: 1 if the first wait returned false (gave up), out[1]: 1 if the second returned false after seeing
// the abort flag, out[2]: elapsed nanoseconds of the whole wait sequence.
__global__ void __launch_bounds__(64) wait_limit_kernel(unsigned long long* out) {
  __shared__ uint64_t never[2];
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&never[0], 1);
    mbar_init(&never[1], 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  const uint64_t t0 = global_timer_ns();
  bool ok = true;
  if (threadIdx.x == 0) ok = mbar_wait(&never[0], 0, &abort_flag);
  __syncthreads();  // the flag is up: the second waiter must leave without serving its own limit
  bool ok2 = true;
  if (threadIdx.x == 32) ok2 = mbar_wait(&never[1], 0, &abort_flag);
  const uint64_t t1 = global_timer_ns();
  if (out != nullptr) {
    if (threadIdx.x == 0) {
      out[0] = ok ? 0ull : 1ull;
      out[2] = t1 - t0;
    }
    if (threadIdx.x == 32) out[1] = ok2 ? 0ull : 1ull;
  }
}

}  // namespace zen

ZEN_DEFINE_TU_STATUS(selftest)

extern "C" int zen_selftest_wait_limit(unsigned long long* result3, void* stream) {
  zen::wait_limit_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(result3);
  return cudaGetLastError() == cudaSuccess ? ZEN_OK : ZEN_ERR_LAUNCH;
}

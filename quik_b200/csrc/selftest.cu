// Self-test of the bounded device-side wait that every tcgen05 kernel of this library uses (tcgen05_ptx.cuh): one CTA
// waits on a barrier that nothing ever arrives on, with a limit of microseconds instead of the kernels' two seconds.
// The wait must give up, raise the CTA's abort flag, set the device status word and let the kernel return normally,
// which is what a host then sees through quik_device_status.  Nothing here faults, traps or spins without a bound.
#include "common.cuh"
#include "tcgen05_ptx.cuh"

namespace quik {
namespace {

__global__ void bounded_wait_selftest_kernel(unsigned long long limit_ns, unsigned int *status, int *result) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // phase 0 of a fresh barrier with one expected arrival that never comes
  const bool done = mbar_wait(smem_u32(&bar), 0, &abort_flag, status, limit_ns);
  __syncthreads();
  if (threadIdx.x == 0 && result) *result = done ? 1 : (abort_flag ? 2 : 3);
}

}  // namespace

int launch_bounded_wait_selftest(unsigned int limit_us, int *result, cudaStream_t st) {
  unsigned int *status = device_status_word();
  if (status == nullptr) return QUIK_ERR_CUDA;
  bounded_wait_selftest_kernel<<<1, 64, 0, st>>>((unsigned long long)limit_us * 1000ull, status, result);
  return check_launch("bounded_wait_selftest_kernel");
}

}  // namespace quik

// Self-test of the bounded wait every tensor-core kernel relies on.
//
// The attention kernels wait on mbarriers through wait_or_abort (sdpa_tc_common.cuh), which gives up after a cycle
// budget, records a code in the device status word and returns false.  In a healthy run that branch never executes,
// so this entry point runs it on purpose in the one way that cannot hang: a single warp waits, with a budget of a
// few thousand cycles, on a barrier that nothing will ever complete.  The wait polls a bounded number of times
// (each poll sleeps at most kWaitHintNs), sees the budget exceeded and returns; the kernel then exits normally.
#include "sdpa_tc_common.cuh"

namespace nb200 {
namespace {

__global__ void __launch_bounds__(32, 1) bounded_wait_selftest_kernel(int* status, int* result) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    sm100::mbar_init(sm100::smem_u32(&bar), 1);   // one arrival expected; none will come
    sm100::mbar_init_fence();
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    const bool completed = tc::wait_or_abort(sm100::smem_u32(&bar), 0, &abort_flag, status, 901, 4096);
    result[0] = completed ? 1 : 0;
    result[1] = abort_flag;
  }
}

}  // namespace
}  // namespace nb200

extern "C" NB200_API int nb200_selftest_bounded_wait(int* result_device, void* cuda_stream) {
  using namespace nb200;
  if (!result_device) { set_error("result pointer is NULL"); return NB200_ERR_INVALID; }
  int* status = device_status_word();
  if (!status) { set_error("device status word is unavailable"); return NB200_ERR_LAUNCH; }
  bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(cuda_stream)>>>(status, result_device);
  count_launch();
  return check_launch("bounded_wait_selftest_kernel");
}

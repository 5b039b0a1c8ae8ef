// Self-test of the bounded wait that every pipelined kernel of this library uses (mbar_wait in
// ptx.cuh): one warp waits, with a short cycle budget, on an mbarrier that nobody ever arrives
// at.  The wait must give up and return, raise the CTA's abort flag and record its code in the
// status word; a second wait in the same CTA must then return at once.  Nothing faults or
// spins without a limit: no TMA, no tensor memory, no other CTA is involved.
#include "ptx.cuh"
#include "errors.h"
#include "../../include/eisen_b200.h"

namespace eisen {
namespace {

__global__ void __launch_bounds__(32) bounded_wait_selftest_kernel(int* status, long long budget, int* report) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    const bool first = mbar_wait(&bar, 0, &abort_flag, status, FAULT_WAIT_SELFTEST, budget);
    const long long t1 = clock64();
    const bool second = mbar_wait(&bar, 0, &abort_flag, status, FAULT_WAIT_FULL, budget);  // abort flag is up: at once
    const long long t2 = clock64();
    if (report) {
      report[0] = first ? 1 : 0;
      report[1] = second ? 1 : 0;
      report[2] = abort_flag;
      report[3] = (t1 - t0) > budget ? 1 : 0;          // the first wait used its whole budget
      report[4] = (t2 - t1) < (t1 - t0) / 4 ? 1 : 0;   // the second one did not wait again
    }
  }
}

}  // namespace
}  // namespace eisen

extern "C" int eisen_selftest_bounded_wait(void* stream, int* status, long long budget_cycles, int* report5) {
  if (!status) return eisen::fail(EISEN_ERR_INVALID, "selftest_bounded_wait: status is null");
  if (budget_cycles < 1000 || budget_cycles > 200000000ll)
    return eisen::fail(EISEN_ERR_INVALID, "selftest_bounded_wait: budget must be between 1e3 and 2e8 cycles");
  eisen::bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, budget_cycles, report5);
  return eisen::check_launch("selftest_bounded_wait");
}

// Self test of the bounded waits every kernel of this library relies on: one CTA waits on an
// mbarrier that nobody arrives at, runs out of its (short) cycle budget, records
// kDevTimeoutProbe in the status word it was given and returns normally.  Nothing traps, spins
// without bound or touches memory it does not own; the context stays usable.  The reference's
// wait helper spins without a limit (src/primitives/33_mbarrier_try_wait.cuh:90-114); this is the
// test of the alternative used here.
#include "gemm_common.cuh"
#include "ptx.cuh"

namespace smb {

namespace {

__global__ void __launch_bounds__(32, 1) wait_probe_kernel(long long budget_cycles, int* status,
                                                           long long* waited_cycles) {
  __shared__ __align__(8) unsigned long long bar_storage;
  const uint32_t bar = smem_u32(&bar_storage);
  if (threadIdx.x == 0) {
    mbar_init(bar, 1);
    fence_mbar_init_cluster();
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    // Phase 0 of a barrier with one expected arrival that never comes.
    const bool arrived = mbar_wait(bar, 0u, budget_cycles);
    if (!arrived) report_status(status, kDevTimeoutProbe);
    if (waited_cycles != nullptr) *waited_cycles = clock64() - t0;
  }
}

}  // namespace

int wait_probe_launch(int* status, long long budget_cycles, long long* waited_cycles, cudaStream_t stream) {
  if (status == nullptr) return set_error(SMB_ERR_INVALID, "wait probe: null status word");
  // At most about a millisecond of SM clocks: the probe is a self test, not a way to stall a GPU.
  if (budget_cycles < 1 || budget_cycles > 2000000)
    return set_error(SMB_ERR_INVALID, "wait probe: budget of %lld cycles outside 1..2000000", budget_cycles);
  wait_probe_kernel<<<1, 32, 0, stream>>>(budget_cycles, status, waited_cycles);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error(e, "wait probe launch");
  return SMB_OK;
}

}  // namespace smb

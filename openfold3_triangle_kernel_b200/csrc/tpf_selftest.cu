// Self-test of the bounded-wait escape that every kernel of this library relies on.
//
// This translation unit is compiled with a wait limit of about one millisecond.  Its one kernel
// initialises an mbarrier that nothing ever arrives on and waits on it with the same mbar_wait()
// the production kernels use: the wait gives up after the limit, raises the CTA's abort flag,
// records kStatusWaitTimeout in the status word and the kernel runs to its normal end.  A second
// wait in the same CTA then returns at once (abort flag already up).  Nothing traps and nothing
// is left spinning; the host reads the status through tpf_device_status().
#define TPF_WAIT_LIMIT_CYCLES 2000000ll

#include "tpf_host.cuh"
#include "tpf_ptx.cuh"

namespace tpf {

static __device__ int g_selftest_status;

int selftest_status_fetch_and_clear(int* out) {
  int v = 0, zero = 0;
  TPF_CUDA_OK(cudaMemcpyFromSymbol(&v, g_selftest_status, sizeof(int)));
  if (v) TPF_CUDA_OK(cudaMemcpyToSymbol(g_selftest_status, &zero, sizeof(int)));
  *out = v;
  return TPF_OK;
}

// report[0] = cycles the first wait took, report[1] = cycles the second wait took (both as
// truncated 32-bit counts), report[2] = 1 when the kernel reached its last statement.
__global__ void __launch_bounds__(32) selftest_bounded_wait_kernel(int* __restrict__ status,
                                                                   unsigned int* __restrict__ report) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const WaitCtx wctx{&abort_flag, status};
    long long t0 = clock64();
    mbar_wait(&bar, 0, wctx);  // nobody arrives: runs into the limit
    long long t1 = clock64();
    mbar_wait(&bar, 0, wctx);  // abort flag is up: returns after the first poll batch
    long long t2 = clock64();
    if (report != nullptr) {
      report[0] = (unsigned int)(t1 - t0);
      report[1] = (unsigned int)(t2 - t1);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && report != nullptr) report[2] = 1u;
}

int selftest_bounded_wait(unsigned int* report, cudaStream_t stream) {
  int* status = nullptr;
  static PerDeviceAddress cache;
  if (int rc = device_symbol_address(g_selftest_status, cache, reinterpret_cast<void**>(&status))) return rc;
  selftest_bounded_wait_kernel<<<1, 32, 0, stream>>>(status, report);
  TPF_LAUNCH_OK();
  return TPF_OK;
}

}  // namespace tpf

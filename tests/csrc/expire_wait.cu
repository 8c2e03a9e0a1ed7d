// Test-only kernel: one thread waits on an mbarrier that nobody ever arrives on, through the library's own
// bounded wait compiled with a tiny poll limit.  The wait gives up by itself, the thread raises the CTA's
// abort flag and stores DAX_ERR_TIMEOUT into the library's device status word, exactly as the production
// kernels do on their tear-down path, and the kernel returns normally: nothing traps, faults or spins
// without a bound.  Built by tests/test_gpu_timeout.py against libdax_b200.so.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace {

__global__ void expire_wait_kernel(int* status, unsigned* polls_done) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_word;
  if (threadIdx.x == 0) {
    dax::mbar_init(&bar, 1);
    abort_word = 0;
    dax::mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool ok = dax::mbar_wait(&bar, 0, &abort_word);  // phase 0 never completes
    *polls_done = dax::kSpinLimit;
    if (!ok && abort_word) atomicExch(status, DAX_ERR_TIMEOUT);
  }
  __syncthreads();
  // a sibling that would have waited on the same barrier sees the abort flag and leaves at once
  if (threadIdx.x == 32) (void)dax::mbar_wait(&bar, 0, &abort_word);
}

}  // namespace

extern "C" int dax_test_expire_wait(unsigned* polls_done_device, void* stream) {
  int* status = dax::device_status_ptr();
  if (status == nullptr) return DAX_ERR_CUDA;
  expire_wait_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(status, polls_done_device);
  return cudaGetLastError() == cudaSuccess ? DAX_OK : DAX_ERR_CUDA;
}

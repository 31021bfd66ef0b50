// pcb_selftest.cu — the one failure the tensor-core kernels can detect on the device, made on
// purpose and harmlessly: a bounded mbarrier wait that runs out.
//
// Every wait of the tcgen05 kernels (on a bulk copy, on tcgen05.commit, on a consumer's release)
// goes through pcbtc::mbar_wait, which gives up after a fixed number of polls, raises the circuit's
// status word and lets the kernel drain and return, so that a lost signal costs one wrong step and
// not the GPU.  The self-test runs that very primitive on a barrier that nothing ever arrives at,
// with a small poll limit, and reports what the host would see: the status word, that the kernel
// went on past the wait and returned, and the time one poll takes (from which the length of a
// production wait follows).  The reference has no counterpart (it has no device-side waits).
#include "pcb_internal.h"
#include "pcb_tc.cuh"

namespace {

__global__ void wait_limit_kernel(int* status, int* after_wait, uint32_t polls) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    pcbtc::mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) ok = pcbtc::mbar_wait(&bar, 0, status, polls);   // nobody arrives
  __syncthreads();
  if (threadIdx.x == 0) *after_wait = ok ? 1 : 2;   // 2: the wait gave up and the kernel carried on
}

}  // namespace

extern "C" int32_t pcb_selftest_wait_limit(int32_t device, uint32_t polls, int32_t* status_out, int32_t* after_out,
                                           float* ms_out, uint32_t* production_polls_out) {
  PCB_REQUIRE(status_out && after_out && ms_out, "null argument");
  PCB_REQUIRE(polls >= 1 && polls <= (1u << 20), "poll limit of the self-test out of range");
  PCB_CUDA(cudaSetDevice(device));
  int* d = nullptr;
  PCB_CUDA(cudaMalloc(&d, 2 * sizeof(int)));
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  int32_t rc = PCB_OK;
  int h[2] = {-1, -1};
  float ms = 0.f;
  do {
    if (cudaMemset(d, 0, 2 * sizeof(int)) != cudaSuccess || cudaEventCreate(&e0) != cudaSuccess ||
        cudaEventCreate(&e1) != cudaSuccess) { rc = pcb_fail(PCB_ERR_CUDA, "self-test set-up failed"); break; }
    cudaEventRecord(e0, 0);
    wait_limit_kernel<<<1, 32>>>(d, d + 1, polls);
    cudaEventRecord(e1, 0);
    cudaError_t e = cudaEventSynchronize(e1);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) { rc = pcb_fail(PCB_ERR_CUDA, std::string("self-test kernel: ") + cudaGetErrorString(e)); break; }
    cudaEventElapsedTime(&ms, e0, e1);
    if (cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost) != cudaSuccess) rc = pcb_fail(PCB_ERR_CUDA, "self-test read-back failed");
  } while (false);
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  cudaFree(d);
  *status_out = h[0];
  *after_out = h[1];
  *ms_out = ms;
  if (production_polls_out) *production_polls_out = pcbtc::WAIT_LIMIT;
  return rc;
}

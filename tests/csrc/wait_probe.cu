// Test-only kernel: makes one bounded wait of the library's own mbar_wait run out.
// One thread waits on an mbarrier that nothing ever arrives on; after the (shortened) limit the
// wait gives up, the kernel records PRISM_ERR_DEVICE_WAIT in the workspace header exactly as the
// product kernels do, and returns normally.  Nothing traps, faults or hangs: the context stays
// usable, which is what the test then shows by running a normal forward on the same workspace.
#define PRISM_WAIT_LIMIT_CYCLES (100000ll)
#include "../../cute_mma_b200/csrc/prism_common.cuh"

__global__ void wait_probe_kernel(int* err) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    prism::mbar_init(&bar, 1);
    prism::fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!prism::mbar_wait(&bar, 0)) atomicExch(err, PRISM_ERR_DEVICE_WAIT);
  }
  __syncthreads();
}

extern "C" int wait_probe_launch(void* workspace, void* stream) {
  wait_probe_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<int*>(workspace));
  return (int)cudaGetLastError();
}

// prism_fwd_noalloc: the forward pass for callers that cannot allocate device memory.
//
// Who needs this: code that runs where cudaMalloc (or a framework allocator that may fall back to
// it) is off limits -- a forward issued from inside a memory-pool callback or an allocator hook,
// an inference server whose device memory was carved up completely at start-up and handed to other
// owners, a plug-in that is only lent input and output buffers by its host application.  The
// regular prism_fwd needs a caller-provided workspace (the status header, and for reconn_sz = 8
// the 16-wide copy of R that the tensor-core rotation reads); such a caller has nowhere to get one.
//
// Here that scratch is a fixed array in the library's own device image.  Consequences the caller
// must know:
//   * the array is PRISM_NOALLOC_SCRATCH_BYTES long on every GPU that loads the library, from
//     load until the process exits, whether or not this entry point is ever called;
//   * shapes whose scratch need exceeds it are refused with PRISM_ERR_WORKSPACE (the need is
//     256 bytes, plus (N / group_size) * 16 * K * 2 bytes when reconn_sz = 8);
//   * all calls on one GPU share the one array and it keeps what the previous call left there.
//     Each call rewrites everything it later reads (the copy of R) and clears the status word
//     before its kernels run, so calls that follow each other on one stream are independent;
//     two calls that may overlap on the GPU (different streams, no event between them) race on
//     the array and give undefined results;
//   * the first call on each GPU looks up the array's device address (cudaGetSymbolAddress, once
//     per device, with that device current).  Make that first call outside any stream capture.
// Nothing on this path calls cudaMalloc, cudaFree or any allocating library routine.
#include <mutex>

#include "prism_host.cuh"

namespace prism {
namespace {

// File-scope scratch.  In host code this name is only a handle for the runtime's symbol lookup --
// it is NOT a device address and must never be passed to a kernel; the address comes from
// cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[PRISM_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_addr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device (set-up on first use).
int scratch_address(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(PRISM_ERR_CUDA, "prism_fwd_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(PRISM_ERR_UNSUPPORTED, "prism_fwd_noalloc: device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      (void)cudaGetLastError();
      return fail(PRISM_ERR_CUDA, "prism_fwd_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev,
                  cudaGetErrorString(e));
    }
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return PRISM_OK;
}

}  // namespace
}  // namespace prism

using namespace prism;

extern "C" int prism_fwd_noalloc(const void* A, const void* B, const void* R, const void* bias, void* C,
                                 int M, int N, int K, int group_size, int reconn_sz, int dtype, int gate,
                                 long long lda, long long ldb, long long ldr, long long ldc,
                                 const int* cfg, int* device_status, void* stream) {
  // the general kernel is the one whose scratch need is small and fixed (status word, 16-wide copy of R):
  // the few-token streaming kernel, which prism_fwd would pick for M <= 128, keeps partial sums whose
  // size grows with the shape, so this entry point never takes it
  int cfg_general[4] = {cfg ? cfg[0] : 0, cfg ? cfg[1] : 0, cfg ? cfg[2] : 0, 1};
  cfg = cfg_general;
  // refuse what does not fit before touching the device
  const size_t need = prism_workspace_bytes(PRISM_KIND_FWD, M, N, K, group_size, reconn_sz, dtype, cfg);
  if (need > (size_t)PRISM_NOALLOC_SCRATCH_BYTES)
    return fail(PRISM_ERR_WORKSPACE,
                "prism_fwd_noalloc: this shape needs %zu bytes of scratch but the built-in array holds %zu "
                "(limit: 256 + (N/group_size)*16*K*2 bytes for reconn_sz=8); use prism_fwd with a caller workspace",
                need, (size_t)PRISM_NOALLOC_SCRATCH_BYTES);
  void* scratch = nullptr;
  int rc = scratch_address(&scratch);
  if (rc) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // the status word must start at zero; the array still holds whatever the last call left
  cudaError_t e = cudaMemsetAsync(scratch, 0, PRISM_WORKSPACE_HEADER_BYTES, s);
  if (e != cudaSuccess) return fail(PRISM_ERR_CUDA, "prism_fwd_noalloc: clearing the status word: %s", cudaGetErrorString(e));
  rc = prism_fwd(A, B, R, bias, nullptr, C, M, N, K, group_size, reconn_sz, dtype, gate, lda, ldb, ldr, ldc, cfg,
                 scratch, (size_t)PRISM_NOALLOC_SCRATCH_BYTES, stream);
  if (rc) return rc;
  if (device_status != nullptr) {
    e = cudaMemcpyAsync(device_status, scratch, sizeof(int), cudaMemcpyDefault, s);
    if (e != cudaSuccess) return fail(PRISM_ERR_CUDA, "prism_fwd_noalloc: copying the status word: %s", cudaGetErrorString(e));
  }
  return PRISM_OK;
}

// Status strings, ABI version and the bounded-wait self-test of the mxk C interface.
#include "mxk_common.cuh"
#include "umma.cuh"

namespace mxk {
namespace {

// One thread waits on an mbarrier phase that nothing will ever complete, with the same bounded
// wait the tensor-core kernels use for their copies and MMAs, and reports the way they do.
__global__ void bounded_wait_selftest_kernel(int* status, int polls) {
  __shared__ uint64_t bar;
  umma::mbar_init(&bar, 1);
  umma::mbar_init_fence();
  const bool completed = umma::mbar_wait(&bar, 0, polls);
  if (!completed && status) atomicExch(status, 1);
}

}  // namespace
}  // namespace mxk

extern "C" {

const char* mxk_status_string(int status) {
  switch (status) {
    case MXK_OK: return "ok";
    case MXK_ERR_NULL: return "a required pointer is NULL";
    case MXK_ERR_DIMS: return "a dimension is non-positive or too large";
    case MXK_ERR_ALIGN: return "a pointer or stride is not sufficiently aligned";
    case MXK_ERR_UNSUPPORTED: return "head dimension or chunk size outside the compiled set";
    case MXK_ERR_WORKSPACE: return "workspace missing or too small";
    case MXK_ERR_SCRATCH_LIMIT: return "problem exceeds the library's built-in scratch buffer (see mxk_linrec_noalloc_max_elements)";
    default: break;
  }
  if (status > 0) return cudaGetErrorString(static_cast<cudaError_t>(status));
  return "unknown mxk status";
}

int mxk_abi_version(void) { return 3; }

int mxk_selftest_bounded_wait(int* status, int polls, mxk_stream_t stream) {
  if (!status) return MXK_ERR_NULL;
  if (polls < 1 || polls > 16) return MXK_ERR_DIMS;
  mxk::bounded_wait_selftest_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(status, polls);
  return mxk::launch_status();
}

}  // extern "C"

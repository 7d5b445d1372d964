// Status strings and ABI version of the mxk C interface.
#include "mxk_common.cuh"

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

int mxk_abi_version(void) { return 1; }

}  // extern "C"

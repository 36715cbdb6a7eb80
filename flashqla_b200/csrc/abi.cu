// Version and status text of the C ABI.
#include <cuda_runtime.h>

#include "fqla_internal.h"

extern "C" int fqla_version(void) { return 3; }

extern "C" const char* fqla_status_string(int status) {
  switch (status) {
    case FQLA_OK: return "ok";
    case FQLA_ERR_INVALID_ARG: return "invalid argument";
    case FQLA_ERR_UNSUPPORTED_DIM: return "unsupported head dimension (64 or 128 only)";
    case FQLA_ERR_TOO_LARGE: return "problem larger than the fixed scratch array of this entry point";
    default: break;
  }
  if (status > 0) return cudaGetErrorString((cudaError_t)status);
  return "unknown status";
}

// Host-side helpers shared by the translation units of libfqla_sm100.so.
#pragma once
#include <cuda_runtime.h>

#include "../../include/fqla.h"

namespace fqla {

// Opt a kernel in to `bytes` of dynamic shared memory on the current device.  Called before
// every launch: the attribute is per device and the call is a few hundred nanoseconds.
inline int configure_smem(const void* func, int bytes) {
  if (bytes <= 48 * 1024) return 0;
  return (int)cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

}  // namespace fqla

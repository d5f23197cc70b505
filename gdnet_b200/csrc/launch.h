// Host-side launch helper: programmatic dependent launch (see pdl_enter() in common.cuh).
#pragma once

#include <cuda_runtime.h>

#include <cstdlib>
#include <utility>

namespace gd {

// GDNET_PDL=1 turns the attribute on; without it kernels run in plain stream order.
inline bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* v = std::getenv("GDNET_PDL");
    on = (v != nullptr && v[0] == '1') ? 1 : 0;
  }
  return on == 1;
}

// Only for kernels whose every thread calls pdl_enter() before touching global memory.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace gd

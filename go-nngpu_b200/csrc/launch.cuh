// Kernel launches with programmatic dependent launch: a kernel of this library may be
// scheduled while the previous kernel on the same stream is still finishing; it runs its
// prologue (barrier set-up, TMEM allocation, descriptor prefetch), and
// ptx::grid_dependency_wait() then holds it until the previous kernel has completed and
// its memory is visible.  Every kernel calls ptx::grid_dependency_release() first, so that
// the kernel after it can be scheduled the same way.  This removes the launch gap between
// the many small dependent kernels of a layer chain.  GONNGPU_PDL=0 turns the launch
// attribute off (the device-side instructions are then no-ops).
#pragma once
#include <cstdlib>
#include <utility>
#include <cuda_runtime.h>

namespace gonn {

inline bool pdl_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("GONNGPU_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, KArgs(std::forward<Args>(args))...);
}

}  // namespace gonn

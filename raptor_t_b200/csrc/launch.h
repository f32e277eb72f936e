// Kernel launch with programmatic dependent launch: the next kernel in the stream may be
// scheduled (and run its prologue up to griddepcontrol.wait) while the previous one drains,
// which hides most of the launch latency between the ~90 dependent kernels of a forward pass.
#pragma once
#include <cuda_runtime.h>

#include "common.h"

namespace rt {

// Kernel attributes (dynamic shared-memory limit, carve-out) belong to a (function, device)
// pair: sets them the first time `func` is launched on the current device.
rt_status ensure_kernel_smem(const void* func, int smem_bytes, bool max_carveout);

template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

}  // namespace rt

// Device side (no-ops when the kernel was not launched with the attribute):
//   pdl_launch_dependents(): the next kernel may start its prologue now;
//   pdl_wait(): everything the previous kernel wrote is visible after this returns.
#define RT_PDL_LAUNCH_DEPENDENTS() asm volatile("griddepcontrol.launch_dependents;" ::: "memory")
#define RT_PDL_WAIT() asm volatile("griddepcontrol.wait;" ::: "memory")

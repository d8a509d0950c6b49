// Programmatic dependent launch for the kernels of a training step.
//
// A kernel whose first instruction is `pdl_prolog()` may be launched with programmatic stream serialization: its
// blocks become resident as soon as every block of the kernel before it on the stream has started (that kernel's own
// prolog releases them), and they wait inside `griddepcontrol.wait` until that kernel has completed and its writes
// are visible. What is saved is the launch latency and ramp-up between dependent kernels, ~1-3 us per boundary inside
// a captured graph; nothing changes in what a kernel may read or write. Launched without the attribute the two
// instructions do nothing.
#pragma once
#include <cuda_runtime.h>
#include <utility>

namespace rb {

// 1 when the kernels of a step (not only the tensor-core kernel) are to be launched with the attribute: planner
// option `pdl` = 2 (RB_GEMM_PDL); defined in gemm_tc.cu.
int pdl_enabled();

__device__ __forceinline__ void pdl_prolog() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <class... KArgs, class... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg;
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute at;
  at.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at.val.programmaticStreamSerializationAllowed = 1;
  const bool on = pdl_enabled() != 0;
  cfg.attrs = on ? &at : nullptr;
  cfg.numAttrs = on ? 1u : 0u;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace rb

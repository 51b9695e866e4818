// Kernel launch with programmatic dependent launch (PDL) for the training step.
//
// A training update is ~5400 dependent kernels on one stream.  Launched normally, each waits for its
// predecessor to drain completely before its own CTAs are even scheduled, and then spends its first
// microseconds on set-up (barrier initialisation, TMEM allocation, descriptor prefetch).  With the
// programmatic-stream-serialization attribute a kernel's CTAs may be scheduled as soon as every CTA of
// the predecessor has executed `griddepcontrol.launch_dependents` (the kernels here do so right after
// their set-up) and an SM has room; the kernel runs its own set-up and then blocks in
// `griddepcontrol.wait`, which returns when the predecessor has completed and its writes are visible.
// Rule every kernel launched through this helper keeps: no global memory access before `pdl_wait()`.
// WS_TRAIN_PDL=0 launches normally.
#pragma once
#include <cuda_runtime.h>

#include <cstdlib>

namespace ws {

inline bool train_pdl_enabled() {
  static const bool enabled = [] {
    const char* e = std::getenv("WS_TRAIN_PDL");
    return e == nullptr || e[0] != '0';
  }();
  return enabled;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_dependent(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = train_pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

}  // namespace ws

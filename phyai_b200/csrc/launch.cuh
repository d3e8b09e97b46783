// One launch path for every kernel of the library: optional thread-block cluster along z
// and optional programmatic dependent launch (PDL). With PDL a kernel may start while
// its predecessor in the stream is still running; each kernel calls
// griddepcontrol.launch_dependents first thing and griddepcontrol.wait before it
// touches memory a predecessor may still read or write, so only set-up work and
// weight prefetch overlap. PDL edges survive stream capture into CUDA graphs.
#pragma once
#include <cuda_runtime.h>

#include <utility>

namespace pb {

bool pdl_enabled();
void set_pdl_enabled(bool on);
void bump_launch_counter(unsigned long long n);

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, int cluster_z, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  if (cluster_z > 1) {
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = 1;
    attrs[na].val.clusterDim.y = 1;
    attrs[na].val.clusterDim.z = unsigned(cluster_z);
    ++na;
  }
  if (pdl_enabled()) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  bump_launch_counter(1);
  return cudaLaunchKernelEx(&cfg, kern, KArgs(std::forward<Args>(args))...);
}

}  // namespace pb

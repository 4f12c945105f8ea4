// Host-side launch helper: cudaLaunchKernelEx with the programmatic-stream-serialisation attribute (so consecutive
// kernels of this library overlap their prologues with their predecessors' tails, also inside captured CUDA graphs)
// and, optionally, a thread-block cluster dimension.  B200RT_PDL=0 turns the attribute off (A/B measurements).
#pragma once
#include <cuda_runtime.h>
#include <cstdlib>
#include "trace.cuh"
#include "debug_check.cuh"

namespace b200 {

inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = std::getenv("B200RT_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v != 0;
}

// internal linkage on purpose: the trace refresh below is per translation unit
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_ex(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_x,
                             Args&&... args) {
  trace_refresh();
  debug_refresh();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 0) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = static_cast<unsigned>(cluster_x);
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// the same with a full cluster shape
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_ex_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                            dim3 cluster, Args&&... args) {
  trace_refresh();
  debug_refresh();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  attr[n].id = cudaLaunchAttributeClusterDimension;
  attr[n].val.clusterDim.x = cluster.x;
  attr[n].val.clusterDim.y = cluster.y;
  attr[n].val.clusterDim.z = cluster.z;
  ++n;
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace b200

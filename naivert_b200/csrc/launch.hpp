// Kernel launch helper: cudaLaunchKernelEx with the programmatic-dependent-launch attribute
// (and an optional thread-block cluster), so consecutive kernels of a stream or a captured
// graph overlap the next kernel's preamble with the previous kernel's tail.  The reference
// gets the same edges by rewriting a captured graph after the fact
// (naivert/runtime/pdl_graph_edges.py:86); here they are requested at launch time.
#pragma once
#include <cuda_runtime.h>

#include <mutex>
#include <unordered_set>

namespace nrt {

// Every kernel asks for the same (maximum) shared-memory carve-out: kernels that follow one
// another with different carve-outs force the SM to drain and reconfigure between them, which
// defeats the overlap programmatic dependent launch is meant to give.
inline void prefer_max_shared(const void* kernel) {
  static std::mutex mu;
  static std::unordered_set<const void*> done;
  std::lock_guard<std::mutex> lock(mu);
  if (done.insert(kernel).second)
    cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

template <typename... KArgs, typename... Args>
int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl,
               Args&&... args) {
  prefer_max_shared(reinterpret_cast<const void*>(kernel));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
int launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, dim3 cluster, size_t smem, cudaStream_t stream,
                   bool pdl, Args&&... args) {
  prefer_max_shared(reinterpret_cast<const void*>(kernel));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  attr[n].id = cudaLaunchAttributeClusterDimension;
  attr[n].val.clusterDim.x = cluster.x;
  attr[n].val.clusterDim.y = cluster.y;
  attr[n].val.clusterDim.z = cluster.z;
  ++n;
  if (pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace nrt

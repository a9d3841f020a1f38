// CUDA graph plumbing in native code: stream capture, instantiation (optionally for device launch),
// upload and launch, plus graph inspection (node count, kernel names, programmatic edges).
//
// The reference reaches the same runtime calls through a ctypes layer
// (naivert/runtime/cuda_backend.py:398ff ``CudaRuntimeGraphApi``: ``graph_instantiate(flags=DEVICE_LAUNCH)``,
// ``graph_upload``, ``graph_launch``, ``inspect_graph``, ``kernel_function_names``) and rewrites captured
// edges into programmatic ones afterwards (naivert/runtime/pdl_graph_edges.py); here programmatic edges are
// requested at launch time by every kernel launch, so capture already yields them.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <vector>

extern "C" int nrt_graph_begin(void* stream) {
  return (int)cudaStreamBeginCapture(reinterpret_cast<cudaStream_t>(stream), cudaStreamCaptureModeThreadLocal);
}
extern "C" int nrt_graph_end(void* stream, void** graph_out) {
  cudaGraph_t g = nullptr;
  cudaError_t e = cudaStreamEndCapture(reinterpret_cast<cudaStream_t>(stream), &g);
  *graph_out = g;
  return (int)e;
}
// device_launch != 0: instantiate for launch from device code (the graph must then be uploaded before use)
extern "C" int nrt_graph_instantiate(void* graph, int device_launch, void** exec_out) {
  cudaGraphExec_t x = nullptr;
  cudaError_t e = cudaGraphInstantiate(&x, reinterpret_cast<cudaGraph_t>(graph),
                                       device_launch ? cudaGraphInstantiateFlagDeviceLaunch : 0);
  *exec_out = x;
  return (int)e;
}
extern "C" int nrt_graph_upload(void* exec, void* stream) {
  return (int)cudaGraphUpload(reinterpret_cast<cudaGraphExec_t>(exec), reinterpret_cast<cudaStream_t>(stream));
}
extern "C" int nrt_graph_launch(void* exec, void* stream) {
  return (int)cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(exec), reinterpret_cast<cudaStream_t>(stream));
}
extern "C" int nrt_graph_destroy(void* graph, void* exec) {
  if (exec) cudaGraphExecDestroy(reinterpret_cast<cudaGraphExec_t>(exec));
  if (graph) cudaGraphDestroy(reinterpret_cast<cudaGraph_t>(graph));
  return 0;
}
// counts[0] = nodes, [1] = kernel nodes, [2] = edges, [3] = programmatic edges
extern "C" int nrt_graph_inspect(void* graph, int* counts) {
  cudaGraph_t g = reinterpret_cast<cudaGraph_t>(graph);
  size_t n = 0;
  cudaError_t e = cudaGraphGetNodes(g, nullptr, &n);
  if (e != cudaSuccess) return (int)e;
  std::vector<cudaGraphNode_t> nodes(n);
  if (n) cudaGraphGetNodes(g, nodes.data(), &n);
  int kernels = 0;
  for (auto nd : nodes) {
    cudaGraphNodeType t;
    if (cudaGraphNodeGetType(nd, &t) == cudaSuccess && t == cudaGraphNodeTypeKernel) ++kernels;
  }
  size_t ne = 0;
  int prog = 0;
  if (cudaGraphGetEdges_v2(g, nullptr, nullptr, nullptr, &ne) == cudaSuccess && ne) {
    std::vector<cudaGraphNode_t> from(ne), to(ne);
    std::vector<cudaGraphEdgeData> data(ne);
    if (cudaGraphGetEdges_v2(g, from.data(), to.data(), data.data(), &ne) == cudaSuccess)
      for (auto& d : data) prog += d.type == cudaGraphDependencyTypeProgrammatic;
  }
  counts[0] = (int)n; counts[1] = kernels; counts[2] = (int)ne; counts[3] = prog;
  return 0;
}

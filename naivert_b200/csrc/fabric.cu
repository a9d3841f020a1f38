// Host side of the peer-memory fabric: device allocations that can be exported to the other
// ranks of the node through CUDA IPC handles, opened there as peer pointers, and a mapped
// pinned host ring for device -> host records.  One process per GPU; handles travel through
// the torch.distributed store.
//
// Reference counterpart: single-process peer access (tests/gpu/naive_n0p5_e2e/run_naive_n0p5_decode.py:103
// ``enable_torch_tp8_peers``) and the mapped pinned ring of naivert/backends/naive_n0p5_draft_round.py:37-39.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

extern "C" int nrt_ipc_alloc(void** out, size_t bytes) {
  cudaError_t e = cudaMalloc(out, bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(*out, 0, bytes);
}
extern "C" int nrt_ipc_free(void* p) { return (int)cudaFree(p); }
extern "C" int nrt_ipc_handle_size() { return (int)sizeof(cudaIpcMemHandle_t); }
extern "C" int nrt_ipc_get_handle(void* p, void* handle_out) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle_out, &h, sizeof(h));
  return 0;
}
extern "C" int nrt_ipc_open(const void* handle, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}
extern "C" int nrt_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }

// mapped pinned host memory: returns host pointer and the device alias
extern "C" int nrt_host_alloc_mapped(void** host, void** dev, size_t bytes) {
  cudaError_t e = cudaHostAlloc(host, bytes, cudaHostAllocMapped | cudaHostAllocPortable);
  if (e != cudaSuccess) return (int)e;
  memset(*host, 0, bytes);
  return (int)cudaHostGetDevicePointer(dev, *host, 0);
}
extern "C" int nrt_host_free(void* host) { return (int)cudaFreeHost(host); }

// Device-side continuation of the speculative round: the last kernel of the round's graph launches the
// same executable graph again (tail launch) unless the control block says the chain stopped, so the host
// launches one graph per request and afterwards only polls the pinned ring.
//
// Backpressure: the host publishes the index of the last ring record it consumed; the round's tail kernel
// compares it with the round counter, max-reduces "must pause" over the ranks and leaves the decision in
// ctrl[13].  The chain pauses (does not relaunch) when that word is set, and the host restarts it with an
// ordinary launch.  Without a decision word from the tail (`host_consumed` given here) this rank decides alone.
// Reference counterpart: naivert/entry/dspark_tail_entry.cu:16-23
// (cudaGraphLaunch(cudaGetCurrentGraphExec(), cudaStreamGraphTailLaunch)).
#include "contract.h"
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

// ctrl[4] stopped, ctrl[5] reason, ctrl[8] round counter, ctrl[12] relaunch failures, ctrl[13] paused
__global__ void relaunch_kernel(int* ctrl, const volatile int* host_consumed, int ring_size) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  if (ctrl[NRT_CTRL_STOPPED]) return;
  if (host_consumed) ctrl[NRT_CTRL_PAUSED] = ctrl[NRT_CTRL_ROUND] - *host_consumed >= ring_size - 8 ? 1 : 0;
  if (ctrl[NRT_CTRL_PAUSED]) return;                                          // let the host catch up
  const cudaError_t e = cudaGraphLaunch(cudaGetCurrentGraphExec(), cudaStreamGraphTailLaunch);
  if (e != cudaSuccess) { ctrl[NRT_CTRL_RELAUNCH_FAIL] += 1; ctrl[NRT_CTRL_STOPPED] = 1; ctrl[NRT_CTRL_REASON] = NRT_STOP_RELAUNCH_FAILED; }   // fail closed: chain launch failed
}

}  // namespace

extern "C" int nrt_relaunch(int* ctrl, const int* host_consumed_dev, int ring_size, void* stream) {
  relaunch_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(ctrl, host_consumed_dev, ring_size);
  return (int)cudaGetLastError();
}

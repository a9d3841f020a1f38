// Small collective helpers over the peer-memory fabric used with the GEMM engine:
//   ag_push    : all-gather of a K-sharded token operand.  Each rank copies its [16 x K/tp] slice into
//                every rank's gather buffer (its own included) and then publishes a tagged flag there;
//                the consuming GEMM waits per source slice, so the gather overlaps the weight stream.
//   l2_flush   : writes a buffer larger than L2 (benchmark hygiene).
// Reference counterparts: the bf16 all-gather / reduce-scatter of the vendored FlashInfer mixed_comm
// (naivert/prefill/native/collectives.py:89-168) and NCCL (naivert/prefill/comms.py:54-147).
#include "gemm.cuh"
#include "launch.hpp"

using namespace nrt;

namespace {

struct AgPushArgs {
  const uint8_t* src;            // local slice: [rows16][slice_bytes] with row stride src_stride
  int src_stride;
  int slice_bytes;               // bytes of one row of the slice (multiple of 16)
  int row_bytes;                 // bytes of one full gathered row
  uint8_t* gather[kMaxPeers];    // gather[p]: rank p's gather buffer [16][row_bytes] (peer mapped)
  uint64_t* flags[kMaxPeers];    // flags[p]: rank p's flag words [tp]
  const uint32_t* epoch;
  int tp, rank, call;
};

// grid = tp CTAs: CTA p serves destination rank (rank + p) % tp.
__global__ void __launch_bounds__(256) ag_push_kernel(const AgPushArgs a) {
  griddep_wait();
  griddep_launch();
  const int dst = (a.rank + blockIdx.x) % a.tp;
  const int vec = a.slice_bytes / 16;
  uint8_t* base = a.gather[dst] + (size_t)a.rank * a.slice_bytes;
  for (int i = threadIdx.x; i < kTok * vec; i += 256) {
    const int r = i / vec, c = i - r * vec;
    const uint4 v = *reinterpret_cast<const uint4*>(a.src + (size_t)r * a.src_stride + c * 16);
    *reinterpret_cast<uint4*>(base + (size_t)r * a.row_bytes + c * 16) = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t tag = (*a.epoch) * 1024u + (uint32_t)a.call + 1u;
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    st_tagged(a.flags[dst] + a.rank, tag, 1u);
  }
}

__global__ void l2_flush_kernel(uint4* buf, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    buf[i] = make_uint4((unsigned)i, 0u, 0u, 0u);
}

}  // namespace

extern "C" int nrt_ag_push_args_size() { return (int)sizeof(AgPushArgs); }
extern "C" int nrt_ag_push(const void* args, void* stream, int pdl) {
  AgPushArgs a;
  memcpy(&a, args, sizeof(a));
  if (a.slice_bytes % 16 || a.src_stride % 16 || a.row_bytes % 16) return -3;
  return launch_pdl(ag_push_kernel, dim3(a.tp), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), pdl != 0, a);
}
extern "C" int nrt_l2_flush(void* buf, size_t bytes, void* stream) {
  l2_flush_kernel<<<592, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>((uint4*)buf, bytes / 16);
  return (int)cudaGetLastError();
}

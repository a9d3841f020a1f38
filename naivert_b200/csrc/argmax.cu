// Greedy tensor-parallel arg-max over vocabulary-sharded logits.
//
// token[r] = argmax over the whole vocabulary of logits[r] (lowest token id on ties).  One CTA per row reduces
// this rank's shard to a packed 64-bit key (order-preserving value << 32 | ~global token id); the last CTA to
// finish exchanges the per-row keys with the other ranks through the small-message fabric (bounded wait) and
// writes the winners.  Used by greedy seq-1 decoding and as a cross-check of the sampler at top-p -> 0.
// Reference counterpart: naivert/entry/tp8_argmax_rows_entry.cu:52,132 (per-rank top-1 published to inboxes by
// the head kernel, then a <<<rows, 8>>> pick).
#include "fabric.cuh"
#include "launch.hpp"

#include <string.h>

using namespace nrt;

namespace {

struct ArgmaxArgs {
  const float* logits;          // [rows][ld] this rank's vocabulary shard
  int ld, rows, vlocal, vbase;
  int* tokens;                  // [rows] out: global token ids (identical on every rank)
  unsigned long long* keys;     // [16] scratch
  unsigned int* ticket;         // zero-initialised, reset by the last CTA
  int call;                     // exchange call index (unique inside one epoch)
  XchgArgs x;
};

__global__ void __launch_bounds__(1024) argmax_rows_kernel(const ArgmaxArgs a) {
  __shared__ unsigned long long sbest;
  __shared__ bool s_last;
  __shared__ uint64_t xv[16];
  griddep_wait();
  griddep_launch();
  const int r = blockIdx.x;
  if (threadIdx.x == 0) sbest = 0ull;
  __syncthreads();
  unsigned long long best = 0ull;
  const float* row = a.logits + (size_t)r * a.ld;
  for (int i = threadIdx.x; i < a.vlocal; i += 1024) {
    const unsigned long long key = ((unsigned long long)float_order(row[i]) << 32) | (unsigned)(~(unsigned)(a.vbase + i));
    best = key > best ? key : best;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if ((threadIdx.x & 31) == 0) atomicMax(&sbest, best);
  __syncthreads();
  if (threadIdx.x == 0) {
    a.keys[r] = sbest;
    __threadfence();
    const unsigned int t = atomicAdd(a.ticket, 1u);
    s_last = t == gridDim.x - 1;
    if (s_last) *a.ticket = 0u;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (threadIdx.x < 16) xv[threadIdx.x] = (int)threadIdx.x < a.rows ? *reinterpret_cast<volatile unsigned long long*>(a.keys + threadIdx.x) : 0ull;
  __syncthreads();
  xchg_reduce_u64<kXMax>(xv, a.rows, a.x, a.call);
  if ((int)threadIdx.x < a.rows) a.tokens[threadIdx.x] = (int)(~(unsigned)(xv[threadIdx.x] & 0xffffffffull));
}

}  // namespace

extern "C" int nrt_argmax_args_size() { return (int)sizeof(ArgmaxArgs); }
extern "C" int nrt_argmax_rows(const void* args, void* stream, int pdl) {
  ArgmaxArgs a;
  memcpy(&a, args, sizeof(a));
  if (a.rows < 1 || a.rows > 16 || a.call < 0 || a.call >= 64) return -3;
  return launch_pdl(argmax_rows_kernel, dim3(a.rows), dim3(1024), 0, reinterpret_cast<cudaStream_t>(stream), pdl != 0, a);
}

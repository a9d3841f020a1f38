// Block-draft specific kernels: block input rows (anchor embedding + mask embeddings) and the
// sequential Markov head (low-rank previous-token bias + Gumbel-max proposal per row).
//
// The reference precomputes a [vocab, vocab/8] bf16 bias table (5.8 GB per rank,
// naivert/entry/dspark_head_markov_entry.cu:31,87) and looks up one row per step; here the
// rank-256 factors stay factored: each step evaluates bias = W2_shard . W1[prev] on the fly
// (W2_shard is 9.7 MB per rank at tp = 8 and stays L2 resident across the seven steps).
// Reference math: naivert/body/dspark_head_markov/markov_body.cuh:6-27,
// naivert/body/dspark_sampling/random.cuh:17-20 (Gumbel-max over (logits + bias) / T).
#include "contract.h"
#include "fabric.cuh"
#include "launch.hpp"

#include <float.h>
#include <string.h>

using namespace nrt;

namespace {

// x[0] = embed[anchor], x[1..rows) = mask embedding, x[rows..16) = 0
__global__ void draft_block_input_kernel(const int* __restrict__ block_ids, const __nv_bfloat16* __restrict__ embed,
                                         const __nv_bfloat16* __restrict__ mask, __nv_bfloat16* __restrict__ x, int hidden,
                                         int rows, int vocab) {
  griddep_wait();
  griddep_launch();
  const int r = blockIdx.x;
  uint4* dst = reinterpret_cast<uint4*>(x + (size_t)r * hidden);
  const uint4* src = nullptr;
  if (r == 0) {
    int t = block_ids[0];
    t = t < 0 ? 0 : (t >= vocab ? vocab - 1 : t);
    src = reinterpret_cast<const uint4*>(embed + (size_t)t * hidden);
  } else if (r < rows) {
    src = reinterpret_cast<const uint4*>(mask);
  }
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = src ? src[i] : make_uint4(0, 0, 0, 0);
}

struct MarkovArgs {
  const float* logits;            // [16][ld] draft head logits (row j proposes token j+1)
  int ld;
  const __nv_bfloat16* w1;        // [vocab][rank]
  const __nv_bfloat16* w2;        // [vlocal][rank]
  int rank_dim, vlocal, vbase, vocab;
  int* block_ids;                 // [8]; block_ids[step] is the previous token, block_ids[step+1] is written
  float* zq;                      // [8][ld] logits + bias (the draft distribution the sampler sees)
  const float* params;            // sampler params ([6] = 1/T of the draft)
  const unsigned long long* seed;
  const int* ctrl;                // round counter at [8]
  unsigned long long* best;       // scratch: packed (ordered value << 32 | ~token)
  unsigned int* ticket;
  XchgArgs x;
};

// grid = ceil(vlocal / 128) CTAs of 256 threads; 8 lanes per token row, 4 rounds of 32 rows.
__global__ void __launch_bounds__(256) markov_step_kernel(const MarkovArgs a, int step) {
  __shared__ float w1s[512];
  __shared__ unsigned long long sbest;
  __shared__ bool s_last;
  __shared__ uint64_t xv[16];
  griddep_wait();
  griddep_launch();
  int prev = a.block_ids[step];
  (void)NRT_INDEX_OK(prev, a.vocab, kBoundsMarkovPrev);
  prev = prev < 0 ? 0 : (prev >= a.vocab ? a.vocab - 1 : prev);
  for (int i = threadIdx.x; i < a.rank_dim; i += 256) w1s[i] = __bfloat162float(a.w1[(size_t)prev * a.rank_dim + i]);
  if (threadIdx.x == 0) sbest = 0ull;
  __syncthreads();
  const float inv_t = a.params[6];
  const unsigned long long seed = *a.seed;
  const uint32_t ctr = (uint32_t)a.ctrl[NRT_CTRL_ROUND] * 8u + (uint32_t)step;
  unsigned long long best = 0ull;
  // 8 lanes cooperate on one token row (rank_dim bf16 = 64 bytes per lane at rank 256), 4 rows per warp
  // at a time: every 16-byte load of a warp is part of a fully used 128-byte line.
  const int sub = threadIdx.x & 7, grp = threadIdx.x >> 3;         // 32 groups per CTA
  const int per_lane = a.rank_dim / 8;                              // elements per lane
  for (int i = 0; i < 4; ++i) {
    const int t = blockIdx.x * 128 + i * 32 + grp;
    float acc = 0.f;
    if (t < a.vlocal) {
      const uint4* wr = reinterpret_cast<const uint4*>(a.w2 + (size_t)t * a.rank_dim + sub * per_lane);
      for (int k = 0; k < per_lane / 8; ++k) {
        const uint4 v = wr[k];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
        const float* w = w1s + sub * per_lane + k * 8;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          acc += f.x * w[2 * j] + f.y * w[2 * j + 1];
        }
      }
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    acc += __shfl_xor_sync(0xffffffffu, acc, 4);
    if (sub == 0 && t < a.vlocal) {
      const float z = a.logits[(size_t)step * a.ld + t] + round_bf16(acc);
      a.zq[(size_t)step * a.ld + t] = z;
      const float u = philox_uniform(seed, 3u, ctr, (uint32_t)(t + a.vbase));
      const float g = -__logf(-__logf(u));
      const float s = z * inv_t + g;
      // larger score wins; ties go to the lower token id
      const unsigned long long key = ((unsigned long long)float_order(s) << 32) | (uint32_t)(~(uint32_t)(t + a.vbase));
      best = key > best ? key : best;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if ((threadIdx.x & 31) == 0) atomicMax(&sbest, best);
  __syncthreads();
  if (threadIdx.x == 0) {
    atomicMax(a.best, sbest);
    __threadfence();
    const unsigned int tk = atomicAdd(a.ticket, 1u);
    s_last = tk == gridDim.x - 1;
    if (s_last) *a.ticket = 0u;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (threadIdx.x < 16) xv[threadIdx.x] = threadIdx.x == 0 ? *reinterpret_cast<volatile unsigned long long*>(a.best) : 0ull;
  __syncthreads();
  xchg_reduce_u64<kXMax>(xv, 1, a.x, 16 + step);
  if (threadIdx.x == 0) {
    a.block_ids[step + 1] = (int)(~(uint32_t)xv[0]);
    *a.best = 0ull;
  }
}

// All proposals of a block in one launch: the same per-step work as markov_step_kernel, with the hand-over of the
// sampled token between steps done inside the grid.  Every CTA adds itself to a monotonic arrival counter after
// folding its best candidate into best[step]; the CTA that completes a step's count runs the tensor-parallel
// exchange, writes block_ids[step + 1] and publishes the step's generation; the others wait for that generation
// (bounded) and go on with the next previous-token row.  The grid must be resident at once (checked at launch).
__global__ void __launch_bounds__(256, 2) markov_chain_kernel(const MarkovArgs a, int steps, unsigned long long* arrive,
                                                           unsigned int* step_gen) {
  __shared__ float w1s[512];
  __shared__ unsigned long long sbest;
  __shared__ unsigned int s_gen;
  __shared__ int s_last, s_ok;
  __shared__ uint64_t xv[16];
  const int sub = threadIdx.x & 7, grp = threadIdx.x >> 3;
  const int per_lane = a.rank_dim / 8;
  // rank 256 (the shipped geometry): a thread's slice of the second factor - four tokens x 32 channels - does not
  // depend on the step, so it is loaded once and stays in registers for all steps; per step only the previous
  // token's row of the first factor and the step's base logits are fetched, all loads in flight together
  const bool fast = a.rank_dim == 256;
  uint4 wv[4][4];
  if (fast) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = blockIdx.x * 128 + i * 32 + grp;
      const bool on = t < a.vlocal;
      const uint4* wr = reinterpret_cast<const uint4*>(a.w2 + (size_t)(on ? t : 0) * 256 + sub * 32);
#pragma unroll
      for (int k = 0; k < 4; ++k) wv[i][k] = on ? __ldg(wr + k) : make_uint4(0u, 0u, 0u, 0u);
    }
  }
  griddep_wait();                                  // the factor is a weight: its loads above overlap the predecessor's tail
  griddep_launch();
  const float inv_t = a.params[6];
  const unsigned long long seed = *a.seed;
  const uint32_t round = (uint32_t)a.ctrl[NRT_CTRL_ROUND];
  for (int step = 0; step < steps; ++step) {
    int prev = step == 0 ? a.block_ids[0] : __ldcg(a.block_ids + step);
    (void)NRT_INDEX_OK(prev, a.vocab, kBoundsMarkovPrev);
    prev = prev < 0 ? 0 : (prev >= a.vocab ? a.vocab - 1 : prev);
    float base[4];
    if (fast) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int t = blockIdx.x * 128 + i * 32 + grp;
        base[i] = (t < a.vlocal && sub == 0) ? a.logits[(size_t)step * a.ld + t] : 0.f;
      }
    }
    for (int i = threadIdx.x; i < a.rank_dim; i += 256) w1s[i] = __bfloat162float(a.w1[(size_t)prev * a.rank_dim + i]);
    if (threadIdx.x == 0) { sbest = 0ull; s_ok = 1; }
    __syncthreads();
    const uint32_t ctr = round * 8u + (uint32_t)step;
    unsigned long long best = 0ull;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int t = blockIdx.x * 128 + i * 32 + grp;
      float acc = 0.f;
      if (fast) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&wv[i][k]);
          const float* w = w1s + sub * 32 + k * 8;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            acc += f.x * w[2 * j] + f.y * w[2 * j + 1];
          }
        }
      } else if (t < a.vlocal) {
        const uint4* wr = reinterpret_cast<const uint4*>(a.w2 + (size_t)t * a.rank_dim + sub * per_lane);
        for (int k = 0; k < per_lane / 8; ++k) {
          const uint4 v = wr[k];
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
          const float* w = w1s + sub * per_lane + k * 8;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            acc += f.x * w[2 * j] + f.y * w[2 * j + 1];
          }
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (sub == 0 && t < a.vlocal) {
        const float z = (fast ? base[i] : a.logits[(size_t)step * a.ld + t]) + round_bf16(acc);
        a.zq[(size_t)step * a.ld + t] = z;
        const float u = philox_uniform(seed, 3u, ctr, (uint32_t)(t + a.vbase));
        const float g = -__logf(-__logf(u));
        const float sc = z * inv_t + g;
        const unsigned long long key = ((unsigned long long)float_order(sc) << 32) | (uint32_t)(~(uint32_t)(t + a.vbase));
        best = key > best ? key : best;
      }
    }
    // 64-bit shared-memory atomics are compare-and-swap loops: fold inside the warp, one lane per warp updates
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
      best = other > best ? other : best;
    }
    if ((threadIdx.x & 31) == 0) atomicMax(&sbest, best);
    __syncthreads();
    if (threadIdx.x == 0) {
      atomicMax(a.best + step, sbest);
      __threadfence();
      const unsigned long long old = atomicAdd(arrive, 1ull);
      s_gen = (unsigned int)(old / gridDim.x + 1ull);
      s_last = (old + 1ull) % gridDim.x == 0ull;
    }
    __syncthreads();
    if (s_last) {
      __threadfence();
      if (threadIdx.x < 16) xv[threadIdx.x] = threadIdx.x == 0 ? *reinterpret_cast<volatile unsigned long long*>(a.best + step) : 0ull;
      __syncthreads();
      xchg_reduce_u64<kXMax>(xv, 1, a.x, 16 + step);
      if (threadIdx.x == 0) {
        a.block_ids[step + 1] = (int)(~(uint32_t)xv[0]);
        a.best[step] = 0ull;
        __threadfence();
        asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(step_gen), "r"(s_gen) : "memory");
      }
    } else if (step + 1 < steps) {
      if (threadIdx.x == 0) {
        const uint64_t deadline = globaltimer() + kWaitLimitNs;
        for (uint32_t i = 0;; ++i) {
          // generations only grow: a later step's value also releases this wait
          if ((int)(ld_acquire_gpu(step_gen) - s_gen) >= 0) break;
          if ((i & 255u) == 255u) {
            if (*reinterpret_cast<volatile uint32_t*>(a.x.status) != 0u) { s_ok = 0; break; }
            if (globaltimer() > deadline) { report(a.x.status, kSiteGrid | 0x20u | (uint32_t)step); s_ok = 0; break; }
          }
        }
      }
    }
    __syncthreads();
    if (!s_ok) return;
  }
}

}  // namespace

#define S(stream) reinterpret_cast<cudaStream_t>(stream)

extern "C" int nrt_draft_block_input(const int* block_ids, const void* embed, const void* mask, void* x, int hidden,
                                     int rows, int vocab, void* stream, int pdl) {
  return launch_pdl(draft_block_input_kernel, dim3(16), dim3(128), 0, S(stream), pdl != 0, block_ids,
                    (const __nv_bfloat16*)embed, (const __nv_bfloat16*)mask, (__nv_bfloat16*)x, hidden, rows, vocab);
}
extern "C" int nrt_markov_args_size() { return (int)sizeof(MarkovArgs); }
NRT_BOUNDS_EXPORT(draft)
// steps proposals in one launch.  `sync`: two 64-bit words (arrival counter, step generation), zero-initialised once.
extern "C" int nrt_markov_chain(const void* args, int steps, void* sync, void* stream, int pdl) {
  MarkovArgs a;
  memcpy(&a, args, sizeof(a));
  if (a.rank_dim > 512 || a.rank_dim % 64 || steps < 1 || steps > 8 || !sync) return -3;
  const int grid = (a.vlocal + 127) / 128;
  static int resident = -1;
  if (resident < 0) {
    int per_sm = 0, dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, markov_chain_kernel, 256, 0) != cudaSuccess) return -3;
    resident = per_sm * sms;
  }
  if (grid > resident) return -9;                 // the in-grid hand-over needs every CTA resident
  unsigned long long* w = reinterpret_cast<unsigned long long*>(sync);
  return launch_pdl(markov_chain_kernel, dim3(grid), dim3(256), 0, S(stream), pdl != 0, a, steps, w,
                    reinterpret_cast<unsigned int*>(w + 1));
}
extern "C" int nrt_markov_step(const void* args, int step, void* stream, int pdl) {
  MarkovArgs a;
  memcpy(&a, args, sizeof(a));
  if (a.rank_dim > 512 || a.rank_dim % 64) return -3;
  return launch_pdl(markov_step_kernel, dim3((a.vlocal + 127) / 128), dim3(256), 0, S(stream), pdl != 0, a, step);
}

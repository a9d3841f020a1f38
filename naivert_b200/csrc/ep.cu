// Expert-parallel all-to-all for prefill: dispatch fused with RMS-normalised activation
// quantisation and the expert permutation, and the combine (return of expert outputs to the
// token owner, probability-weighted sum + residual), all over peer memory.
//
//   ep_count     every rank histograms its (token, k) -> expert choices, the [ranks x experts] count
//                matrix is exchanged with tagged words, and every rank derives (a) the destination row of
//                each of its (token, k) pairs - rows land *expert-sorted and contiguous* in the expert
//                rank's receive buffer, each expert segment padded to 16 rows - and (b) the work list
//                (expert, first row) of 16-row groups for the grouped GEMM on its own experts.
//   ep_dispatch  one CTA per token: e4m3 + power-of-two scale per 128 channels, then one 4 KiB row + scales
//                + metadata stored straight into the destination rank's receive buffer for each of the
//                token's experts; the last CTA publishes a per-source "dispatch complete" flag to every rank.
//   (grouped block-scaled GEMMs run on the receive buffer: csrc/gemm.cuh, group-item mode)
//   ep_return    epilogue helper of the down projection: bf16 expert outputs are pushed as tagged words
//                into the owner's combine buffer slot (token, k).
//   ep_combine   owner side: waits for the top-k slots of each token, adds them in fixed k order weighted by
//                the routing probability in fp32 on top of the residual.
//
// Reference counterparts: vendored DeepEP intranode dispatch (naivert/prefill/native/deepep.py),
// Triton scatter/permute (naivert/kernels/naive_n0p5/prefill_sglang/), sgl per-token-group fp8 quant, and
// naivert/prefill/native/native_combine.cu (tagged-word combine).
#include "fabric.cuh"
#include "gemm.cuh"
#include "launch.hpp"

#include <string.h>

using namespace nrt;

namespace {

constexpr int kEpMaxExperts = 512;

struct EpArgs {
  // routing of the local tokens
  const int* topk_ids;        // [tokens][top_k] global expert ids
  const float* topk_p;        // [tokens][top_k]
  int tokens, top_k, experts, experts_local, hidden;
  // count outputs (local)
  int* slot_of;               // [tokens*top_k] destination row of each pair
  int* n_items;               // grouped-GEMM work list of this rank's experts
  int* item_expert;           // [max_items] local expert id
  int* item_row;              // [max_items] first row of the item's row group
  int* seg_rows;              // [experts_local] rows received per local expert (unpadded)
  int max_items;
  int cap_rows;               // receive buffer capacity in rows
  // dispatch
  const __nv_bfloat16* x;     // [tokens][hidden] residual rows
  const __nv_bfloat16* gamma; // RMSNorm weight (null: rows are already normalised)
  float eps;
  uint8_t* recv8[kXchgPeers];    // [cap_rows][hidden] e4m3
  float* recvs[kXchgPeers];      // [cap_rows][hidden/128]
  int4* meta[kXchgPeers];        // [cap_rows] {src rank, token, k, tag}
  uint64_t* flags[kXchgPeers];   // [tp] dispatch-complete words
  unsigned int* ticket;
  int call;                      // tag call index of this layer's dispatch
  int item_rows;                 // rows per grouped-GEMM work item and segment padding (16 or 64; 0 = 16)
  XchgArgs x_args;
};

// ----------------------------------------------------------------------------- counts + layout
__global__ void __launch_bounds__(1024) ep_count_kernel(const EpArgs a) {
  __shared__ unsigned int hist[kEpMaxExperts + 1];
  __shared__ uint64_t xv[kXchgMaxWords];          // [tp][experts]
  __shared__ int seg_base[kEpMaxExperts + 1];
  griddep_wait();
  griddep_launch();
  const int tp = a.x_args.tp, rank = a.x_args.rank;
  const int n = a.tokens * a.top_k;
  const int ir = a.item_rows > 0 ? a.item_rows : 16;
  for (int i = threadIdx.x; i < a.experts; i += 1024) hist[i] = 0u;
  for (int i = threadIdx.x; i < tp * a.experts; i += 1024) xv[i] = 0ull;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += 1024) atomicAdd(&hist[a.topk_ids[i]], 1u);
  __syncthreads();
  for (int e = threadIdx.x; e < a.experts; e += 1024) xv[rank * a.experts + e] = hist[e];
  __syncthreads();
  xchg_reduce_u64<kXSum>(xv, tp * a.experts, a.x_args, 32 + (a.call & 15));
  // padded segment bases on every destination rank (all ranks compute the same table)
  if (threadIdx.x < tp) {
    const int d = threadIdx.x;
    int base = 0;
    for (int el = 0; el < a.experts_local; ++el) {
      const int e = d * a.experts_local + el;
      int rows = 0;
      for (int s = 0; s < tp; ++s) rows += (int)xv[s * a.experts + e];
      seg_base[e] = base;
      base += (rows + ir - 1) / ir * ir;
    }
  }
  __syncthreads();
  // destination row of each local (token, k): segment base + rows of lower ranks + stable local rank.
  // `hist` becomes the running count per expert; pairs are ranked in index order: chunks of 1024 in order,
  // warps of a chunk in order, lanes of a warp by their position among equal experts.
  for (int e = threadIdx.x; e < a.experts; e += 1024) {
    int pos = seg_base[e];
    for (int s = 0; s < rank; ++s) pos += (int)xv[s * a.experts + e];
    hist[e] = (unsigned)pos;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (a.experts <= 256 && tp * a.experts <= kXchgMaxWords / 2) {
    // Every warp owns one contiguous range of the pairs.  Pass 1 counts the range's pairs per expert (warp-private
    // row of 16-bit counters), a prefix over the warps turns the counts into each range's offset inside the expert's
    // segment, pass 2 walks the range in index order and hands out rows.  Same stable order as ranking the pairs one
    // by one (lower index first), with three block barriers instead of two thousand.
    // (the counters live in the unused upper half of the exchange buffer: 32 x 256 x 2 bytes)
    unsigned short (*wc)[256] = reinterpret_cast<unsigned short (*)[256]>(xv + kXchgMaxWords / 2);
    for (int i = threadIdx.x; i < 32 * 256; i += 1024) (&wc[0][0])[i] = 0;
    __syncthreads();
    const int per = (n + 31) / 32;
    const int lo = warp * per, hi = min(n, lo + per);
    for (int i0 = lo; i0 < hi; i0 += 32) {
      const int i = i0 + lane;
      const int e = i < hi ? a.topk_ids[i] : -1;
      const unsigned peers = __match_any_sync(0xffffffffu, e);
      if (e >= 0 && (peers & ((1u << lane) - 1u)) == 0u) wc[warp][e] += (unsigned short)__popc(peers);
      __syncwarp();
    }
    __syncthreads();
    if ((int)threadIdx.x < a.experts) {
      unsigned run = 0;
      for (int w = 0; w < 32; ++w) { const unsigned t = wc[w][threadIdx.x]; wc[w][threadIdx.x] = (unsigned short)run; run += t; }
    }
    __syncthreads();
    for (int i0 = lo; i0 < hi; i0 += 32) {
      const int i = i0 + lane;
      const int e = i < hi ? a.topk_ids[i] : -1;
      const unsigned peers = __match_any_sync(0xffffffffu, e);
      const int below = __popc(peers & ((1u << lane) - 1u));
      if (e >= 0) {
        unsigned base = 0;
        if (below == 0) { base = hist[e] + wc[warp][e]; wc[warp][e] += (unsigned short)__popc(peers); }
        base = __shfl_sync(peers, base, __ffs(peers) - 1);
        a.slot_of[i] = (int)base + below;
      }
      __syncwarp();
    }
    __syncthreads();
  } else
  for (int c0 = 0; c0 < n; c0 += 1024) {
    const int i = c0 + threadIdx.x;
    const int e = i < n ? a.topk_ids[i] : -1;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int below = __popc(peers & ((1u << lane) - 1u));
    const bool lead = below == 0;
    for (int w = 0; w < 32; ++w) {
      if (warp == w && e >= 0) {
        unsigned base = 0;
        if (lead) { base = hist[e]; hist[e] = base + __popc(peers); }
        base = __shfl_sync(peers, base, __ffs(peers) - 1);
        a.slot_of[i] = (int)base + below;
      }
      __syncthreads();
    }
  }
  // work list of my own experts: one thread per local expert counts its row groups, a prefix over the experts gives
  // each its first item, then every thread writes its own items (same list as a sequential walk over the experts)
  {
    int* first_item = reinterpret_cast<int*>(hist);          // hist is free again: [experts_local + 1]
    int my_rows = 0, my_items = 0;
    const int el = threadIdx.x;
    if (el < a.experts_local) {
      const int e = rank * a.experts_local + el;
      for (int s = 0; s < tp; ++s) my_rows += (int)xv[s * a.experts + e];
      a.seg_rows[el] = my_rows;
      my_items = (my_rows + ir - 1) / ir;
    }
    __syncthreads();                                          // everybody is done with hist as running positions
    if (el < a.experts_local) first_item[el + 1] = my_items;
    if (el == 0) first_item[0] = 0;
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int i = 0; i < a.experts_local; ++i) first_item[i + 1] += first_item[i];
      *a.n_items = first_item[a.experts_local] < a.max_items ? first_item[a.experts_local] : a.max_items;
    }
    __syncthreads();
    if (el < a.experts_local) {
      const int e = rank * a.experts_local + el;
      for (int k = 0; k < my_items; ++k) {
        const int idx = first_item[el] + k;
        if (idx < a.max_items) { a.item_expert[idx] = el; a.item_row[idx] = seg_base[e] + k * ir; }
      }
    }
  }
}

__device__ __forceinline__ uint8_t e4m3_of(float v) {
  const __nv_fp8_e4m3 q(v);
  return *reinterpret_cast<const uint8_t*>(&q);
}

// ----------------------------------------------------------------------------- dispatch
// One CTA (256 threads) per local token.
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const EpArgs a) {
  __shared__ float red[8];
  __shared__ bool s_last;
  griddep_wait();
  griddep_launch();
  const int t = blockIdx.x;
  const int per = a.hidden / 8;
  const int tp = a.x_args.tp, rank = a.x_args.rank;
  const uint32_t tag = (*a.x_args.epoch) * 1024u + (uint32_t)a.call + 1u;
  const uint4* src = reinterpret_cast<const uint4*>(a.x + (size_t)t * a.hidden);
  float rs = 1.f;
  if (a.gamma) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < per; i += 256) {
      const uint4 v = src[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); ss += f.x * f.x + f.y * f.y; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    ss = 0.f;
    for (int i = 0; i < 8; ++i) ss += red[i];
    rs = rsqrtf(ss / (float)a.hidden + a.eps);
  }
  for (int i = threadIdx.x; i < per; i += 256) {
    const uint4 v = src[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    float o[8];
    float am = 0.f;
    if (a.gamma) {
      const uint4 gv = reinterpret_cast<const uint4*>(a.gamma)[i];
      const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]), g = __bfloat1622float2(gh[j]);
        o[2 * j] = round_bf16(f.x * rs * g.x);
        o[2 * j + 1] = round_bf16(f.y * rs * g.y);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); o[2 * j] = f.x; o[2 * j + 1] = f.y; }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) am = fmaxf(am, fabsf(o[j]));
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, off));
    const float sc = pow2_scale(am);
    uint2 q;
    uint8_t* qb = reinterpret_cast<uint8_t*>(&q);
#pragma unroll
    for (int j = 0; j < 8; ++j) qb[j] = e4m3_of(o[j] / sc);
    for (int k = 0; k < a.top_k; ++k) {
      const int e = a.topk_ids[t * a.top_k + k];
      const int d = e / a.experts_local;
      const int row = a.slot_of[t * a.top_k + k];
      if (row >= a.cap_rows) continue;
      reinterpret_cast<uint2*>(a.recv8[d] + (size_t)row * a.hidden)[i] = q;
      if ((i & 15) == 0) a.recvs[d][(size_t)row * (a.hidden / 128) + (i >> 4)] = sc;
    }
  }
  if (threadIdx.x < a.top_k) {
    const int k = threadIdx.x;
    const int e = a.topk_ids[t * a.top_k + k];
    const int row = a.slot_of[t * a.top_k + k];
    if (row < a.cap_rows) a.meta[e / a.experts_local][row] = make_int4(rank, t, k, (int)tag);
  }
  // last CTA: everything this rank sends is out -> publish the flag on every rank
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int tk = atomicAdd(a.ticket, 1u);
    s_last = tk == gridDim.x - 1;
    if (s_last) *a.ticket = 0u;
  }
  __syncthreads();
  if (s_last && threadIdx.x < tp) {
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    st_tagged(a.flags[threadIdx.x] + rank, tag, 1u);
  }
}

// ----------------------------------------------------------------------------- combine (owner side)
struct EpCombineArgs {
  const uint64_t* slots;      // [tokens*top_k][hidden/2] tagged words {tag, bf16x2}
  const float* topk_p;        // [tokens][top_k]
  const __nv_bfloat16* resid; // [tokens][hidden]
  __nv_bfloat16* out;         // [tokens][hidden]
  const uint32_t* epoch;
  uint32_t* status;
  int tokens, top_k, hidden, call;
  unsigned long long timeout_ns;
};

__global__ void __launch_bounds__(256) ep_combine_kernel(const EpCombineArgs a) {
  griddep_wait();
  griddep_launch();
  const int t = blockIdx.x;
  const uint32_t tag = (*a.epoch) * 1024u + (uint32_t)a.call + 1u;
  const int words = a.hidden / 2;
  const uint64_t deadline = globaltimer() + a.timeout_ns;
  for (int w = threadIdx.x; w < words; w += 256) {
    const float2 r = __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(a.resid + (size_t)t * a.hidden)[w]);
    float lo = r.x, hi = r.y;
    bool ok = true;
    for (int k = 0; k < a.top_k && ok; ++k) {                 // fixed k order
      uint32_t v;
      ok = wait_tagged(a.slots + ((size_t)(t * a.top_k + k)) * words + w, tag, v, deadline, a.status, kSiteMailbox | 0x80 | (uint32_t)k);
      const float p = a.topk_p[t * a.top_k + k];
      lo += p * bf16_lo(v);
      hi += p * bf16_hi(v);
    }
    reinterpret_cast<__nv_bfloat162*>(a.out + (size_t)t * a.hidden)[w] = __floats2bfloat162_rn(lo, hi);
  }
}

}  // namespace

#define S(stream) reinterpret_cast<cudaStream_t>(stream)
extern "C" int nrt_ep_args_size() { return (int)sizeof(EpArgs); }
extern "C" int nrt_ep_combine_args_size() { return (int)sizeof(EpCombineArgs); }
extern "C" int nrt_ep_count(const void* args, void* stream, int pdl) {
  EpArgs a;
  memcpy(&a, args, sizeof(a));
  if (a.experts > kEpMaxExperts || a.x_args.tp * a.experts > kXchgMaxWords) return -3;
  return launch_pdl(ep_count_kernel, dim3(1), dim3(1024), 0, S(stream), pdl != 0, a);
}
extern "C" int nrt_ep_dispatch(const void* args, void* stream, int pdl) {
  EpArgs a;
  memcpy(&a, args, sizeof(a));
  if (a.hidden % 256 || a.top_k > 32) return -3;
  return launch_pdl(ep_dispatch_kernel, dim3(a.tokens), dim3(256), 0, S(stream), pdl != 0, a);
}
extern "C" int nrt_ep_combine(const void* args, void* stream, int pdl) {
  EpCombineArgs a;
  memcpy(&a, args, sizeof(a));
  return launch_pdl(ep_combine_kernel, dim3(a.tokens), dim3(256), 0, S(stream), pdl != 0, a);
}

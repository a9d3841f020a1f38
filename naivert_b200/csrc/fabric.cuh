// Small-message exchange over the peer-memory fabric: every rank pushes its values to every
// peer as tagged words and combines the tp contributions locally (integers: order-free; the
// float variants combine in rank order); many values go through a reduce-scatter form in which
// each group of values has one owning rank.  Used by the sampler, the draft head and the tail
// for maxima, integer masses, histograms and token broadcasts.  All waits are bounded.
//
// Reference counterpart: the per-stage rendezvous and tagged inbox exchange of
// naivert/body/dspark_sampling/{sharded,persistent}.cuh and naivert/body/dspark_common/rendezvous.cuh.
#pragma once
#include "ptx.cuh"

namespace nrt {

constexpr int kXchgMaxWords = 4096;     // 64-bit values per exchange
constexpr int kXchgSlabs = 4;
constexpr int kXchgPeers = 8;

struct XchgArgs {
  uint64_t* box[kXchgPeers];   // box[p] = rank p's exchange region (peer mapped); box[rank] is local
  const uint32_t* epoch;
  uint32_t* status;
  int tp;
  int rank;
  unsigned long long timeout_ns;
};

enum XchgOp : int { kXSum = 0, kXMax = 1 };

// Collects kVB values of this thread from every peer's slot of the local box: vals[idx[b]] (idx < 0: none) becomes the
// reduction of the local value with the tp - 1 words pairs tagged `tag`.  All outstanding words of the kVB values are
// requested before any answer is examined - the guards test a snapshot of the masks - so the loads of a sweep overlap
// instead of each waiting for the previous comparison.  Bounded: gives up at `deadline` or when the status word is set.
template <int OP, int kVB>
__device__ __forceinline__ bool xchg_collect(uint64_t* vals, const int (&idx)[kVB], const XchgArgs& x, uint32_t tag, size_t slab,
                                             int call, uint64_t deadline) {
  bool ok = true;
  uint32_t lo[kVB][kXchgPeers], hi[kVB][kXchgPeers];
  uint32_t need[kVB], any = 0u;
#pragma unroll
  for (int b = 0; b < kVB; ++b) {
    need[b] = 0u;
#pragma unroll
    for (int s = 0; s < kXchgPeers; ++s) {
      lo[b][s] = hi[b][s] = 0u;
      if (idx[b] >= 0 && s < x.tp && s != x.rank) need[b] |= 3u << (2 * s);
    }
    any |= need[b];
  }
  for (uint32_t sweep = 0; any != 0u; ++sweep) {
    uint32_t snap[kVB], t[kVB][2 * kXchgPeers], v[kVB][2 * kXchgPeers];
#pragma unroll
    for (int b = 0; b < kVB; ++b) {
      snap[b] = need[b];
      const uint64_t* base = x.box[x.rank] + (slab * kXchgMaxWords + (size_t)max(idx[b], 0)) * 2;
#pragma unroll
      for (int q = 0; q < 2 * kXchgPeers; ++q) {
        t[b][q] = ~tag;
        v[b][q] = 0u;
        if (snap[b] & (1u << q)) ld_tagged(base + (size_t)(q >> 1) * kXchgMaxWords * 2 + (q & 1), t[b][q], v[b][q]);
      }
    }
    any = 0u;
#pragma unroll
    for (int b = 0; b < kVB; ++b) {
#pragma unroll
      for (int q = 0; q < 2 * kXchgPeers; ++q)
        if ((snap[b] & (1u << q)) && t[b][q] == tag) {
          if (q & 1) hi[b][q >> 1] = v[b][q]; else lo[b][q >> 1] = v[b][q];
          need[b] &= ~(1u << q);
        }
      any |= need[b];
    }
    if ((sweep & 255u) == 255u) {
      if (*reinterpret_cast<volatile uint32_t*>(x.status) != 0u) { ok = false; break; }
      if (globaltimer() > deadline) { report(x.status, kSiteRendezvous | (uint32_t)call); ok = false; break; }
    }
  }
#pragma unroll
  for (int b = 0; b < kVB; ++b) {
    if (idx[b] >= 0) {
      uint64_t acc = vals[idx[b]];
#pragma unroll
      for (int s = 0; s < kXchgPeers; ++s) {
        if (s < x.tp && s != x.rank) {
          const uint64_t o = ((uint64_t)hi[b][s] << 32) | lo[b][s];
          acc = OP == kXSum ? acc + o : (o > acc ? o : acc);
        }
      }
      vals[idx[b]] = acc;
    }
  }
  return ok;
}

// Called by all threads of ONE CTA.  vals[0..n) (shared or global, local to this rank) are
// replaced by the reduction over ranks.  `call` must be unique inside one epoch (< 64).  Consecutive calls of a rank
// must use different slabs (call % kXchgSlabs): a peer may already push the next call's words while this rank still
// polls the current one.  kVB values of a thread are polled together (costs registers).
template <int OP, int kVB = 1>
__device__ __forceinline__ bool xchg_reduce_u64(uint64_t* vals, int n, const XchgArgs& x, int call) {
  if (x.tp <= 1) return true;
  const uint32_t tag = (*x.epoch) * 64u + (uint32_t)call + 1u;
  const size_t slab = (size_t)(call % kXchgSlabs) * x.tp;
  bool ok = true;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const uint64_t v = vals[i];
    for (int d = 1; d < x.tp; ++d) {
      const int peer = (x.rank + d) % x.tp;
      uint64_t* dst = x.box[peer] + ((slab + x.rank) * kXchgMaxWords + i) * 2;
      st_tagged(dst, tag, (uint32_t)v);
      st_tagged(dst + 1, tag, (uint32_t)(v >> 32));
    }
  }
  const uint64_t deadline = globaltimer() + x.timeout_ns;
  for (int i0 = threadIdx.x; i0 < n && ok; i0 += kVB * blockDim.x) {
    int idx[kVB];
#pragma unroll
    for (int b = 0; b < kVB; ++b) idx[b] = i0 + b * (int)blockDim.x < n ? i0 + b * (int)blockDim.x : -1;
    ok = xchg_collect<OP, kVB>(vals, idx, x, tag, slab, call, deadline);
  }
  __syncthreads();
  return ok;
}

// Reduce-scatter form for many values: vals holds `groups` groups of `gsize` values; group g is owned by rank
// g % tp.  Every rank pushes the values of the live groups (bit g of `live`) it does not own to their owners only -
// 1/tp of the stores of the all-to-all form - and afterwards an owner's groups hold the sums over ranks; the groups of
// other owners keep the local values.  Same slab rule as xchg_reduce_u64.
template <int kVB>
__device__ __forceinline__ bool xchg_reduce_scatter_u64(uint64_t* vals, int groups, int gsize, uint32_t live, const XchgArgs& x,
                                                        int call) {
  if (x.tp <= 1) return true;
  const uint32_t tag = (*x.epoch) * 64u + (uint32_t)call + 1u;
  const size_t slab = (size_t)(call % kXchgSlabs) * x.tp;
  for (int g = 0; g < groups; ++g) {
    const int owner = g % x.tp;
    if (owner == x.rank || !((live >> g) & 1u)) continue;
    for (int t = threadIdx.x; t < gsize; t += blockDim.x) {
      const int i = g * gsize + t;
      const uint64_t v = vals[i];
      uint64_t* dst = x.box[owner] + ((slab + x.rank) * kXchgMaxWords + i) * 2;
      st_tagged(dst, tag, (uint32_t)v);
      st_tagged(dst + 1, tag, (uint32_t)(v >> 32));
    }
  }
  const uint64_t deadline = globaltimer() + x.timeout_ns;
  bool ok = true;
  for (int t = threadIdx.x; t < gsize; t += blockDim.x) {
    for (int g0 = x.rank; g0 < groups && ok; g0 += kVB * x.tp) {
      int idx[kVB];
#pragma unroll
      for (int b = 0; b < kVB; ++b) {
        const int g = g0 + b * x.tp;
        idx[b] = (g < groups && ((live >> g) & 1u)) ? g * gsize + t : -1;
      }
      ok = xchg_collect<kXSum, kVB>(vals, idx, x, tag, slab, call, deadline);
    }
  }
  __syncthreads();
  return ok;
}

// order-preserving map float -> uint32 (so a max over uints is a max over floats)
__device__ __forceinline__ uint32_t float_order(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float float_unorder(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}

// Philox4x32-10; uniform in (0, 1) from (seed, domain, a, b)
__host__ __device__ inline uint32_t philox_u32(uint64_t seed, uint32_t domain, uint32_t a, uint32_t b) {
  uint32_t c0 = domain, c1 = a, c2 = b, c3 = 0;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
    const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
    const uint32_t n1 = (uint32_t)p1;
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
    const uint32_t n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c0;
}
__host__ __device__ inline float philox_uniform(uint64_t seed, uint32_t domain, uint32_t a, uint32_t b) {
  return ((philox_u32(seed, domain, a, b) >> 9) + 0.5f) * (1.0f / 8388608.0f);   // 23 bits + 1/2: exact in fp32
}

}  // namespace nrt

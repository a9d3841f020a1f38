// Vocabulary-sharded speculative sampler, verify and tail commit.
//
// Every distribution is handled in *integer masses*: after the exact row maximum m is known
// on all ranks, e(t) = rint(exp(z(t) - m) * 2^31) is a 32-bit integer per token.  Sums of
// integers do not depend on summation order, so the nucleus threshold, the normaliser, the
// accept test and the inverse-CDF draw are bit-identical from run to run and identical for
// every tensor-parallel degree.
//
//   z      = penalised logit / T
//   e      = rint(exp(z - max z) * 2^31)
//   nucleus: the largest threshold tau with  sum_{e >= tau} e  >=  top_p * sum e  (radix select
//            over the 32-bit codes, four 8-bit passes on mass histograms); kept = {e >= tau}, Z = kept mass
//   accept draft token d_j  iff  u * q'(d_j) < p'(d_j),  p' = e_p/Z_p on the kept set (0 outside)
//   first rejection at row m: draw from max(p' - q', 0) in vocabulary order; all accepted: draw from p' of the last row
//   forced mode: the accept decision of every position is replaced by a seeded Bernoulli(p_force) draw
//
// Rows 0..7 are the target distributions, rows 8..14 the draft distributions.
// Reference: naivert/body/dspark_sampling/{sharded,persistent,parallel}.cuh (math),
// random.cuh (Philox domains), naivert/body/dspark_tail/{body,commit}.cuh (accept prefix, commit).
#include "contract.h"
#include "fabric.cuh"
#include "launch.hpp"

#include <string.h>

using namespace nrt;

namespace {

constexpr int kRowsP = 8, kRowsQ = 7, kDist = kRowsP + kRowsQ;
constexpr int kTile = 2048;                 // vocabulary entries per CTA
constexpr int kThreads = 256;
constexpr int kPer = kTile / kThreads;      // vocabulary entries per thread and tile

enum Domain : uint32_t { kDomAccept = 0, kDomResample = 1, kDomForced = 2, kDomDraft = 3, kDomAnchor = 4 };

struct SamplerState {          // device-resident scratch of one rank
  float rowmax[16];
  unsigned long long total[16];      // sum of e
  unsigned long long above[16];      // mass strictly above the current prefix bin
  unsigned long long kept[16];       // Z (valid after the last pass)
  unsigned int prefix[16];           // threshold code tau (valid after the last pass)
  unsigned long long hist[kDist * 256];
  unsigned long long tile_mass[16 * 128];   // per-tile masses of the row being resampled (<= 128 tiles... see launcher)
  unsigned int ticket[8];
  int accepted;                      // m: accepted draft tokens (0..7)
  int extra_token;                   // resampled / bonus token
  int accept_flags[8];
};

struct SamplerArgs {
  const float* zp;             // target logits [16][ldp]
  int ldp;
  const float* zq;             // draft logits (+ Markov bias) [8][ldq]
  int ldq;
  int vlocal;                  // vocabulary entries of this rank
  int vbase;                   // first global token id of this rank
  unsigned int* e;             // [kDist][vlocal] integer codes
  const unsigned short* counts;   // [vlocal] occurrences of each token in the context (penalties) or null
  const float* params;         // [8]: inv_T, top_p, rep_penalty, freq_penalty, pres_penalty, forced_p (<0: off), inv_T_draft
  const unsigned long long* seed;
  const int* ctrl;             // control block (round counter at [8])
  const int* block_ids;        // [8]: anchor + 7 proposals
  int n_rows_p, n_rows_q;      // 8,7 for a round; 1,0 for the anchor sample
  SamplerState* st;
  XchgArgs x;
  // opt-in phase stamps of the single-launch sampler (%globaltimer, ns), [32]: word 2p = the last CTA of phase p has
  // arrived, 2p + 1 = phase p released (phases: 0 maxima, 1 codes, 2..5 nucleus passes (+ accept after the last),
  // 6 tile masses / draw done); word 30 = kernel entry of CTA (0, 0).  Null: none.
  unsigned long long* stamps;
};

__device__ __forceinline__ float penalised(const SamplerArgs& a, const float* params, float z, int t) {
  if (a.counts) {
    const float c = (float)a.counts[t];
    if (c > 0.f) {
      const float rp = params[2];
      z = z > 0.f ? z / rp : z * rp;
      z -= params[3] * c + params[4];
    }
  }
  return z;
}
__device__ __forceinline__ const float* row_logits(const SamplerArgs& a, int d, float& inv_t) {
  if (d < kRowsP) { inv_t = a.params[0]; return a.zp + (size_t)d * a.ldp; }
  inv_t = a.params[6];
  return a.zq + (size_t)(d - kRowsP) * a.ldq;
}
__device__ __forceinline__ bool row_active(const SamplerArgs& a, int d) {
  return d < kRowsP ? d < a.n_rows_p : (d - kRowsP) < a.n_rows_q;
}

// ticket: true for the last CTA of the grid to arrive (and resets the counter)
__device__ __forceinline__ bool last_block(unsigned int* ticket) {
  __shared__ bool s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int total = gridDim.x * gridDim.y;
    const unsigned int t = atomicAdd(ticket, 1u);
    s_last = (t == total - 1);
    if (s_last) *ticket = 0u;
  }
  __syncthreads();
  __threadfence();
  return s_last;
}

// State written by another CTA inside one launch (persistent form) must not come from a stale L1 line.
template <typename T>
__device__ __forceinline__ T ldg2(const T* p) { return __ldcg(p); }

// 64-bit shared-memory atomics are compare-and-swap loops: 256 threads adding to one word serialise for microseconds.
// Sums are therefore folded inside the warp first and one lane per warp touches shared memory.
__device__ __forceinline__ unsigned long long warp_sum_u64(unsigned long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---------------------------------------------------------------- pass A: row maxima
__device__ __forceinline__ void work_max(const SamplerArgs& a, int bx, int d) {
  __shared__ unsigned int smax;
  if (threadIdx.x == 0) smax = 0u;
  __syncthreads();
  if (row_active(a, d)) {
    float inv_t;
    const float* z = row_logits(a, d, inv_t);
    unsigned int best = 0u;
    const int t0 = bx * kTile;
    // a thread's eight entries are requested together (one memory round trip instead of eight)
    float zv[kPer];
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int t = t0 + threadIdx.x + j * kThreads;
      zv[j] = t < a.vlocal ? z[t] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int t = t0 + threadIdx.x + j * kThreads;
      if (t < a.vlocal) {
        float v = d < kRowsP ? penalised(a, a.params, zv[j], t) : zv[j];
        best = max(best, float_order(__fmul_rn(v, inv_t)));
      }
    }
    atomicMax(&smax, best);
    __syncthreads();
    if (threadIdx.x == 0) atomicMax(reinterpret_cast<unsigned int*>(&a.st->hist[d]), smax);   // hist[] doubles as scratch
  }
}
__device__ __forceinline__ void post_max(const SamplerArgs& a, uint64_t* xv) {
  if (threadIdx.x < 16) {
    const unsigned int v = threadIdx.x < kDist ? *reinterpret_cast<volatile unsigned int*>(&a.st->hist[threadIdx.x]) : 0u;
    xv[threadIdx.x] = v;
  }
  __syncthreads();
  xchg_reduce_u64<kXMax>(xv, 16, a.x, 0);
  if (threadIdx.x < 16) {
    a.st->rowmax[threadIdx.x] = float_unorder((uint32_t)xv[threadIdx.x]);
    a.st->hist[threadIdx.x] = 0ull;
    a.st->total[threadIdx.x] = 0ull;
  }
}
__global__ void __launch_bounds__(kThreads) samp_max_kernel(const SamplerArgs a) {
  __shared__ uint64_t xv[16];
  griddep_wait();
  griddep_launch();
  work_max(a, blockIdx.x, blockIdx.y);
  if (!last_block(&a.st->ticket[0])) return;
  post_max(a, xv);
}

// ---------------------------------------------------------------- pass B: integer codes + totals
__device__ __forceinline__ void work_exp(const SamplerArgs& a, int bx, int d) {
  __shared__ unsigned long long ssum;
  if (threadIdx.x == 0) ssum = 0ull;
  __syncthreads();
  if (row_active(a, d)) {
    float inv_t;
    const float* z = row_logits(a, d, inv_t);
    const float m = ldg2(&a.st->rowmax[d]);
    unsigned long long acc = 0ull;
    const int t0 = bx * kTile;
    float zv[kPer];
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int t = t0 + threadIdx.x + j * kThreads;
      zv[j] = t < a.vlocal ? z[t] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int t = t0 + threadIdx.x + j * kThreads;
      if (t < a.vlocal) {
        float v = d < kRowsP ? penalised(a, a.params, zv[j], t) : zv[j];
        const unsigned int e = (unsigned int)rintf(expf(__fsub_rn(__fmul_rn(v, inv_t), m)) * 2147483648.0f);
        a.e[(size_t)d * a.vlocal + t] = e;
        acc += e;
      }
    }
    acc = warp_sum_u64(acc);
    if ((threadIdx.x & 31) == 0) atomicAdd(&ssum, acc);
    __syncthreads();
    if (threadIdx.x == 0) atomicAdd(&a.st->total[d], ssum);
  }
}
__device__ __forceinline__ void post_exp(const SamplerArgs& a, uint64_t* xv) {
  if (threadIdx.x < 16) xv[threadIdx.x] = *reinterpret_cast<volatile unsigned long long*>(&a.st->total[threadIdx.x]);
  __syncthreads();
  xchg_reduce_u64<kXSum>(xv, 16, a.x, 1);
  if (threadIdx.x < 16) {
    a.st->total[threadIdx.x] = xv[threadIdx.x];
    a.st->above[threadIdx.x] = 0ull;
    a.st->prefix[threadIdx.x] = 0u;
  }
  for (int i = threadIdx.x; i < kDist * 256; i += kThreads) a.st->hist[i] = 0ull;
}
__global__ void __launch_bounds__(kThreads) samp_exp_kernel(const SamplerArgs a) {
  __shared__ uint64_t xv[16];
  griddep_wait();
  griddep_launch();
  work_exp(a, blockIdx.x, blockIdx.y);
  if (!last_block(&a.st->ticket[1])) return;
  post_exp(a, xv);
}

// ---------------------------------------------------------------- passes C0..C3: nucleus radix select
__device__ __forceinline__ void work_hist(const SamplerArgs& a, int bx, int d, int pass) {
  // Bin sums are kept as two 32-bit words (low / high 16 bits of the codes: a tile's sums fit) because 32-bit
  // shared-memory atomics are native while 64-bit ones are compare-and-swap loops.
  __shared__ unsigned int sh_lo[256], sh_hi[256];
  const int shift = 24 - 8 * pass;
  const unsigned int mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
  for (int i = threadIdx.x; i < 256; i += kThreads) { sh_lo[i] = 0u; sh_hi[i] = 0u; }
  __syncthreads();
  if (row_active(a, d)) {
    const unsigned int prefix = ldg2(&a.st->prefix[d]);
    const unsigned int* e = a.e + (size_t)d * a.vlocal;
    const int t0 = bx * kTile;
    unsigned int ev[kPer];
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const int t = t0 + threadIdx.x + j * kThreads;
      ev[j] = t < a.vlocal ? __ldcg(e + t) : 0u;
    }
    // In the first pass nearly all codes of a warp fall into one bin (tiny probabilities): then the warp adds once.
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
      const unsigned int v = ev[j];
      const bool in = (v & mask) == prefix && v != 0u;
      const unsigned int bin = in ? (v >> shift) & 255u : 0xFFFFFFFFu;
      const unsigned int b0 = __shfl_sync(0xffffffffu, bin, 0);
      if (__all_sync(0xffffffffu, bin == b0)) {
        if (b0 != 0xFFFFFFFFu) {
          const unsigned int lo = __reduce_add_sync(0xffffffffu, v & 0xFFFFu), hi = __reduce_add_sync(0xffffffffu, v >> 16);
          if ((threadIdx.x & 31) == 0) { atomicAdd(&sh_lo[b0], lo); atomicAdd(&sh_hi[b0], hi); }
        }
      } else if (in) {
        atomicAdd(&sh_lo[bin], v & 0xFFFFu);
        atomicAdd(&sh_hi[bin], v >> 16);
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 256; i += kThreads) {
      const unsigned long long tot = ((unsigned long long)sh_hi[i] << 16) + sh_lo[i];
      if (tot) atomicAdd(&a.st->hist[d * 256 + i], tot);
    }
  }
}
__device__ __forceinline__ void post_hist(const SamplerArgs& a, uint64_t* xv, int pass) {
  // The 256 bins of a distribution are summed over ranks at ONE rank (distribution r at rank r mod tp), which finds
  // the threshold digit and tells everybody the three numbers that come out of it: the all-to-all form would push
  // tp times as many words through one CTA.
  __shared__ uint64_t res[48];                       // [r] suffix mass at the digit, [16 + r] mass of its bin, [32 + r] digit
  const int shift = 24 - 8 * pass;
  const int tp = a.x.tp > 1 ? a.x.tp : 1, rank = a.x.tp > 1 ? a.x.rank : 0;
  uint32_t live = 0u;
#pragma unroll
  for (int j = 0; j < kDist; ++j) {                  // fifteen independent L2 loads per thread, in flight together
    xv[threadIdx.x + j * kThreads] = __ldcg(reinterpret_cast<const unsigned long long*>(&a.st->hist[threadIdx.x + j * kThreads]));
    live |= row_active(a, j) ? 1u << j : 0u;
  }
  if (threadIdx.x < 48) res[threadIdx.x] = 0ull;
  __syncthreads();
  xchg_reduce_scatter_u64<2>(xv, kDist, 256, live, a.x, 2 + 2 * pass);
  // Threshold digit of every distribution: the largest bin b >= 1 whose suffix sum S(b) = sum of bins >= b reaches
  // the target (bin 0 when none does).  One warp per distribution; a lane holds eight bins and their suffix sums.
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = warp; r < kDist; r += kThreads / 32) {
    if (!((live >> r) & 1u) || r % tp != rank) continue;                // uniform over the warp
    const double top_p = (double)a.params[1];
    const unsigned long long target = (unsigned long long)ceil(top_p * (double)ldg2(&a.st->total[r]));
    const unsigned long long above = ldg2(&a.st->above[r]);
    unsigned long long bin[8], suf[8];
    unsigned long long mine = 0ull;
#pragma unroll
    for (int i = 7; i >= 0; --i) { bin[i] = xv[r * 256 + lane * 8 + i]; mine += bin[i]; suf[i] = mine; }   // suffix inside the lane
    unsigned long long higher = mine;                                  // inclusive suffix over lanes, then made exclusive
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long v = __shfl_down_sync(0xffffffffu, higher, o);
      if (lane + o < 32) higher += v;
    }
    higher -= mine;
    int cand = -1;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (lane * 8 + i >= 1 && above + higher + suf[i] >= target) cand = lane * 8 + i;      // ascending i keeps the largest
    const int b = max(0, (int)__reduce_max_sync(0xffffffffu, cand));
    const int owner = b >> 3;
    unsigned long long cum = 0ull, in_bin = 0ull;
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i == (b & 7)) { cum = higher + suf[i]; in_bin = bin[i]; }
    cum = __shfl_sync(0xffffffffu, cum, owner);
    in_bin = __shfl_sync(0xffffffffu, in_bin, owner);
    if (lane == 0) { res[r] = cum; res[16 + r] = in_bin; res[32 + r] = (unsigned long long)b; }
  }
  __syncthreads();
  xchg_reduce_u64<kXSum>(res, 48, a.x, 3 + 2 * pass);   // every entry has one non-zero contributor
  if (threadIdx.x < kDist && ((live >> threadIdx.x) & 1u)) {
    const int r = threadIdx.x;
    const unsigned long long above = ldg2(&a.st->above[r]);
    a.st->above[r] = above + res[r] - res[16 + r];
    a.st->prefix[r] = ldg2(&a.st->prefix[r]) | ((unsigned int)res[32 + r] << shift);
    if (pass == 3) a.st->kept[r] = above + res[r];     // Z: everything with e >= tau
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < kDist; ++j) a.st->hist[threadIdx.x + j * kThreads] = 0ull;
}
__global__ void __launch_bounds__(kThreads) samp_hist_kernel(const SamplerArgs a, int pass) {
  __shared__ uint64_t xv[kDist * 256];
  griddep_wait();
  griddep_launch();
  work_hist(a, blockIdx.x, blockIdx.y, pass);
  if (!last_block(&a.st->ticket[2])) return;
  post_hist(a, xv, pass);
}

// ---------------------------------------------------------------- verify: accept prefix
// One CTA.  Gathers e_p(d_j), e_q(d_j) from the owning ranks, decides acceptance.
__device__ __forceinline__ void do_accept(const SamplerArgs& a, uint64_t* xv) {
  const int j = threadIdx.x;                  // proposal j+1 is judged by target row j / draft row j
  if (j < 16) xv[j] = 0ull;
  __syncthreads();
  if (j < a.n_rows_q) {
    const int tok = a.block_ids[j + 1] - a.vbase;
    if (tok >= 0 && tok < a.vlocal) {
      unsigned int ep = ldg2(&a.e[(size_t)j * a.vlocal + tok]);
      unsigned int eq = ldg2(&a.e[(size_t)(kRowsP + j) * a.vlocal + tok]);
      if (ep < ldg2(&a.st->prefix[j])) ep = 0u;
      if (eq < ldg2(&a.st->prefix[kRowsP + j])) eq = 0u;
      xv[j] = ((uint64_t)ep << 32) | eq;
    }
  }
  __syncthreads();
  xchg_reduce_u64<kXSum>(xv, 8, a.x, 10);
  if (threadIdx.x == 0) {
    const unsigned long long seed = *a.seed;
    const uint32_t round = (uint32_t)a.ctrl[NRT_CTRL_ROUND];
    const float forced = a.params[5];
    int m = 0;
    for (; m < a.n_rows_q; ++m) {
      const double ep = (double)(uint32_t)(xv[m] >> 32), eq = (double)(uint32_t)xv[m];
      bool acc;
      if (forced >= 0.f) {
        acc = philox_uniform(seed, kDomForced, round, (uint32_t)m) < forced;
      } else {
        const double u = (double)philox_uniform(seed, kDomAccept, round, (uint32_t)m);
        acc = u * eq * (double)ldg2(&a.st->kept[m]) < ep * (double)ldg2(&a.st->kept[kRowsP + m]);
      }
      a.st->accept_flags[m] = acc ? 1 : 0;
      if (!acc) break;
    }
    a.st->accepted = m;
  }
  __syncthreads();
}
__global__ void __launch_bounds__(64) samp_accept_kernel(const SamplerArgs a) {
  __shared__ uint64_t xv[16];
  griddep_wait();
  griddep_launch();
  do_accept(a, xv);
}

// residual / bonus mass of token t of the row being resampled (40-bit fixed point of a probability).  The row's
// scalars are fetched once (ResampleRow); the per-token part works on the two loaded codes.
struct ResampleRow {
  unsigned int prefix_p, prefix_q;
  double kept_p, kept_q;
  bool has_q;
  const unsigned int* ep;     // codes of the target row
  const unsigned int* eq;     // codes of the draft row (valid when has_q)
};
__device__ __forceinline__ ResampleRow resample_row(const SamplerArgs& a, int m) {
  ResampleRow r;
  r.has_q = m < a.n_rows_q;
  r.ep = a.e + (size_t)m * a.vlocal;
  r.eq = a.e + (size_t)(kRowsP + (r.has_q ? m : 0)) * a.vlocal;
  r.prefix_p = ldg2(&a.st->prefix[m]);
  r.prefix_q = r.has_q ? ldg2(&a.st->prefix[kRowsP + m]) : 0u;
  r.kept_p = (double)ldg2(&a.st->kept[m]);
  r.kept_q = r.has_q ? (double)ldg2(&a.st->kept[kRowsP + m]) : 1.0;
  return r;
}
__device__ __forceinline__ unsigned long long resample_mass_of(const ResampleRow& r, unsigned int ep, unsigned int eq, bool from_p) {
  if (ep < r.prefix_p) ep = 0u;
  if (from_p || !r.has_q) return (unsigned long long)ep;          // bonus / anchor row / empty residual: sample from p'
  if (eq < r.prefix_q) eq = 0u;
  const double v = (double)ep / r.kept_p - (double)eq / r.kept_q;
  return v > 0.0 ? (unsigned long long)(v * 1099511627776.0) : 0ull;
}

// ---------------------------------------------------------------- resample: per-tile masses
__device__ __forceinline__ void work_tile_mass(const SamplerArgs& a, int bx) {
  __shared__ unsigned long long ssum, ssum_p;
  if (threadIdx.x == 0) { ssum = 0ull; ssum_p = 0ull; }
  __syncthreads();
  const int m = ldg2(&a.st->accepted);
  const ResampleRow rr = resample_row(a, m);
  unsigned long long acc = 0ull, acc_p = 0ull;
  const int t0 = bx * kTile;
  unsigned int ep[kPer], eq[kPer];
#pragma unroll
  for (int j = 0; j < kPer; ++j) {                  // all of a thread's codes are requested together
    const int t = t0 + threadIdx.x + j * kThreads;
    ep[j] = t < a.vlocal ? __ldcg(rr.ep + t) : 0u;
    eq[j] = (t < a.vlocal && rr.has_q) ? __ldcg(rr.eq + t) : 0u;
  }
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    acc += resample_mass_of(rr, ep[j], eq[j], false);
    acc_p += resample_mass_of(rr, ep[j], eq[j], true);
  }
  acc = warp_sum_u64(acc);
  acc_p = warp_sum_u64(acc_p);
  if ((threadIdx.x & 31) == 0) { atomicAdd(&ssum, acc); atomicAdd(&ssum_p, acc_p); }
  __syncthreads();
  if (threadIdx.x == 0) { a.st->tile_mass[bx] = ssum; a.st->tile_mass[128 + bx] = ssum_p; }
}
__global__ void __launch_bounds__(kThreads) samp_tile_mass_kernel(const SamplerArgs a) {
  griddep_wait();
  griddep_launch();
  work_tile_mass(a, blockIdx.x);
}

// ---------------------------------------------------------------- resample: inverse CDF in vocabulary order
__device__ __forceinline__ void do_draw(const SamplerArgs& a, int tiles, int domain, uint64_t* xv) {
  __shared__ unsigned long long part[kThreads];
  __shared__ int s_tok;
  __shared__ unsigned long long tmass[256];        // tile masses of this rank: residual [0, 128), bonus [128, 256)
  __shared__ int s_th;
  __shared__ unsigned long long s_rem;
  const int m = ldg2(&a.st->accepted);
  if (threadIdx.x < 16) xv[threadIdx.x] = 0ull;
  tmass[threadIdx.x] = (threadIdx.x & 127) < tiles ? ldg2(&a.st->tile_mass[threadIdx.x]) : 0ull;   // one round of loads
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long tot = 0ull, tot_p = 0ull;
    for (int i = 0; i < tiles; ++i) { tot += tmass[i]; tot_p += tmass[128 + i]; }
    xv[a.x.rank] = tot;
    xv[8 + a.x.rank] = tot_p;
    s_tok = -1;
  }
  __syncthreads();
  xchg_reduce_u64<kXSum>(xv, 16, a.x, 11);        // everyone learns every rank's totals
  unsigned long long total = 0ull, before = 0ull;
  for (int r = 0; r < a.x.tp; ++r) total += xv[r];
  const bool from_p = total == 0ull;               // empty residual (p' <= q' everywhere): draw from p'
  const int xo = from_p ? 8 : 0, mo = from_p ? 128 : 0;
  total = 0ull;
  for (int r = 0; r < a.x.tp; ++r) { if (r < a.x.rank) before += xv[xo + r]; total += xv[xo + r]; }
  const double u = (double)philox_uniform(*a.seed, (uint32_t)domain, (uint32_t)a.ctrl[NRT_CTRL_ROUND], (uint32_t)m);
  unsigned long long target = (unsigned long long)(u * (double)total);
  if (total > 0ull && target >= total) target = total - 1ull;
  const bool mine = total > 0ull && target >= before && target < before + xv[xo + a.x.rank];
  if (mine) {
    unsigned long long local = target - before;       // uniform across the CTA
    int tile = 0;
    for (; tile < tiles - 1; ++tile) {
      const unsigned long long tm = tmass[mo + tile];
      if (local < tm) break;
      local -= tm;
    }
    // scan the tile: each thread owns 8 consecutive tokens, whose codes it requests together and keeps
    const ResampleRow rr = resample_row(a, m);
    const int t0 = tile * kTile + threadIdx.x * kPer;
    unsigned long long w[kPer];
    {
      unsigned int ep[kPer], eq[kPer];
#pragma unroll
      for (int i = 0; i < kPer; ++i) {
        ep[i] = t0 + i < a.vlocal ? __ldcg(rr.ep + t0 + i) : 0u;
        eq[i] = (t0 + i < a.vlocal && rr.has_q) ? __ldcg(rr.eq + t0 + i) : 0u;
      }
#pragma unroll
      for (int i = 0; i < kPer; ++i) w[i] = t0 + i < a.vlocal ? resample_mass_of(rr, ep[i], eq[i], from_p) : 0ull;
    }
    unsigned long long mine_sum = 0ull;
#pragma unroll
    for (int i = 0; i < kPer; ++i) mine_sum += w[i];
    part[threadIdx.x] = mine_sum;
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long run = 0ull;
      int th = 0;
      for (; th < kThreads - 1; ++th) {
        if (local < run + part[th]) break;
        run += part[th];
      }
      s_th = th;
      s_rem = local - run;
    }
    __syncthreads();
    if ((int)threadIdx.x == s_th) {                  // the owner of the eight tokens walks its own masses
      unsigned long long rem = s_rem;
      int tok = t0;
#pragma unroll
      for (int i = 0; i < kPer; ++i) {
        if (t0 + i >= a.vlocal) break;
        tok = t0 + i;
        if (rem < w[i]) break;
        rem -= w[i];
      }
      s_tok = tok + a.vbase;
    }
  }
  __syncthreads();
  if (threadIdx.x < 16) xv[threadIdx.x] = (threadIdx.x == 0 && s_tok >= 0) ? (uint64_t)(s_tok + 1) : 0ull;
  __syncthreads();
  xchg_reduce_u64<kXSum>(xv, 1, a.x, 12);
  if (threadIdx.x == 0) {
    int tok = (int)xv[0] - 1;
    if (tok < 0) tok = 0;                          // unreachable while the kept set is non-empty
    a.st->extra_token = tok;
  }
}
__global__ void __launch_bounds__(kThreads) samp_draw_kernel(const SamplerArgs a, int tiles, int domain) {
  __shared__ uint64_t xv[16];
  griddep_wait();
  griddep_launch();
  do_draw(a, tiles, domain, xv);
}

// ---------------------------------------------------------------- the whole sampler in one launch
// Same phases, same arithmetic, same exchanges as the chain of nine kernels; the hand-over between phases happens
// inside the grid.  After its share of a phase every CTA adds itself to a monotonic arrival counter; the CTA that
// completes the count runs the phase's cross-rank exchange and state update and publishes the phase generation,
// the others wait for it (bounded: a wait that gives up records a status word and the CTA leaves).  grid =
// (vocabulary tiles, 15 distributions), all resident at once (checked at launch).
// Reference counterpart: the persistent cooperative sampler, naivert/body/dspark_sampling/persistent.cuh:15-42,1208.
struct PhaseSync {
  unsigned long long* arrive;
  unsigned int* gen;
  uint32_t* status;
  unsigned int n_ctas;
};
// true for the CTA that completed this phase's count; my_gen = generation the others wait for
__device__ __forceinline__ bool phase_arrive(const PhaseSync& ps, unsigned int& my_gen) {
  __shared__ unsigned int s_gen;
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned long long old = atomicAdd(ps.arrive, 1ull);
    s_gen = (unsigned int)(old / ps.n_ctas + 1ull);
    s_last = (old + 1ull) % ps.n_ctas == 0ull;
  }
  __syncthreads();
  my_gen = s_gen;
  __threadfence();
  return s_last != 0;
}
__device__ __forceinline__ void phase_release(const PhaseSync& ps, unsigned int my_gen) {
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(ps.gen), "r"(my_gen) : "memory");
}
__device__ __forceinline__ bool phase_wait(const PhaseSync& ps, unsigned int my_gen, int site) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    s_ok = 1;
    const uint64_t deadline = globaltimer() + kWaitLimitNs;
    for (uint32_t i = 0;; ++i) {
      if ((int)(ld_acquire_gpu(ps.gen) - my_gen) >= 0) break;        // generations only grow
      if ((i & 255u) == 255u) {
        if (*reinterpret_cast<volatile uint32_t*>(ps.status) != 0u) { s_ok = 0; break; }
        if (globaltimer() > deadline) { report(ps.status, kSiteGrid | 0x40u | (uint32_t)site); s_ok = 0; break; }
      }
    }
  }
  __syncthreads();
  return s_ok != 0;
}

__global__ void __launch_bounds__(kThreads, 2) samp_persistent_kernel(const SamplerArgs a, int tiles, int domain,
                                                                   unsigned long long* arrive, unsigned int* gen) {
  __shared__ uint64_t xv[kDist * 256];
  griddep_wait();
  griddep_launch();
  const int bx = blockIdx.x, d = blockIdx.y;
  PhaseSync ps{arrive, gen, a.x.status, gridDim.x * gridDim.y};
  unsigned int g;
#define NRT_SSTAMP(i) do { if (a.stamps && threadIdx.x == 0) a.stamps[i] = globaltimer(); } while (0)
  if (bx == 0 && d == 0) NRT_SSTAMP(30);
  work_max(a, bx, d);
  if (phase_arrive(ps, g)) { NRT_SSTAMP(0); post_max(a, xv); phase_release(ps, g); NRT_SSTAMP(1); } else if (!phase_wait(ps, g, 0)) return;
  work_exp(a, bx, d);
  if (phase_arrive(ps, g)) { NRT_SSTAMP(2); post_exp(a, xv); phase_release(ps, g); NRT_SSTAMP(3); } else if (!phase_wait(ps, g, 1)) return;
  for (int pass = 0; pass < 4; ++pass) {
    work_hist(a, bx, d, pass);
    if (phase_arrive(ps, g)) {
      NRT_SSTAMP(4 + 2 * pass);
      post_hist(a, xv, pass);
      if (pass == 3) { __syncthreads(); do_accept(a, xv); }
      phase_release(ps, g);
      NRT_SSTAMP(5 + 2 * pass);
    } else if (!phase_wait(ps, g, 2 + pass)) return;
  }
  if (d == 0) work_tile_mass(a, bx);
  if (phase_arrive(ps, g)) { NRT_SSTAMP(12); do_draw(a, tiles, domain, xv); NRT_SSTAMP(13); }
#undef NRT_SSTAMP
}

// ---------------------------------------------------------------- tail: commit + next-round geometry
struct RingRecord {              // 64 bytes, host-visible
  unsigned int generation;       // written last: round index + 1
  int count;                     // tokens committed by this round (0..8)
  int tokens[8];
  int pos0;                      // position of the anchor row of this round
  int stop_reason;               // 0 none, 1 eos, 2 output limit, 3 position limit, 4 cancelled, 5 device wait failed
  unsigned long long t_end_ns;
  int accepted;
  int pad[1];
};

struct TailArgs {
  int* ctrl;                     // [0] pos0 [1] n_ingest [2] ingest_pos0 [4] stopped [5] reason [6] produced [7] max_tokens [8] round [9] capacity
  int* block_ids;                // [8]
  uint32_t* epoch;
  SamplerState* st;
  RingRecord* ring;              // mapped pinned host memory
  int ring_size;
  const volatile int* cancel;    // mapped pinned host word (non-zero: stop)
  const int* stop_ids;           // device [n_stop]
  int n_stop;
  unsigned short* counts;        // [vlocal] penalty counts of this rank's shard or null
  int vbase, vlocal;
  const uint32_t* status;
  int n_rows_q;
  const volatile int* host_consumed;   // mapped pinned host word: rounds the host has read (null: host-launched rounds)
  XchgArgs x;                    // cancel / failure / pause consensus across ranks
};

__global__ void tail_commit_kernel(const TailArgs a) {
  __shared__ uint64_t xv[16];
  griddep_wait();
  griddep_launch();
  // Every rank must take the same stop decision in the same round: the host cancel word (set on one
  // rank only) and a failed device wait on any rank are max-reduced over the ranks first.
  // A self-relaunching chain pauses when the host is a ring length behind.  Each rank sees its own host's
  // progress, so the pause is a consensus too: one rank that must wait makes every rank wait, otherwise the
  // others would run into the next round's exchanges alone.
  if (threadIdx.x < 16) {
    uint64_t v = 0ull;
    if (threadIdx.x == 0) v = (uint64_t)(*a.cancel != 0);
    else if (threadIdx.x == 1) v = (uint64_t)(*a.status != 0u);
    else if (threadIdx.x == 2 && a.host_consumed) v = (uint64_t)(a.ctrl[NRT_CTRL_ROUND] + 1 - *a.host_consumed >= a.ring_size - 8);
    xv[threadIdx.x] = v;
  }
  __syncthreads();
  xchg_reduce_u64<kXMax>(xv, 3, a.x, 13);
  __syncthreads();
  const bool cancel_any = xv[0] != 0ull, failed_any = xv[1] != 0ull;
  if (threadIdx.x != 0) return;
  int* c = a.ctrl;
  c[NRT_CTRL_PAUSED] = xv[2] != 0ull ? 1 : 0;
  const int round = c[NRT_CTRL_ROUND];
  if (c[NRT_CTRL_STOPPED]) {                                  // already stopped: keep the fabric epoch moving, publish nothing
    // The round that just ran completed the draft context of the last committed rows; any further
    // round must not overwrite it with features of rows that were never committed.
    c[NRT_CTRL_INGEST_POS] = c[NRT_CTRL_POS];
    *a.epoch += 1u;
    c[NRT_CTRL_ROUND] = round + 1;
    return;
  }
  const int m = a.st->accepted;
  const int pos0 = c[NRT_CTRL_POS];
  int reason = 0, n = 0;
  int out[8];
  if (failed_any) reason = NRT_STOP_DEVICE_WAIT_FAILED;
  else if (cancel_any) reason = NRT_STOP_CANCELLED;
  for (int j = 0; j <= m && reason == 0; ++j) {
    const int tok = j < m ? a.block_ids[j + 1] : a.st->extra_token;
    out[n++] = tok;
    c[NRT_CTRL_GENERATED] += 1;
    const int local = tok - a.vbase;
    if (a.counts && local >= 0 && local < a.vlocal && a.counts[local] < 65535) a.counts[local] += 1;
    for (int s = 0; s < a.n_stop; ++s)
      if (tok == a.stop_ids[s]) reason = NRT_STOP_EOS;
    if (reason == 0 && c[NRT_CTRL_GENERATED] >= c[NRT_CTRL_MAX_TOKENS]) reason = NRT_STOP_MAX_TOKENS;
  }
  if (reason == 0 && pos0 + n + 16 >= c[NRT_CTRL_CAPACITY]) reason = NRT_STOP_CAPACITY;
  RingRecord* rec = a.ring + (round % a.ring_size);
  rec->count = n;
  for (int j = 0; j < 8; ++j) rec->tokens[j] = j < n ? out[j] : -1;
  rec->pos0 = pos0;
  rec->stop_reason = reason;
  rec->accepted = m;
  rec->t_end_ns = globaltimer();
  __threadfence_system();
  *reinterpret_cast<volatile unsigned int*>(&rec->generation) = (unsigned int)round + 1u;
  // next round: rows 0..n-1 of this verify are committed context
  if (n > 0) {
    c[NRT_CTRL_INGEST_POS] = pos0;
    c[NRT_CTRL_COMMITTED] = n;
    c[NRT_CTRL_POS] = pos0 + n;
    a.block_ids[0] = out[n - 1];
  }
  if (reason) { c[NRT_CTRL_STOPPED] = 1; c[NRT_CTRL_REASON] = reason; }
  c[NRT_CTRL_ROUND] = round + 1;
  *a.epoch += 1u;
}

// Prompt replay cursor: loads the next `rows` prompt tokens into the step's token buffer, points
// the step (ctrl[0]) and the draft ingest (ctrl[2]) at their position and advances ctrl[10].
__global__ void prefill_cursor_kernel(const int* __restrict__ prompt, int n_prompt, int rows, int* ctrl, int* tokens) {
  griddep_wait();
  griddep_launch();
  const int cur = ctrl[NRT_CTRL_CURSOR];
  if (n_prompt < 0) n_prompt = ctrl[NRT_CTRL_PROMPT_CTX];          // length kept in the control block (graph replays)
  if (threadIdx.x < 16) {
    const int t = cur + (int)threadIdx.x;
    tokens[threadIdx.x] = ((int)threadIdx.x < rows && t < n_prompt) ? prompt[t] : 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) { ctrl[NRT_CTRL_POS] = cur; ctrl[NRT_CTRL_INGEST_POS] = cur; ctrl[NRT_CTRL_CURSOR] = cur + rows; }
}

// advance the fabric epoch (eager steps outside a round)
__global__ void epoch_advance_kernel(uint32_t* epoch) {
  griddep_wait();
  griddep_launch();
  if (threadIdx.x == 0) *epoch += 1u;
}

}  // namespace

#define S(stream) reinterpret_cast<cudaStream_t>(stream)

extern "C" int nrt_sampler_args_size() { return (int)sizeof(SamplerArgs); }
extern "C" int nrt_sampler_state_size() { return (int)sizeof(SamplerState); }
extern "C" int nrt_tail_args_size() { return (int)sizeof(TailArgs); }
extern "C" int nrt_ring_record_size() { return (int)sizeof(RingRecord); }

// Runs the whole sampler chain: maxima, codes, four nucleus passes, accept, resample.
// domain: Philox domain of the final draw (1 = residual/bonus of a round, 4 = anchor sample).
extern "C" int nrt_sampler_run(const void* args, int domain, void* stream, int pdl) {
  SamplerArgs a;
  memcpy(&a, args, sizeof(a));
  const int tiles = (a.vlocal + kTile - 1) / kTile;
  if (tiles > 128) return -3;
  const bool p = pdl != 0;
  int rc;
  if ((rc = launch_pdl(samp_max_kernel, dim3(tiles, kDist), dim3(kThreads), 0, S(stream), p, a))) return rc;
  if ((rc = launch_pdl(samp_exp_kernel, dim3(tiles, kDist), dim3(kThreads), 0, S(stream), p, a))) return rc;
  for (int pass = 0; pass < 4; ++pass)
    if ((rc = launch_pdl(samp_hist_kernel, dim3(tiles, kDist), dim3(kThreads), 0, S(stream), p, a, pass))) return rc;
  if ((rc = launch_pdl(samp_accept_kernel, dim3(1), dim3(64), 0, S(stream), p, a))) return rc;
  if ((rc = launch_pdl(samp_tile_mass_kernel, dim3(tiles), dim3(kThreads), 0, S(stream), p, a))) return rc;
  return launch_pdl(samp_draw_kernel, dim3(1), dim3(kThreads), 0, S(stream), p, a, tiles, domain);
}

// The same sampler in one launch.  `sync`: two 64-bit words (arrival counter, phase generation), zeroed once.
// Returns -9 when the grid cannot be resident at once (use nrt_sampler_run).
extern "C" int nrt_sampler_persistent(const void* args, int domain, void* sync, void* stream, int pdl) {
  SamplerArgs a;
  memcpy(&a, args, sizeof(a));
  const int tiles = (a.vlocal + kTile - 1) / kTile;
  if (tiles > 128 || !sync) return -3;
  static int resident = -1;
  if (resident < 0) {
    int per_sm = 0, dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, samp_persistent_kernel, kThreads, 0) != cudaSuccess) return -3;
    resident = per_sm * sms;
  }
  if (tiles * kDist > resident) return -9;
  unsigned long long* w = reinterpret_cast<unsigned long long*>(sync);
  return launch_pdl(samp_persistent_kernel, dim3(tiles, kDist), dim3(kThreads), 0, S(stream), pdl != 0, a, tiles, domain, w,
                    reinterpret_cast<unsigned int*>(w + 1));
}

extern "C" int nrt_tail_commit(const void* args, void* stream, int pdl) {
  TailArgs a;
  memcpy(&a, args, sizeof(a));
  return launch_pdl(tail_commit_kernel, dim3(1), dim3(32), 0, S(stream), pdl != 0, a);
}

extern "C" int nrt_epoch_advance(void* epoch, void* stream, int pdl) {
  return launch_pdl(epoch_advance_kernel, dim3(1), dim3(32), 0, S(stream), pdl != 0, (uint32_t*)epoch);
}

extern "C" int nrt_prefill_cursor(const int* prompt, int n_prompt, int rows, int* ctrl, int* tokens, void* stream, int pdl) {
  return launch_pdl(prefill_cursor_kernel, dim3(1), dim3(32), 0, S(stream), pdl != 0, prompt, n_prompt, rows, ctrl, tokens);
}

extern "C" float nrt_philox_uniform(unsigned long long seed, unsigned int domain, unsigned int a, unsigned int b) {
  return philox_uniform(seed, domain, a, b);
}

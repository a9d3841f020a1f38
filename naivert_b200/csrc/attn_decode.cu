// Tensor-core row attention for the decode / verify / draft step.
//
// One CTA (8 warps) per (KV head, query row, key split).  The query heads that share the KV head are the
// M = 16 side of bf16 m16n8k16 MMAs, so every key / value row is gathered once per KV head (at tp = 8 the eight
// local query heads share one KV head: the scalar per-head kernel read each key eight times).  Keys come in
// chunks of 128 (a sliding window, or one of sixteen splits of a 2048-key selection, is a single chunk: one gather,
// one soft-max pass) - the row's sliding window, its dense prefix, its top-k selection list, or the draft's context
// window followed by the block's own rows - staged with cp.async in two buffers (the next chunk's gather runs
// under the current chunk's math), scored (S = Q K^T), soft-maxed online per head and accumulated (O += P V,
// V fragments through ldmatrix.trans).  Long key lists (2048 selected keys) are split over grid.z CTAs; each
// writes its (max, sum, unnormalised O) and the last CTA of a (KV head, row) to arrive merges the splits in
// split order, adds the sink column, normalises and emits bf16 o and / or the e4m3 packet for o_proj.
// Every result depends only on its own row's inputs and on a fixed merge order: bitwise repeatable and
// independent of which other rows share the step.
//
// Reference counterparts: naivert/body/attn_dsa/attn_dsa_body.cuh:675-716 (mma m16n8k16 + ldmatrix 8-head
// path), :768-860 (wmma 16-head path, 16 key splits + combine), naivert/body/attn_swa/attn_swa_body.cuh,
// naivert/body/dspark_attention/body.cuh (draft window attention).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>
#include <string.h>

#include "gemm.cuh"
#include "launch.hpp"

using namespace nrt;

namespace {

struct AttnArgs {               // must match target_kernels.cu
  const __nv_bfloat16* q;
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  const int* pos0;
  int rows, heads, kv_heads, head_dim, v_dim;
  float scale;
  int mode;
  int window, ring;
  const __nv_bfloat16* sink;
  const int* sel;
  int top_k;
  const __nv_bfloat16* k_blk;
  const __nv_bfloat16* v_blk;
  __nv_bfloat16* o_bf16;
  uint8_t* o8;
  float* o_scale;
  float* part;
  unsigned int* tickets;
  unsigned long long* stamps;   // opt-in phase stamps of the tensor-core decode kernel (%globaltimer, ns), [CTA][8]; null: none
};

constexpr int kVd = 128, kChunk = 128, kM = 16, kStagesKV = 2;
constexpr int kVStride = kVd + 8;        // 272-byte rows: ldmatrix rows fall into distinct 16-byte bank groups
constexpr int kSStride = kVd + 4;        // fp32; also carries the 128 output channels at the end
constexpr int kPStride = kChunk + 8;     // bf16
constexpr int kPartStride = kVd + 2;     // per (split, head): max, sum, 128 channels

template <int HD>
struct Smem {
  static constexpr int kQStride = HD + 8;   // row stride in bf16 elements: fragment loads hit distinct banks
  __nv_bfloat16 q[kM][kQStride];
  __nv_bfloat16 k[kStagesKV][kChunk][kQStride];
  __nv_bfloat16 v[kStagesKV][kChunk][kVStride];
  float s[kM][kSStride];
  __nv_bfloat16 p[kM][kPStride];
  float m[kM], l[kM], corr[kM];
  int last;
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma16816(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, const void* p) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}

// key j of the row's list -> cache row (>= 0) or block row -(id + 1) (draft block mode)
struct KeyList {
  int mode, lo, ctx, count, top_k, ring, base;
  bool use_sel;
  const int* sel;
  __device__ __forceinline__ int id(int j) const {
    if (mode == 1) return use_sel ? sel[j] : j;
    if (mode == 2) return j < ctx ? lo + j : -(j - ctx) - 1;
    return lo + j;
  }
  // cache row of a non-negative id; consecutive window keys wrap around the ring at most once (base = lo % ring)
  __device__ __forceinline__ size_t slot(int id, int j) const {
    if (ring <= 0) return (size_t)id;
    if (mode == 0) { const int s = base + j; return (size_t)(s >= ring ? s - ring : s); }
    return (size_t)(id % ring);
  }
};

template <int HD>
__global__ void __launch_bounds__(256, 2) attn_decode_kernel(const AttnArgs a) {
  extern __shared__ uint4 smem_raw[];
  Smem<HD>& sm = *reinterpret_cast<Smem<HD>*>(smem_raw);
  unsigned long long* stamp = a.stamps ? a.stamps + (size_t)((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 8 : nullptr;
#define NRT_ASTAMP(i) do { if (stamp && threadIdx.x == 0) stamp[i] = globaltimer(); } while (0)
  NRT_ASTAMP(0);
  const int g = blockIdx.x, r = blockIdx.y, sp = blockIdx.z, splits = gridDim.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hpg = a.heads / a.kv_heads;                      // live query heads (<= 16)
  const int h0 = g * hpg;
  // The position word was written by the previous round's tail (or the step's cursor kernel), at least two launches
  // back: with programmatic dependent launch that work is complete before this grid may start, so the word - and the
  // cache rows of earlier steps - are read before the wait for the immediate predecessor (the projection that
  // appends this step's rows).
  const int p0 = *a.pos0;
  const int pos = p0 + r;
  const int qr = lane >> 2, qc = (lane & 3) * 2;             // fragment row / column pair of this lane

  KeyList kl;
  kl.mode = a.mode; kl.top_k = a.top_k; kl.ring = a.ring; kl.lo = 0; kl.ctx = 0; kl.use_sel = false; kl.base = 0;
  kl.sel = a.sel + (size_t)r * a.top_k;
  if (a.mode == 0) { kl.lo = max(0, pos - a.window + 1); kl.count = pos - kl.lo + 1; kl.base = a.ring > 0 ? kl.lo % a.ring : 0; }
  else if (a.mode == 1) { kl.use_sel = pos + 1 > a.top_k; kl.count = kl.use_sel ? a.top_k : pos + 1; }
  else { kl.lo = max(0, p0 - a.window); kl.ctx = p0 - kl.lo; kl.count = kl.ctx + a.rows; }
  const int count = kl.count;
  const int nchunks_all = (count + kChunk - 1) / kChunk;
  const int per = (nchunks_all + splits - 1) / splits;
  const int c_first = sp * per, c_last = min(nchunks_all, (sp + 1) * per);      // this CTA's chunks
  const int nchunks = max(0, c_last - c_first);

  // Two threads per key: the row address is worked out once per key, then the thread copies its half of the row's
  // 16-byte pieces.  `which`: 0 = keys appended by earlier steps (cache rows before this step's first position),
  // 1 = this step's own rows (written by the predecessor kernel), 2 = all.
  auto issue = [&](int c0, int stage, int which) {
    const int t = tid >> 1, half = tid & 1;
    const int j = c0 + t;
    bool valid = j < count;
    const int id = valid ? kl.id(j) : 0;
    valid = valid && (id < 0 || NRT_INDEX_OK(id, pos + 1, kBoundsAttnKey));   // a key of the cache is never beyond the query
    const bool own = id < 0 || (a.mode != 1 && id >= p0);       // a row of the running step
    const bool take = which == 2 || (which == 1) == own;
    if (!take) return;
    const __nv_bfloat16 *ksrc, *vsrc;
    if (id < 0) {
      ksrc = a.k_blk + ((size_t)(-id - 1) * a.kv_heads + g) * HD;
      vsrc = a.v_blk + ((size_t)(-id - 1) * a.kv_heads + g) * kVd;
    } else {
      const size_t row = kl.slot(id, j);
      ksrc = a.k_cache + (row * a.kv_heads + g) * HD;
      vsrc = a.v_cache + (row * a.kv_heads + g) * kVd;
    }
#pragma unroll
    for (int c = 0; c < HD / 16; ++c) cp_async16(&sm.k[stage][t][(half * (HD / 16) + c) * 8], ksrc + (half * (HD / 16) + c) * 8, valid);
#pragma unroll
    for (int c = 0; c < kVd / 16; ++c) cp_async16(&sm.v[stage][t][(half * (kVd / 16) + c) * 8], vsrc + (half * (kVd / 16) + c) * 8, valid);
  };
  // sliding window / draft context: the rows of earlier steps are requested before the wait for the predecessor
  const bool early = a.mode != 1 && nchunks > 0 && r < a.rows;
  if (early) issue(c_first * kChunk, 0, 0);
  griddep_wait();
  griddep_launch();
  NRT_ASTAMP(1);
  if (r >= a.rows) return;
  // the first gather is in flight while Q is staged
  if (nchunks > 0) issue(c_first * kChunk, 0, early ? 1 : 2);
  cp_async_commit();
  for (int i = tid; i < kM * (HD / 8); i += 256) {
    const int h = i / (HD / 8), c = i - h * (HD / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (h < hpg) v = reinterpret_cast<const uint4*>(a.q + ((size_t)r * a.heads + h0 + h) * HD)[c];
    *reinterpret_cast<uint4*>(&sm.q[h][c * 8]) = v;
  }
  if (tid < kM) { sm.m[tid] = -FLT_MAX; sm.l[tid] = 0.f; }
  __syncthreads();
  uint32_t qa[HD / 16][4];
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
    qa[ks][0] = *reinterpret_cast<const uint32_t*>(&sm.q[qr][ks * 16 + qc]);
    qa[ks][1] = *reinterpret_cast<const uint32_t*>(&sm.q[qr + 8][ks * 16 + qc]);
    qa[ks][2] = *reinterpret_cast<const uint32_t*>(&sm.q[qr][ks * 16 + qc + 8]);
    qa[ks][3] = *reinterpret_cast<const uint32_t*>(&sm.q[qr + 8][ks * 16 + qc + 8]);
  }

  float oc[2][4];
#pragma unroll
  for (int t = 0; t < 2; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) oc[t][j] = 0.f;

  for (int ci = 0; ci < nchunks; ++ci) {
    const int c0 = (c_first + ci) * kChunk, st = ci & 1;
    const int n = min(kChunk, count - c0);
    if (ci + 1 < nchunks) issue(c0 + kChunk, st ^ 1, 2);
    cp_async_commit();                                        // (possibly empty) group of chunk ci + 1
    cp_async_wait<1>();                                       // this thread's copies of chunk ci have landed
    __syncthreads();                                          // ... and everybody else's
    if (ci == 0) NRT_ASTAMP(2);
    // ---- S = Q K^T: warp w scores keys [8w, 8w + 8) and [64 + 8w, 64 + 8w + 8) for all heads
#pragma unroll
    for (int nt = 0; nt < kChunk / 64; ++nt) {
      const int key0 = nt * 64 + warp * 8;
      if (key0 >= n) {                                        // whole tile beyond the chunk's keys (uniform per warp)
        if (lane < 16) {
#pragma unroll
          for (int j = 0; j < 8; ++j) sm.s[lane][key0 + j] = -FLT_MAX;
        }
        continue;
      }
      float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(&sm.k[st][key0 + qr][ks * 16 + qc]);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(&sm.k[st][key0 + qr][ks * 16 + qc + 8]);
        mma16816(c, qa[ks], b0, b1);
      }
      const int kc = key0 + qc;
      sm.s[qr][kc] = kc < n ? c[0] * a.scale : -FLT_MAX;
      sm.s[qr][kc + 1] = kc + 1 < n ? c[1] * a.scale : -FLT_MAX;
      sm.s[qr + 8][kc] = kc < n ? c[2] * a.scale : -FLT_MAX;
      sm.s[qr + 8][kc + 1] = kc + 1 < n ? c[3] * a.scale : -FLT_MAX;
    }
    __syncthreads();
    // ---- online softmax: warp w owns heads 2w and 2w + 1
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int h = warp * 2 + t;
      float v[kChunk / 32];
      float mx = -FLT_MAX;
#pragma unroll
      for (int j = 0; j < kChunk / 32; ++j) { v[j] = sm.s[h][lane + 32 * j]; mx = fmaxf(mx, v[j]); }
      mx = warp_max_f(mx);
      const float m_old = sm.m[h];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < kChunk / 32; ++j) {
        const int kc = lane + 32 * j;
        const float p = kc < n ? round_bf16(__expf(v[j] - m_new)) : 0.f;
        sm.p[h][kc] = __float2bfloat16_rn(p);
        sum += p;
      }
      sum = warp_sum_f(sum);
      if (lane == 0) {
        const float corr = __expf(m_old - m_new);
        sm.corr[h] = corr;
        sm.l[h] = sm.l[h] * corr + sum;
        sm.m[h] = m_new;
      }
    }
    __syncthreads();
    // ---- O = O * corr + P V: warp w owns channels [16w, 16w + 16)
    {
      const float c_lo = sm.corr[qr], c_hi = sm.corr[qr + 8];
#pragma unroll
      for (int t = 0; t < 2; ++t) { oc[t][0] *= c_lo; oc[t][1] *= c_lo; oc[t][2] *= c_hi; oc[t][3] *= c_hi; }
#pragma unroll
      for (int kk = 0; kk < kChunk / 16; ++kk) {
        if (kk * 16 >= n) break;                              // probabilities beyond the chunk's keys are zero
        uint32_t pa[4];
        pa[0] = *reinterpret_cast<const uint32_t*>(&sm.p[qr][kk * 16 + qc]);
        pa[1] = *reinterpret_cast<const uint32_t*>(&sm.p[qr + 8][kk * 16 + qc]);
        pa[2] = *reinterpret_cast<const uint32_t*>(&sm.p[qr][kk * 16 + qc + 8]);
        pa[3] = *reinterpret_cast<const uint32_t*>(&sm.p[qr + 8][kk * 16 + qc + 8]);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          uint32_t b0, b1;
          ldmatrix_x2_trans(b0, b1, &sm.v[st][kk * 16 + (lane & 15)][warp * 16 + t * 8]);
          mma16816(oc[t], pa, b0, b1);
        }
      }
    }
    __syncthreads();                                          // stage st is free for chunk ci + 2
  }
  cp_async_wait<0>();
  __syncthreads();
  NRT_ASTAMP(3);

  // unnormalised O of this CTA -> shared memory (heads x channels)
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int ch = warp * 16 + t * 8 + qc;
    sm.s[qr][ch] = oc[t][0];
    sm.s[qr][ch + 1] = oc[t][1];
    sm.s[qr + 8][ch] = oc[t][2];
    sm.s[qr + 8][ch + 1] = oc[t][3];
  }
  __syncthreads();

  if (splits > 1) {
    // publish (max, sum, O) of this split; the last CTA of the (KV head, row) merges all splits in split order
    float* mine = a.part + (((size_t)r * a.kv_heads + g) * splits + sp) * kM * kPartStride;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int h = warp * 2 + t;
      float* dst = mine + h * kPartStride;
      if (lane == 0) { dst[0] = sm.m[h]; dst[1] = sm.l[h]; }
#pragma unroll
      for (int j = 0; j < 4; ++j) dst[2 + lane + 32 * j] = sm.s[h][lane + 32 * j];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const unsigned int tk = atomicAdd(&a.tickets[r * a.kv_heads + g], 1u);
      sm.last = tk == (unsigned)splits - 1;
      if (sm.last) a.tickets[r * a.kv_heads + g] = 0u;
    }
    __syncthreads();
    if (!sm.last) return;
    __threadfence();
    NRT_ASTAMP(4);
    const float* all = a.part + ((size_t)r * a.kv_heads + g) * splits * kM * kPartStride;
    // one live head per warp at a time (heads warp, warp + 8): with eight query heads per KV head all warps work
#pragma unroll 1
    for (int h = warp; h < hpg; h += 8) {
      float m_run = -FLT_MAX, l_run = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
      // eight splits per batch: their 48 loads are in flight together, then they are folded in split order
#pragma unroll 1
      for (int q0 = 0; q0 < splits; q0 += 8) {
        float mq[8], lq[8], aq[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int q = min(q0 + i, splits - 1);
          const float* o = all + ((size_t)q * kM + h) * kPartStride;
          mq[i] = __ldcg(o);
          lq[i] = __ldcg(o + 1);
#pragma unroll
          for (int j = 0; j < 4; ++j) aq[i][j] = __ldcg(o + 2 + lane + 32 * j);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (q0 + i < splits) {                              // fixed merge order: deterministic
            const float m_new = fmaxf(m_run, mq[i]);
            const float c_old = __expf(m_run - m_new), c_new = __expf(mq[i] - m_new);
            l_run = l_run * c_old + lq[i] * c_new;
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] = acc[j] * c_old + aq[i][j] * c_new;
            m_run = m_new;
          }
        }
      }
      if (lane == 0) { sm.m[h] = m_run; sm.l[h] = l_run; }
#pragma unroll
      for (int j = 0; j < 4; ++j) sm.s[h][lane + 32 * j] = acc[j];
    }
    __syncthreads();
  }

  // ---- sink column (no value), normalisation, bf16 rounding, outputs: warp w finishes heads 2w and 2w + 1
  const size_t ldo = (size_t)a.heads * kVd;
#pragma unroll 1
  for (int h = warp; h < hpg; h += 8) {
    float m = sm.m[h], l = sm.l[h], corr = 1.f;
    if (a.sink) {
      const float sv = __bfloat162float(a.sink[h0 + h]);
      const float m_new = fmaxf(m, sv);
      corr = __expf(m - m_new);
      l = l * corr + __expf(sv - m_new);
    }
    const float inv = l > 0.f ? corr / l : 0.f;
    float v[4];
    float am = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) { v[j] = round_bf16(sm.s[h][lane + 32 * j] * inv); am = fmaxf(am, fabsf(v[j])); }
    am = warp_max_f(am);
    const size_t base = (size_t)r * ldo + (size_t)(h0 + h) * kVd;
    if (a.o_bf16)
#pragma unroll
      for (int j = 0; j < 4; ++j) a.o_bf16[base + lane + 32 * j] = __float2bfloat16_rn(v[j]);
    if (a.o8) {
      const float sc = pow2_scale(am);
#pragma unroll
      for (int j = 0; j < 4; ++j) a.o8[base + lane + 32 * j] = e4m3_bits(v[j] / sc);
      if (lane == 0) a.o_scale[(size_t)r * (ldo / 128) + h0 + h] = sc;
    }
  }
  NRT_ASTAMP(5);
#undef NRT_ASTAMP
}

template <int HD>
int launch_decode(const AttnArgs& a, int splits, cudaStream_t stream, int pdl) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem<HD>));
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return launch_pdl(attn_decode_kernel<HD>, dim3(a.kv_heads, a.rows, splits), dim3(256), sizeof(Smem<HD>), stream, pdl != 0, a);
}

}  // namespace

extern "C" int nrt_attn_decode_args_size() { return (int)sizeof(AttnArgs); }
NRT_BOUNDS_EXPORT(attn_decode)
// floats of `part` needed for (rows, kv_heads, splits)
extern "C" long long nrt_attn_decode_part_floats(int rows, int kv_heads, int splits) {
  return (long long)rows * kv_heads * splits * kM * kPartStride;
}

// Row attention on tensor cores; modes 0 (sliding window), 1 (dense prefix / selection list), 2 (draft block),
// head_dim 192 or 128, v_dim 128, at most 16 query heads per KV head.  Returns -3 for other geometries
// (use nrt_attn_rows).  splits > 1 needs `part` (nrt_attn_decode_part_floats) and zeroed `tickets` [rows * kv_heads].
extern "C" int nrt_attn_decode(const void* args, int splits, void* stream, int pdl) {
  AttnArgs a;
  memcpy(&a, args, sizeof(a));
  if (a.v_dim != kVd || a.kv_heads < 1 || a.heads % a.kv_heads || a.heads / a.kv_heads > kM) return -3;
  if (a.mode < 0 || a.mode > 2 || a.rows < 1 || a.rows > 65535 || splits < 1 || splits > 64) return -3;
  if (splits > 1 && (!a.part || !a.tickets)) return -3;
  if (a.mode == 2 && (!a.k_blk || !a.v_blk)) return -3;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (a.head_dim == 192) return launch_decode<192>(a, splits, s, pdl);
  if (a.head_dim == 128) return launch_decode<128>(a, splits, s, pdl);
  return -3;
}

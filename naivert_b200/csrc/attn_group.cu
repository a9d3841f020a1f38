// Row attention for prefill chunks with the query heads of one KV head handled together.
//
// One CTA (8 warps) per (KV head, query row): the up to 16 query heads that share the KV head form the
// M = 16 side of bf16 tensor-core tiles, so every gathered key/value row is read once per KV head instead of
// once per query head (grouped-query attention: 16 heads per KV head in the sparse layers at tp = 1, 8 at
// tp = 8).  Keys come in chunks of 64 (the row's sliding window, its dense prefix, or its top-k selection
// list), are staged in shared memory with cp.async (two buffers: the next chunk's gather overlaps the current
// chunk's math), scored with m16n8k16 MMAs (S = Q K^T, 16 heads x 64 keys), soft-maxed online per head, and accumulated with a second set of MMAs
// (O += P V, V fragments through ldmatrix.trans).  The work per CTA is a gather of ~1.3 MB at top-k 2048, so
// the kernel is bound by L2/HBM gather bandwidth, not by tensor throughput; with M = 16 live rows there is no
// 128-lane UMMA shape to fill, which is why this kernel uses warp-level MMAs rather than tcgen05.
//
// Output: bf16-rounded o, written as bf16 and/or as the e4m3 packet (one power-of-two scale per head) that
// the o_proj GEMM consumes.  Probabilities are rounded to bf16 before P V (and summed as rounded), so results
// differ from attn_rows_kernel in the last bits; the step/verify path keeps attn_rows_kernel.
//
// Reference counterpart: naivert/kernels/naive_n0p5/prefill_ext (FA4 CuTe sliding-window attention,
// naive_ops sparse attention); same math, different tiling.
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

constexpr int kHd = 192, kVd = 128, kChunk = 64, kM = 16, kStagesKV = 2;
constexpr int kQStride = kHd + 8;        // bf16 elements; 400-byte rows: fragment loads hit 32 distinct banks
constexpr int kVStride = kVd + 8;        // 272-byte rows: ldmatrix rows fall into distinct 16-byte bank groups
constexpr int kSStride = kVd + 4;        // fp32; also carries the 128 output channels at the end
constexpr int kPStride = kChunk + 8;     // bf16

struct Smem {
  __nv_bfloat16 q[kM][kQStride];
  __nv_bfloat16 k[kStagesKV][kChunk][kQStride];
  __nv_bfloat16 v[kStagesKV][kChunk][kVStride];
  float s[kM][kSStride];
  __nv_bfloat16 p[kM][kPStride];
  float m[kM], l[kM], corr[kM];
};

// 16-byte asynchronous copy global -> shared; `valid` false writes zeros (nothing is read)
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
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float rbf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__global__ void __launch_bounds__(256, 2) attn_group_kernel(const AttnArgs a) {
  extern __shared__ uint4 smem_raw[];
  Smem& sm = *reinterpret_cast<Smem*>(smem_raw);
  const int g = blockIdx.x, r = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hpg = a.heads / a.kv_heads;                      // live query heads (<= 16)
  const int h0 = g * hpg;
  const int pos = *a.pos0 + r;
  const int qr = lane >> 2, qc = (lane & 3) * 2;             // fragment row / column pair of this lane

  // ---- stage Q (dead rows zero) and reset the running statistics
  for (int i = tid; i < kM * (kHd / 8); i += 256) {
    const int h = i / (kHd / 8), c = i - h * (kHd / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (h < hpg) v = reinterpret_cast<const uint4*>(a.q + ((size_t)r * a.heads + h0 + h) * kHd)[c];
    *reinterpret_cast<uint4*>(&sm.q[h][c * 8]) = v;
  }
  if (tid < kM) { sm.m[tid] = -FLT_MAX; sm.l[tid] = 0.f; }
  __syncthreads();
  uint32_t qa[kHd / 16][4];
#pragma unroll
  for (int ks = 0; ks < kHd / 16; ++ks) {
    qa[ks][0] = *reinterpret_cast<const uint32_t*>(&sm.q[qr][ks * 16 + qc]);
    qa[ks][1] = *reinterpret_cast<const uint32_t*>(&sm.q[qr + 8][ks * 16 + qc]);
    qa[ks][2] = *reinterpret_cast<const uint32_t*>(&sm.q[qr][ks * 16 + qc + 8]);
    qa[ks][3] = *reinterpret_cast<const uint32_t*>(&sm.q[qr + 8][ks * 16 + qc + 8]);
  }

  int lo = 0, count = 0;
  bool use_sel = false;
  if (a.mode == 0) { lo = max(0, pos - a.window + 1); count = pos - lo + 1; }
  else { use_sel = pos + 1 > a.top_k; count = use_sel ? a.top_k : pos + 1; }

  float oc[2][4];
#pragma unroll
  for (int t = 0; t < 2; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) oc[t][j] = 0.f;

  // Key chunks of 64 are staged with cp.async into two buffers: the gather of chunk c + 1 is in flight while
  // chunk c is scored, so a CTA covers its own gather latency (two CTAs per SM cover the rest).
  auto issue = [&](int c0, int stage) {
    for (int i = tid; i < kChunk * (kHd / 8); i += 256) {
      const int t = i / (kHd / 8), c = i - t * (kHd / 8);
      const int j = c0 + t;
      const bool valid = j < count;
      const int id = !valid ? 0 : (a.mode == 1 ? (use_sel ? a.sel[(size_t)r * a.top_k + j] : j) : lo + j);
      const size_t slot = a.ring > 0 ? (size_t)(id % a.ring) : (size_t)id;
      cp_async16(&sm.k[stage][t][c * 8], a.k_cache + (slot * a.kv_heads + g) * kHd + c * 8, valid);
    }
    for (int i = tid; i < kChunk * (kVd / 8); i += 256) {
      const int t = i / (kVd / 8), c = i - t * (kVd / 8);
      const int j = c0 + t;
      const bool valid = j < count;
      const int id = !valid ? 0 : (a.mode == 1 ? (use_sel ? a.sel[(size_t)r * a.top_k + j] : j) : lo + j);
      const size_t slot = a.ring > 0 ? (size_t)(id % a.ring) : (size_t)id;
      cp_async16(&sm.v[stage][t][c * 8], a.v_cache + (slot * a.kv_heads + g) * kVd + c * 8, valid);
    }
  };
  const int nchunks = (count + kChunk - 1) / kChunk;
  issue(0, 0);
  cp_async_commit();
  for (int ci = 0; ci < nchunks; ++ci) {
    const int c0 = ci * kChunk, st = ci & 1;
    const int n = min(kChunk, count - c0);
    if (ci + 1 < nchunks) issue(c0 + kChunk, st ^ 1);
    cp_async_commit();                                        // (possibly empty) group of chunk ci + 1
    cp_async_wait<1>();                                       // this thread's copies of chunk ci have landed
    __syncthreads();                                          // ... and everybody else's
    // ---- S = Q K^T: warp w scores keys [8w, 8w + 8) for all heads
    {
      const int key0 = warp * 8;
      float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < kHd / 16; ++ks) {
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
      mx = wmax(mx);
      const float m_old = sm.m[h];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < kChunk / 32; ++j) {
        const int kc = lane + 32 * j;
        const float p = kc < n ? rbf16(__expf(v[j] - m_new)) : 0.f;
        sm.p[h][kc] = __float2bfloat16_rn(p);
        sum += p;
      }
      sum = wsum(sum);
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
  // ---- sink column (no value), normalisation, bf16 rounding; o goes through shared memory for the packet
  if (tid < kM) {
    float m = sm.m[tid], l = sm.l[tid], corr = 1.f;
    if (a.sink && tid < hpg) {
      const float sv = __bfloat162float(a.sink[h0 + tid]);
      const float m_new = fmaxf(m, sv);
      corr = __expf(m - m_new);
      l = l * corr + __expf(sv - m_new);
    }
    sm.corr[tid] = l > 0.f ? corr / l : 0.f;
  }
  __syncthreads();
  {
    const float c_lo = sm.corr[qr], c_hi = sm.corr[qr + 8];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int ch = warp * 16 + t * 8 + qc;
      sm.s[qr][ch] = rbf16(oc[t][0] * c_lo);
      sm.s[qr][ch + 1] = rbf16(oc[t][1] * c_lo);
      sm.s[qr + 8][ch] = rbf16(oc[t][2] * c_hi);
      sm.s[qr + 8][ch + 1] = rbf16(oc[t][3] * c_hi);
    }
  }
  __syncthreads();
  const size_t ldo = (size_t)a.heads * kVd;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int h = warp * 2 + t;
    if (h >= hpg) continue;
    float v[4];
    float am = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) { v[j] = sm.s[h][lane + 32 * j]; am = fmaxf(am, fabsf(v[j])); }
    am = wmax(am);
    const size_t base = (size_t)r * ldo + (size_t)(h0 + h) * kVd;
    if (a.o_bf16)
#pragma unroll
      for (int j = 0; j < 4; ++j) a.o_bf16[base + lane + 32 * j] = __float2bfloat16_rn(v[j]);
    if (a.o8) {
      const float sc = pow2_scale(am);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __nv_fp8_e4m3 q8(v[j] / sc);
        a.o8[base + lane + 32 * j] = *reinterpret_cast<const uint8_t*>(&q8);
      }
      if (lane == 0) a.o_scale[(size_t)r * (ldo / 128) + h0 + h] = sc;
    }
  }
}

}  // namespace

extern "C" int nrt_attn_group_args_size() { return (int)sizeof(AttnArgs); }

// Grouped-head row attention; modes 0 (sliding window) and 1 (dense prefix / selection list), head_dim 192,
// v_dim 128, at most 16 query heads per KV head.  Returns -3 for other geometries (use nrt_attn_rows).
extern "C" int nrt_attn_group(const void* args, void* stream, int pdl) {
  AttnArgs a;
  memcpy(&a, args, sizeof(a));
  if (a.head_dim != kHd || a.v_dim != kVd || a.kv_heads < 1 || a.heads % a.kv_heads || a.heads / a.kv_heads > kM) return -3;
  if (a.mode != 0 && a.mode != 1) return -3;
  if (a.rows > 65535) return -3;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_group_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem));
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return launch_pdl(attn_group_kernel, dim3(a.kv_heads, a.rows), dim3(256), sizeof(Smem), reinterpret_cast<cudaStream_t>(stream),
                    pdl != 0, a);
}

// Non-GEMM kernels of the target (and draft) decode/verify body: embedding gather, RoPE table,
// RMSNorm + e4m3 packet, q/k/v post-processing (RoPE, KV-cache append, indexer key/query
// quantisation), row attention (sliding window with sink, dense range, or top-k index list),
// lightning-indexer logits, exact top-k selection, and the MoE router.
//
// Reference counterparts: naivert/kernels/model_ops/extension/embed_gather_bindings.cu,
// naivert/body/attn_dsa/attn_dsa_body.cuh (publish_query/kv/ki, compute_attention),
// naivert/body/attn_swa/attn_swa_body.cuh, naivert/body/attn_dsa/topk_grid_select.cuh,
// naivert/body/rmsnorm_expert_proj/, naivert/body/expert_select_up_gate_silu/ (compute_route).
#include "gemm.cuh"
#include "launch.hpp"
#include "router.cuh"

#include <float.h>

using namespace nrt;

namespace {

constexpr int kMaxRows = 16;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < THREADS / 32; ++i) t += red[i];
  return t;
}
template <int THREADS>
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = -FLT_MAX;
#pragma unroll
  for (int i = 0; i < THREADS / 32; ++i) t = fmaxf(t, red[i]);
  return t;
}
__device__ __forceinline__ uint8_t to_e4m3(float v) {
  const __nv_fp8_e4m3 q(v);
  return *reinterpret_cast<const uint8_t*>(&q);
}
__device__ __forceinline__ float from_e4m3(uint8_t b) {
  __nv_fp8_e4m3 q;
  *reinterpret_cast<uint8_t*>(&q) = b;
  return float(q);
}

// ----------------------------------------------------------------------------- embedding gather
__global__ void embed_rows_kernel(const int* __restrict__ tokens, const __nv_bfloat16* __restrict__ table,
                                  __nv_bfloat16* __restrict__ x, int hidden, int rows, int vocab) {
  griddep_wait();
  griddep_launch();
  const int r = blockIdx.x;
  if (r >= rows) return;
  int t = tokens[r];
  (void)NRT_INDEX_OK(t, vocab, kBoundsToken);                 // recorded in the checking build; clamped in every build
  t = t < 0 ? 0 : (t >= vocab ? vocab - 1 : t);
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)t * hidden);
  uint4* dst = reinterpret_cast<uint4*>(x + (size_t)r * hidden);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = src[i];
}

// ----------------------------------------------------------------------------- RoPE tables for this step
// table[r][i] = (cos, sin)(pos_r * theta^(-2i/dim)), evaluated in fp64 and rounded to fp32.
__global__ void rope_table_kernel(const int* __restrict__ pos0, int rows, int dim, double theta, float2* __restrict__ out) {
  griddep_wait();
  griddep_launch();
  const int r = blockIdx.x, i = threadIdx.x;
  if (r >= rows || i >= dim / 2) return;
  const double inv = pow(theta, -2.0 * (double)i / (double)dim);
  const double ang = (double)(*pos0 + r) * inv;
  out[r * (dim / 2) + i] = make_float2((float)cos(ang), (float)sin(ang));
}

// ----------------------------------------------------------------------------- step prologue
// One launch for everything a step needs before its first projection: the input rows (embedding gather, or the
// draft block: anchor embedding + mask embeddings), the per-128-feature sums of squares of those rows (the first
// RMSNorm is fused into the projection that follows and only needs these partials) and the RoPE tables of the
// step's positions.  CTAs 0..15 take one row each, CTA 16 + t fills table t.
struct PrologueArgs {
  const int* tokens;               // mode 0: [rows] token ids; mode 1: [0] is the anchor token
  const __nv_bfloat16* table;      // [vocab][hidden]
  const __nv_bfloat16* mask;       // mode 1: [hidden] mask embedding of rows 1..rows-1
  __nv_bfloat16* x;                // [16][hidden]
  float* ssq;                      // [hidden/128][16]
  int hidden, rows, vocab, mode;
  int n_tabs;
  const int* tab_pos0[4];
  int tab_dim[4];
  double tab_theta[4];
  float2* tab_out[4];              // [rows][dim/2]
};

__global__ void __launch_bounds__(128) step_prologue_kernel(const PrologueArgs a) {
  griddep_wait();
  griddep_launch();
  if (blockIdx.x >= kMaxRows) {
    const int t = blockIdx.x - kMaxRows;
    const int half = a.tab_dim[t] / 2;
    const int p0 = *a.tab_pos0[t];
    for (int i = threadIdx.x; i < a.rows * half; i += 128) {
      const int r = i / half, c = i - r * half;
      const double inv = pow(a.tab_theta[t], -2.0 * (double)c / (double)a.tab_dim[t]);
      const double ang = (double)(p0 + r) * inv;
      a.tab_out[t][i] = make_float2((float)cos(ang), (float)sin(ang));
    }
    return;
  }
  const int r = blockIdx.x;
  const uint4* src = nullptr;
  if (r < a.rows) {
    if (a.mode == 0 || r == 0) {
      int t = a.tokens[r];
      (void)NRT_INDEX_OK(t, a.vocab, kBoundsToken);
      t = t < 0 ? 0 : (t >= a.vocab ? a.vocab - 1 : t);
      src = reinterpret_cast<const uint4*>(a.table + (size_t)t * a.hidden);
    } else {
      src = reinterpret_cast<const uint4*>(a.mask);
    }
  }
  uint4* dst = reinterpret_cast<uint4*>(a.x + (size_t)r * a.hidden);
  // 16 consecutive threads cover one 128-feature tile
  for (int i = threadIdx.x; i < a.hidden / 8; i += 128) {
    const uint4 v = src ? src[i] : make_uint4(0u, 0u, 0u, 0u);
    dst[i] = v;
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); ss += f.x * f.x + f.y * f.y; }
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if ((i & 15) == 0) a.ssq[(i >> 4) * kMaxRows + r] = ss;
  }
}

// ----------------------------------------------------------------------------- RMSNorm (+ e4m3 packet)
// One CTA per row (16 CTAs; rows >= `rows` are zero-filled so the padded GEMM operand is clean).
// xn = bf16(x * rsqrt(mean(x^2) + eps) * g); optional packet: e4m3(xn / s) with one power-of-two
// scale s per 128 channels.
__global__ void __launch_bounds__(256)
prep_norm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma, int hidden, int rows,
                 float eps, __nv_bfloat16* __restrict__ xn, uint8_t* __restrict__ x8, float* __restrict__ xs) {
  __shared__ float red[8];
  griddep_wait();
  griddep_launch();
  const int r = blockIdx.x;
  const int per = hidden / 8;              // 8-element vectors per row
  if (r >= rows) {
    for (int i = threadIdx.x; i < per; i += 256) {
      if (xn) reinterpret_cast<uint4*>(xn + (size_t)r * hidden)[i] = make_uint4(0, 0, 0, 0);
      if (x8) reinterpret_cast<uint2*>(x8 + (size_t)r * hidden)[i] = make_uint2(0, 0);
    }
    if (xs) for (int i = threadIdx.x; i < hidden / 128; i += 256) xs[(size_t)r * (hidden / 128) + i] = 1.f;
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)r * hidden);
  float ss = 0.f;
  for (int i = threadIdx.x; i < per; i += 256) {
    uint4 v = src[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(h[j]); ss += f.x * f.x + f.y * f.y; }
  }
  ss = block_sum<256>(ss, red);
  const float rs = rsqrtf(ss / (float)hidden + eps);
  for (int i = threadIdx.x; i < per; i += 256) {
    uint4 v = src[i];
    uint4 gv = reinterpret_cast<const uint4*>(gamma)[i];
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv);
    float o[8];
    float am = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(h[j]);
      float2 g = __bfloat1622float2(gh[j]);
      o[2 * j] = round_bf16(f.x * rs * g.x);
      o[2 * j + 1] = round_bf16(f.y * rs * g.y);
      am = fmaxf(am, fmaxf(fabsf(o[2 * j]), fabsf(o[2 * j + 1])));
    }
    if (xn) {
      uint4 w;
      __nv_bfloat162* wh = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
      for (int j = 0; j < 4; ++j) wh[j] = __floats2bfloat162_rn(o[2 * j], o[2 * j + 1]);
      reinterpret_cast<uint4*>(xn + (size_t)r * hidden)[i] = w;
    }
    if (x8) {
      // 16 consecutive threads cover one 128-channel block
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, off));
      const float s = pow2_scale(am);
      uint2 q;
      uint8_t* qb = reinterpret_cast<uint8_t*>(&q);
#pragma unroll
      for (int j = 0; j < 8; ++j) qb[j] = to_e4m3(o[j] / s);
      reinterpret_cast<uint2*>(x8 + (size_t)r * hidden)[i] = q;
      if ((i & 15) == 0) xs[(size_t)r * (hidden / 128) + (i >> 4)] = s;
    }
  }
}

// ----------------------------------------------------------------------------- q/k/v post-processing
// One CTA per row; warps take whole heads.
__global__ void __launch_bounds__(256) attn_post_kernel(const AttnPostArgs a) {
  __shared__ float red[8];
  __shared__ float kbuf[256];
  griddep_wait();
  griddep_launch();
  const int r = blockIdx.x;
  if (r >= a.rows) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* src = a.qkv + (size_t)r * a.ld;
  const int pos = *a.pos0 + r;
  const size_t slot = a.ring > 0 ? (size_t)(pos % a.ring) : (a.ring < 0 ? (size_t)r : (size_t)pos);
  const float2* rt = a.rope + (size_t)r * (a.rope_dim / 2);

  // q heads and k heads: [optional head RMS norm] -> bf16 -> RoPE on adjacent pairs -> bf16
  const int qk_heads = a.heads + a.kv_heads;
  const int part = blockIdx.y, parts = gridDim.y;          // heads are spread over grid.y CTAs per row
  for (int h = part * 8 + warp; h < qk_heads; h += 8 * parts) {
    const bool is_q = h < a.heads;
    const float* hs = is_q ? src + a.col_q + h * a.head_dim : src + a.col_k + (h - a.heads) * a.head_dim;
    __nv_bfloat16* dst = is_q ? a.q_out + ((size_t)r * a.heads + h) * a.head_dim
                              : a.k_cache + (slot * a.kv_heads + (h - a.heads)) * a.head_dim;
    const __nv_bfloat16* nw = is_q ? a.q_norm : a.k_norm;
    float rs = 1.f;
    if (nw) {
      float ss = 0.f;
      for (int d = lane; d < a.head_dim; d += 32) { const float v = round_bf16(hs[d]); ss += v * v; }
      ss = warp_sum(ss);
      rs = rsqrtf(ss / (float)a.head_dim + a.norm_eps);
    }
    for (int i = lane; i < a.head_dim / 2; i += 32) {
      float x0 = round_bf16(hs[2 * i]), x1 = round_bf16(hs[2 * i + 1]);
      if (nw) {
        x0 = round_bf16(x0 * rs * __bfloat162float(nw[2 * i]));
        x1 = round_bf16(x1 * rs * __bfloat162float(nw[2 * i + 1]));
      }
      if (2 * i < a.rope_dim) rope_pair(x0, x1, rt[i]);
      reinterpret_cast<__nv_bfloat162*>(dst)[i] = __floats2bfloat162_rn(x0, x1);
    }
  }
  // v heads
  if (part == parts - 1)
    for (int i = threadIdx.x; i < a.kv_heads * a.v_dim; i += 256)
      a.v_cache[slot * a.kv_heads * a.v_dim + i] = __float2bfloat16_rn(src[a.col_v + i] * a.value_scale);

  if (a.idx_heads == 0) return;
  const float2* it = a.idx_rope_tab + (size_t)r * (a.idx_rope / 2);
  // indexer queries: bf16 -> RoPE -> bf16 -> e4m3 with a per-(row, head) scale folded into the head weight
  for (int h = part * 8 + warp; h < a.idx_heads; h += 8 * parts) {
    const float* hs = src + a.col_iq + h * a.idx_dim;
    float v[8];                                   // idx_dim <= 256: 4 pairs per lane
    float am = 0.f;
    const int pairs = a.idx_dim / 2;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int i = lane + 32 * t;
      float x0 = 0.f, x1 = 0.f;
      if (i < pairs) {
        x0 = round_bf16(hs[2 * i]);
        x1 = round_bf16(hs[2 * i + 1]);
        if (2 * i < a.idx_rope) { rope_pair(x0, x1, it[i]); x0 = round_bf16(x0); x1 = round_bf16(x1); }
      }
      v[2 * t] = x0;
      v[2 * t + 1] = x1;
      am = fmaxf(am, fmaxf(fabsf(x0), fabsf(x1)));
    }
    am = warp_max(am);
    const float s = am > 0.f ? am / 448.f : 1.f;
    uint8_t* dst = a.iq8 + ((size_t)r * a.idx_heads + h) * a.idx_dim;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const int i = lane + 32 * t;
      if (i < pairs) { dst[2 * i] = to_e4m3(v[2 * t] / s); dst[2 * i + 1] = to_e4m3(v[2 * t + 1] / s); }
    }
    if (lane == 0) {
      if (a.iq_scale) { a.ihw[r * a.idx_heads + h] = src[a.col_iw + h] * a.idx_weight_scale; a.iq_scale[r * a.idx_heads + h] = s; }
      else a.ihw[r * a.idx_heads + h] = src[a.col_iw + h] * a.idx_weight_scale * s;
    }
  }
  // indexer key: LayerNorm (fp32) -> bf16 -> RoPE -> bf16 -> e4m3 with a per-row scale amax/448
  if (part == 0) {
    const int d = threadIdx.x;
    const float kv = d < a.idx_dim ? src[a.col_ik + d] : 0.f;
    const float mean = block_sum<256>(kv, red) / (float)a.idx_dim;
    const float dv = d < a.idx_dim ? kv - mean : 0.f;
    const float var = block_sum<256>(dv * dv, red) / (float)a.idx_dim;
    float kn = 0.f;
    if (d < a.idx_dim)
      kn = round_bf16(dv * rsqrtf(var + a.ln_eps) * __bfloat162float(a.ik_w[d]) + __bfloat162float(a.ik_b[d]));
    kbuf[d] = kn;
    __syncthreads();
    if (d < a.idx_rope) {
      float x0 = kbuf[d & ~1], x1 = kbuf[d | 1];
      rope_pair(x0, x1, it[d >> 1]);
      kn = round_bf16((d & 1) ? x1 : x0);
    }
    const float am = block_max<256>(d < a.idx_dim ? fabsf(kn) : 0.f, red);
    const float s = am > 0.f ? am / 448.f : 1.f;
    if (d < a.idx_dim) a.ik_cache[(size_t)pos * a.idx_dim + d] = to_e4m3(kn / s);
    if (d == 0) a.ik_scale[pos] = s;
  }
}

// ----------------------------------------------------------------------------- row attention
struct AttnArgs {
  const __nv_bfloat16* q;        // [rows][heads][head_dim]
  const __nv_bfloat16* k_cache;  // [cap][kv_heads][head_dim]
  const __nv_bfloat16* v_cache;  // [cap][kv_heads][v_dim]
  const int* pos0;
  int rows, heads, kv_heads, head_dim, v_dim;
  float scale;
  int mode;                      // 0: sliding window (ring)   1: dense [0, pos] or index list   2: draft block
  int window, ring;
  const __nv_bfloat16* sink;     // [heads] or null
  const int* sel;                // mode 1: [16][top_k] ascending key ids (used when pos + 1 > top_k)
  int top_k;
  const __nv_bfloat16* k_blk;    // mode 2: block rows' own keys/values [rows][kv_heads][dim]
  const __nv_bfloat16* v_blk;
  // outputs: bf16 o [rows][heads*v_dim], and/or the e4m3 packet (one K block per head when v_dim == 128)
  __nv_bfloat16* o_bf16;
  uint8_t* o8;
  float* o_scale;                // [16][heads*v_dim/128]
  // key-split: grid.z CTAs share one (head, row); partial (max, sum, acc) go through `part`
  // and the last CTA to arrive merges them in split order.
  float* part;                   // [16][heads][splits][v_dim + 2]
  unsigned int* tickets;         // [16][heads], zero between launches
  unsigned long long* stamps;   // opt-in phase stamps of the tensor-core decode kernel (%globaltimer, ns), [CTA][8]; null: none
};

// One CTA (128 threads) per (head, row); keys are processed in chunks of 128 with an online softmax.
// Each chunk's K and V rows are staged in shared memory with one wave of independent 16-byte
// loads (a single L2 round trip), then scored warp-per-key and accumulated thread-per-channel.
constexpr int kAttnChunk = 128;
constexpr int kAttnKPad = 8;       // bf16 elements of row padding (keeps 16-byte alignment, breaks bank aliasing)

__device__ __forceinline__ const __nv_bfloat16* attn_key_ptr(const AttnArgs& a, int id, int g, bool value) {
  const int dim = value ? a.v_dim : a.head_dim;
  if (id < 0) return (value ? a.v_blk : a.k_blk) + ((size_t)(-id - 1) * a.kv_heads + g) * dim;
  const size_t slot = a.ring > 0 ? (size_t)(id % a.ring) : (size_t)id;
  return (value ? a.v_cache : a.k_cache) + (slot * a.kv_heads + g) * dim;
}

__global__ void __launch_bounds__(128) attn_rows_kernel(const AttnArgs a) {
  extern __shared__ uint4 attn_smem[];
  __shared__ float qs[256];
  __shared__ float sc[kAttnChunk];
  __shared__ float red[4];
  __shared__ int kid[kAttnChunk];
  griddep_wait();
  griddep_launch();
  const int h = blockIdx.x, r = blockIdx.y;
  if (r >= a.rows) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = h / (a.heads / a.kv_heads);
  const int p0 = *a.pos0;
  const int pos = p0 + r;
  const int kvec = a.head_dim / 8, vvec = a.v_dim / 8;            // uint4 per row
  const int kstride = (a.head_dim + kAttnKPad) / 8;                // uint4 per padded K row
  uint4* ks = attn_smem;
  uint4* vs = attn_smem + kAttnChunk * kstride;
  for (int d = tid; d < a.head_dim; d += 128)
    qs[d] = __bfloat162float(a.q[((size_t)r * a.heads + h) * a.head_dim + d]);

  int lo = 0, count = 0, ctx = 0;
  bool use_sel = false;
  if (a.mode == 0) { lo = max(0, pos - a.window + 1); count = pos - lo + 1; }
  else if (a.mode == 1) { use_sel = pos + 1 > a.top_k; count = use_sel ? a.top_k : pos + 1; }
  else { lo = max(0, p0 - a.window); ctx = p0 - lo; count = ctx + a.rows; }

  float m_run = -FLT_MAX, l_run = 0.f, acc = 0.f;      // acc: output channel tid (v_dim <= 128)
  const int splits = gridDim.z, sp = blockIdx.z;
  const int chunks = (count + kAttnChunk - 1) / kAttnChunk;
  const int per = (chunks + splits - 1) / splits;
  const int c_begin = sp * per * kAttnChunk, c_end = min(count, (sp + 1) * per * kAttnChunk);
  for (int c0 = c_begin; c0 < c_end; c0 += kAttnChunk) {
    const int n = min(kAttnChunk, c_end - c0);
    __syncthreads();                                   // previous chunk fully consumed
    if (tid < n) {
      const int j = c0 + tid;
      int id;                                          // negative = block row -(id+1) in mode 2
      if (a.mode == 1) id = use_sel ? a.sel[r * a.top_k + j] : j;
      else if (a.mode == 2) id = j < ctx ? lo + j : -(j - ctx) - 1;
      else id = lo + j;
      kid[tid] = id;
    }
    __syncthreads();
    for (int i = tid; i < n * kvec; i += 128) {
      const int t = i / kvec, c = i - t * kvec;
      ks[t * kstride + c] = reinterpret_cast<const uint4*>(attn_key_ptr(a, kid[t], g, false))[c];
    }
    for (int i = tid; i < n * vvec; i += 128) {
      const int t = i / vvec, c = i - t * vvec;
      vs[t * vvec + c] = reinterpret_cast<const uint4*>(attn_key_ptr(a, kid[t], g, true))[c];
    }
    __syncthreads();
    // scores: each warp takes keys warp, warp+4, ...; lanes split the head dimension
    for (int t = warp; t < n; t += 4) {
      const __nv_bfloat16* kp = reinterpret_cast<const __nv_bfloat16*>(ks + t * kstride);
      float s = 0.f;
      for (int d = lane * 2; d < a.head_dim; d += 64) {
        const float2 kv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(kp + d));
        s += qs[d] * kv.x + qs[d + 1] * kv.y;
      }
      s = warp_sum(s);
      if (lane == 0) sc[t] = s * a.scale;
    }
    __syncthreads();
    const float v = tid < n ? sc[tid] : -FLT_MAX;
    const float cm = block_max<128>(v, red);
    const float m_new = fmaxf(m_run, cm);
    const float e = tid < n ? __expf(v - m_new) : 0.f;
    __syncthreads();
    sc[tid] = e;
    const float cs = block_sum<128>(e, red);           // contains a __syncthreads after sc[] is written
    const float corr = __expf(m_run - m_new);
    l_run = l_run * corr + cs;
    acc *= corr;
    if (tid < a.v_dim) {
      const __nv_bfloat16* vp = reinterpret_cast<const __nv_bfloat16*>(vs) + tid;
#pragma unroll 8
      for (int t = 0; t < n; ++t) acc += sc[t] * __bfloat162float(vp[t * a.v_dim]);
    }
    m_run = m_new;
  }
  if (splits > 1) {
    __shared__ bool s_last;
    float* mine = a.part + (((size_t)r * a.heads + h) * splits + sp) * (a.v_dim + 2);
    if (tid < a.v_dim) mine[2 + tid] = acc;
    if (tid == 0) { mine[0] = m_run; mine[1] = l_run; }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const unsigned int t = atomicAdd(&a.tickets[r * a.heads + h], 1u);
      s_last = t == (unsigned)splits - 1;
      if (s_last) a.tickets[r * a.heads + h] = 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    m_run = -FLT_MAX; l_run = 0.f; acc = 0.f;
    for (int q = 0; q < splits; ++q) {                   // fixed merge order: deterministic
      const float* o = a.part + (((size_t)r * a.heads + h) * splits + q) * (a.v_dim + 2);
      const float mq = __ldcg(o), lq = __ldcg(o + 1);
      const float aq = tid < a.v_dim ? __ldcg(o + 2 + tid) : 0.f;
      const float m_new = fmaxf(m_run, mq);
      const float c_old = __expf(m_run - m_new), c_new = __expf(mq - m_new);
      l_run = l_run * c_old + lq * c_new;
      acc = acc * c_old + aq * c_new;
      m_run = m_new;
    }
  }
  if (a.sink) {                                   // extra softmax column that carries no value
    const float sv = __bfloat162float(a.sink[h]);
    const float m_new = fmaxf(m_run, sv);
    const float corr = __expf(m_run - m_new);
    l_run = l_run * corr + __expf(sv - m_new);
    acc *= corr;
  }
  const float o = tid < a.v_dim ? round_bf16(acc / l_run) : 0.f;
  const size_t col = (size_t)h * a.v_dim + tid;
  const size_t ldo = (size_t)a.heads * a.v_dim;
  if (a.o_bf16 && tid < a.v_dim) a.o_bf16[r * ldo + col] = __float2bfloat16_rn(o);
  if (a.o8) {
    const float am = block_max<128>(fabsf(o), red);
    const float s = pow2_scale(am);
    if (tid < a.v_dim) a.o8[r * ldo + col] = to_e4m3(o / s);
    if (tid == 0) a.o_scale[r * (ldo / 128) + h] = s;
  }
}

// ----------------------------------------------------------------------------- indexer logits (CUDA-core form)
// logit[r][t] = sum_h relu(q8[r,h] . k8[t]) * hw[r,h] * ks[t] for t <= pos_r.  Used for short
// contexts and as the cross-check of the tcgen05 sweep.
struct IndexArgs {
  const uint8_t* iq8;   // [16*heads][dim]
  const float* ihw;     // [16][heads]
  const uint8_t* ik;    // [cap][dim]
  const float* iks;     // [cap]
  const int* pos0;
  int rows, heads, dim, top_k;
  float* logits;        // [16][ld]
  int ld;
  const float* iq_scale;   // [16][heads] or null (scale already folded into ihw)
};

__global__ void __launch_bounds__(256) index_logits_simple_kernel(const IndexArgs a) {
  extern __shared__ float qf[];                    // [rows*heads][dim] as float
  griddep_wait();
  griddep_launch();
  const int p0 = *a.pos0;
  if (p0 + a.rows <= a.top_k) return;              // every row is still dense
  const int total = p0 + a.rows;
  const int nq = a.rows * a.heads;
  for (int i = threadIdx.x; i < nq * a.dim; i += 256) qf[i] = from_e4m3(a.iq8[i]);
  __syncthreads();
  for (int t = blockIdx.x * 256 + threadIdx.x; t < total; t += gridDim.x * 256) {
    float kf[128];
    const uint4* kp = reinterpret_cast<const uint4*>(a.ik + (size_t)t * a.dim);
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      if (v * 16 < a.dim) {
        uint4 w = kp[v];
        const uint8_t* b = reinterpret_cast<const uint8_t*>(&w);
#pragma unroll
        for (int j = 0; j < 16; ++j) kf[v * 16 + j] = from_e4m3(b[j]);
      }
    }
    const float ks = a.iks[t];
    for (int r = 0; r < a.rows; ++r) {
      float lg = 0.f;
      for (int h = 0; h < a.heads; ++h) {
        const float* q = qf + (r * a.heads + h) * a.dim;
        float d = 0.f;
#pragma unroll 16
        for (int j = 0; j < a.dim; ++j) d += q[j] * kf[j];
        lg += fmaxf(d, 0.f) * (a.ihw[r * a.heads + h] * (a.iq_scale ? a.iq_scale[r * a.heads + h] : 1.f));
      }
      a.logits[(size_t)r * a.ld + t] = lg * ks;
    }
  }
}

// ----------------------------------------------------------------------------- exact top-k
// Per row: the k largest logits among positions [0, pos_r], ties to the lowest index, emitted
// in ascending position order.  Four 8-bit radix passes over order-preserving 32-bit keys
// find the threshold; one ordered sweep compacts the winners.
__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One CTA per row.  Thread t owns the contiguous index segment [t * per, (t + 1) * per) (16-byte loads, the warp
// covers a contiguous span), so the final sweep can emit winners in ascending index order from one block-wide
// prefix sum.  Each radix pass builds a 256-bin shared histogram; warp 0 locates the threshold bin with a
// shuffle scan (lane l owns bins 255 - 8l .. 248 - 8l).
__global__ void __launch_bounds__(1024) topk_rows_kernel(const float* __restrict__ logits, int ld, const int* pos0,
                                                         int rows, int top_k, int* __restrict__ sel) {
  __shared__ uint32_t hist[256];
  __shared__ uint32_t s_prefix, s_need;
  __shared__ uint32_t wsum_gt[32], wsum_eq[32];
  griddep_wait();
  griddep_launch();
  const int r = blockIdx.x;
  if (r >= rows) return;
  const int n = *pos0 + r + 1;
  if (n <= top_k) return;                           // dense row: no selection needed
  const float* row = logits + (size_t)r * ld;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool vec = ((reinterpret_cast<uintptr_t>(row) & 15) == 0);
  const int per = (((n + 1023) / 1024) + 3) & ~3;   // elements per thread, a multiple of 4
  const int lo = tid * per, hi = min(n, lo + per);

  // Rows of up to 16,384 keys: a thread's (at most sixteen) keys are loaded once and stay in registers for the four
  // radix passes and the final sweep, instead of five trips to L2.
  constexpr int kCache = 16;
  const bool cached = per <= kCache;
  uint32_t kc[kCache];
  uint32_t vmask = 0u;
  if (cached) {
#pragma unroll
    for (int q = 0; q < kCache; q += 4) {
      const int i = lo + q;
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      if (q < per && i < hi) {
        if (vec && i + 4 <= n) { const float4 f = *reinterpret_cast<const float4*>(row + i); v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w; }
        else { for (int c = 0; c < 4; ++c) v[c] = i + c < n ? row[i + c] : 0.f; }
      }
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        kc[q + c] = order_key(v[c]);
        if (q < per && i + c < hi) vmask |= 1u << (q + c);
      }
    }
  }
  uint32_t prefix = 0, mask = 0, need = top_k;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    if (cached) {
#pragma unroll
      for (int q = 0; q < kCache; ++q)
        if (((vmask >> q) & 1u) && (kc[q] & mask) == prefix) atomicAdd(&hist[(kc[q] >> shift) & 255u], 1u);
    } else {
      for (int i = lo; i < hi; i += 4) {
        float v[4];
        if (vec && i + 4 <= n) { const float4 f = *reinterpret_cast<const float4*>(row + i); v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w; }
        else { for (int c = 0; c < 4; ++c) v[c] = i + c < n ? row[i + c] : 0.f; }
#pragma unroll
        for (int c = 0; c < 4; ++c)
          if (i + c < hi) {
            const uint32_t k = order_key(v[c]);
            if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1u);
          }
      }
    }
    __syncthreads();
    if (warp == 0) {
      uint32_t c[8], tot = 0;
#pragma unroll
      for (int b = 0; b < 8; ++b) { c[b] = hist[255 - 8 * lane - b]; tot += c[b]; }
      uint32_t incl = tot;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += t; }
      const uint32_t excl = incl - tot;
      // the first lane whose bins reach `need` (bin 0 takes the rest, as a sequential walk from bin 255 would)
      const bool hit = incl >= need || lane == 31;
      const int first = __ffs(__ballot_sync(0xffffffffu, hit)) - 1;
      if (lane == first) {
        uint32_t acc = excl;
        int b = 0;
        for (; b < 8; ++b) {
          if (255 - 8 * lane - b == 0) break;
          if (acc + c[b] >= need) break;
          acc += c[b];
        }
        s_prefix = prefix | ((uint32_t)(255 - 8 * lane - b) << shift);
        s_need = need - acc;                                     // winners still to take from inside that bin
      }
    }
    __syncthreads();
    prefix = s_prefix;
    need = s_need;
    mask |= 255u << shift;
  }
  // prefix = exact threshold key; `need` elements equal to it are taken, lowest index first
  const uint32_t thr = prefix;
  unsigned long long m_gt = 0ull, m_eq = 0ull;      // winners of this thread's segment (per <= 64: rows up to 65536)
  if (cached) {
#pragma unroll
    for (int q = 0; q < kCache; ++q)
      if ((vmask >> q) & 1u) {
        if (kc[q] > thr) m_gt |= 1ull << q;
        else if (kc[q] == thr) m_eq |= 1ull << q;
      }
  } else if (per <= 64) {
    for (int i = lo; i < hi; i += 4) {
      float v[4];
      if (vec && i + 4 <= n) { const float4 f = *reinterpret_cast<const float4*>(row + i); v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w; }
      else { for (int c = 0; c < 4; ++c) v[c] = i + c < n ? row[i + c] : 0.f; }
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (i + c < hi) {
          const uint32_t k = order_key(v[c]);
          if (k > thr) m_gt |= 1ull << (i + c - lo);
          else if (k == thr) m_eq |= 1ull << (i + c - lo);
        }
    }
  }
  if (per <= 64) {
    const uint32_t my_gt = __popcll(m_gt), my_eq = __popcll(m_eq);
    uint32_t ig = my_gt, ie = my_eq;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t tg = __shfl_up_sync(0xffffffffu, ig, o), te = __shfl_up_sync(0xffffffffu, ie, o);
      if (lane >= o) { ig += tg; ie += te; }
    }
    if (lane == 31) { wsum_gt[warp] = ig; wsum_eq[warp] = ie; }
    __syncthreads();
    uint32_t bg = 0, be = 0;
    for (int w = 0; w < warp; ++w) { bg += wsum_gt[w]; be += wsum_eq[w]; }
    uint32_t gt_before = bg + ig - my_gt, eq_before = be + ie - my_eq;
    uint32_t out = gt_before + min(eq_before, need);
    for (int i = lo; i < hi; ++i) {
      const unsigned long long bit = 1ull << (i - lo);
      if (m_gt & bit) { if (out < (uint32_t)top_k) sel[r * top_k + out] = i; ++out; }
      else if (m_eq & bit) {
        if (eq_before < need) { if (out < (uint32_t)top_k) sel[r * top_k + out] = i; ++out; }
        ++eq_before;
      }
    }
    return;
  }
  // rows longer than 65536 entries: chunked ordered sweep (1024 consecutive indices at a time)
  __shared__ uint32_t base_out, base_eq;
  if (tid == 0) { base_out = 0; base_eq = 0; }
  __syncthreads();
  for (int c0 = 0; c0 < n; c0 += 1024) {
    const int i = c0 + tid;
    const uint32_t k = i < n ? order_key(row[i]) : 0u;
    const bool gt = i < n && k > thr;
    const bool eq = i < n && k == thr;
    const uint32_t bgm = __ballot_sync(0xffffffffu, gt), bem = __ballot_sync(0xffffffffu, eq);
    if (lane == 0) { wsum_gt[warp] = __popc(bgm); wsum_eq[warp] = __popc(bem); }
    __syncthreads();
    uint32_t eq_before = base_eq, gt_before = 0;
    for (int w = 0; w < warp; ++w) { eq_before += wsum_eq[w]; gt_before += wsum_gt[w]; }
    const uint32_t lm = (1u << lane) - 1u;
    const uint32_t my_eq_rank = eq_before + __popc(bem & lm);
    const uint32_t taken_eq_before = min(my_eq_rank, need) - min(base_eq, need);
    const uint32_t outpos = base_out + gt_before + __popc(bgm & lm) + taken_eq_before;
    if ((gt || (eq && my_eq_rank < need)) && outpos < (uint32_t)top_k) sel[r * top_k + outpos] = i;
    __syncthreads();
    if (tid == 0) {
      uint32_t tg = 0, te = 0;
      for (int w = 0; w < 32; ++w) { tg += wsum_gt[w]; te += wsum_eq[w]; }
      const uint32_t new_eq = base_eq + te;
      base_out += tg + (min(new_eq, need) - min(base_eq, need));
      base_eq = new_eq;
    }
    __syncthreads();
  }
}

// ----------------------------------------------------------------------------- exact top-k, many CTAs per row
// Long contexts (hundreds of thousands of keys): `gridDim.x` CTAs share one row.  Four histogram launches
// fix the 32-bit threshold one byte at a time (per-CTA shared histograms merged with one global add per
// non-empty bin; the last CTA of a row picks the bin), one launch counts winners per CTA segment and one
// writes them in ascending position order at offsets derived from the per-segment counts.  Same result as
// topk_rows_kernel: value descending, ties to the lowest index, emitted in ascending index order.
struct TopkGridState {          // per row
  unsigned int prefix, need, ticket, pad;
  unsigned int hist[256];
  unsigned int seg_gt[64], seg_eq[64];
};

__global__ void __launch_bounds__(1024) topk_grid_hist_kernel(const float* __restrict__ logits, int ld, const int* pos0,
                                                               int rows, int top_k, TopkGridState* st, int pass) {
  __shared__ unsigned int sh[256];
  __shared__ bool s_last;
  griddep_wait();
  griddep_launch();
  const int r = blockIdx.y;
  const int n = *pos0 + r + 1;
  if (r >= rows || n <= top_k) return;
  TopkGridState& S = st[r];
  const int shift = 24 - 8 * pass;
  const unsigned int mask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
  const unsigned int prefix = pass == 0 ? 0u : S.prefix;
  if (threadIdx.x < 256) sh[threadIdx.x] = 0u;
  __syncthreads();
  const int seg = (n + gridDim.x - 1) / gridDim.x;
  const int lo = blockIdx.x * seg, hi = min(n, lo + seg);
  const float* row = logits + (size_t)r * ld;
  for (int i = lo + threadIdx.x; i < hi; i += 1024) {
    const unsigned int k = order_key(row[i]);
    if ((k & mask) == prefix) atomicAdd(&sh[(k >> shift) & 255u], 1u);
  }
  __syncthreads();
  if (threadIdx.x < 256 && sh[threadIdx.x]) atomicAdd(&S.hist[threadIdx.x], sh[threadIdx.x]);
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int t = atomicAdd(&S.ticket, 1u);
    s_last = t == gridDim.x - 1;
    if (s_last) S.ticket = 0u;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (threadIdx.x == 0) {
    unsigned int need = pass == 0 ? (unsigned)top_k : S.need, acc = 0;
    int b = 255;
    for (; b > 0; --b) {
      const unsigned int h = *reinterpret_cast<volatile unsigned int*>(&S.hist[b]);
      if (acc + h >= need) break;
      acc += h;
    }
    S.prefix = prefix | ((unsigned int)b << shift);
    S.need = need - acc;
  }
  __syncthreads();
  if (threadIdx.x < 256) S.hist[threadIdx.x] = 0u;
}

__global__ void __launch_bounds__(1024) topk_grid_count_kernel(const float* __restrict__ logits, int ld, const int* pos0,
                                                                int rows, int top_k, TopkGridState* st) {
  __shared__ unsigned int s_gt, s_eq;
  griddep_wait();
  griddep_launch();
  const int r = blockIdx.y;
  const int n = *pos0 + r + 1;
  if (r >= rows || n <= top_k) return;
  TopkGridState& S = st[r];
  if (threadIdx.x == 0) { s_gt = 0u; s_eq = 0u; }
  __syncthreads();
  const unsigned int thr = S.prefix;
  const int seg = (n + gridDim.x - 1) / gridDim.x;
  const int lo = blockIdx.x * seg, hi = min(n, lo + seg);
  const float* row = logits + (size_t)r * ld;
  unsigned int gt = 0, eq = 0;
  for (int i = lo + threadIdx.x; i < hi; i += 1024) {
    const unsigned int k = order_key(row[i]);
    gt += k > thr;
    eq += k == thr;
  }
  if (gt) atomicAdd(&s_gt, gt);
  if (eq) atomicAdd(&s_eq, eq);
  __syncthreads();
  if (threadIdx.x == 0) { S.seg_gt[blockIdx.x] = s_gt; S.seg_eq[blockIdx.x] = s_eq; }
}

__global__ void __launch_bounds__(1024) topk_grid_write_kernel(const float* __restrict__ logits, int ld, const int* pos0,
                                                                int rows, int top_k, TopkGridState* st, int* __restrict__ sel) {
  __shared__ uint32_t wsum_gt[32], wsum_eq[32];
  __shared__ uint32_t base_out, base_eq;
  griddep_wait();
  griddep_launch();
  const int r = blockIdx.y;
  const int n = *pos0 + r + 1;
  if (r >= rows || n <= top_k) return;
  const TopkGridState& S = st[r];
  const unsigned int thr = S.prefix, need = S.need;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    unsigned int g = 0, e = 0;
    for (int c = 0; c < (int)blockIdx.x; ++c) { g += S.seg_gt[c]; e += S.seg_eq[c]; }
    base_eq = e;
    base_out = g + min(e, need);
  }
  __syncthreads();
  const int seg = (n + gridDim.x - 1) / gridDim.x;
  const int lo = blockIdx.x * seg, hi = min(n, lo + seg);
  const float* row = logits + (size_t)r * ld;
  for (int c0 = lo; c0 < hi; c0 += 1024) {
    const int i = c0 + tid;
    const unsigned int k = i < hi ? order_key(row[i]) : 0u;
    const bool gt = i < hi && k > thr;
    const bool eq = i < hi && k == thr;
    const uint32_t bg = __ballot_sync(0xffffffffu, gt), be = __ballot_sync(0xffffffffu, eq);
    if (lane == 0) { wsum_gt[warp] = __popc(bg); wsum_eq[warp] = __popc(be); }
    __syncthreads();
    uint32_t eq_before = base_eq, gt_before = 0;
    for (int w = 0; w < warp; ++w) { eq_before += wsum_eq[w]; gt_before += wsum_gt[w]; }
    const uint32_t lm = (1u << lane) - 1u;
    const uint32_t my_eq_rank = eq_before + __popc(be & lm);
    const uint32_t taken_eq_before = min(my_eq_rank, need) - min(base_eq, need);
    const uint32_t outpos = base_out + gt_before + __popc(bg & lm) + taken_eq_before;
    if ((gt || (eq && my_eq_rank < need)) && outpos < (uint32_t)top_k) sel[r * top_k + outpos] = i;
    __syncthreads();
    if (tid == 0) {
      uint32_t tg = 0, te = 0;
      for (int w = 0; w < 32; ++w) { tg += wsum_gt[w]; te += wsum_eq[w]; }
      const uint32_t new_eq = base_eq + te;
      base_out += tg + (min(new_eq, need) - min(base_eq, need));
      base_eq = new_eq;
    }
    __syncthreads();
  }
}

// ----------------------------------------------------------------------------- MoE router
// grid = experts / 2 CTAs: one CTA computes 2 experts x 16 rows; the last CTA to finish performs the per-row
// top-k and builds the ascending active-expert list.
__global__ void __launch_bounds__(256) router_kernel(const RouterArgs a_in) {
  // grid.y row groups of 16 rows (prefill chunks): each group is routed independently
  RouterArgs a = a_in;
  if (gridDim.y > 1) {
    const int g0 = blockIdx.y * kMaxRows;
    a.xn = a_in.xn + (size_t)g0 * a_in.hidden;
    a.rows = min(kMaxRows, a_in.rows - g0);
    a.scores = a_in.scores + (size_t)g0 * a_in.experts;
    a.ticket = a_in.ticket + blockIdx.y;
    a.topk_ids = a_in.topk_ids + (size_t)g0 * a_in.top_k;
    a.topk_p = a_in.topk_p + (size_t)g0 * a_in.top_k;
  }
  __shared__ RouterSmem sm;
  __shared__ bool last;
  const int tid = threadIdx.x;
  unsigned long long* stamp = (a.stamps && gridDim.y == 1) ? a.stamps + (size_t)blockIdx.x * 16 : nullptr;
  if (stamp && tid == 0) stamp[0] = globaltimer();
  if (a.w == nullptr) {
    // selection only: the score matrix was filled by the caller (chunked prefill computes it as one fp32 matrix
    // product for thousands of rows); one CTA per group of 16 rows
    griddep_wait();
    griddep_launch();
    router_select(a, sm, true, nullptr, nullptr, nullptr);
    return;
  }
  router_scores(a, blockIdx.x, gridDim.x, sm, stamp);
  // The CTA's score stores are ordered before the ticket by the barrier (CTA scope) followed by thread 0's fence
  // (cumulative, GPU scope); the last CTA reads the scores from L2 after the same pair on the acquiring side.
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const unsigned int t = atomicAdd(a.ticket, 1u);
    last = (t == gridDim.x - 1);
    if (last) { *a.ticket = 0u; __threadfence(); }
    if (stamp) stamp[1] = globaltimer();
  }
  __syncthreads();
  // the activation packet is off the selection's critical path: the other CTAs write their share while the last
  // one selects
  if (!last) { router_packet(a, blockIdx.x, gridDim.x, sm); return; }
  if (stamp && tid == 0) stamp[2] = globaltimer();
  router_select(a, sm, true, nullptr, nullptr, stamp);
  if (stamp && tid == 0) stamp[3] = globaltimer();
  router_packet(a, blockIdx.x, gridDim.x, sm);
}

}  // namespace

// ============================================================================= C ABI
#define S(stream) reinterpret_cast<cudaStream_t>(stream)

NRT_BOUNDS_EXPORT(target_kernels)
extern "C" int nrt_embed_rows(const int* tokens, const void* table, void* x, int hidden, int rows, int vocab,
                              void* stream, int pdl) {
  return launch_pdl(embed_rows_kernel, dim3(rows > kMaxRows ? rows : kMaxRows), dim3(128), 0, S(stream), pdl != 0, tokens,
                    (const __nv_bfloat16*)table, (__nv_bfloat16*)x, hidden, rows, vocab);
}
extern "C" int nrt_prologue_args_size() { return (int)sizeof(PrologueArgs); }
extern "C" int nrt_step_prologue(const void* args, void* stream, int pdl) {
  PrologueArgs a;
  memcpy(&a, args, sizeof(a));
  if (a.hidden % 128 || a.n_tabs < 0 || a.n_tabs > 4 || a.rows < 1 || a.rows > kMaxRows) return -3;
  return launch_pdl(step_prologue_kernel, dim3(kMaxRows + a.n_tabs), dim3(128), 0, S(stream), pdl != 0, a);
}
extern "C" int nrt_rope_table(const int* pos0, int rows, int dim, double theta, void* out, void* stream, int pdl) {
  return launch_pdl(rope_table_kernel, dim3(rows), dim3(dim / 2 < 32 ? 32 : dim / 2), 0, S(stream), pdl != 0, pos0, rows,
                    dim, theta, (float2*)out);
}
// rows <= 16: the operand is padded to 16 rows (dead rows zero-filled); larger row counts (prefill chunks)
// launch one CTA per row.
extern "C" int nrt_prep_norm(const void* x, const void* gamma, int hidden, int rows, float eps, void* xn, void* x8,
                             void* xs, void* stream, int pdl) {
  return launch_pdl(prep_norm_kernel, dim3(rows > kMaxRows ? rows : kMaxRows), dim3(256), 0, S(stream), pdl != 0, (const __nv_bfloat16*)x,
                    (const __nv_bfloat16*)gamma, hidden, rows, eps, (__nv_bfloat16*)xn, (uint8_t*)x8, (float*)xs);
}
extern "C" int nrt_attn_post_args_size() { return (int)sizeof(AttnPostArgs); }
extern "C" int nrt_attn_post(const void* args, void* stream, int pdl) {
  AttnPostArgs a;
  memcpy(&a, args, sizeof(a));
  const int heads = a.heads + a.kv_heads;
  const int parts = heads > 32 ? 8 : (heads > 8 ? 2 : 1);
  return launch_pdl(attn_post_kernel, dim3(a.rows, parts), dim3(256), 0, S(stream), pdl != 0, a);
}
extern "C" int nrt_attn_args_size() { return (int)sizeof(AttnArgs); }
extern "C" int nrt_attn_rows(const void* args, int splits, void* stream, int pdl) {
  AttnArgs a;
  memcpy(&a, args, sizeof(a));
  const size_t smem = (size_t)kAttnChunk * ((a.head_dim + kAttnKPad) + a.v_dim) * 2;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(attn_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024);
    configured = true;
  }
  if (a.head_dim % 8 || a.v_dim % 8 || a.head_dim > 256 || a.v_dim > 128 || smem > 128 * 1024) return -3;
  if (splits > 1 && (!a.part || !a.tickets)) return -3;
  return launch_pdl(attn_rows_kernel, dim3(a.heads, a.rows, splits < 1 ? 1 : splits), dim3(128), smem, S(stream), pdl != 0, a);
}
extern "C" int nrt_index_args_size() { return (int)sizeof(IndexArgs); }
extern "C" int nrt_index_logits_simple(const void* args, int blocks, void* stream, int pdl) {
  IndexArgs a;
  memcpy(&a, args, sizeof(a));
  const size_t smem = (size_t)a.rows * a.heads * a.dim * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(index_logits_simple_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    configured = true;
  }
  return launch_pdl(index_logits_simple_kernel, dim3(blocks), dim3(256), smem, S(stream), pdl != 0, a);
}
extern "C" int nrt_topk_rows(const float* logits, int ld, const int* pos0, int rows, int top_k, int* sel, void* stream,
                             int pdl) {
  return launch_pdl(topk_rows_kernel, dim3(rows), dim3(1024), 0, S(stream), pdl != 0, logits, ld, pos0, rows, top_k, sel);
}
extern "C" int nrt_topk_grid_state_bytes() { return (int)sizeof(TopkGridState); }
// ctas: CTAs per row (<= 64).  `state` holds rows x TopkGridState, zero-initialised once.
extern "C" int nrt_topk_rows_grid(const float* logits, int ld, const int* pos0, int rows, int top_k, int* sel, void* state,
                                  int ctas, void* stream, int pdl) {
  if (ctas < 1 || ctas > 64) return -3;
  TopkGridState* st = reinterpret_cast<TopkGridState*>(state);
  int rc;
  for (int pass = 0; pass < 4; ++pass)
    if ((rc = launch_pdl(topk_grid_hist_kernel, dim3(ctas, rows), dim3(1024), 0, S(stream), pdl != 0, logits, ld, pos0, rows,
                         top_k, st, pass)))
      return rc;
  if ((rc = launch_pdl(topk_grid_count_kernel, dim3(ctas, rows), dim3(1024), 0, S(stream), pdl != 0, logits, ld, pos0, rows,
                       top_k, st)))
    return rc;
  return launch_pdl(topk_grid_write_kernel, dim3(ctas, rows), dim3(1024), 0, S(stream), pdl != 0, logits, ld, pos0, rows,
                    top_k, st, sel);
}
extern "C" int nrt_router_args_size() { return (int)sizeof(RouterArgs); }
extern "C" int nrt_router(const void* args, void* stream, int pdl) {
  RouterArgs a;
  memcpy(&a, args, sizeof(a));
  const size_t smem = 0;
  if (a.x && (!a.ssq || !a.gamma || a.hidden % 128)) return -3;
  // the packet's (row, block) pairs are spread over the CTAs, 16 groups of 16 threads each
  if (a.x && a.x8 && (!a.xs || a.rows * (a.hidden / 128) > 16 * ((a.experts + 1) / 2))) return -3;
  const int groups = a.rows > kMaxRows ? (a.rows + kMaxRows - 1) / kMaxRows : 1;
  if (groups > 1 && (a.x || a.probs)) return -3;                      // row groups: plain routing of normed rows only
  if (!a.w && (!a.scores || a.x)) return -3;                          // selection only: needs the caller's score matrix
  return launch_pdl(router_kernel, dim3(a.w ? (a.experts + 1) / 2 : 1, groups), dim3(256), smem, S(stream), pdl != 0, a);
}

// ============================================================================= allocation-free routing
#include "no_alloc.h"

#include <mutex>

// Scratch of nrt_router_route_noalloc: score matrix followed by the arrival counter.  In host code this
// name is only a handle for cudaGetSymbolAddress; the device address is resolved once per device.
static __device__ __align__(256) unsigned char g_noalloc_router_scratch[NRT_NOALLOC_SCRATCH_BYTES];

extern "C" int nrt_router_route_noalloc(const void* xn, const float* w, const float* bias, int hidden, int experts, int rows,
                                        int top_k, int sigmoid, int normalize, float route_scale, int* n_active,
                                        int* active_ids, float* probs, int* topk_ids, float* topk_p, int max_slots,
                                        void* stream) {
  if (!xn || !w || !n_active || !active_ids || !probs || !topk_ids || !topk_p) return NRT_NOALLOC_E_ARG;
  if (rows < 1 || top_k < 1 || top_k > experts || max_slots < 1 || hidden < 4 || hidden % 4) return NRT_NOALLOC_E_ARG;
  if (rows > NRT_NOALLOC_MAX_ROWS || experts > NRT_NOALLOC_MAX_EXPERTS || top_k > 32) return NRT_NOALLOC_E_LIMIT;
  static std::mutex mu;
  static void* scratch_of_device[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return NRT_NOALLOC_E_SETUP;
  void* base = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!scratch_of_device[dev]) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_noalloc_router_scratch);       // with `dev` current
      if (e != cudaSuccess || !p) return e != cudaSuccess ? (int)e : NRT_NOALLOC_E_SETUP;
      scratch_of_device[dev] = p;
    }
    base = scratch_of_device[dev];
  }
  float* scores = reinterpret_cast<float*>(base);
  unsigned int* ticket = reinterpret_cast<unsigned int*>(reinterpret_cast<unsigned char*>(base) +
                                                         NRT_NOALLOC_MAX_ROWS * NRT_NOALLOC_MAX_EXPERTS * 4);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  e = cudaMemsetAsync(ticket, 0, sizeof(unsigned int), s);           // the counter must start at zero
  if (e != cudaSuccess) return (int)e;
  RouterArgs a;
  memset(&a, 0, sizeof(a));
  a.xn = reinterpret_cast<const __nv_bfloat16*>(xn);
  a.w = w;
  a.bias = bias;
  a.hidden = hidden; a.experts = experts; a.rows = rows; a.top_k = top_k;
  a.sigmoid = sigmoid; a.normalize = normalize; a.route_scale = route_scale;
  a.scores = scores; a.ticket = ticket;
  a.n_active = n_active; a.active_ids = active_ids; a.probs = probs;
  a.topk_ids = topk_ids; a.topk_p = topk_p; a.max_slots = max_slots;
  router_kernel<<<dim3((experts + 1) / 2), dim3(256), 0, s>>>(a);
  return (int)cudaGetLastError();
}

// MoE router shared by the stand-alone router kernel and the fused MoE layer kernel: two device phases.
//   router_scores : CTA `cta` computes the scores of experts 2*cta and 2*cta + 1 for every row (fp32 FMA over
//                   the fp32 router weights; RMSNorm applied on the fly from per-tile sums of squares) and
//                   quantises a few (row, 128-channel block) pairs of the e4m3 packet the expert GEMMs read.
//   router_select : per-row top-k (sigmoid + bias or softmax, ties to the lowest index, probabilities
//                   normalised over the choice) and the ascending list of distinct experts with each row's
//                   probability per list slot.
// Reference counterparts: naivert/body/rmsnorm_expert_proj/ (scores + prepared packet),
// naivert/body/expert_select_up_gate_silu/ (compute_route, distinct-expert item list).
#pragma once
#include "gemm.cuh"

#include <float.h>

namespace nrt {

constexpr int kRouterRows = 16;

struct RouterArgs {
  const __nv_bfloat16* xn;   // [16][hidden] normed activations (plain router) or null (inline-norm form)
  const __nv_bfloat16* x;    // inline-norm form: residual rows [16][hidden], normalised while they are read
  const __nv_bfloat16* gamma;
  float eps;
  const float* ssq;          // inline-norm form: [hidden/128][16] sums of squares of x per 128-feature tile
  float* xs;                 // inline-norm form: scales [16][hidden/128] of the e4m3 packet below (null: no packet)
  const float* w;            // [experts][hidden] fp32
  const float* bias;         // [experts] or null
  int hidden, experts, rows, top_k;
  int sigmoid;               // 1: sigmoid(+bias for the choice); 0: softmax
  int normalize;
  float route_scale;
  float* scores;             // [16][experts] scratch
  unsigned int* ticket;      // zero-initialised counter (reset by the last CTA)
  int* n_active;             // outputs
  int* active_ids;           // [max_slots]
  float* probs;              // [max_slots][16]
  int* topk_ids;             // [16][top_k]
  float* topk_p;             // [16][top_k]
  int max_slots;
  uint8_t* x8;               // inline-norm form: e4m3 packet [16][hidden] of the normalised rows for the expert GEMMs;
                             // each CTA quantises a few (row, 128-channel block) pairs, so nobody repeats the work
  // opt-in phase stamps of the router kernel (%globaltimer, ns), [CTA][16]: 0 entry, 12 upstream grid done, 13 row scales
  // ready, 14 dot products done, 1 scores published, 2 selection begins (last CTA), 10 choices made, 15 lists built, 3 end
  unsigned long long* stamps;
};


struct RouterSmem {
  float part[8][2][kRouterRows];
  float rs[kRouterRows];
  unsigned int used[8];            // bitmap over <= 256 experts
  int slot_of[256];
  int n_active;
  int tk_id[kRouterRows][32];      // per-row choices (top_k <= 32)
  float tk_p[kRouterRows][32];
};

__device__ __forceinline__ float router_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float router_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ uint32_t router_order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// 256 threads.  Waits for the upstream grid itself (after the loads that do not depend on it).
__device__ __forceinline__ void router_scores(const RouterArgs& a, int cta, int n_ctas, RouterSmem& sm, unsigned long long* stamp = nullptr) {
  constexpr int kMaxRows = kRouterRows;
  float (*part)[2][kMaxRows] = sm.part;
  float* rs_s = sm.rs;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int e0 = cta * 2;
  const bool inline_norm = a.x != nullptr;
  const bool fast = a.hidden == 4096;
  // The two experts' weights and the norm weights never depend on earlier kernels: their loads are issued before
  // this kernel waits for its predecessor, so the HBM round trip overlaps the predecessor's tail.
  float4 w0[4], w1[4], gm[4];
  if (fast) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = tid * 4 + 1024 * i;
      gm[i] = make_float4(1.f, 1.f, 1.f, 1.f);
      if (inline_norm) {
        const uint2 gv = __ldg(reinterpret_cast<const uint2*>(a.gamma + k));
        const float2 g01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gv.x));
        const float2 g23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gv.y));
        gm[i] = make_float4(g01.x, g01.y, g23.x, g23.y);
      }
      // CTAs beyond the expert list (a grid wider than experts / 2) read nothing
      w0[i] = (e0 < a.experts) ? __ldg(reinterpret_cast<const float4*>(a.w + (size_t)e0 * 4096 + k)) : make_float4(0, 0, 0, 0);
      w1[i] = (e0 + 1 < a.experts) ? __ldg(reinterpret_cast<const float4*>(a.w + (size_t)(e0 + 1) * 4096 + k)) : make_float4(0, 0, 0, 0);
    }
  }
  griddep_wait();
  griddep_launch();
  if (stamp && threadIdx.x == 0) stamp[12] = globaltimer();
  const __nv_bfloat16* xsrc = inline_norm ? a.x : a.xn;
  const int xld = a.hidden;
  const int blocks = a.hidden / 128;
  // The first four rows' activations are requested before anything waits (they do not depend on the row scales).
  uint2 xv[4][4];
  if (fast) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int rr = 0; rr < 4; ++rr)
        xv[i][rr] = (rr < a.rows) ? *reinterpret_cast<const uint2*>(xsrc + (size_t)rr * xld + tid * 4 + 1024 * i) : make_uint2(0u, 0u);
  }
  // 1 / rms per row from the per-tile sums of squares left behind by the producer of x.  (The phases below are rolled
  // loops with small bodies on purpose - a kernel that runs once per layer executes mostly cold code, and instruction
  // fetch is then the top stall reason.)
  if (inline_norm) {
#pragma unroll 1
    for (int r = warp; r < a.rows; r += 8) {
      float ss = 0.f;
#pragma unroll 1
      for (int t = lane; t < blocks; t += 32) ss += __ldcg(a.ssq + t * kMaxRows + r);
      ss = router_warp_sum(ss);
      if (lane == 0) rs_s[r] = rsqrtf(ss / (float)a.hidden + a.eps);
    }
    __syncthreads();
  }
  if (stamp && threadIdx.x == 0) stamp[13] = globaltimer();
  if (fast) {
    // four rows at a time: their sixteen loads are in flight together, then the FMAs, then the warp sums
#pragma unroll 1
    for (int r0 = 0; r0 < a.rows; r0 += 4) {
      if (r0 > 0) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int rr = 0; rr < 4; ++rr)
            xv[i][rr] = (r0 + rr < a.rows) ? *reinterpret_cast<const uint2*>(xsrc + (size_t)(r0 + rr) * xld + tid * 4 + 1024 * i)
                                           : make_uint2(0u, 0u);
      }
      float acc0[4], acc1[4];
#pragma unroll
      for (int rr = 0; rr < 4; ++rr) { acc0[rr] = 0.f; acc1[rr] = 0.f; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int rr = 0; rr < 4; ++rr) {
          float2 x01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xv[i][rr].x));
          float2 x23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xv[i][rr].y));
          if (inline_norm) {
            const float rs = rs_s[min(r0 + rr, kMaxRows - 1)];
            x01.x = round_bf16(x01.x * rs * gm[i].x); x01.y = round_bf16(x01.y * rs * gm[i].y);
            x23.x = round_bf16(x23.x * rs * gm[i].z); x23.y = round_bf16(x23.y * rs * gm[i].w);
          }
          acc0[rr] += x01.x * w0[i].x + x01.y * w0[i].y + x23.x * w0[i].z + x23.y * w0[i].w;
          acc1[rr] += x01.x * w1[i].x + x01.y * w1[i].y + x23.x * w1[i].z + x23.y * w1[i].w;
        }
#pragma unroll
      for (int rr = 0; rr < 4; ++rr) {
        const float v0 = router_warp_sum(acc0[rr]), v1 = router_warp_sum(acc1[rr]);
        if (lane == 0 && r0 + rr < a.rows) { part[warp][0][r0 + rr] = v0; part[warp][1][r0 + rr] = v1; }
      }
    }
  } else {
    // any other width: one row at a time, the K steps of a thread in ascending order
#pragma unroll 1
    for (int r = 0; r < a.rows; ++r) {
      float a0 = 0.f, a1 = 0.f;
      const float rs = inline_norm ? rs_s[r] : 1.f;
#pragma unroll 1
      for (int k = tid * 4; k < a.hidden; k += 1024) {
        const float4 v0 = (e0 < a.experts) ? *reinterpret_cast<const float4*>(a.w + (size_t)e0 * a.hidden + k) : make_float4(0, 0, 0, 0);
        const float4 v1 = (e0 + 1 < a.experts) ? *reinterpret_cast<const float4*>(a.w + (size_t)(e0 + 1) * a.hidden + k)
                                               : make_float4(0, 0, 0, 0);
        const uint2 xv = *reinterpret_cast<const uint2*>(xsrc + (size_t)r * xld + k);
        float2 x01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xv.x));
        float2 x23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xv.y));
        if (inline_norm) {
          const uint2 gv = *reinterpret_cast<const uint2*>(a.gamma + k);
          const float2 g01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gv.x));
          const float2 g23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gv.y));
          x01.x = round_bf16(x01.x * rs * g01.x); x01.y = round_bf16(x01.y * rs * g01.y);
          x23.x = round_bf16(x23.x * rs * g23.x); x23.y = round_bf16(x23.y * rs * g23.y);
        }
        a0 += x01.x * v0.x + x01.y * v0.y + x23.x * v0.z + x23.y * v0.w;
        a1 += x01.x * v1.x + x01.y * v1.y + x23.x * v1.z + x23.y * v1.w;
      }
      a0 = router_warp_sum(a0);
      a1 = router_warp_sum(a1);
      if (lane == 0) { part[warp][0][r] = a0; part[warp][1][r] = a1; }
    }
  }
  if (stamp && threadIdx.x == 0) stamp[14] = globaltimer();
  __syncthreads();
  if (tid < 2 * kMaxRows) {
    const int j = tid / kMaxRows, r = tid % kMaxRows;
    float s = 0.f;
#pragma unroll 1
    for (int w = 0; w < 8; ++w) s += part[w][j][r];
    if (e0 + j < a.experts && r < a.rows) a.scores[r * a.experts + e0 + j] = s;
  }
}

// This CTA's share of the e4m3 packet of the normalised rows (inline-norm form): pair (row, 128-channel block) number
// cta + n_ctas * g goes to the g-th group of 16 threads.  Uses the row scales router_scores left in shared memory.
__device__ __forceinline__ void router_packet(const RouterArgs& a, int cta, int n_ctas, RouterSmem& sm) {
  if (a.x == nullptr || a.x8 == nullptr) return;
  const int tid = threadIdx.x;
  const int blocks = a.hidden / 128;
  const int pairs = a.rows * blocks;
  const int my_pair = cta + n_ctas * (tid >> 4);
  const bool pk_on = my_pair < pairs;
  const int pk_r = pk_on ? my_pair % a.rows : 0, pk_b = pk_on ? my_pair / a.rows : 0;
  if (cta >= pairs) return;                          // no group of this CTA has a pair (uniform over the CTA)
  uint4 pk_x = make_uint4(0u, 0u, 0u, 0u), pk_g = pk_x;
  if (pk_on) {
    const int k = pk_b * 128 + (tid & 15) * 8;
    pk_x = *reinterpret_cast<const uint4*>(a.x + (size_t)pk_r * a.hidden + k);
    pk_g = __ldg(reinterpret_cast<const uint4*>(a.gamma + k));
  }
  const float rs = sm.rs[pk_r];
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pk_x);
  const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&pk_g);
  float o[8];
  float am = 0.f;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const float2 f = __bfloat1622float2(h[q]), g = __bfloat1622float2(gh[q]);
    o[2 * q] = round_bf16(f.x * rs * g.x);
    o[2 * q + 1] = round_bf16(f.y * rs * g.y);
    am = fmaxf(am, fmaxf(fabsf(o[2 * q]), fabsf(o[2 * q + 1])));
  }
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, off));
  const float sc = pow2_scale(am);
  const float inv = 1.0f / sc;                       // a power of two: the product is the exact quotient
  uint2 q8;
  uint8_t* qb = reinterpret_cast<uint8_t*>(&q8);
#pragma unroll
  for (int q = 0; q < 8; ++q) qb[q] = e4m3_bits(o[q] * inv);
  if (pk_on) {
    *reinterpret_cast<uint2*>(a.x8 + (size_t)pk_r * a.hidden + pk_b * 128 + (tid & 15) * 8) = q8;
    if ((tid & 15) == 0) a.xs[(size_t)pk_r * blocks + pk_b] = sc;
  }
}

// 256 threads; every score must be visible (the caller has synchronised the CTAs).  Results: sm.used / sm.slot_of /
// sm.n_active, and - when `publish` - the global outputs of RouterArgs.  `probs_s` / `active_s` (shared memory,
// may be null) receive the slot table for a consumer in the same CTA.
__device__ __forceinline__ void router_select(const RouterArgs& a, RouterSmem& sm, bool publish, float* probs_s, int* active_s,
                                              unsigned long long* stamp = nullptr) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  unsigned int* used = sm.used;
  int* slot_of = sm.slot_of;
  if (tid < 8) used[tid] = 0u;
  __syncthreads();
  // one warp per row: iterative arg-max with lowest-index ties
#pragma unroll 1
  for (int r = warp; r < a.rows; r += 8) {
    float sc[8], ch[8];                             // experts lane, lane+32, ... (<= 256 experts)
    // all sixteen loads (scores from L2, selection bias) are issued before anything depends on them
    float raw[8], bv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = min(lane + 32 * j, a.experts - 1);
      raw[j] = __ldcg(a.scores + r * a.experts + e);
      bv[j] = a.bias ? __ldg(a.bias + e) : 0.f;
    }
    float mx = -FLT_MAX;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const bool in = lane + 32 * j < a.experts;
      sc[j] = in ? raw[j] : -FLT_MAX;
      mx = fmaxf(mx, sc[j]);
    }
    if (a.sigmoid) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const bool in = lane + 32 * j < a.experts;
        sc[j] = in ? __frcp_rn(1.f + __expf(-sc[j])) : 0.f;      // rcp.rn == 1 / y, without the division's slow path
        ch[j] = in ? sc[j] + bv[j] : -FLT_MAX;
      }
    } else {
      mx = router_warp_max(mx);
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int e = lane + 32 * j;
        sc[j] = e < a.experts ? __expf(sc[j] - mx) : 0.f;
        sum += sc[j];
      }
      sum = router_warp_sum(sum);
#pragma unroll
      for (int j = 0; j < 8; ++j) { sc[j] /= sum; ch[j] = (lane + 32 * j) < a.experts ? sc[j] : -FLT_MAX; }
    }
    // Every lane sorts its eight candidates once (descending key, lower expert first among equals - the experts of
    // a lane ascend with j, and the network below never swaps equal keys out of order); a selection step is then
    // two warp reductions over the lanes' heads and a pop on the winning lane.
    uint32_t kk[8];                                 // order-preserving keys; 0 once taken
    uint32_t ee[8];                                 // expert of each candidate
#pragma unroll
    for (int j = 0; j < 8; ++j) { kk[j] = router_order_key(ch[j]); ee[j] = (uint32_t)(lane + 32 * j); }
#define NRT_CAS(i, j)                                                                                      \
    if (kk[j] > kk[i] || (kk[j] == kk[i] && ee[j] < ee[i])) {                                              \
      const uint32_t tk = kk[i]; kk[i] = kk[j]; kk[j] = tk;                                                \
      const uint32_t te = ee[i]; ee[i] = ee[j]; ee[j] = te;                                                \
      const float tp = sc[i]; sc[i] = sc[j]; sc[j] = tp;                                                   \
    }
    NRT_CAS(0, 1) NRT_CAS(2, 3) NRT_CAS(4, 5) NRT_CAS(6, 7)
    NRT_CAS(0, 2) NRT_CAS(1, 3) NRT_CAS(4, 6) NRT_CAS(5, 7)
    NRT_CAS(1, 2) NRT_CAS(5, 6) NRT_CAS(0, 4) NRT_CAS(3, 7)
    NRT_CAS(1, 5) NRT_CAS(2, 6)
    NRT_CAS(1, 4) NRT_CAS(3, 6)
    NRT_CAS(2, 4) NRT_CAS(3, 5)
    NRT_CAS(3, 4)
#undef NRT_CAS
    float psum = 0.f;
    float my_p = 0.f;
    int my_id = -1;
#pragma unroll 1
    for (int t = 0; t < a.top_k; ++t) {
      const uint32_t best = __reduce_max_sync(0xffffffffu, kk[0]);
      const int bi = (int)__reduce_min_sync(0xffffffffu, kk[0] == best ? ee[0] : 0xffffffffu);
      const float pv = __shfl_sync(0xffffffffu, sc[0], bi & 31);
      if ((bi & 31) == lane) {                      // pop the head of the winning lane
#pragma unroll
        for (int j = 0; j < 7; ++j) { kk[j] = kk[j + 1]; ee[j] = ee[j + 1]; sc[j] = sc[j + 1]; }
        kk[7] = 0u;
      }
      psum += pv;
      if (lane == t) { my_p = pv; my_id = bi; }
    }
    const float denom = a.normalize ? psum + 1e-20f : 1.f;
    if (lane < a.top_k) {
      const float p = my_p / denom * a.route_scale;
      sm.tk_id[r][lane] = my_id;
      sm.tk_p[r][lane] = p;
      if (publish && a.topk_ids) a.topk_ids[r * a.top_k + lane] = my_id;
      if (publish && a.topk_p) a.topk_p[r * a.top_k + lane] = p;
      atomicOr(&used[my_id >> 5], 1u << (my_id & 31));
    }
  }
  if (stamp && threadIdx.x == 0) stamp[10] = globaltimer();
  __syncthreads();
  if (a.probs == nullptr && probs_s == nullptr) return;   // prefill: only the per-token choices are needed
  // ascending list of distinct experts -> slots
  if (tid < 256) {
    const bool on = tid < a.experts && (used[tid >> 5] >> (tid & 31)) & 1u;
    int before = 0;
#pragma unroll 1
    for (int w = 0; w < (tid >> 5); ++w) before += __popc(used[w]);
    before += __popc(used[tid >> 5] & ((1u << (tid & 31)) - 1u));
    slot_of[tid] = on ? before : -1;
    if (on && before < a.max_slots) {
      if (publish && a.active_ids) a.active_ids[before] = tid;
      if (active_s) active_s[before] = tid;
    }
    if (tid == 0) {
      int tot = 0;
#pragma unroll 1
      for (int w = 0; w < 8; ++w) tot += __popc(used[w]);
      sm.n_active = min(tot, a.max_slots);
      if (publish && a.n_active) *a.n_active = sm.n_active;
    }
  }
  if (stamp && threadIdx.x == 0) stamp[15] = globaltimer();
#pragma unroll 1
  for (int i = tid; i < a.max_slots * kTok; i += 256) {
    if (publish && a.probs) a.probs[i] = 0.f;
    if (probs_s) probs_s[i] = 0.f;
  }
  __syncthreads();
#pragma unroll 1
  for (int i = tid; i < a.rows * a.top_k; i += 256) {
    const int r = i / a.top_k, k = i - r * a.top_k;
    const int s = slot_of[sm.tk_id[r][k]];
    if (s >= 0 && s < a.max_slots) {
      if (publish && a.probs) a.probs[s * kTok + r] = sm.tk_p[r][k];
      if (probs_s) probs_s[s * kTok + r] = sm.tk_p[r][k];
    }
  }
  __syncthreads();
}

}  // namespace nrt

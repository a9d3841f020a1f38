// Skinny-M tcgen05 GEMM engine for decode / verify / draft rows (1..16 token rows).
//
// Operands are swapped relative to the usual orientation: the *weight* tile is the UMMA
// A operand (M = 128 output features fill the 128 TMEM lanes) and the token rows are the
// B operand (N = 16 columns).  One CTA owns one 128-feature output tile.  Warp roles:
//   warp 0     : TMA producer  (weights: 128 x 128-byte swizzled tiles; tokens: 16 x 128-byte tiles)
//   warp 1     : TMEM allocator + UMMA issuer (one elected lane)
//   warps 2..5 : epilogue, one TMEM lane quadrant each (thread = one output feature,
//                registers = the 16 token columns)
// Block-scaled e4m3 (W8A8): every 128-wide K block gets a fresh TMEM accumulator
// (ring of NBUF buffers); the epilogue multiplies by weight-block scale x activation-block
// scale and promotes in fp32 registers in ascending K order, so results do not depend on
// pipeline timing.  bf16 weights accumulate all of K in one TMEM buffer.
//
// Grouped modes cover the MoE: kGroupItem (grid.y = active expert slot; gate/up) and
// kGroupLoop (the CTA walks every active expert, weighting by the routing probability;
// down projection).  Epilogues: plain store, SiLU(gate)*up + e4m3 re-quantisation, and the
// fused tensor-parallel all-reduce (+ residual) over peer memory.
//
// Reference counterparts (mma.sync based unless noted): naivert/body/unproj_o_allreduce/,
// naivert/body/down_allreduce/, naivert/body/expert_select_up_gate_silu/,
// naivert/body/expert_down_allreduce/expert_down_w8a8.cuh (tcgen05 M128xN8),
// naivert/body/rmsnorm_head_proj/, naivert/common/tp8_mailbox.cuh.
#pragma once
#include "ptx.cuh"

namespace nrt {

constexpr int kTileN = 128;        // output features per CTA (UMMA M)
constexpr int kTok = 16;           // token columns (UMMA N)
constexpr int kKBytes = 128;       // bytes of K per stage row (one swizzle atom)
constexpr int kATileBytes = kTileN * kKBytes;   // 16 KiB
constexpr int kBTileBytes = kTok * kKBytes;     // 2 KiB
constexpr int kMaxPeers = 8;
constexpr int kRowPairs = kTok / 2;             // mailbox stride: tagged words per feature per source rank
constexpr int kArRows = 8;                      // rows the fused all-reduce / cluster split handle (verify = 8)
constexpr int kArPairs = kArRows / 2;
constexpr int kMailboxSlabs = 4;
constexpr int kMaxSplit = 8;                    // CTAs of one cluster that share an output tile (split K / split experts)

enum GroupMode : int { kGroupNone = 0, kGroupItem = 1, kGroupLoop = 2 };
enum Epilogue : int { kEpiStoreF32 = 0, kEpiStoreBF16 = 1, kEpiSiluQuant = 2, kEpiAllReduce = 3, kEpiSiluBF16 = 4, kEpiReturn = 5,
                      kEpiQkvPost = 6 };
// Where the token (B) operand comes from: a TMA load of a prepared tensor, or rows the CTA normalises itself
// (RMSNorm fused into the operand build: no separate normalisation launch, no normalised copy in global memory).
enum BSource : int { kBTma = 0, kBNorm = 1 };

// q/k/v(/indexer) post-processing: per-head RMS norm (draft), RoPE on adjacent pairs, KV-cache append, value
// scaling, indexer query / key quantisation.  Used by attn_post_kernel on stored projections and by the
// kEpiQkvPost epilogue straight from the accumulators.
struct AttnPostArgs {
  const float* qkv;          // [rows][ld] fp32 projection outputs: q | k | v | iq | ik | iw   (attn_post_kernel only)
  int ld;
  int rows;
  const int* pos0;
  int heads, kv_heads, head_dim, v_dim, rope_dim;
  float value_scale;
  const float2* rope;        // [rows][rope_dim/2]
  __nv_bfloat16* q_out;      // [rows][heads][head_dim]
  __nv_bfloat16* k_cache;    // [cap][kv_heads][head_dim]
  __nv_bfloat16* v_cache;    // [cap][kv_heads][v_dim]
  int ring;                  // > 0: position p is stored at p % ring; < 0: row r is stored at r (block buffers)
  // optional per-head RMS norms (draft q_norm / k_norm), applied before RoPE
  const __nv_bfloat16* q_norm;
  const __nv_bfloat16* k_norm;
  float norm_eps;
  // indexer (idx_heads == 0: none)
  int idx_heads, idx_dim, idx_rope;
  const float2* idx_rope_tab;   // [rows][idx_rope/2]
  const __nv_bfloat16* ik_w;
  const __nv_bfloat16* ik_b;
  float ln_eps, idx_weight_scale;
  uint8_t* iq8;              // [16*idx_heads][idx_dim] e4m3 (row r, head h at r*idx_heads + h)
  float* ihw;                // [16][idx_heads] head weight (x query scale when iq_scale is null)
  uint8_t* ik_cache;         // [cap][idx_dim]
  float* ik_scale;           // [cap]
  int col_q, col_k, col_v, col_iq, col_ik, col_iw;
  float* iq_scale;           // [16][idx_heads] query quantisation scale kept apart from the head weight (epilogue form)
  // epilogue form, several layers' k | v projections in one GEMM (draft context ingest): the columns repeat every
  // group_cols features; group g appends to k_cache + g * k_group_stride (elements) with k_norm + g * norm_group_stride
  int group_cols;            // 0: one group
  int norm_group_stride;
  long long k_group_stride;
  long long v_group_stride;
};

struct FabricArgs {
  uint64_t* mailbox[kMaxPeers];   // mailbox[p] = base of rank p's mailbox (peer-mapped); mailbox[rank] is local
  const uint32_t* epoch;          // device word; advanced once per step/round
  uint32_t* status;               // local error status word
  int tp;
  int rank;
  int call_idx;                   // position of this all-reduce inside one step (tag + slab selection)
  int features;                   // row width of the all-reduced tensor (mailbox stride)
  unsigned long long timeout_ns;
  int mode;                       // 0: all-reduce (every rank gets every feature)  1: reduce-scatter (rank r owns slice r)
  int ag_call;                    // >= 0: the token operand is all-gathered; K slice s is valid once ag_flags[s] carries this call's tag
  const uint64_t* ag_flags;       // [tp] tagged words in local memory, written by the peers' ag_push
};

struct GemmArgs {
  int n_total;                    // output features of one group (weight rows)
  int k_total;                    // K in elements
  int rows;                       // valid token rows (<= 16)
  int a_group;                    // fixed weight group (z coordinate) for kGroupNone
  // grouped modes
  const int* n_active;            // number of active expert slots
  const int* active_ids;          // [slots] expert id per slot (ascending)
  const float* probs;             // [slots][16] routing probability of token r for slot
  int max_slots;
  int n_experts;                  // kGroupLoop: total experts; a cluster splits the list by expert-id range
  // block scales (fp8 only)
  const float* w_scale0;          // [groups][n_total/128][k_total/128]
  const float* w_scale1;          // second matrix in dual mode
  const float* a_scale;           // [slots or 1][16][k_total/128]
  // outputs
  float* out_f32;                 // kEpiStoreF32: [rows][ld_out]
  __nv_bfloat16* out_bf16;        // kEpiStoreBF16 / kEpiAllReduce result / kEpiSiluBF16
  int ld_out;
  float out_scale;                // multiplies the stored value (kEpiStore*)
  uint8_t* out_q;                 // kEpiSiluQuant: e4m3 [slots*16][n_total]
  float* out_qscale;              // kEpiSiluQuant: [slots*16][n_total/128]
  const __nv_bfloat16* resid;     // kEpiAllReduce: residual [rows][ld_out]
  __nv_bfloat16* out_copy;        // kEpiAllReduce: optional second copy (draft feature tap)
  int ld_copy;                    // row stride of out_copy
  FabricArgs fab;
  uint32_t* status;
  // expert-parallel prefill (group-item mode over a receive buffer)
  const int* row_offsets;         // [items] first token row of each 16-row group (null: shared packet / slot * 16)
  const int4* ep_meta;            // kEpiReturn: [rows] {owner rank, token, k, dispatch tag}
  uint64_t* ep_combine[kMaxPeers];  // kEpiReturn: owner's combine slots [tokens*top_k][n_total/2] tagged words
  int ep_top_k;
  int ep_dispatch_call;           // tag call index the metadata rows must carry
  int ep_return_call;             // tag call index of the returned words
  // fused RMSNorm of the token operand (kBNorm): xn = bf16(nx * rsqrt(sum(nssq) / k_total + neps) * ngamma)
  const __nv_bfloat16* nx;        // [16][k_total] un-normalised rows
  const __nv_bfloat16* ngamma;    // [k_total]
  const float* nssq;              // [k_total/128][16] sums of squares of nx per 128-feature tile (written by nx's producer)
  float neps;
  // kEpiAllReduce: sums of squares of the result rows per 128-feature tile, [n_total/128][16] (null: none)
  float* ssq_out;
  AttnPostArgs post;              // kEpiQkvPost
  // opt-in phase stamps (%globaltimer, ns): [CTA][16] words, CTA = blockIdx.y * gridDim.x + blockIdx.x.
  // 0 entry, 1 barriers + TMEM ready, 2 upstream grid done, 3 token operand built, 4 first weight stage landed,
  // 5 last MMA issued, 6 accumulators read, 7 cluster partials merged, 8 peer words pushed, 9 peer words arrived
  // (word 10: polls of the local mailbox), 11 epilogue done, 12 row scales of the fused RMSNorm ready, 14 normalised
  // operand stored.  Null: no stamps.
  unsigned long long* stamps;
  unsigned int publish_delay_ns;  // test knob: this rank delays its mailbox publish by this long (a late peer that still arrives)
  // Region a later kernel streams from HBM (the next projection's weights): every CTA requests its share into L2 once
  // its own weight loads are issued, so the next kernel's loads - and the small loads queued behind them - hit L2.
  const void* pf_ptr;
  unsigned long long pf_bytes;
};

constexpr int kOutStageBytes = kTok * kTileN * 4;      // accumulators of a tile as [row][feature] for row-wise epilogues

template <bool FP8, bool DUAL, int BSRC = kBTma>
struct GemmCfg {
  static constexpr int kABytes = (DUAL ? 2 : 1) * kATileBytes;
  // kBNorm keeps the whole token operand of the CTA beside the ring, so a stage carries weights only
  static constexpr int kStageBytes = kABytes + (BSRC == kBTma ? kBTileBytes : 0);
  // single-matrix tiles keep the footprint near 100 KiB so two CTAs (typically of consecutive kernels,
  // overlapped by programmatic dependent launch) share an SM
  // (kBNorm, single matrix: 8 stages, so a CTA's whole K slice of weights is in flight while it builds the operand)
  static constexpr int kStages = BSRC != kBTma ? (DUAL ? 4 : 8) : 5;
  static constexpr int kAccCols = DUAL ? 2 * kTok : kTok;          // TMEM columns per accumulator buffer
  static constexpr int kAccBufs = FP8 ? (DUAL ? 4 : 8) : 1;
  static constexpr int kTmemCols = (kAccCols * kAccBufs < 32) ? 32 : kAccCols * kAccBufs;
  // split partials of the cluster peers (leader only): (split - 1) x rows x 128 floats, twice for a dual GEMM
  __host__ __device__ static constexpr int part_bytes(int split) {
    return split > 1 ? (DUAL ? 2 : 1) * (split - 1) * kArRows * kTileN * 4 : 0;
  }
  static constexpr int kRingBytes = kStages * kStageBytes;
  // token operand built in shared memory: one 2 KiB swizzled chunk per K block (+ activation scales for e4m3)
  __host__ __device__ static constexpr int operand_bytes(int kb_count) {
    return BSRC == kBTma ? 0 : kb_count * kBTileBytes + (FP8 ? ((kb_count * kTok * 4 + 1023) & ~1023) : 0);
  }
  __host__ __device__ static constexpr int smem_bytes(int kb_count, int split) {
    return kRingBytes + operand_bytes(kb_count) + 1024 /*align*/ + 1024 /*barriers + scratch*/ + kOutStageBytes + part_bytes(split);
  }
};

struct GemmSmemTail {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t acc_full[8];
  uint64_t acc_empty[8];
  uint64_t split_bar;          // leader: arrivals of the cluster peers' partials
  uint64_t b_ready;            // kBNorm: the token operand is complete in shared memory
  uint32_t tmem_base;
  uint32_t pad;
  float red[4][kTok];
  float rs[kTok];              // kBNorm: 1 / rms of each row
};

__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }

// smallest power of two >= amax / 448 (exact exponent arithmetic); 1 for amax == 0
__device__ __forceinline__ float pow2_scale(float amax) {
  if (!(amax > 0.0f)) return 1.0f;
  float t = amax * (1.0f / 448.0f);
  int e;
  float m = frexpf(t, &e);            // t = m * 2^e, m in [0.5, 1)
  if (m == 0.5f) e -= 1;
  return ldexpf(1.0f, e);
}

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Reduction of 16 per-thread values over the 128 epilogue threads of a CTA (fixed order: warp butterfly,
// then the four warps in order).  `red` is [4][16] shared floats; SUM = false takes the maximum.
template <bool SUM>
__device__ __forceinline__ void epi_reduce16(float (&v)[kTok], int rows, float (*red)[kTok], int quad, int lane) {
#pragma unroll
  for (int r = 0; r < kTok; ++r)
    if (r < rows) {
      const float t = SUM ? warp_sum_f(v[r]) : warp_max_f(v[r]);
      if (lane == 0) red[quad][r] = t;
    }
  epi_bar();
#pragma unroll
  for (int r = 0; r < kTok; ++r)
    if (r < rows)
      v[r] = SUM ? ((red[0][r] + red[1][r]) + (red[2][r] + red[3][r]))
                 : fmaxf(fmaxf(red[0][r], red[1][r]), fmaxf(red[2][r], red[3][r]));
  epi_bar();
}

__device__ __forceinline__ void rope_pair(float& a, float& b, float2 cs) {
  const float re = a * cs.x - b * cs.y;
  const float im = a * cs.y + b * cs.x;
  a = re;
  b = im;
}
// RoPE of the element a thread holds when its pair partner sits in the neighbouring lane (feature index
// parity = lane parity): both lanes evaluate the same pair and keep their own half.
__device__ __forceinline__ float rope_lane(float x, float other, bool odd, float2 cs) {
  float a = odd ? other : x, b = odd ? x : other;
  rope_pair(a, b, cs);
  return odd ? b : a;
}
__device__ __forceinline__ uint8_t e4m3_bits(float v) {
  const __nv_fp8_e4m3 q(v);
  return *reinterpret_cast<const uint8_t*>(&q);
}

// ----------------------------------------------------------------------------- fused RMSNorm operand build
// Called by the 128 epilogue threads (et = 0..127).  Writes the CTA's K blocks [kb_first, kb_first + kb_count)
// of the normalised rows into `ball` in the layout a 128-byte-swizzled TMA box {128 B, 16 rows} would produce:
// chunk c at c * 2 KiB, row r at (r / 8) * 1024 + (r % 8) * 128, 16-byte unit j at ((j ^ (r % 8)) * 16).
// bf16: 64 elements per chunk; e4m3: 128 elements per chunk with one power-of-two scale per (row, chunk)
// stored in bscale[r * kb_count + c].  Rows >= p.rows are zero.
template <bool FP8>
__device__ __forceinline__ void build_norm_operand(const GemmArgs& p, uint8_t* ball, float* bscale, float* rs_s,
                                                   int kb_first, int kb_count, int et, unsigned long long* stamp = nullptr) {
  const int rows = p.rows;
  const int tiles = p.k_total / 128;
  // Rows >= p.rows are left as they are: an MMA column depends on its own token row only, and the columns of
  // dead rows are never stored.
  // A unit is 16 bytes of operand: 8 bf16 elements, or 16 e4m3 elements (two 16-byte loads of x).  A thread owns one
  // column unit (chunk c, unit j) - its norm weights are loaded once - and walks token rows in batches of eight (four for e4m3) whose
  // loads are all in flight together.  With fewer than 128 column units the threads form 128 / units row groups.
  constexpr int kLoads = FP8 ? 2 : 1;
  constexpr int kRB = FP8 ? 4 : 8;              // token rows per batch: every load of a batch is in flight together
  constexpr int kElems = FP8 ? 128 : 64;
  const int units = kb_count * 8;
  const int groups = units < 128 ? 128 / units : 1;
  const int g = units < 128 ? et / units : 0;
  // The first batch of activations and norm weights does not depend on the row scales: it is requested before them,
  // so the two memory round trips overlap.
  const int cu0 = units < 128 ? et % units : et;
  uint4 gv[kLoads];
  uint4 xv[kRB][kLoads];
  auto load_batch = [&](int cu, int r0) {
    const int k = (kb_first + (cu >> 3)) * kElems + (cu & 7) * (kElems / 8);
#pragma unroll
    for (int l = 0; l < kLoads; ++l) gv[l] = __ldg(reinterpret_cast<const uint4*>(p.ngamma + k + 8 * l));
#pragma unroll
    for (int b = 0; b < kRB; ++b) {
      const int r = r0 + b * groups;
#pragma unroll
      for (int l = 0; l < kLoads; ++l)
        xv[b][l] = r < rows ? *reinterpret_cast<const uint4*>(p.nx + (size_t)r * p.k_total + k + 8 * l) : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  const bool active = cu0 < units && g < groups && g < rows;
  // 1 / rms of every row: 8 threads per row, each adds the tiles t = sub, sub + 8, ...  These loads gate everything
  // else, so they are issued first; the operand's own loads queue up behind them.
  {
    const int r = et >> 3, sub = et & 7;
    float sv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int t = sub + 8 * i;
      sv[i] = (r < rows && t < tiles) ? __ldcg(p.nssq + t * kTok + r) : 0.f;
    }
    if (active) load_batch(cu0, g);
    float ssum = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) ssum += sv[i];
    for (int t = sub + 64; t < tiles && r < rows; t += 8) ssum += __ldcg(p.nssq + t * kTok + r);     // hidden > 8192
#pragma unroll
    for (int off = 4; off > 0; off >>= 1) ssum += __shfl_xor_sync(0xffffffffu, ssum, off);
    if (sub == 0 && r < rows) rs_s[r] = rsqrtf(ssum / (float)p.k_total + p.neps);
    if (stamp && et == 0) stamp[12] = globaltimer();
  }
  epi_bar();
#pragma unroll 1
  for (int cu = cu0; cu < units && g < groups; cu += 128) {
    const int c = cu >> 3, j = cu & 7;
#pragma unroll 1
    for (int r0 = g; r0 < rows; r0 += kRB * groups) {
      if (cu != cu0 || r0 != g) load_batch(cu, r0);
#pragma unroll
      for (int b = 0; b < kRB; ++b) {
        const int r = r0 + b * groups;
        const bool on = r < rows;
        const float rs = rs_s[on ? r : 0];
        float o[8 * kLoads];
#pragma unroll
        for (int l = 0; l < kLoads; ++l) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&xv[b][l]);
          const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv[l]);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 f = __bfloat1622float2(h[q]), gg = __bfloat1622float2(gh[q]);
            o[8 * l + 2 * q] = round_bf16(f.x * rs * gg.x);
            o[8 * l + 2 * q + 1] = round_bf16(f.y * rs * gg.y);
          }
        }
        uint4 w;
        if (!FP8) {
          __nv_bfloat162* wh = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
          for (int q = 0; q < 4; ++q) wh[q] = __floats2bfloat162_rn(o[2 * q], o[2 * q + 1]);
        } else {
          // the 8 units of a (row, chunk) sit in 8 consecutive lanes (same row group, same chunk)
          float am = 0.f;
#pragma unroll
          for (int q = 0; q < 8 * kLoads; ++q) am = fmaxf(am, fabsf(o[q]));
#pragma unroll
          for (int off = 4; off > 0; off >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffu << (et & 24), am, off));
          const float sc = pow2_scale(am);
          const float inv = 1.0f / sc;                 // a power of two: the product is the exact quotient
          uint8_t* wb = reinterpret_cast<uint8_t*>(&w);
#pragma unroll
          for (int q = 0; q < 8 * kLoads; ++q) wb[q] = e4m3_bits(o[q] * inv);
          if (on && j == 0) bscale[r * kb_count + c] = sc;
        }
        if (on)
          *reinterpret_cast<uint4*>(ball + c * kBTileBytes + (r >> 3) * 1024 + (r & 7) * 128 + ((j ^ (r & 7)) << 4)) = w;
      }
    }
  }
}

// ----------------------------------------------------------------------------- q/k/v post-processing epilogue
// The accumulators of a tile (thread = feature, register = token row) are staged in shared memory as
// [row][128 features]; then every epilogue warp takes whole token rows (warp w: rows w, w + 4, ...), a lane four
// adjacent features.  All reductions of a row (LayerNorm, per-head RMS norm, quantisation maximum) are warp
// reductions, RoPE pairs sit in one lane, stores are 8-byte (bf16) or 4-byte (e4m3) per lane, and the per-row code
// is one rolled loop - this epilogue runs once per launch, and a short loop body that is fetched once beats sixteen
// unrolled copies of it.
// Tiles of indexer heads, the indexer key and per-head-normed heads (head_dim == 128) must be 128-aligned; region
// boundaries (q | k | v | iq | ik | iw) and head sizes are multiples of 4 features.
enum PostKind : int { kPostNone = 0, kPostQ, kPostK, kPostV, kPostIw, kPostIq, kPostIk };

struct PostCtx {             // per-lane constants, fetched while the MMAs still run
  int p0;
  int kind, h, d;            // region of the lane's four features, head index, first feature inside the head
  bool rope, head_norm;
  float w[4], b[4];          // per-feature norm weight / LayerNorm weight and bias
  const float2* tab;         // RoPE table of the region, row stride `half` pairs
  int half;
  float4 cs0, cs1;           // (cos, sin) of the lane's two pairs for this warp's first two rows
};

__device__ __forceinline__ void post_group(AttnPostArgs& a, int& n0) {
  if (a.group_cols > 0) {
    const int g = n0 / a.group_cols;
    n0 -= g * a.group_cols;
    a.k_cache += (size_t)g * a.k_group_stride;
    a.v_cache += (size_t)g * a.v_group_stride;
    if (a.k_norm) a.k_norm += (size_t)g * a.norm_group_stride;
  }
}

__device__ __forceinline__ PostCtx qkv_post_prepare(const AttnPostArgs& a_in, int n0, int quad, int lane, int rows) {
  AttnPostArgs a = a_in;
  post_group(a, n0);
  PostCtx c;
  c.p0 = *a.pos0;
  c.kind = kPostNone; c.h = 0; c.d = 0; c.rope = false; c.head_norm = false; c.tab = nullptr; c.half = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) { c.w[i] = 1.f; c.b[i] = 0.f; }
  c.cs0 = c.cs1 = make_float4(1.f, 0.f, 1.f, 0.f);
  const int f = n0 + lane * 4;                       // first of the lane's four features
  const int q_end = a.col_q + a.heads * a.head_dim;
  const int k_end = a.col_k + a.kv_heads * a.head_dim;
  const int v_end = a.col_v + a.kv_heads * a.v_dim;
  const __nv_bfloat16* nw = nullptr;
  if (a.idx_heads > 0 && n0 >= a.col_iq && n0 < a.col_iq + a.idx_heads * a.idx_dim) {
    c.kind = kPostIq; c.h = (n0 - a.col_iq) / a.idx_dim; c.d = f - n0;
    if (c.d < a.idx_rope) { c.rope = true; c.tab = a.idx_rope_tab; c.half = a.idx_rope / 2; }
  } else if (a.idx_heads > 0 && n0 == a.col_ik) {
    c.kind = kPostIk; c.d = f - n0;
    if (c.d < a.idx_rope) { c.rope = true; c.tab = a.idx_rope_tab; c.half = a.idx_rope / 2; }
    if (c.d < a.idx_dim) {
#pragma unroll
      for (int i = 0; i < 4; ++i) { c.w[i] = __bfloat162float(a.ik_w[c.d + i]); c.b[i] = __bfloat162float(a.ik_b[c.d + i]); }
    }
  } else if (f >= a.col_q && f < q_end) {
    c.kind = kPostQ; c.h = (f - a.col_q) / a.head_dim; c.d = (f - a.col_q) - c.h * a.head_dim; nw = a.q_norm;
  } else if (f >= a.col_k && f < k_end) {
    c.kind = kPostK; c.h = (f - a.col_k) / a.head_dim; c.d = (f - a.col_k) - c.h * a.head_dim; nw = a.k_norm;
  } else if (f >= a.col_v && f < v_end) {
    c.kind = kPostV; c.d = f - a.col_v;
  } else if (a.idx_heads > 0 && f >= a.col_iw && f < a.col_iw + a.idx_heads) {
    c.kind = kPostIw; c.d = f - a.col_iw;
  }
  if (c.kind == kPostQ || c.kind == kPostK) {
    if (c.d < a.rope_dim) { c.rope = true; c.tab = a.rope; c.half = a.rope_dim / 2; }
    if (nw) {
      c.head_norm = true;
#pragma unroll
      for (int i = 0; i < 4; ++i) c.w[i] = __bfloat162float(nw[c.d + i]);
    }
  }
  if (c.rope) {
    const float4* t = reinterpret_cast<const float4*>(c.tab + (c.d >> 1));      // two pairs = 16 bytes, 16-byte aligned
    if (quad < rows) c.cs0 = __ldg(t + (size_t)quad * (c.half >> 1));
    if (quad + 4 < rows) c.cs1 = __ldg(t + (size_t)(quad + 4) * (c.half >> 1));
  }
  return c;
}

// `v`: the thread's accumulators (feature n0 + quad * 32 + lane, one per token row).  `stage`: [16][128] floats of
// shared memory owned by the epilogue warps.  Called by all 128 epilogue threads of the CTA that holds the full sums.
__device__ __forceinline__ void qkv_post_epilogue(const AttnPostArgs& a_in, const PostCtx& c, int n0, int quad, int lane,
                                                  const float (&v)[kTok], int rows, float* stage, bool live) {
  AttnPostArgs a = a_in;
  post_group(a, n0);
  const int col = quad * 32 + lane;
#pragma unroll
  for (int r = 0; r < kTok; ++r)
    if (r < rows) stage[r * kTileN + col] = v[r];
  epi_bar();
  if (!live) return;
  int it = 0;
#pragma unroll 1
  for (int r = quad; r < rows; r += 4, ++it) {
    const float4 v4 = *reinterpret_cast<const float4*>(stage + r * kTileN + lane * 4);
    float x[4] = {v4.x, v4.y, v4.z, v4.w};
    const int pos = c.p0 + r;
    float4 cs = make_float4(1.f, 0.f, 1.f, 0.f);
    if (c.rope) cs = it == 0 ? c.cs0 : (it == 1 ? c.cs1 : __ldg(reinterpret_cast<const float4*>(c.tab + (c.d >> 1)) + (size_t)r * (c.half >> 1)));
    if (c.kind == kPostIq || c.kind == kPostIk) {
      // whole tile = one indexer head / the indexer key (uniform over the warp)
      if (c.kind == kPostIk) {
        // LayerNorm in fp32 over idx_dim features
        const bool in = c.d < a.idx_dim;
        float t = in ? (x[0] + x[1]) + (x[2] + x[3]) : 0.f;
        const float mean = warp_sum_f(t) / (float)a.idx_dim;
        float dv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) dv[i] = in ? x[i] - mean : 0.f;
        t = (dv[0] * dv[0] + dv[1] * dv[1]) + (dv[2] * dv[2] + dv[3] * dv[3]);
        const float inv = rsqrtf(warp_sum_f(t) / (float)a.idx_dim + a.ln_eps);
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = in ? round_bf16(dv[i] * inv * c.w[i] + c.b[i]) : 0.f;
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = round_bf16(x[i]);
      }
      if (c.rope) {
        rope_pair(x[0], x[1], make_float2(cs.x, cs.y));
        rope_pair(x[2], x[3], make_float2(cs.z, cs.w));
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = round_bf16(x[i]);
      }
      const float am = warp_max_f(fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3]))));
      const float sc = am > 0.f ? am / 448.f : 1.f;
      uint32_t q4 = 0u;
#pragma unroll
      for (int i = 0; i < 4; ++i) q4 |= (uint32_t)e4m3_bits(x[i] / sc) << (8 * i);
      if (c.kind == kPostIq) {
        *reinterpret_cast<uint32_t*>(a.iq8 + ((size_t)r * a.idx_heads + c.h) * a.idx_dim + c.d) = q4;
        if (lane == 0) a.iq_scale[r * a.idx_heads + c.h] = sc;
      } else if (c.d < a.idx_dim) {
        *reinterpret_cast<uint32_t*>(a.ik_cache + (size_t)pos * a.idx_dim + c.d) = q4;
        if (lane == 0) a.ik_scale[pos] = sc;
      }
      continue;
    }
    const size_t slot = a.ring > 0 ? (size_t)(pos % a.ring) : (a.ring < 0 ? (size_t)r : (size_t)pos);
    if (c.kind == kPostQ || c.kind == kPostK) {
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] = round_bf16(x[i]);
      if (c.head_norm) {                               // heads are whole tiles here: uniform over the warp
        const float ss = warp_sum_f((x[0] * x[0] + x[1] * x[1]) + (x[2] * x[2] + x[3] * x[3]));
        const float inv = rsqrtf(ss / (float)a.head_dim + a.norm_eps);
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = round_bf16(x[i] * inv * c.w[i]);
      }
      if (c.rope) {
        rope_pair(x[0], x[1], make_float2(cs.x, cs.y));
        rope_pair(x[2], x[3], make_float2(cs.z, cs.w));
      }
      uint2 o;
      *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(x[0], x[1]);
      *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(x[2], x[3]);
      __nv_bfloat16* dst = c.kind == kPostQ ? a.q_out + ((size_t)r * a.heads + c.h) * a.head_dim + c.d
                                            : a.k_cache + (slot * a.kv_heads + c.h) * a.head_dim + c.d;
      *reinterpret_cast<uint2*>(dst) = o;
    } else if (c.kind == kPostV) {
      uint2 o;
      *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(x[0] * a.value_scale, x[1] * a.value_scale);
      *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(x[2] * a.value_scale, x[3] * a.value_scale);
      *reinterpret_cast<uint2*>(a.v_cache + slot * a.kv_heads * a.v_dim + c.d) = o;
    } else if (c.kind == kPostIw) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (c.d + i < a.idx_heads) a.ihw[r * a.idx_heads + c.d + i] = x[i] * a.idx_weight_scale;
    }
  }
}

// ----------------------------------------------------------------------------- fused all-reduce epilogue
// Thread = feature n of the output tile, mix0[r] = this rank's fp32 partial for token row r (leader CTA of a
// cluster split).  The partial is rounded to bf16, pushed to every peer's mailbox as tagged words, the peers'
// words are polled from the local mailbox and all ranks' values are added in rank order in fp32 on top of the
// residual; the bf16 result (and optionally its per-tile sums of squares for the next RMSNorm) is stored.
#define NRT_STAMP(i) do { if (stamp) stamp[i] = globaltimer(); } while (0)
// `resid_pre`: the residual values of this thread's feature for rows 0..7, loaded by the caller while the MMAs were
// still running (null: they are loaded here).
__device__ __forceinline__ void allreduce_epilogue(const GemmArgs& p, float (&mix0)[kTok], int n, int n_tile, int row, int lane,
                                                   int quad, bool leader, GemmSmemTail* tail, unsigned long long* stamp,
                                                   const float* resid_pre = nullptr) {
  const FabricArgs& f = p.fab;
  const int owner = f.mode == 1 ? n / (p.n_total / f.tp) : f.rank;        // reduce-scatter: one owner per feature
  const bool col_ok = leader && n < p.n_total;
  const bool mine = owner == f.rank;
  // Each rank rounds its partial to bf16, pushes it to every peer as tagged words and adds
  // the partials of all ranks in rank order in fp32 on top of the residual.
  uint32_t w[kMaxPeers][kArPairs];
  const int pairs = (p.rows + 1) >> 1;
  float sum[kArRows];
#pragma unroll
  for (int r = 0; r < kArRows; ++r)
    sum[r] = resid_pre ? (col_ok ? resid_pre[r] : 0.f)
                       : ((p.resid && r < p.rows && col_ok) ? __bfloat162float(p.resid[(size_t)r * p.ld_out + n]) : 0.f);
  uint32_t own[kArPairs];
#pragma unroll
  for (int j = 0; j < kArPairs; ++j) own[j] = pack_bf16x2(mix0[2 * j], mix0[2 * j + 1]);
  if (f.tp > 1 && col_ok) {
    const uint32_t tag = (*f.epoch) * 1024u + (uint32_t)f.call_idx + 1u;
    const size_t slab = (size_t)(f.call_idx % kMailboxSlabs) * f.tp;
    if (p.publish_delay_ns) {                    // a late peer (skew experiment): bounded, it still arrives
      const uint64_t until = globaltimer() + p.publish_delay_ns;
      while (globaltimer() < until) __nanosleep(200);
    }
    for (int d = 1; d < f.tp; ++d) {
      const int peer = (f.rank + d) % f.tp;
      if (f.mode == 1 && peer != owner) continue;
      // layout [slab][source][row pair][feature]: a warp's 32 stores of one pair are contiguous
      uint64_t* dst = f.mailbox[peer] + (slab + f.rank) * kRowPairs * f.features + n;
#pragma unroll
      for (int j = 0; j < kArPairs; ++j)
        if (j < pairs) st_tagged(dst + (size_t)j * f.features, tag, own[j]);
    }
    if (threadIdx.x == 64) NRT_STAMP(8);
    // Batched poll: every missing word of every source is re-read per sweep, so the
    // loads of one sweep overlap instead of paying one fabric round trip each.
    uint64_t missing = 0;
#pragma unroll
    for (int s = 0; s < kMaxPeers; ++s)
#pragma unroll
      for (int j = 0; j < kArPairs; ++j) {
        if (s == f.rank) w[s][j] = own[j];
        else if (mine && s < f.tp && j < pairs) missing |= 1ull << (s * kArPairs + j);
        else w[s][j] = 0u;
      }
    const uint64_t deadline = globaltimer() + f.timeout_ns;
    const uint64_t* base = f.mailbox[f.rank] + slab * kRowPairs * f.features + n;
    for (uint32_t sweep = 0; missing != 0; ++sweep) {
      // One sweep = every outstanding word requested before any answer is looked at: the guards test a snapshot of
      // the mask, so no load waits for the previous load's comparison and the fabric round trips overlap.
      const uint64_t need = missing;
      uint32_t tt[kMaxPeers][kArPairs], vv[kMaxPeers][kArPairs];
#pragma unroll
      for (int s = 0; s < kMaxPeers; ++s)
#pragma unroll
        for (int j = 0; j < kArPairs; ++j) {
          tt[s][j] = ~tag;
          vv[s][j] = 0u;
          if (need & (1ull << (s * kArPairs + j))) ld_tagged(base + ((size_t)s * kRowPairs + j) * f.features, tt[s][j], vv[s][j]);
        }
#pragma unroll
      for (int s = 0; s < kMaxPeers; ++s)
#pragma unroll
        for (int j = 0; j < kArPairs; ++j)
          if ((need & (1ull << (s * kArPairs + j))) && tt[s][j] == tag) { w[s][j] = vv[s][j]; missing &= ~(1ull << (s * kArPairs + j)); }
      if ((sweep & 255u) == 255u) {
        if (*reinterpret_cast<volatile uint32_t*>(f.status) != 0u) break;
        if (globaltimer() > deadline) { report(f.status, kSiteMailbox | (uint32_t)__ffsll((long long)missing)); break; }
      }
      if (missing == 0 && threadIdx.x == 64 && stamp) stamp[10] = sweep + 1;
    }
    if (threadIdx.x == 64) NRT_STAMP(9);
#pragma unroll
    for (int s = 0; s < kMaxPeers; ++s)
#pragma unroll
      for (int j = 0; j < kArPairs; ++j)
        if (s < f.tp) { sum[2 * j] += bf16_lo(w[s][j]); sum[2 * j + 1] += bf16_hi(w[s][j]); }
  } else {
#pragma unroll
    for (int r = 0; r < kArRows; ++r) sum[r] += round_bf16(mix0[r]);
  }
  float sq[kArRows];
#pragma unroll
  for (int r = 0; r < kArRows; ++r) {
    sq[r] = 0.f;
    if (r < p.rows && col_ok && mine) {
      const __nv_bfloat16 o = __float2bfloat16_rn(sum[r]);
      p.out_bf16[(size_t)r * p.ld_out + n] = o;
      if (p.out_copy) p.out_copy[(size_t)r * p.ld_copy + n] = o;
      const float of = __bfloat162float(o);
      sq[r] = of * of;
    }
  }
  if (p.ssq_out != nullptr) {
    // sums of squares of this tile's result rows: the next RMSNorm adds the tiles' partials in tile order
#pragma unroll
    for (int r = 0; r < kArRows; ++r) {
      const float t = warp_sum_f(sq[r]);
      if (lane == 0) tail->red[quad][r] = t;
    }
    epi_bar();
    if (leader && row < kTok)
      p.ssq_out[n_tile * kTok + row] =
          row < kArRows ? ((tail->red[0][row] + tail->red[1][row]) + (tail->red[2][row] + tail->red[3][row])) : 0.f;
  }
}
#undef NRT_STAMP

template <bool FP8, bool DUAL, int EPI, int GROUP, int BSRC = kBTma>
__global__ void __launch_bounds__(192, (DUAL || BSRC != kBTma) ? 1 : 2)
skinny_gemm_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
                   const __grid_constant__ CUtensorMap tmB, const GemmArgs p) {
  using Cfg = GemmCfg<FP8, DUAL, BSRC>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x;
  const int n0 = n_tile * kTileN;
  const int kb_total = p.k_total / (FP8 ? 128 : 64);
  constexpr int kElemsPerStage = FP8 ? 128 : 64;
  // Cluster split: grid.y CTAs (one cluster) share this output tile.  kGroupNone splits K,
  // kGroupLoop splits the expert list; the leader (cluster rank 0) adds the partials in rank order.
  const int split = GROUP == kGroupItem ? 1 : (int)gridDim.y;
  const int crank = split > 1 ? (int)cluster_ctarank() : 0;
  const int kb_count = GROUP == kGroupNone ? kb_total / split : kb_total;   // K blocks this CTA walks per group
  const int kb_first = GROUP == kGroupNone ? crank * kb_count : 0;
  uint8_t* ball = smem + Cfg::kRingBytes;                                    // kBNorm: the CTA's token operand
  float* bscale = reinterpret_cast<float*>(ball + kb_count * kBTileBytes);   // kBNorm e4m3: [16][kb_count]
  GemmSmemTail* tail = reinterpret_cast<GemmSmemTail*>(smem + Cfg::kRingBytes + Cfg::operand_bytes(kb_count));
  float* out_stage = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(tail) + 1024);      // [16][128] epilogue staging
  float* part = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(tail) + 1024 + kOutStageBytes);

  unsigned long long* stamp = p.stamps ? p.stamps + (size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 16 : nullptr;
#define NRT_STAMP(i) do { if (stamp) stamp[i] = globaltimer(); } while (0)
  if (threadIdx.x == 0) {
    NRT_STAMP(0);
    for (int i = 0; i < Cfg::kStages; ++i) { mbar_init(&tail->full[i], 1); mbar_init(&tail->empty[i], 1); }
    for (int i = 0; i < Cfg::kAccBufs; ++i) { mbar_init(&tail->acc_full[i], 1); mbar_init(&tail->acc_empty[i], 128); }
    mbar_init(&tail->split_bar, 128 * (split > 1 ? split - 1 : 1));
    mbar_init(&tail->b_ready, 128);
    mbar_fence_init();
    tma_prefetch_desc(&tmA0);
    if (BSRC == kBTma) tma_prefetch_desc(&tmB);
    if (DUAL) tma_prefetch_desc(&tmA1);
  }
  if (warp == 1) { tmem_alloc(&tail->tmem_base, Cfg::kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  if (split > 1) cluster_sync_all();           // peers' barriers are initialised before any remote arrive
  tc_fence_after();
  const uint32_t tmem = tail->tmem_base;
  if (threadIdx.x == 0) NRT_STAMP(1);

  // Weights never depend on earlier kernels, so (ungrouped) the producer streams the first weight
  // tiles *before* waiting for the upstream grid; token tiles, scales, residuals and expert lists are
  // read after the wait.  The dependent kernel is released only after this kernel's own wait, so at
  // most one successor is resident early (a chain of waiting grids clogs the CTA scheduler).
  // stages whose weight tile is issued before the wait
  const int early = GROUP == kGroupNone ? min(kb_count, Cfg::kStages) : 0;
  // weight tiles are read once per step: they are the first to leave L2, so the step's activations, KV rows and
  // hand-off buffers stay resident while gigabytes of weights stream through
  const uint64_t stream_once = l2_policy_evict_first();
  if (GROUP == kGroupNone) {
    if (warp == 0 && elect_one()) {
      for (int u = 0; u < early; ++u) {
        uint8_t* sa = smem + u * Cfg::kStageBytes;
        mbar_expect_tx(&tail->full[u], Cfg::kStageBytes);
        const int kx = (kb_first + u) * kElemsPerStage;
        tma_load_3d_hint(sa, &tmA0, &tail->full[u], kx, n0, p.a_group, stream_once);
        if (DUAL) tma_load_3d_hint(sa + kATileBytes, &tmA1, &tail->full[u], kx, n0, p.a_group, stream_once);
      }
    }
  }
  if (BSRC != kBTma && warp >= 2) {
    // the norm weights of this thread's first operand unit are a cold HBM line once per step: requested into L2 now,
    // so the load after the wait does not pay the DRAM (and page-table) round trip
    const int et = (int)threadIdx.x - 64, units = kb_count * 8;
    const int cu0 = units < 128 ? et % units : et;
    if (cu0 < units) prefetch_l2(p.ngamma + (kb_first + (cu0 >> 3)) * kElemsPerStage + (cu0 & 7) * (kElemsPerStage / 8));
  }
  griddep_wait();
  griddep_launch();
  if (threadIdx.x == 0) NRT_STAMP(2);

  int n_groups = 1, g_first = 0, g_step = 1;
  if (GROUP == kGroupItem) {
    const int na = min(*p.n_active, p.max_slots);
    n_groups = (int)blockIdx.y < na ? 1 : 0;
    g_first = blockIdx.y;
  } else if (GROUP == kGroupLoop) {
    // CTA y of the cluster takes the active experts whose id lies in the y-th range of the expert ids (the list is
    // ascending, so that is one contiguous run of slots).  A token's experts are then always added in the same
    // grouping and order, whatever other tokens share the step: a row's result does not depend on its batch.
    const int na = min(*p.n_active, p.max_slots);
    const int per = (p.n_experts + (int)gridDim.y - 1) / (int)gridDim.y;
    const int id_lo = (int)blockIdx.y * per, id_hi = id_lo + per;
    // every warp counts the list entries below each bound with one round of loads (the list is ascending)
    int lo = 0, hi = 0;
    for (int i0 = 0; i0 < na; i0 += 32) {
      const int i = i0 + lane;
      const int id = i < na ? __ldg(p.active_ids + i) : 0x7fffffff;
      lo += __popc(__ballot_sync(0xffffffffu, id < id_lo));
      hi += __popc(__ballot_sync(0xffffffffu, id < id_hi));
    }
    g_first = lo;
    g_step = 1;
    n_groups = hi - lo;
  }
  const int units = n_groups * kb_count;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int ag_seen = -1;
      for (int u = 0; u < units; ++u) {
        const int st = u % Cfg::kStages;
        if (u >= Cfg::kStages &&
            !mbar_wait(&tail->empty[st], ((u / Cfg::kStages) & 1) ^ 1, p.status, kSiteStageEmpty | st)) break;
        const int g = u / kb_count, kb = u - g * kb_count;
        const int slot = g_first + g * g_step;
        const int z = GROUP == kGroupNone ? p.a_group : p.active_ids[slot];
        uint8_t* sa = smem + st * Cfg::kStageBytes;
        const int kx = (kb_first + kb) * kElemsPerStage;
        if (u >= early) {
          mbar_expect_tx(&tail->full[st], Cfg::kStageBytes);
          tma_load_3d_hint(sa, &tmA0, &tail->full[st], kx, n0, z, stream_once);
          if (DUAL) tma_load_3d_hint(sa + kATileBytes, &tmA1, &tail->full[st], kx, n0, z, stream_once);
        }
        if (BSRC != kBTma) continue;
        const int brow = (GROUP == kGroupLoop) ? slot * kTok : ((GROUP == kGroupItem && p.row_offsets) ? p.row_offsets[slot] : 0);
        if (GROUP == kGroupItem && p.fab.ag_call >= 0 && p.fab.tp > 1 && ag_seen < 0) {
          // expert-parallel dispatch: rows of every source rank must have landed before the first token tile
          const uint32_t tag = (*p.fab.epoch) * 1024u + (uint32_t)p.fab.ag_call + 1u;
          bool all = true;
          for (int s = 0; s < p.fab.tp && all; ++s) {
            uint32_t v;
            all = wait_tagged(p.fab.ag_flags + s, tag, v, globaltimer() + p.fab.timeout_ns, p.status, kSiteMailbox | 0x60 | s);
          }
          if (!all) break;
          asm volatile("fence.acq_rel.sys;" ::: "memory");
          asm volatile("fence.proxy.async;" ::: "memory");
          ag_seen = 0;
        }
        if (GROUP == kGroupNone && p.fab.ag_call >= 0 && p.fab.tp > 1) {
          // all-gather -> GEMM: the K slice of source rank `src` was pushed into local memory by that rank;
          // wait for its flag (acquire), then order the generic-proxy writes before the TMA read
          const int src = (kb_first + kb) / (kb_total / p.fab.tp);
          if (src != ag_seen) {
            const uint32_t tag = (*p.fab.epoch) * 1024u + (uint32_t)p.fab.ag_call + 1u;
            uint32_t v;
            if (!wait_tagged(p.fab.ag_flags + src, tag, v, globaltimer() + p.fab.timeout_ns, p.status, kSiteMailbox | 0x40 | src)) break;
            asm volatile("fence.acq_rel.sys;" ::: "memory");
            asm volatile("fence.proxy.async;" ::: "memory");
            ag_seen = src;
          }
        }
        tma_load_2d(sa + Cfg::kABytes, &tmB, &tail->full[st], kx, brow);
      }
      prefetch_share_l2(p.pf_ptr, p.pf_bytes, (int)(blockIdx.y * gridDim.x + blockIdx.x), (int)(gridDim.x * gridDim.y));
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ UMMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc(FP8 ? 0u : 1u, kTileN, kTok);
      bool ok = true;
      if (BSRC != kBTma && units > 0) ok = mbar_wait(&tail->b_ready, 0, p.status, kSiteTmaFull | 0x40);
      for (int u = 0; u < units && ok; ++u) {
        const int st = u % Cfg::kStages;
        const int kb = u % kb_count;
        const int buf = FP8 ? (u % Cfg::kAccBufs) : 0;
        if (FP8 && u >= Cfg::kAccBufs &&
            !mbar_wait(&tail->acc_empty[buf], ((u / Cfg::kAccBufs) & 1) ^ 1, p.status, kSiteAccEmpty | buf)) break;
        if (!mbar_wait(&tail->full[st], (u / Cfg::kStages) & 1, p.status, kSiteTmaFull | st)) break;
        if (u == 0) NRT_STAMP(4);
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + st * Cfg::kStageBytes);
        const uint64_t da0 = umma_desc_sw128(sa);
        const uint64_t da1 = umma_desc_sw128(sa + kATileBytes);
        const uint64_t db = umma_desc_sw128(BSRC == kBTma ? sa + Cfg::kABytes : smem_u32(ball + kb * kBTileBytes));
        const uint32_t d0 = tmem + buf * Cfg::kAccCols;
#pragma unroll
        for (int j = 0; j < 4; ++j) {          // 4 x 32 bytes of K per 128-byte swizzle atom
          const uint32_t acc = FP8 ? (j > 0) : (kb > 0 || j > 0);
          if (FP8) {
            umma_f8(d0, da0 + 2 * j, db + 2 * j, idesc, acc);
            if (DUAL) umma_f8(d0 + kTok, da1 + 2 * j, db + 2 * j, idesc, acc);
          } else {
            umma_bf16(d0, da0 + 2 * j, db + 2 * j, idesc, acc);
            if (DUAL) umma_bf16(d0 + kTok, da1 + 2 * j, db + 2 * j, idesc, acc);
          }
        }
        umma_commit(&tail->empty[st]);                                  // frees the smem stage
        if (FP8 || kb == kb_count - 1) umma_commit(&tail->acc_full[buf]);
      }
      NRT_STAMP(5);
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int quad = warp & 3;                       // TMEM lane quadrant this warp may read
    const int row = quad * 32 + lane;                // feature within the tile
    const int n = n0 + row;
    const uint32_t lane_addr = tmem + (uint32_t(quad * 32) << 16);
    const int nt_count = p.n_total / kTileN;
    if (BSRC != kBTma) {
      // the epilogue warps are idle until the first accumulator completes: they normalise (and quantise)
      // the CTA's token rows into shared memory while the weight tiles stream in
      if (units > 0) build_norm_operand<FP8>(p, ball, bscale, tail->rs, kb_first, kb_count, (int)threadIdx.x - 64, stamp);
      if (threadIdx.x == 64) NRT_STAMP(14);
      fence_proxy_async_smem();
      mbar_arrive(&tail->b_ready);
      epi_bar();                                     // bscale of every thread is visible to the epilogue
      if (threadIdx.x == 64) NRT_STAMP(3);
    }
    PostCtx post_ctx;
    if (EPI == kEpiQkvPost) post_ctx = qkv_post_prepare(p.post, n0, quad, lane, p.rows);
    // the residual rows were written by an earlier kernel: fetched now, added when the sums are complete
    float resid_pre[kArRows];
    if (EPI == kEpiAllReduce) {
#pragma unroll
      for (int r = 0; r < kArRows; ++r)
        resid_pre[r] = (p.resid && r < p.rows && crank == 0 && n < p.n_total) ? __bfloat162float(p.resid[(size_t)r * p.ld_out + n]) : 0.f;
    }
    float mix0[kTok];
#pragma unroll
    for (int r = 0; r < kTok; ++r) mix0[r] = 0.f;
    float mix1[kTok];
#pragma unroll
    for (int r = 0; r < kTok; ++r) mix1[r] = 0.f;
    bool ok = true;
    int u = 0;
    for (int g = 0; g < n_groups && ok; ++g) {
      const int slot = g_first + g * g_step;
      const int z = GROUP == kGroupNone ? p.a_group : p.active_ids[slot];
      float acc0[kTok], acc1[kTok];
#pragma unroll
      for (int r = 0; r < kTok; ++r) { acc0[r] = 0.f; acc1[r] = 0.f; }
      if (FP8) {
        const size_t in_row = GROUP == kGroupLoop ? (size_t)slot * kTok
                                                   : ((GROUP == kGroupItem && p.row_offsets) ? (size_t)p.row_offsets[slot] : 0);
        const float* as = BSRC == kBTma ? p.a_scale + in_row * kb_total + kb_first : nullptr;
        const float* ws0 = p.w_scale0 + ((size_t)z * nt_count + n_tile) * kb_total + kb_first;
        const float* ws1 = DUAL ? p.w_scale1 + ((size_t)z * nt_count + n_tile) * kb_total + kb_first : nullptr;
        for (int kb = 0; kb < kb_count; ++kb, ++u) {
          const int buf = u % Cfg::kAccBufs;
          // scales are fetched before the wait so their latency hides behind the MMA of this block
          float sc[kTok];
          const bool gathered = BSRC == kBTma && GROUP != kGroupLoop && p.fab.ag_call >= 0 && p.fab.tp > 1;
          if (BSRC != kBTma) {
#pragma unroll
            for (int r = 0; r < kTok; ++r) sc[r] = r < p.rows ? bscale[r * kb_count + kb] : 0.f;
          } else if (!gathered) {
#pragma unroll
            for (int r = 0; r < kTok; ++r) sc[r] = __ldg(as + r * kb_total + kb);
          }
          const float w0 = __ldg(ws0 + kb);
          const float w1 = DUAL ? __ldg(ws1 + kb) : 0.f;
          if (!mbar_wait(&tail->acc_full[buf], (u / Cfg::kAccBufs) & 1, p.status, kSiteAccFull | buf)) { ok = false; break; }
          if (gathered) {
            // scales of a gathered operand arrive with the peer's slice: read them (coherently) only after
            // the accumulator of that slice is complete, i.e. after the producer has seen the slice's flag
#pragma unroll
            for (int r = 0; r < kTok; ++r) sc[r] = __ldcv(as + r * kb_total + kb);
          }
          tc_fence_after();
          float v0[kTok], v1[kTok];
          tmem_ld16(lane_addr + buf * Cfg::kAccCols, v0);
          if (DUAL) tmem_ld16(lane_addr + buf * Cfg::kAccCols + kTok, v1);
          tc_fence_before();
          mbar_arrive(&tail->acc_empty[buf]);
#pragma unroll
          for (int r = 0; r < kTok; ++r) {
            acc0[r] += v0[r] * (sc[r] * w0);
            if (DUAL) acc1[r] += v1[r] * (sc[r] * w1);
          }
        }
      } else {
        if (!mbar_wait(&tail->acc_full[0], 0, p.status, kSiteAccFull)) { ok = false; break; }
        tc_fence_after();
        tmem_ld16(lane_addr, acc0);
        if (DUAL) tmem_ld16(lane_addr + kTok, acc1);
        tc_fence_before();
      }
      if (GROUP == kGroupLoop) {
        const float* pr = p.probs + (size_t)slot * kTok;
#pragma unroll
        for (int r = 0; r < kTok; ++r) mix0[r] += pr[r] * acc0[r];
      } else {
#pragma unroll
        for (int r = 0; r < kTok; ++r) { mix0[r] = acc0[r]; mix1[r] = acc1[r]; }
      }
    }

    if (threadIdx.x == 64) NRT_STAMP(6);
    // ---------------------------------------------------------------- cluster split: partials -> leader
    bool leader = true;
    if (split > 1) {
      if (crank != 0) {
        leader = false;
        const uint32_t dst = mapa_shared(smem_u32(part), 0);
#pragma unroll
        for (int r = 0; r < kArRows; ++r) {
          st_cluster_f32(dst + (uint32_t)((((crank - 1) * kArRows + r) * kTileN + row) * 4), mix0[r]);
          if (DUAL)
            st_cluster_f32(dst + (uint32_t)(((((split - 1) + crank - 1) * kArRows + r) * kTileN + row) * 4), mix1[r]);
        }
        mbar_arrive_cluster(mapa_shared(smem_u32(&tail->split_bar), 0));
      } else {
        if (mbar_wait_cluster(&tail->split_bar, 0, p.status, kSiteCluster)) {
          for (int y = 1; y < split; ++y)
#pragma unroll
            for (int r = 0; r < kArRows; ++r) {
              mix0[r] += part[((y - 1) * kArRows + r) * kTileN + row];
              if (DUAL) mix1[r] += part[(((split - 1) + y - 1) * kArRows + r) * kTileN + row];
            }
        }
      }
    }

    if (threadIdx.x == 64) NRT_STAMP(7);
    // ---------------------------------------------------------------- epilogue op
    const bool live = leader && (n_groups > 0 || split > 1) && n < p.n_total;
    // group-item mode over a long row buffer: this CTA's 16 rows start at row_offsets[item]
    const size_t out_row0 = (GROUP == kGroupItem && p.row_offsets && n_groups > 0) ? (size_t)p.row_offsets[g_first] : 0;
    if (EPI == kEpiStoreF32) {
#pragma unroll
      for (int r = 0; r < kTok; ++r)
        if (live && r < p.rows) p.out_f32[(out_row0 + r) * p.ld_out + n] = mix0[r] * p.out_scale;
    } else if (EPI == kEpiStoreBF16) {
#pragma unroll
      for (int r = 0; r < kTok; ++r)
        if (live && r < p.rows) p.out_bf16[(out_row0 + r) * p.ld_out + n] = __float2bfloat16_rn(mix0[r] * p.out_scale);
    } else if (EPI == kEpiSiluBF16) {
#pragma unroll
      for (int r = 0; r < kTok; ++r)
        if (live && r < p.rows) p.out_bf16[(size_t)r * p.ld_out + n] = __float2bfloat16_rn(silu(mix0[r]) * mix1[r]);
    } else if (EPI == kEpiQkvPost) {
      if (leader) qkv_post_epilogue(p.post, post_ctx, n0, quad, lane, mix0, p.rows, out_stage, leader && (n_groups > 0 || split > 1) && n0 < p.n_total);
    } else if (EPI == kEpiSiluQuant) {
      if (n_groups > 0) {
        // y = silu(gate) * up in fp32; one power-of-two scale per (token, this 128-feature tile).  Live rows only;
        // the scale of a row is derived once (thread r of the tile) and applied as an exact reciprocal.
        float y[kTok];
#pragma unroll
        for (int r = 0; r < kTok; ++r) {
          y[r] = 0.f;
          if (r < p.rows) {
            y[r] = silu(mix0[r]) * mix1[r];
            const float m = warp_max_f(fabsf(y[r]));
            if (lane == 0) tail->red[quad][r] = m;
          }
        }
        epi_bar();
        if (row < p.rows) {
          const float am = fmaxf(fmaxf(tail->red[0][row], tail->red[1][row]), fmaxf(tail->red[2][row], tail->red[3][row]));
          tail->rs[row] = pow2_scale(am);
        }
        epi_bar();
        const size_t qrow = GROUP == kGroupNone ? 0 : (p.row_offsets ? (size_t)p.row_offsets[g_first] : (size_t)g_first * kTok);
#pragma unroll
        for (int r = 0; r < kTok; ++r) {
          if (r < p.rows && leader) {               // K split over a cluster: only the leader holds the full sums
            const float s = tail->rs[r];
            p.out_q[(qrow + r) * p.n_total + n] = e4m3_bits(y[r] * (1.0f / s));
            if (row == 0) p.out_qscale[(qrow + r) * nt_count + n_tile] = s;
          }
        }
      }
    } else if (EPI == kEpiReturn) {
      // Expert outputs go straight back to the token owner: bf16 pairs of adjacent features as tagged
      // words into slot (token, k) of the owner's combine buffer (peer memory).
      if (n_groups > 0) {
        const uint32_t dtag = (*p.fab.epoch) * 1024u + (uint32_t)p.ep_dispatch_call + 1u;
        const uint32_t rtag = (*p.fab.epoch) * 1024u + (uint32_t)p.ep_return_call + 1u;
        const size_t row0 = p.row_offsets ? (size_t)p.row_offsets[g_first] : 0;
        const int words = p.n_total / 2;
#pragma unroll
        for (int r = 0; r < kTok; ++r) {
          const int4 m = p.ep_meta[row0 + r];
          const float other = __shfl_down_sync(0xffffffffu, mix0[r], 1);
          if ((uint32_t)m.w == dtag && (lane & 1) == 0 && n + 1 < p.n_total + 1) {
            uint64_t* dst = p.ep_combine[m.x] + ((size_t)(m.y * p.ep_top_k + m.z)) * words + (n >> 1);
            st_tagged(dst, rtag, pack_bf16x2(mix0[r], other));
          }
        }
      }
    } else if (EPI == kEpiAllReduce) {
      allreduce_epilogue(p, mix0, n, n_tile, row, lane, quad, leader, tail, stamp, resid_pre);
    }
    (void)ok;
    if (threadIdx.x == 64) NRT_STAMP(11);
  }
#undef NRT_STAMP

  drain_on_error(p.status);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, Cfg::kTmemCols); }
}

}  // namespace nrt

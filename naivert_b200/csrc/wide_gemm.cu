// Chunk GEMM for prefill: the same swapped-operand tcgen05 engine as gemm.cuh with 64 token columns per tile.
//
// The 16-column engine re-reads every 16 KiB weight tile from L2 once per 16 tokens, which bounds a
// prefill chunk by L2 -> SM bandwidth (~18 KiB per 0.5 MFLOP).  Here one CTA owns 128 output features x
// 64 token rows of one work item (grid.y = item; an item is 64 consecutive rows of the token operand that
// share one weight group: a row group of a prefill chunk, or a padded expert segment of the expert-parallel
// receive buffer), so a weight tile feeds four times the math.
//   warp 0     : TMA producer (weights 128 x 128 B, tokens 64 x 128 B, 128-byte swizzle, no multicast)
//   warp 1     : TMEM allocator + UMMA issuer (M = 128, N = 64; kind::f8f6f4 or kind::f16)
//   warps 2..9 : epilogue; thread = output feature x one half (32) of the token columns: two warps per TMEM
//                lane quadrant, so every scheduler has two epilogue warps to hide TMEM-load latency
// Block-scaled e4m3: one fresh TMEM accumulator per 128-wide K block (ring of 4), scaled by weight-block x
// activation-block scale and promoted in fp32 registers in ascending K order (the same arithmetic as the
// 16-column engine, so both produce identical values).  Activation scales of the item are staged in shared
// memory once (after the first accumulator is ready, i.e. after the producer has seen the rows arrive).
// Epilogues: fp32 / bf16 store, SiLU(gate) * up with e4m3 re-quantisation, and the expert-parallel return
// (tagged bf16 pairs into the token owner's combine slots in peer memory).
//
// Reference counterpart: DeepGEMM contiguous grouped fp8 GEMM and cuBLAS bf16 GEMMs of the reference's prefill
// (naivert/kernels/naive_n0p5/prefill.py:1044-1146).
#include "gemm.cuh"
#include "launch.hpp"

#include <string.h>

using namespace nrt;

namespace {

constexpr int kWTok = 64;
constexpr int kWBTileBytes = kWTok * kKBytes;    // 8 KiB

template <bool FP8, bool DUAL>
struct WideCfg {
  static constexpr int kStageBytes = (DUAL ? 2 : 1) * kATileBytes + kWBTileBytes;
  static constexpr int kStages = DUAL ? 4 : 6;
  static constexpr int kAccCols = DUAL ? 2 * kWTok : kWTok;
  static constexpr int kAccBufs = FP8 ? 4 : 2;                     // bf16: one accumulator per tile, two tiles in flight
  static constexpr int kTmemCols = kAccCols * kAccBufs;            // 128, 256 or 512
  static constexpr int kMaxKBlocks = 128;                          // K <= 16384 for e4m3
  static constexpr int kScaleBytes = kMaxKBlocks * kWTok * 4;      // activation scales [K blocks][64]
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 2048 /*barriers + scratch*/ + kScaleBytes;
};

struct WideTail {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t acc_full[4];
  uint64_t acc_empty[4];
  uint32_t tmem_base;
  uint32_t pad;
  float red[4][kWTok];
};

constexpr int kWThreads = 320;
constexpr int kWHalf = kWTok / 2;                // token columns per epilogue thread

// Persistent CTAs (one per SM) walk the (feature tile, item) work list with a fixed stride, so the TMA producer
// and the MMA issuer run ahead into the next tile while the epilogue warps still store the previous one; the
// stage ring and the accumulator ring simply continue across tiles.
// order 0: feature tiles vary fastest over the work list (consecutive CTAs share the item's token tile: grouped
// experts; or a weight matrix that fits the L2); order 1: items vary fastest (consecutive CTAs share a weight
// tile: one big weight matrix that must stream from HBM only once per chunk).
template <bool FP8, bool DUAL, int EPI>
__global__ void __launch_bounds__(kWThreads, 1)
wide_gemm_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
                 const __grid_constant__ CUtensorMap tmB, const GemmArgs p, const int order, const int n_tiles, const int items) {
  using Cfg = WideCfg<FP8, DUAL>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  WideTail* tail = reinterpret_cast<WideTail*>(smem + Cfg::kStages * Cfg::kStageBytes);
  float* as_s = reinterpret_cast<float*>(smem + Cfg::kStages * Cfg::kStageBytes + 2048);   // [kb][64]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kElemsPerStage = FP8 ? 128 : 64;
  const int kb_total = p.k_total / kElemsPerStage;

  if (threadIdx.x == 0) {
    for (int i = 0; i < Cfg::kStages; ++i) { mbar_init(&tail->full[i], 1); mbar_init(&tail->empty[i], 1); }
    for (int i = 0; i < Cfg::kAccBufs; ++i) { mbar_init(&tail->acc_full[i], 1); mbar_init(&tail->acc_empty[i], 256); }
    mbar_fence_init();
    tma_prefetch_desc(&tmA0);
    tma_prefetch_desc(&tmB);
    if (DUAL) tma_prefetch_desc(&tmA1);
  }
  if (warp == 1) { tmem_alloc(&tail->tmem_base, Cfg::kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tail->tmem_base;
  griddep_wait();
  griddep_launch();

  const int na = min(min(*p.n_active, p.max_slots), items);
  const int total = n_tiles * items;
  // every role walks the same list: work w -> (feature tile, item); items >= na are skipped by all roles alike
#define NRT_WIDE_DECODE(w, n_tile, item)                               \
  const int n_tile = order ? (w) / items : (w) % n_tiles;              \
  const int item = order ? (w) % items : (w) / n_tiles;

  if (warp == 0) {
    if (elect_one()) {
      bool ready = !(p.fab.ag_call >= 0 && p.fab.tp > 1);
      bool ok = true;
      int u = 0;                                               // stage counter over all tiles of this CTA
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
        NRT_WIDE_DECODE(w, n_tile, item)
        if (item >= na) continue;
        const int z = p.active_ids[item];
        const int brow = p.row_offsets ? p.row_offsets[item] : item * kWTok;
        for (int kb = 0; kb < kb_total; ++kb, ++u) {
          const int st = u % Cfg::kStages;
          if (u >= Cfg::kStages &&
              !mbar_wait(&tail->empty[st], ((u / Cfg::kStages) & 1) ^ 1, p.status, kSiteStageEmpty | st)) { ok = false; break; }
          uint8_t* sa = smem + st * Cfg::kStageBytes;
          const int kx = kb * kElemsPerStage;
          mbar_expect_tx(&tail->full[st], Cfg::kStageBytes);
          tma_load_3d(sa, &tmA0, &tail->full[st], kx, n_tile * kTileN, z);
          if (DUAL) tma_load_3d(sa + kATileBytes, &tmA1, &tail->full[st], kx, n_tile * kTileN, z);
          if (!ready) {
            // expert-parallel dispatch: the rows of every source rank must have landed before the first token tile
            const uint32_t tag = (*p.fab.epoch) * 1024u + (uint32_t)p.fab.ag_call + 1u;
            bool all = true;
            for (int s = 0; s < p.fab.tp && all; ++s) {
              uint32_t v;
              all = wait_tagged(p.fab.ag_flags + s, tag, v, globaltimer() + p.fab.timeout_ns, p.status, kSiteMailbox | 0x60 | s);
            }
            if (!all) { ok = false; break; }
            asm volatile("fence.acq_rel.sys;" ::: "memory");
            asm volatile("fence.proxy.async;" ::: "memory");
            ready = true;
          }
          tma_load_2d(sa + (DUAL ? 2 : 1) * kATileBytes, &tmB, &tail->full[st], kx, brow);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc(FP8 ? 0u : 1u, kTileN, kWTok);
      bool ok = true;
      int u = 0, v = 0, t = 0;                                 // stages, accumulator uses, live tiles of this CTA
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
        NRT_WIDE_DECODE(w, n_tile, item)
        (void)n_tile;
        if (item >= na) continue;
        for (int kb = 0; kb < kb_total; ++kb, ++u) {
          const int st = u % Cfg::kStages;
          // e4m3: a fresh accumulator per K block; bf16: one accumulator per tile, two tiles in flight
          const bool new_acc = FP8 || kb == 0;
          const int buf = FP8 ? (v % Cfg::kAccBufs) : (t % Cfg::kAccBufs);
          if (new_acc) {
            const int uses = FP8 ? v : t;
            if (uses >= Cfg::kAccBufs &&
                !mbar_wait(&tail->acc_empty[buf], ((uses / Cfg::kAccBufs) & 1) ^ 1, p.status, kSiteAccEmpty | buf)) { ok = false; break; }
          }
          if (!mbar_wait(&tail->full[st], (u / Cfg::kStages) & 1, p.status, kSiteTmaFull | st)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + st * Cfg::kStageBytes);
          const uint64_t da0 = umma_desc_sw128(sa);
          const uint64_t da1 = umma_desc_sw128(sa + kATileBytes);
          const uint64_t db = umma_desc_sw128(sa + (DUAL ? 2 : 1) * kATileBytes);
          const uint32_t d0 = tmem + buf * Cfg::kAccCols;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t acc = FP8 ? (j > 0) : (kb > 0 || j > 0);
            if (FP8) {
              umma_f8(d0, da0 + 2 * j, db + 2 * j, idesc, acc);
              if (DUAL) umma_f8(d0 + kWTok, da1 + 2 * j, db + 2 * j, idesc, acc);
            } else {
              umma_bf16(d0, da0 + 2 * j, db + 2 * j, idesc, acc);
            }
          }
          umma_commit(&tail->empty[st]);
          if (FP8 || kb == kb_total - 1) umma_commit(&tail->acc_full[buf]);
          if (FP8) ++v;
        }
        ++t;
      }
    }
  } else {
    const int quad = warp & 3;                       // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;                // which 32 token columns
    const int c0 = half * kWHalf;
    const int row = quad * 32 + lane;                // feature within the tile
    const int e = threadIdx.x - 64;                  // 0..255 among the epilogue threads
    const uint32_t lane_addr = tmem + (uint32_t(quad * 32) << 16);
    const int nt_count = p.n_total / kTileN;
    bool ok = true;
    int v = 0, t = 0;
    for (int w = blockIdx.x; w < total && ok; w += gridDim.x) {
      NRT_WIDE_DECODE(w, n_tile, item)
      if (item >= na) continue;
      const int z = p.active_ids[item];
      const int brow = p.row_offsets ? p.row_offsets[item] : item * kWTok;
      const int n = n_tile * kTileN + row;
      float acc0[kWHalf];
      float acc1[DUAL ? kWHalf : 1];
#pragma unroll
      for (int r = 0; r < kWHalf; ++r) acc0[r] = 0.f;
      if (DUAL) {
#pragma unroll
        for (int r = 0; r < kWHalf; ++r) acc1[r] = 0.f;
      }
      if (FP8) {
        const float* ws0 = p.w_scale0 + ((size_t)z * nt_count + n_tile) * kb_total;
        const float* ws1 = DUAL ? p.w_scale1 + ((size_t)z * nt_count + n_tile) * kb_total : nullptr;
        for (int kb = 0; kb < kb_total; ++kb, ++v) {
          const int buf = v % Cfg::kAccBufs;
          const float w0 = __ldg(ws0 + kb);
          const float w1 = DUAL ? __ldg(ws1 + kb) : 0.f;
          if (!mbar_wait(&tail->acc_full[buf], (v / Cfg::kAccBufs) & 1, p.status, kSiteAccFull | buf)) { ok = false; break; }
          if (kb == 0) {
            // activation scales of the item's 64 rows, transposed to [K block][row]; read coherently after the first
            // accumulator is ready (in the expert-parallel path peers wrote them shortly before).  The first barrier
            // keeps a fast warp from overwriting the table while a slow one still reads the previous tile's scales.
            asm volatile("bar.sync 1, 256;" ::: "memory");
            const float* as = p.a_scale + (size_t)brow * kb_total;
            for (int i = e; i < kWTok * kb_total; i += 256) {
              const int r = i / kb_total, k = i - r * kb_total;
              as_s[k * kWTok + r] = __ldcv(as + i);
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
          }
          tc_fence_after();
          uint32_t v0[kWHalf], v1[DUAL ? kWHalf : 1];
          const uint32_t t0 = lane_addr + buf * Cfg::kAccCols + c0;
          tmem_ld16_nowait(t0, v0);
          tmem_ld16_nowait(t0 + 16, v0 + 16);
          if (DUAL) {
            tmem_ld16_nowait(t0 + kWTok, v1);
            tmem_ld16_nowait(t0 + kWTok + 16, v1 + 16);
          }
          tmem_ld_wait();
          tc_fence_before();
          mbar_arrive(&tail->acc_empty[buf]);            // values are in registers: the buffer can be reused
          const float4* sc4 = reinterpret_cast<const float4*>(as_s + kb * kWTok + c0);
#pragma unroll
          for (int q = 0; q < kWHalf / 4; ++q) {
            const float4 s = sc4[q];
            const float sv[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              acc0[q * 4 + j] += __uint_as_float(v0[q * 4 + j]) * (sv[j] * w0);
              if (DUAL) acc1[q * 4 + j] += __uint_as_float(v1[DUAL ? q * 4 + j : 0]) * (sv[j] * w1);
            }
          }
        }
        if (!ok) break;
      } else {
        const int buf = t % Cfg::kAccBufs;
        if (!mbar_wait(&tail->acc_full[buf], (t / Cfg::kAccBufs) & 1, p.status, kSiteAccFull | buf)) { ok = false; break; }
        tc_fence_after();
        uint32_t v0[kWHalf];
        tmem_ld16_nowait(lane_addr + buf * Cfg::kAccCols + c0, v0);
        tmem_ld16_nowait(lane_addr + buf * Cfg::kAccCols + c0 + 16, v0 + 16);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&tail->acc_empty[buf]);
#pragma unroll
        for (int r = 0; r < kWHalf; ++r) acc0[r] = __uint_as_float(v0[r]);
      }
      ++t;

      const bool live = n < p.n_total;
      const size_t out_row0 = (size_t)brow + c0;
      if (EPI == kEpiStoreF32) {
        if (live)
#pragma unroll
          for (int r = 0; r < kWHalf; ++r) p.out_f32[(out_row0 + r) * p.ld_out + n] = acc0[r] * p.out_scale;
      } else if (EPI == kEpiStoreBF16) {
        if (live)
#pragma unroll
          for (int r = 0; r < kWHalf; ++r) p.out_bf16[(out_row0 + r) * p.ld_out + n] = __float2bfloat16_rn(acc0[r] * p.out_scale);
      } else if (EPI == kEpiSiluQuant) {
#pragma unroll
        for (int r = 0; r < kWHalf; ++r) {
          acc0[r] = silu(acc0[r]) * acc1[DUAL ? r : 0];
          float m = fabsf(acc0[r]);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
          if (lane == 0) tail->red[quad][c0 + r] = m;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
#pragma unroll
        for (int r = 0; r < kWHalf; ++r) {
          const int c = c0 + r;
          const float am = fmaxf(fmaxf(tail->red[0][c], tail->red[1][c]), fmaxf(tail->red[2][c], tail->red[3][c]));
          const float s = pow2_scale(am);
          const __nv_fp8_e4m3 q(acc0[r] / s);
          p.out_q[(out_row0 + r) * p.n_total + n] = *reinterpret_cast<const uint8_t*>(&q);
          if (row == 0) p.out_qscale[(out_row0 + r) * nt_count + n_tile] = s;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");      // the amax scratch is reused by the next tile
      } else if (EPI == kEpiReturn) {
        const uint32_t dtag = (*p.fab.epoch) * 1024u + (uint32_t)p.ep_dispatch_call + 1u;
        const uint32_t rtag = (*p.fab.epoch) * 1024u + (uint32_t)p.ep_return_call + 1u;
        const int words = p.n_total / 2;
#pragma unroll
        for (int r = 0; r < kWHalf; ++r) {
          const int4 m = p.ep_meta[out_row0 + r];
          const float other = __shfl_down_sync(0xffffffffu, acc0[r], 1);
          if ((uint32_t)m.w == dtag && (lane & 1) == 0) {
            uint64_t* dst = p.ep_combine[m.x] + ((size_t)(m.y * p.ep_top_k + m.z)) * words + (n >> 1);
            st_tagged(dst, rtag, pack_bf16x2(acc0[r], other));
          }
        }
      }
    }
  }
#undef NRT_WIDE_DECODE

  drain_on_error(p.status);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, Cfg::kTmemCols); }
}

template <bool FP8, bool DUAL, int EPI>
int launch_wide(const CUtensorMap& a0, const CUtensorMap& a1, const CUtensorMap& b, const GemmArgs& args, int n_tiles, int items,
                int order, cudaStream_t stream, int pdl) {
  using Cfg = WideCfg<FP8, DUAL>;
  auto* kern = wide_gemm_kernel<FP8, DUAL, EPI>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if (FP8 && args.k_total / 128 > Cfg::kMaxKBlocks) return -6;        // scale table size
  if (n_tiles < 1 || items < 1 || (long long)n_tiles * items > 0x7fffffffLL) return -3;
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms < 1) sms = 148;
  }
  const int total = n_tiles * items;
  const dim3 grid(total < sms ? total : sms, 1, 1);                    // persistent: one CTA per SM
  return launch_pdl(kern, grid, dim3(kWThreads, 1, 1), Cfg::kSmemBytes, stream, pdl != 0, a0, a1, b, args, order, n_tiles, items);
}

}  // namespace

extern "C" int nrt_wide_tok() { return kWTok; }

// variant = fp8 | dual<<1 | epi<<2 (item mode only; items of 64 rows).  The token tensor map must have 64-row
// boxes.  order: 0 = feature tiles vary fastest over the grid, 1 = items vary fastest.
extern "C" int nrt_wide_gemm_launch(int variant, const void* tmA0, const void* tmA1, const void* tmB, const void* args,
                                    int n_tiles, int items, int order, void* stream, int pdl) {
  CUtensorMap a0, a1, b;
  memcpy(&a0, tmA0, sizeof(a0));
  memcpy(&a1, tmA1 ? tmA1 : tmA0, sizeof(a1));
  memcpy(&b, tmB, sizeof(b));
  GemmArgs g;
  memcpy(&g, args, sizeof(g));
  if (!g.n_active || !g.active_ids) return -3;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define NRT_WCASE(FP8, DUAL, EPI)                    \
  case ((FP8) | ((DUAL) << 1) | ((EPI) << 2)):      \
    return launch_wide<(FP8) != 0, (DUAL) != 0, EPI>(a0, a1, b, g, n_tiles, items, order, s, pdl);
  switch (variant & 31) {
    NRT_WCASE(1, 1, kEpiSiluQuant)
    NRT_WCASE(1, 0, kEpiReturn)
    NRT_WCASE(1, 0, kEpiStoreBF16)
    NRT_WCASE(0, 0, kEpiStoreF32)
    NRT_WCASE(0, 0, kEpiStoreBF16)
    default:
      return -2;
  }
#undef NRT_WCASE
}

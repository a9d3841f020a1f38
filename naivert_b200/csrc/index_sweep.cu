// Lightning-indexer logit sweep on tcgen05.
//
//   logit[r][t] = ( sum_h relu(q8[r,h] . k8[t]) * w'[r,h] ) * k_scale[t]      for every cached position t
//
// The e4m3 key cache [capacity, 128] is streamed once per step: each 128-position tile
// (16 KiB) is one TMA load (128-byte swizzle) and the A operand of a UMMA (M = 128 positions);
// the e4m3 queries of all rows and heads (rows x 16 heads = 128 columns per 8 rows) sit in
// shared memory as the B operand (N = 128).  Four K = 32 UMMAs produce a 128 x 128 fp32 tile in
// TMEM; the epilogue thread of a position reads its TMEM lane, applies relu and the per-
// (row, head) weight, sums the heads and scales by the key's quantisation scale.  Persistent
// CTAs walk the tiles with a 4-stage TMA ring and double-buffered accumulators, so at long
// context the sweep runs at the HBM rate of the key cache (128 B per position per DSA layer).
//
// Reference counterpart: naivert/body/attn_dsa/index_sweep_tcgen05.cuh (tcgen05 M128, 3-stage
// bulk-copy ring, keys pre-swizzled in the cache; here the cache stays row-major and TMA swizzles).
#include "gemm.cuh"
#include "launch.hpp"

#include <string.h>

using namespace nrt;

namespace {

constexpr int kSweepStages = 4;
constexpr int kTilePos = 128;
constexpr int kSweepThreads = 192;

struct SweepArgs {
  const float* ihw;      // [16][heads] head weight x query scale
  const float* iks;      // [capacity] key scales
  const int* pos0;
  int rows, heads, top_k;
  float* logits;         // [16][ld]
  int ld;
  uint32_t* status;
  int group0, ngroups;   // row groups [group0, group0 + ngroups) are swept (ngroups == 0: all); query-row sharding
  const float* iq_scale; // [16][heads] query quantisation scales kept apart from ihw (null: already folded into ihw)
};

struct SweepTail {
  uint64_t full[kSweepStages], empty[kSweepStages];
  uint64_t acc_full[2], acc_empty[2];
  uint64_t qbar;
  uint32_t tmem_base;
  uint32_t pad;
  float hw[256];
};

// dim must be 128 (one swizzle atom of e4m3); rows*heads <= 256, a multiple of 16.
__global__ void __launch_bounds__(kSweepThreads, 1)
index_sweep_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmQ, const SweepArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* qsm = smem + kSweepStages * kATileBytes;                       // up to 256 x 128 B of queries
  SweepTail* tail = reinterpret_cast<SweepTail*>(qsm + 256 * 128);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid.y row groups (prefill chunks): group g holds rows g*16.. with queries at row g*256 of the query map
  const int rg = blockIdx.y + p.group0;
  const int grows = min(16, p.rows - rg * 16);
  const int ncol = grows * p.heads;                                        // UMMA N (<= 256)

  if (threadIdx.x == 0) {
    for (int i = 0; i < kSweepStages; ++i) { mbar_init(&tail->full[i], 1); mbar_init(&tail->empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&tail->acc_full[i], 1); mbar_init(&tail->acc_empty[i], 128); }
    mbar_init(&tail->qbar, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmQ);
  }
  if (warp == 1) { tmem_alloc(&tail->tmem_base, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tail->tmem_base;
  griddep_wait();
  griddep_launch();

  const int p0 = *p.pos0 + rg * 16;
  const int total = p0 + grows;                        // positions visible to the last row of this group
  const bool active = total > p.top_k;                 // otherwise every row is still dense
  const int tiles = active ? (total + kTilePos - 1) / kTilePos : 0;
  int my_tiles = 0;
  for (int t = blockIdx.x; t < tiles; t += gridDim.x) ++my_tiles;

  if (warp == 0) {
    if (elect_one() && my_tiles > 0) {
      mbar_expect_tx(&tail->qbar, 256 * 128);
      tma_load_2d(qsm, &tmQ, &tail->qbar, 0, rg * 256);
      int u = 0;
      for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++u) {
        const int st = u % kSweepStages;
        if (u >= kSweepStages && !mbar_wait(&tail->empty[st], ((u / kSweepStages) & 1) ^ 1, p.status, kSiteStageEmpty | st)) break;
        mbar_expect_tx(&tail->full[st], kATileBytes);
        tma_load_2d(smem + st * kATileBytes, &tmK, &tail->full[st], 0, t * kTilePos);
      }
    }
  } else if (warp == 1) {
    if (elect_one() && my_tiles > 0) {
      const uint32_t idesc = umma_idesc(0u, 128, (uint32_t)ncol);
      const uint64_t db = umma_desc_sw128(smem_u32(qsm));
      bool ok = mbar_wait(&tail->qbar, 0, p.status, kSiteTmaFull | 0x80);
      for (int u = 0; u < my_tiles && ok; ++u) {
        const int st = u % kSweepStages, buf = u & 1;
        if (u >= 2 && !mbar_wait(&tail->acc_empty[buf], ((u >> 1) & 1) ^ 1, p.status, kSiteAccEmpty | buf)) break;
        if (!mbar_wait(&tail->full[st], (u / kSweepStages) & 1, p.status, kSiteTmaFull | st)) break;
        tc_fence_after();
        const uint64_t da = umma_desc_sw128(smem_u32(smem + st * kATileBytes));
#pragma unroll
        for (int j = 0; j < 4; ++j) umma_f8(tmem + buf * 256, da + 2 * j, db + 2 * j, idesc, j > 0);
        umma_commit(&tail->empty[st]);
        umma_commit(&tail->acc_full[buf]);
      }
    }
  } else {
    const int quad = warp & 3;
    const int e = threadIdx.x - 64;                     // 0..127
    for (int i = e; i < 256; i += 128) tail->hw[i] = i < ncol ? p.ihw[(size_t)rg * 16 * p.heads + i] * (p.iq_scale ? p.iq_scale[(size_t)rg * 16 * p.heads + i] : 1.f) : 0.f;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const uint32_t lane_addr = tmem + (uint32_t(quad * 32) << 16);
    int u = 0;
    for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++u) {
      const int buf = u & 1;
      const int pos = t * kTilePos + quad * 32 + lane;
      const float ks = pos < total ? p.iks[pos] : 0.f;
      if (!mbar_wait(&tail->acc_full[buf], (u >> 1) & 1, p.status, kSiteAccFull | buf)) break;
      tc_fence_after();
      for (int r = 0; r < grows; ++r) {
        float acc = 0.f;
        for (int c = 0; c < p.heads; c += 16) {
          float v[16];
          tmem_ld16(lane_addr + buf * 256 + r * p.heads + c, v);
#pragma unroll
          for (int j = 0; j < 16; ++j) acc += fmaxf(v[j], 0.f) * tail->hw[r * p.heads + c + j];
        }
        if (pos < total) p.logits[(size_t)(rg * 16 + r) * p.ld + pos] = acc * ks;
      }
      tc_fence_before();
      mbar_arrive(&tail->acc_empty[buf]);
    }
  }
  drain_on_error(p.status);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

}  // namespace

extern "C" int nrt_sweep_args_size() { return (int)sizeof(SweepArgs); }

// tmK: 2-D map over the e4m3 key cache [capacity][128], box 128 x 128 B, 128-byte swizzle.
// tmQ: 2-D map over the e4m3 queries [256][128] (row = token_row * heads + head), box 128 B x 256 rows.
extern "C" int nrt_index_sweep(const void* tmK, const void* tmQ, const void* args, int blocks, void* stream, int pdl) {
  CUtensorMap k, q;
  memcpy(&k, tmK, sizeof(k));
  memcpy(&q, tmQ, sizeof(q));
  SweepArgs a;
  memcpy(&a, args, sizeof(a));
  int groups = (a.rows + 15) / 16;
  if (a.heads != 16 && groups > 1) return -3;           // row groups assume 256 query rows per group
  if (a.group0 < 0 || a.group0 + a.ngroups > groups) return -3;
  if (a.ngroups > 0) groups = a.ngroups;
  else if (a.group0 > 0) return -3;
  const int ncol = (a.rows > 16 ? 16 : a.rows) * a.heads;
  if (a.heads % 16 || ncol > 256 || ncol % 16) return -3;
  constexpr int smem = kSweepStages * kATileBytes + 256 * 128 + 2048 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(index_sweep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return launch_pdl(index_sweep_kernel, dim3(blocks, groups), dim3(kSweepThreads), smem, reinterpret_cast<cudaStream_t>(stream),
                    pdl != 0, k, q, a);
}

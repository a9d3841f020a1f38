// One launch for a whole MoE block of the decode / verify step:
//
//   phase R  router: every CTA scores two experts for all rows (fp32 FMA, RMSNorm applied on the fly from the
//            per-tile sums of squares the previous all-reduce left behind) and quantises a share of the e4m3
//            activation packet; a grid-wide arrival counter separates it from the selection, which every CTA
//            then repeats for itself (8 rows x 256 scores: cheaper than a second hand-off through memory);
//   phase G  gate/up: work items (active expert, 128-feature tile) on the dual tcgen05 pipeline (weights by TMA,
//            block-scaled e4m3, fresh TMEM accumulator per 128-wide K block), SiLU(gate) * up re-quantised to
//            e4m3 and left in L2 with a per-(expert, tile) flag;
//   phase D  down: CTA (output tile, expert-id range) streams its experts' down weights - the weight tiles are
//            requested before the flags of their activations are checked, so HBM streaming never stops between
//            the phases - weights each expert by the routing probability, hands its partial to the range-0 CTA
//            of the tile (fixed order), which runs the fused tensor-parallel all-reduce + residual epilogue.
//
// 128 CTAs, one per SM, all resident (the launcher checks the occupancy): the arrival counter and the flags are
// bounded waits that record a status word instead of hanging.  Nothing depends on which other rows share the
// step, and every sum has a fixed order: results equal those of the three separate kernels
// (router_kernel, grouped gate/up, grouped down) bit for bit.
//
// Reference counterparts: naivert/body/rmsnorm_expert_proj/, naivert/body/expert_select_up_gate_silu_rows8_body.cuh,
// naivert/body/expert_down_allreduce/expert_down_w8a8.cuh (three launches there).
#include "gemm.cuh"
#include "launch.hpp"
#include "router.cuh"

#include <stdlib.h>
#include <string.h>

using namespace nrt;

namespace {

constexpr int kMoeCtas = 128, kMoeThreads = 256, kMoeStages = 5;
constexpr int kMoeStageA = 2 * kATileBytes;                 // gate + up tile
constexpr int kMoeStageBytes = kMoeStageA + 2 * kBTileBytes;   // 36 KiB: | gate | up | token tile | second token tile |
// The down phase cuts every stage into two half slots (a 16 KiB weight tile each, and one of the two token tiles), so
// ten down tiles per CTA are in flight while the phases hand over instead of five.
constexpr int kDnSlots = 2 * kMoeStages;
constexpr int kSlotsMax = 128;
constexpr int kGuBufs = 4, kGuCols = 2 * kTok;               // TMEM columns [0, 128): dual accumulators
constexpr int kDnBufs = 8, kDnCols = kTok, kDnBase = 128;    // TMEM columns [128, 256)
constexpr int kMoeTmemCols = 256;
constexpr int kRanges = 4;                                    // expert-id ranges that share one output tile
constexpr int kGuTilesMax = 16;
// Requesting the down tiles into L2 behind the gate/up stages was measured and is off: the block is HBM bound end to
// end, the prefetch only takes bandwidth from the gate/up stream (39.4 -> 42.0 us per block at 8-way shapes).
constexpr bool kPrefetchDown = false;
constexpr int kDnStaged = 256;                                // down units whose scales are staged in shared memory

struct MoeArgs {
  RouterArgs r;
  int inter;                      // local expert intermediate size
  const float* gate_s;            // [experts][inter/128][hidden/128]
  const float* up_s;
  const float* down_s;            // [experts][hidden/128][inter/128]
  uint8_t* y8;                    // [slots * 16][inter] e4m3 hand-off between the phases (stays in L2)
  float* ys;                      // [slots * 16][inter/128]
  unsigned long long* sync;       // grid arrival counter (monotonic over launches)
  unsigned int* slot_flags;       // [kSlotsMax][kGuTilesMax] launch generation once (slot, tile) of y is complete
  float* part;                    // [hidden/128][kRanges - 1][8][128] partial sums of ranges 1..3
  unsigned int* part_flags;       // [hidden/128][kRanges - 1]
  GemmArgs ar;                    // epilogue of the down phase: rows, n_total, out_bf16, ld_out, resid, out_copy, fab, ssq_out
};

struct MoeSmem {
  GemmSmemTail tail;              // full / empty: weight ring; acc_full / acc_empty: down accumulators; red: reductions
  uint64_t gu_full[kGuBufs], gu_empty[kGuBufs];
  uint64_t dn_full[kDnSlots], dn_empty[kDnSlots];   // half slots of the down phase
  uint32_t gen;
  int ok;
  RouterSmem router;
  float probs[kSlotsMax * kTok];
  int active[kSlotsMax];
  alignas(16) float xs_t[64][kArRows];        // read as float4; gate/up activation scales, [K block][row] (hidden <= 8192)
  alignas(16) float dn_sc[kDnStaged][kArRows];   // read as float4; down: y scales of this CTA's first kDnStaged units, [unit][row]
  float dn_w[kDnStaged];          // and their weight-block scales
  float part_s[(kRanges - 1) * kArRows * kTileN];   // cluster launch: partial sums of ranges 1..3, written by the peers
};

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_u32(unsigned int* p, unsigned int v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// bounded wait for a generation tag written by another CTA of this launch
__device__ __forceinline__ bool wait_flag(const unsigned int* p, unsigned int gen, uint32_t* status, uint32_t site) {
  const uint64_t deadline = globaltimer() + kWaitLimitNs;
  for (uint32_t i = 0;; ++i) {
    if (ld_acquire_gpu(p) == gen) return true;
    if ((i & 255u) == 255u) {
      if (status && *reinterpret_cast<volatile uint32_t*>(status) != 0u) return false;
      if (globaltimer() > deadline) break;
    }
  }
  report(status, site);
  return false;
}

template <bool ROUTE>
__global__ void __launch_bounds__(kMoeThreads, 1)
moe_layer_kernel(const __grid_constant__ CUtensorMap tmGate, const __grid_constant__ CUtensorMap tmUp,
                 const __grid_constant__ CUtensorMap tmDown, const __grid_constant__ CUtensorMap tmX8,
                 const __grid_constant__ CUtensorMap tmY8, const MoeArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  MoeSmem& sm = *reinterpret_cast<MoeSmem*>(smem + kMoeStages * kMoeStageBytes);
  GemmSmemTail* tail = &sm.tail;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x;
  uint32_t* status = p.ar.status;
  unsigned long long* stamp = p.ar.stamps ? p.ar.stamps + (size_t)cta * 16 : nullptr;
#define NRT_STAMP(i) do { if (stamp) stamp[i] = globaltimer(); } while (0)

  if (tid == 0) {
    NRT_STAMP(0);
    for (int i = 0; i < kMoeStages; ++i) { mbar_init(&tail->full[i], 1); mbar_init(&tail->empty[i], 1); }
    for (int i = 0; i < kGuBufs; ++i) { mbar_init(&sm.gu_full[i], 1); mbar_init(&sm.gu_empty[i], 128); }
    for (int i = 0; i < kDnBufs; ++i) { mbar_init(&tail->acc_full[i], 1); mbar_init(&tail->acc_empty[i], 128); }
    for (int i = 0; i < kDnSlots; ++i) { mbar_init(&sm.dn_full[i], 1); mbar_init(&sm.dn_empty[i], 1); }
    mbar_init(&tail->split_bar, 128 * (kRanges - 1));
    mbar_fence_init();
    tma_prefetch_desc(&tmGate);
    tma_prefetch_desc(&tmUp);
    tma_prefetch_desc(&tmDown);
    tma_prefetch_desc(&tmX8);
    tma_prefetch_desc(&tmY8);
    sm.ok = 1;
  }
  if (warp == 1) { tmem_alloc(&tail->tmem_base, kMoeTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  // Launched as clusters of kRanges CTAs (the four expert-id ranges of one output tile) where the device can keep all
  // of them resident: the ranges then merge through distributed shared memory instead of global memory and flags.
  uint32_t cluster_x;
  asm volatile("mov.u32 %0, %%cluster_nctaid.x;" : "=r"(cluster_x));
  const bool clustered = cluster_x == (uint32_t)kRanges;
  if (clustered) cluster_sync_all();             // the peers' barriers are initialised before any remote arrive
  tc_fence_after();
  const uint32_t tmem = tail->tmem_base;

  int n_active = 0;
  uint32_t gen = 0;
  if (ROUTE) {
    // ---------------------------------------------------------------- phase R: scores + packet, arrival, selection
    router_scores(p.r, cta, kMoeCtas, sm.router, stamp);     // waits for the upstream grid inside
    router_packet(p.r, cta, kMoeCtas, sm.router);             // read by other CTAs' TMA after the arrival counter
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      NRT_STAMP(1);
      const unsigned long long old = atomicAdd(p.sync, 1ull);
      const unsigned long long target = (old / kMoeCtas + 1ull) * kMoeCtas;
      sm.gen = (uint32_t)(old / kMoeCtas + 1ull);
      const uint64_t deadline = globaltimer() + kWaitLimitNs;
      for (uint32_t i = 0; ld_acquire_u64(p.sync) < target; ++i) {
        if ((i & 63u) == 63u) {
          if (*reinterpret_cast<volatile uint32_t*>(status) != 0u) { sm.ok = 0; break; }
          if (globaltimer() > deadline) { report(status, kSiteGrid | 1u); sm.ok = 0; break; }
        }
      }
      NRT_STAMP(2);
    }
    __syncthreads();
    griddep_launch();                                         // every CTA of this grid is resident by now
    gen = sm.gen;
    router_select(p.r, sm.router, cta == 0, sm.probs, sm.active, stamp);
    n_active = sm.ok ? sm.router.n_active : 0;
  } else {
    // ---------------------------------------------------------------- routed by the preceding router kernel: its
    // active-expert list, slot probabilities and activation packet are read from global memory.  The arrival counter
    // only numbers this launch (the flags of a launch carry its generation); nobody waits on it.
    griddep_wait();
    griddep_launch();
    if (tid == 0) sm.gen = (uint32_t)(atomicAdd(p.sync, 1ull) / kMoeCtas + 1ull);
    n_active = min(*p.r.n_active, p.r.max_slots);
    for (int i = tid; i < n_active; i += kMoeThreads) sm.active[i] = p.r.active_ids[i];
    for (int i = tid; i < n_active * kTok; i += kMoeThreads) sm.probs[i] = p.r.probs[i];
    __syncthreads();
    gen = sm.gen;
  }
  if (tid == 0) NRT_STAMP(3);
#ifdef NRT_BOUNDS_CHECK
  for (int i = tid; i < n_active; i += kMoeThreads)
    if (!NRT_INDEX_OK(sm.active[i], p.r.experts, kBoundsExpert)) sm.active[i] = 0;
  __syncthreads();
#endif

  const int kbH = p.r.hidden / 128;                         // K blocks of gate/up
  const int kbI = p.inter / 128;                            // K blocks of down = gate/up tiles per expert
  const int gu_items = n_active * kbI;
  int my_items = 0;
  for (int it = cta; it < gu_items; it += kMoeCtas) ++my_items;
  const int gu_units = my_items * kbH;
  // down: CTA -> (output tile, expert-id range); the active list is ascending, so a range is a run of slots
  const int tilesH = p.r.hidden / 128;
  const bool dn_on = cta < tilesH * kRanges;
  const int dn_tile = cta / kRanges, dn_range = cta % kRanges;
  int dn_lo = 0, dn_hi = 0;
  if (dn_on) {
    const int per = (p.r.experts + kRanges - 1) / kRanges;
    const int id_lo = dn_range * per, id_hi = id_lo + per;
    for (int i0 = 0; i0 < n_active; i0 += 32) {             // every warp counts with one round of reads
      const int i = i0 + lane;
      const int id = i < n_active ? sm.active[i] : 0x7fffffff;
      dn_lo += __popc(__ballot_sync(0xffffffffu, id < id_lo));
      dn_hi += __popc(__ballot_sync(0xffffffffu, id < id_hi));
    }
  }
  const int dn_slots = dn_hi - dn_lo;
  const int dn_units = dn_slots * kbI;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both phases)
    const bool issuer = elect_one();                          // one lane issues every copy; all lanes poll flags
    int u = 0;
    int ok = 1;
    if (issuer) {
      // the packet was written by plain stores: by other CTAs of this launch when the routing runs in here (order them
      // before the TMA reads); by the preceding router kernel otherwise (the kernel boundary already orders them)
      if (ROUTE) asm volatile("fence.proxy.async;" ::: "memory");
      // gate/up tiles are read once: they leave L2 first, so that the down tiles requested below stay until the
      // down phase reads them
      const uint64_t stream_once = l2_policy_evict_first();
      int pf = 0;                                             // down units already requested into L2
      for (int it = cta; it < gu_items && ok; it += kMoeCtas) {
        const int slot = it / kbI, tile = it - slot * kbI;
        const int z = sm.active[slot];
        for (int kb = 0; kb < kbH; ++kb, ++u) {
          const int st = u % kMoeStages;
          if (u >= kMoeStages && !mbar_wait(&tail->empty[st], ((u / kMoeStages) & 1) ^ 1, status, kSiteStageEmpty | st)) { ok = 0; break; }
          uint8_t* sa = smem + st * kMoeStageBytes;
          mbar_expect_tx(&tail->full[st], kMoeStageA + kBTileBytes);
          tma_load_3d_hint(sa, &tmGate, &tail->full[st], kb * 128, tile * kTileN, z, stream_once);
          tma_load_3d_hint(sa + kATileBytes, &tmUp, &tail->full[st], kb * 128, tile * kTileN, z, stream_once);
          tma_load_2d(sa + kMoeStageA, &tmX8, &tail->full[st], kb * 128, 0);
          // Behind every gate/up stage one down tile of this CTA is requested into L2: the down weights arrive while
          // the gate/up stream runs and while the phases hand over, so HBM never idles between them.
          if (kPrefetchDown && u >= kMoeStages && pf < dn_units) {
            tma_prefetch_l2_3d(&tmDown, (pf % kbI) * 128, dn_tile * kTileN, sm.active[dn_lo + pf / kbI]);
            ++pf;
          }
        }
      }
      if (kPrefetchDown && ok)
        for (; pf < dn_units; ++pf) tma_prefetch_l2_3d(&tmDown, (pf % kbI) * 128, dn_tile * kTileN, sm.active[dn_lo + pf / kbI]);
    }
    // down: the weight tiles of the first ring-full of units are requested before anything waits for their
    // activations; then every lane polls a share of the (slot, tile) flags of this CTA's experts (one round of
    // loads for all of them), and the activation tiles follow
    // Half slot h of the down phase lives in stage h % kMoeStages (weights at + (h / kMoeStages) * 16 KiB, token tile
    // number h / kMoeStages).  Its first use has to wait for the last gate/up unit that used that stage.
    const int npre = min(dn_units, kDnSlots);
    auto slot_free = [&](int i) -> bool {                     // down unit i may overwrite its half slot
      const int h = i % kDnSlots;
      if (i >= kDnSlots) return mbar_wait(&sm.dn_empty[h], ((i / kDnSlots) & 1) ^ 1, status, kSiteStageEmpty | 0x10 | h);
      const int st = h % kMoeStages;
      if (gu_units <= st) return true;                        // the gate/up phase never used this stage
      const int last = ((gu_units - 1 - st) / kMoeStages) * kMoeStages + st;       // last gate/up unit of the stage
      return mbar_wait(&tail->empty[st], (last / kMoeStages) & 1, status, kSiteStageEmpty | st);
    };
    auto slot_w = [&](int i) -> uint8_t* { const int h = i % kDnSlots; return smem + (h % kMoeStages) * kMoeStageBytes + (h / kMoeStages) * kATileBytes; };
    auto slot_b = [&](int i) -> uint8_t* { const int h = i % kDnSlots; return smem + (h % kMoeStages) * kMoeStageBytes + kMoeStageA + (h / kMoeStages) * kBTileBytes; };
    if (issuer && ok) {
      for (int i = 0; i < npre; ++i) {
        if (!slot_free(i)) { ok = 0; break; }
        const int slot = dn_lo + i / kbI, kb = i % kbI;
        mbar_expect_tx(&sm.dn_full[i % kDnSlots], kATileBytes + kBTileBytes);
        tma_load_3d_hint(slot_w(i), &tmDown, &sm.dn_full[i % kDnSlots], kb * 128, dn_tile * kTileN, sm.active[slot],
                         l2_policy_evict_first());
      }
    }
    ok = __shfl_sync(0xffffffffu, ok, __ffs(__ballot_sync(0xffffffffu, issuer)) - 1);
    if (ok) {
      for (int i = lane; i < dn_slots * kbI; i += 32) {
        const int slot = dn_lo + i / kbI, t = i % kbI;
        if (!wait_flag(p.slot_flags + slot * kGuTilesMax + t, gen, status, kSiteGrid | 2u)) ok = 0;
      }
    }
    ok = __all_sync(0xffffffffu, ok);
    if (issuer && ok) {
      asm volatile("fence.proxy.async;" ::: "memory");
      for (int i = 0; i < dn_units; ++i) {
        const int slot = dn_lo + i / kbI, kb = i % kbI;
        if (i >= npre) {
          if (!slot_free(i)) break;
          mbar_expect_tx(&sm.dn_full[i % kDnSlots], kATileBytes + kBTileBytes);
          tma_load_3d_hint(slot_w(i), &tmDown, &sm.dn_full[i % kDnSlots], kb * 128, dn_tile * kTileN, sm.active[slot], l2_policy_evict_first());
        }
        tma_load_2d(slot_b(i), &tmY8, &sm.dn_full[i % kDnSlots], kb * 128, slot * kTok);
      }
    }
    // the down stream of this CTA is issued: HBM goes quiet during the merge and the all-reduce - the next kernel's
    // weights are requested into L2 in that gap
    if (issuer) prefetch_share_l2(p.ar.pf_ptr, p.ar.pf_bytes, cta, kMoeCtas);
  } else if (warp == 1) {
    // ------------------------------------------------------------------ UMMA issuer (both phases)
    if (elect_one()) {
      constexpr uint32_t idesc = umma_idesc(0u, kTileN, kTok);
      int u = 0;
      bool ok = true;
      for (int ug = 0; ug < gu_units && ok; ++ug, ++u) {
        const int st = u % kMoeStages, buf = ug % kGuBufs;
        if (ug >= kGuBufs && !mbar_wait(&sm.gu_empty[buf], ((ug / kGuBufs) & 1) ^ 1, status, kSiteAccEmpty | buf)) { ok = false; break; }
        if (!mbar_wait(&tail->full[st], (u / kMoeStages) & 1, status, kSiteTmaFull | st)) { ok = false; break; }
        if (ug == 0) NRT_STAMP(4);
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + st * kMoeStageBytes);
        const uint64_t da0 = umma_desc_sw128(sa), da1 = umma_desc_sw128(sa + kATileBytes);
        const uint64_t db = umma_desc_sw128(sa + kMoeStageA);
        const uint32_t d0 = tmem + buf * kGuCols;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          umma_f8(d0, da0 + 2 * j, db + 2 * j, idesc, j > 0);
          umma_f8(d0 + kTok, da1 + 2 * j, db + 2 * j, idesc, j > 0);
        }
        umma_commit(&tail->empty[st]);
        umma_commit(&sm.gu_full[buf]);
      }
      NRT_STAMP(5);
      for (int ud = 0; ud < dn_units && ok; ++ud) {
        const int h = ud % kDnSlots, buf = ud % kDnBufs;
        if (ud >= kDnBufs && !mbar_wait(&tail->acc_empty[buf], ((ud / kDnBufs) & 1) ^ 1, status, kSiteAccEmpty | 0x10 | buf)) { ok = false; break; }
        if (!mbar_wait(&sm.dn_full[h], (ud / kDnSlots) & 1, status, kSiteTmaFull | 0x10 | h)) { ok = false; break; }
        tc_fence_after();
        const uint32_t base = smem_u32(smem + (h % kMoeStages) * kMoeStageBytes);
        const uint64_t da = umma_desc_sw128(base + (h / kMoeStages) * kATileBytes);
        const uint64_t db = umma_desc_sw128(base + kMoeStageA + (h / kMoeStages) * kBTileBytes);
        const uint32_t d0 = tmem + kDnBase + buf * kDnCols;
#pragma unroll
        for (int j = 0; j < 4; ++j) umma_f8(d0, da + 2 * j, db + 2 * j, idesc, j > 0);
        umma_commit(&sm.dn_empty[h]);
        umma_commit(&tail->acc_full[buf]);
      }
      NRT_STAMP(6);
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue warps (both phases)
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = tmem + (uint32_t(quad * 32) << 16);
    const int rows = p.r.rows;
    bool ok = true;
    // the residual rows of the down epilogue (written by the predecessor kernel) are fetched now, long before use
    float resid_pre[kArRows];
    {
      const int nres = dn_tile * kTileN + row;
#pragma unroll
      for (int r = 0; r < kArRows; ++r)
        resid_pre[r] = (p.ar.resid && r < p.ar.rows && dn_on && dn_range == 0 && nres < p.ar.n_total)
                           ? __bfloat162float(p.ar.resid[(size_t)r * p.ar.ld_out + nres]) : 0.f;
    }
    // ---- gate/up items
    // Steps have at most eight token rows: the epilogue reads the first eight columns of an accumulator.  The
    // activation scales are the same for every item: staged once as [K block][row].
    constexpr int kR = kArRows;
    for (int i = tid - 64; i < kbH * kR; i += 128) {
      const int kb = i / kR, r = i - kb * kR;
      sm.xs_t[kb][r] = r < rows ? p.r.xs[r * kbH + kb] : 0.f;
    }
    epi_bar();
    int ug = 0;
#pragma unroll 1
    for (int it = cta; it < gu_items && ok; it += kMoeCtas) {
      const int slot = it / kbI, tile = it - slot * kbI;
      const int z = sm.active[slot];
      const int n = tile * kTileN + row;
      float acc0[kR], acc1[kR];
#pragma unroll
      for (int r = 0; r < kR; ++r) { acc0[r] = 0.f; acc1[r] = 0.f; }
      const float* ws0 = p.gate_s + ((size_t)z * kbI + tile) * kbH;
      const float* ws1 = p.up_s + ((size_t)z * kbI + tile) * kbH;
#pragma unroll 1
      for (int kb = 0; kb < kbH; ++kb, ++ug) {
        const int buf = ug % kGuBufs;
        const float4 s0 = *reinterpret_cast<const float4*>(&sm.xs_t[kb][0]), s1 = *reinterpret_cast<const float4*>(&sm.xs_t[kb][4]);
        const float sc[kR] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        const float w0 = __ldg(ws0 + kb), w1 = __ldg(ws1 + kb);
        if (!mbar_wait(&sm.gu_full[buf], (ug / kGuBufs) & 1, status, kSiteAccFull | buf)) { ok = false; break; }
        tc_fence_after();
        float v0[kR], v1[kR];
        tmem_ld8(lane_addr + buf * kGuCols, v0);
        tmem_ld8(lane_addr + buf * kGuCols + kTok, v1);
        tc_fence_before();
        mbar_arrive(&sm.gu_empty[buf]);
#pragma unroll
        for (int r = 0; r < kR; ++r) {
          acc0[r] += v0[r] * (sc[r] * w0);
          acc1[r] += v1[r] * (sc[r] * w1);
        }
      }
      if (!ok) break;
      // y = silu(gate) * up, one power-of-two scale per (row, this tile), e4m3
      float y[kR];
#pragma unroll
      for (int r = 0; r < kR; ++r) {
        y[r] = silu(acc0[r]) * acc1[r];
        const float m = warp_max_f(fabsf(y[r]));
        if (lane == 0) tail->red[quad][r] = m;
      }
      epi_bar();
      if (row < rows) {
        const float am = fmaxf(fmaxf(tail->red[0][row], tail->red[1][row]), fmaxf(tail->red[2][row], tail->red[3][row]));
        tail->rs[row] = pow2_scale(am);
      }
      epi_bar();
#pragma unroll
      for (int r = 0; r < kR; ++r)
        if (r < rows) {
          const float s = tail->rs[r];
          p.y8[((size_t)slot * kTok + r) * p.inter + n] = e4m3_bits(y[r] * (1.0f / s));
          if (row == 0) p.ys[((size_t)slot * kTok + r) * kbI + tile] = s;
        }
      __threadfence();
      epi_bar();
      if (row == 0) st_release_u32(p.slot_flags + slot * kGuTilesMax + tile, gen);
    }
    if (tid == 64) NRT_STAMP(7);
    // ---- down: probability-weighted sum over this CTA's experts
    float mix0[kTok];
#pragma unroll
    for (int r = 0; r < kTok; ++r) mix0[r] = 0.f;
    const int n = dn_tile * kTileN + row;
    int ud = 0;
    // The y scales of a slot are final once the producer has seen the slot flags, i.e. once this CTA's first down
    // accumulator has completed (all flags are polled before the first activation tile is requested).  At that point
    // the epilogue warps fetch the scales of all their units in one round of loads into shared memory; without that
    // every unit would pay an L2 round trip of its own and the accumulator ring would fill up behind the epilogue.
    bool staged = false;
#pragma unroll 1
    for (int s = 0; s < dn_slots && ok; ++s) {
      const int slot = dn_lo + s;
      float acc[kR];
#pragma unroll
      for (int r = 0; r < kR; ++r) acc[r] = 0.f;
#pragma unroll 1
      for (int kb = 0; kb < kbI; ++kb, ++ud) {
        const int buf = ud % kDnBufs;
        if (!mbar_wait(&tail->acc_full[buf], (ud / kDnBufs) & 1, status, kSiteAccFull | 0x10 | buf)) { ok = false; break; }
        if (!staged) {
          for (int i = tid - 64; i < min(dn_units, kDnStaged) * kR; i += 128) {
            const int uu = i / kR, r = i - uu * kR;
            const int sl = dn_lo + uu / kbI, k2 = uu % kbI;
            sm.dn_sc[uu][r] = r < rows ? p.ys[((size_t)sl * kTok + r) * kbI + k2] : 0.f;
            if (r == 0) sm.dn_w[uu] = __ldg(p.down_s + ((size_t)sm.active[sl] * tilesH + dn_tile) * kbI + k2);
          }
          epi_bar();
          staged = true;
        }
        float sc[kR];
        float w0;
        if (ud < kDnStaged) {
          const float4 s0 = *reinterpret_cast<const float4*>(&sm.dn_sc[ud][0]), s1 = *reinterpret_cast<const float4*>(&sm.dn_sc[ud][4]);
          sc[0] = s0.x; sc[1] = s0.y; sc[2] = s0.z; sc[3] = s0.w; sc[4] = s1.x; sc[5] = s1.y; sc[6] = s1.z; sc[7] = s1.w;
          w0 = sm.dn_w[ud];
        } else {
#pragma unroll
          for (int r = 0; r < kR; ++r) sc[r] = r < rows ? p.ys[((size_t)slot * kTok + r) * kbI + kb] : 0.f;
          w0 = __ldg(p.down_s + ((size_t)sm.active[slot] * tilesH + dn_tile) * kbI + kb);
        }
        tc_fence_after();
        float v[kR];
        tmem_ld8(lane_addr + kDnBase + buf * kDnCols, v);
        tc_fence_before();
        mbar_arrive(&tail->acc_empty[buf]);
#pragma unroll
        for (int r = 0; r < kR; ++r) acc[r] += v[r] * (sc[r] * w0);
      }
      const float* pr = sm.probs + slot * kTok;
#pragma unroll
      for (int r = 0; r < kR; ++r) mix0[r] += pr[r] * acc[r];
    }
    if (tid == 64) NRT_STAMP(8);
    // ---- ranges 1..3 hand their partial to range 0 of the tile, which adds them in range order
    bool leader = dn_on && dn_range == 0;
    if (clustered) {
      if (dn_on && dn_range != 0) {
        const uint32_t dst = mapa_shared(smem_u32(sm.part_s), 0);
#pragma unroll
        for (int r = 0; r < kArRows; ++r)
          st_cluster_f32(dst + (uint32_t)((((dn_range - 1) * kArRows + r) * kTileN + row) * 4), mix0[r]);
        mbar_arrive_cluster(mapa_shared(smem_u32(&tail->split_bar), 0));
      } else if (leader) {
        if (mbar_wait_cluster(&tail->split_bar, 0, status, kSiteCluster)) {
#pragma unroll 1
          for (int y = 1; y < kRanges; ++y)
#pragma unroll
            for (int r = 0; r < kArRows; ++r) mix0[r] += sm.part_s[((y - 1) * kArRows + r) * kTileN + row];
        } else {
          ok = false;
        }
      }
    } else if (dn_on && dn_range != 0) {
      float* dst = p.part + ((size_t)(dn_tile * (kRanges - 1) + dn_range - 1) * kArRows) * kTileN + row;
#pragma unroll
      for (int r = 0; r < kArRows; ++r) dst[(size_t)r * kTileN] = mix0[r];
      __threadfence();
      epi_bar();
      if (row == 0) st_release_u32(p.part_flags + dn_tile * (kRanges - 1) + dn_range - 1, gen);
    } else if (leader) {
      for (int y = 1; y < kRanges && ok; ++y) {
        ok = wait_flag(p.part_flags + dn_tile * (kRanges - 1) + y - 1, gen, status, kSiteGrid | 3u);
        const float* src = p.part + ((size_t)(dn_tile * (kRanges - 1) + y - 1) * kArRows) * kTileN + row;
#pragma unroll
        for (int r = 0; r < kArRows; ++r) mix0[r] += __ldcg(src + (size_t)r * kTileN);
      }
    }
    if (tid == 64) NRT_STAMP(9);
    // every CTA takes part in the epilogue's barriers; only the leaders exchange and store
    allreduce_epilogue(p.ar, mix0, n, dn_tile, row, lane, quad, leader, tail, nullptr, resid_pre);
    if (tid == 64) NRT_STAMP(11);
  }
#undef NRT_STAMP

  drain_on_error(status);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, kMoeTmemCols); }
}

}  // namespace

extern "C" int nrt_moe_args_size() { return (int)sizeof(MoeArgs); }
NRT_BOUNDS_EXPORT(moe_fused)
extern "C" int nrt_moe_slot_flag_words() { return kSlotsMax * kGuTilesMax; }
extern "C" long long nrt_moe_part_floats(int hidden) { return (long long)(hidden / 128) * (kRanges - 1) * kArRows * kTileN; }

// Returns -3 when the geometry does not fit this kernel (the caller keeps the three separate launches) and -9 when
// the device cannot hold all 128 CTAs at once (the arrival counter needs every CTA resident).
extern "C" int nrt_moe_layer(const void* tmGate, const void* tmUp, const void* tmDown, const void* tmX8, const void* tmY8,
                             const void* args, void* stream, int pdl) {
  MoeArgs a;
  memcpy(&a, args, sizeof(a));
  const RouterArgs& r = a.r;
  if (r.hidden % 128 || a.inter % 128 || !r.x8 || !r.xs) return -3;
  if (r.w != nullptr && (!r.x || !r.ssq || !r.gamma || !r.scores)) return -3;                 // routing inside the kernel
  if (r.w == nullptr && (!r.n_active || !r.active_ids || !r.probs)) return -3;               // routed by nrt_router
  if (r.experts > 2 * kMoeCtas || r.experts > 256 || r.rows < 1 || r.rows > kArRows || r.top_k > 32) return -3;
  if (r.max_slots > kSlotsMax || a.inter / 128 > kGuTilesMax || (r.hidden / 128) * kRanges > kMoeCtas) return -3;
  if (r.rows * (r.hidden / 128) > 16 * kMoeCtas || r.hidden / 128 > 64) return -3;
  if (!a.sync || !a.slot_flags || !a.part || !a.part_flags || !a.y8 || !a.ys || !a.ar.status) return -3;
  constexpr int smem = kMoeStages * kMoeStageBytes + 1024 + (int)sizeof(MoeSmem);
  static int resident = -1;
  if (resident < 0) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int worst = 1 << 30;
    for (int route = 0; route < 2; ++route) {
      const void* k = route ? (const void*)moe_layer_kernel<true> : (const void*)moe_layer_kernel<false>;
      cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return (int)e;
      int per_sm = 0;
      e = route ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, moe_layer_kernel<true>, kMoeThreads, smem)
                : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, moe_layer_kernel<false>, kMoeThreads, smem);
      if (e != cudaSuccess) return (int)e;
      worst = per_sm * sms < worst ? per_sm * sms : worst;
    }
    resident = worst;
  }
  if (resident < kMoeCtas) return -9;
  // clusters of kRanges CTAs when all 32 of them fit on the device at once (checked per instantiation)
  static int cluster_ok[2] = {-1, -1};
  const int inst = r.w != nullptr ? 1 : 0;
  if (cluster_ok[inst] < 0) {
    const char* env = getenv("NAIVERT_MOE_CLUSTER");
    int n = 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kMoeCtas);
    cfg.blockDim = dim3(kMoeThreads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = kRanges;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    cudaError_t e = inst ? cudaOccupancyMaxActiveClusters(&n, moe_layer_kernel<true>, &cfg)
                         : cudaOccupancyMaxActiveClusters(&n, moe_layer_kernel<false>, &cfg);
    cluster_ok[inst] = (e == cudaSuccess && n >= kMoeCtas / kRanges && !(env && env[0] == '0')) ? 1 : 0;
    if (e != cudaSuccess) cudaGetLastError();
  }
  CUtensorMap g, u, d, x, y;
  memcpy(&g, tmGate, sizeof(g));
  memcpy(&u, tmUp, sizeof(u));
  memcpy(&d, tmDown, sizeof(d));
  memcpy(&x, tmX8, sizeof(x));
  memcpy(&y, tmY8, sizeof(y));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (cluster_ok[inst]) {
    if (inst) return launch_cluster(moe_layer_kernel<true>, dim3(kMoeCtas), dim3(kMoeThreads), dim3(kRanges), smem, st, pdl != 0, g, u, d, x, y, a);
    return launch_cluster(moe_layer_kernel<false>, dim3(kMoeCtas), dim3(kMoeThreads), dim3(kRanges), smem, st, pdl != 0, g, u, d, x, y, a);
  }
  if (inst) return launch_pdl(moe_layer_kernel<true>, dim3(kMoeCtas), dim3(kMoeThreads), smem, st, pdl != 0, g, u, d, x, y, a);
  return launch_pdl(moe_layer_kernel<false>, dim3(kMoeCtas), dim3(kMoeThreads), smem, st, pdl != 0, g, u, d, x, y, a);
}

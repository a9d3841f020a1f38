// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (non-multicast bulk tensor copies),
// tcgen05 (TMEM alloc, UMMA issue/commit, TMEM loads), PDL grid dependencies, system-scope
// tagged loads/stores for the peer-memory fabric, and bounded waits.
//
// Every wait in this file is bounded: it gives up after a fixed number of polls, records
// a site code in a status word and returns false, so a lost peer or a broken pipeline
// ends the kernel with an error status instead of hanging the device.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nrt {

// ----------------------------------------------------------------------------- status words
// status[0]: first error site (0 = ok), written with atomicCAS so the first failure wins.
enum StatusSite : uint32_t {
  kOk = 0,
  kSiteTmaFull = 0x100,      // consumer waited for a TMA stage that never filled
  kSiteStageEmpty = 0x200,   // producer waited for a stage that was never released
  kSiteAccFull = 0x300,      // epilogue waited for an accumulator commit
  kSiteAccEmpty = 0x400,     // MMA issuer waited for an accumulator buffer
  kSiteMailbox = 0x500,      // a peer's tagged word did not arrive
  kSiteCluster = 0x600,      // cluster partner did not arrive
  kSiteRendezvous = 0x700,   // small-message rendezvous
  kSiteGrid = 0x800,         // grid barrier
};

__device__ __forceinline__ void report(uint32_t* status, uint32_t site) {
  if (status) atomicCAS(status, 0u, site);
}

// ----------------------------------------------------------------------------- debug bounds checks
// In a library built with -DNRT_BOUNDS_CHECK (python -m naivert_b200.ops.build --bounds) every index that comes out of
// data - selected key ids, expert ids, token ids - is tested before it addresses memory.  A violation records
// (site, index) in a word of the translation unit, first one wins, and the access is skipped or clamped, so the
// context stays usable and the host reads what went wrong (nrt_bounds_<unit>() returns and clears the word).  In the
// regular build the test is the constant `true` and the word does not exist.
enum BoundsSite : uint32_t { kBoundsAttnKey = 1, kBoundsExpert = 2, kBoundsToken = 3, kBoundsMarkovPrev = 4 };
#ifdef NRT_BOUNDS_CHECK
static __device__ unsigned long long g_bounds_first = 0ull;
__device__ __forceinline__ bool index_ok(long long i, long long n, uint32_t site) {
  if (i >= 0 && i < n) return true;
  atomicCAS(&g_bounds_first, 0ull, ((unsigned long long)(site | 0x80000000u) << 32) | (unsigned long long)(uint32_t)i);
  return false;
}
#define NRT_INDEX_OK(i, n, site) nrt::index_ok((long long)(i), (long long)(n), (site))
#define NRT_BOUNDS_EXPORT(unit)                                                     \
  extern "C" unsigned long long nrt_bounds_##unit() {                               \
    unsigned long long v = 0ull, z = 0ull;                                          \
    if (cudaMemcpyFromSymbol(&v, nrt::g_bounds_first, sizeof(v)) != cudaSuccess) return ~0ull; \
    cudaMemcpyToSymbol(nrt::g_bounds_first, &z, sizeof(z));                         \
    return v;                                                                       \
  }
#else
#define NRT_INDEX_OK(i, n, site) true
#define NRT_BOUNDS_EXPORT(unit) \
  extern "C" unsigned long long nrt_bounds_##unit() { return 0ull; }
#endif

// ----------------------------------------------------------------------------- misc
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ uint64_t globaltimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// PDL: wait for the grids this launch depends on / let dependents start their preamble.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ----------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: polls until a wall-clock deadline (kWaitLimitNs after the first slow poll).
constexpr uint64_t kWaitLimitNs = 2000000000ull;
// The deadline logic is one out-of-line function: a wait appears at dozens of sites in a kernel, and code that runs
// once per launch is paid for in instruction fetch.
static __device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, uint32_t* status, uint32_t site) {
  const uint64_t deadline = globaltimer() + kWaitLimitNs;
#pragma unroll 1
  for (uint32_t i = 0;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 63u) {
      if (status && *reinterpret_cast<volatile uint32_t*>(status) != 0u) return false;
      if (globaltimer() > deadline) break;
    }
  }
  report(status, site);
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t* status, uint32_t site) {
#pragma unroll 1
  for (uint32_t i = 0; i < 64; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, status, site);
}
// After a failed wait, give this CTA's asynchronous copies time to land before it exits.
__device__ __forceinline__ void drain_on_error(const uint32_t* status) {
  if (status && *reinterpret_cast<const volatile uint32_t*>(status) != 0u)
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
}

// ----------------------------------------------------------------------------- thread-block clusters / DSMEM
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// All threads of all CTAs of the cluster (co-scheduled by the hardware, so this cannot starve).
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t local_addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(cta_rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t remote_bar_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
static __device__ __noinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, uint32_t* status, uint32_t site) {
  const uint64_t deadline = globaltimer() + kWaitLimitNs;
#pragma unroll 1
  for (uint32_t i = 0;; ++i) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((i & 63u) == 63u) {
      if (status && *reinterpret_cast<volatile uint32_t*>(status) != 0u) return false;
      if (globaltimer() > deadline) break;
    }
  }
  report(status, site);
  return false;
}

// ----------------------------------------------------------------------------- TMA (never multicast)
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// L2 eviction policies for streams: weights that are read once should not push out what is read again (activations,
// KV rows, tiles another phase has prefetched).
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void tma_load_3d_hint(void* dst, const CUtensorMap* m, uint64_t* bar, int x, int y, int z, uint64_t pol) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "l"(pol)
      : "memory");
}
// Ask the TMA unit to bring one box of a tensor into L2 (no shared memory, no barrier): the later load of the
// same box finds it there.
__device__ __forceinline__ void tma_prefetch_l2_3d(const CUtensorMap* m, int x, int y, int z) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];"
               ::"l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
// Ask for `bytes` (a multiple of 16, 16-byte aligned) of global memory to be brought into L2; nothing waits for it.
__device__ __forceinline__ void bulk_prefetch_l2(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
// This CTA's share of a region that a later kernel will stream (typically the next projection's weights): requested
// into L2 in 8 KiB pieces by one thread, at a point where this kernel's own HBM traffic is over.
__device__ __forceinline__ void prefetch_share_l2(const void* base, unsigned long long bytes, int part, int parts) {
  if (base == nullptr || bytes == 0ull) return;
  const unsigned long long per = ((bytes / (unsigned long long)parts) + 15ull) & ~15ull;
  unsigned long long lo = per * (unsigned long long)part;
  const unsigned long long hi = lo + per < bytes ? lo + per : bytes;
  const char* p8 = reinterpret_cast<const char*>(base);
  for (; lo + 16ull <= hi; lo += 8192ull) {
    const unsigned long long n = hi - lo < 8192ull ? (hi - lo) & ~15ull : 8192ull;
    bulk_prefetch_l2(p8 + lo, (uint32_t)n);
  }
}
__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p) : "memory");
}
// generic-proxy writes to shared memory -> visible to the async proxy (UMMA / TMA reads)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ----------------------------------------------------------------------------- tcgen05 / TMEM
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t cols) {   // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {     // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// commit all prior UMMAs of this thread; the mbarrier gets one arrival when they have finished
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle: rows of 128 bytes,
// 8-row groups 1024 bytes apart (SBO), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);       // start address, bits [0,14)
  d |= static_cast<uint64_t>(1) << 16;                           // leading byte offset (unused with swizzle)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                   // stride byte offset, bits [32,46)
  d |= static_cast<uint64_t>(1) << 46;                           // version = 1
  d |= static_cast<uint64_t>(2) << 61;                           // layout = SWIZZLE_128B
  return d;
}
// Instruction descriptor: fp32 accumulate, both operands K-major.
// fmt: kind::f16 -> 0 f16 / 1 bf16 ; kind::f8f6f4 -> 0 e4m3 / 1 e5m2
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t fmt, uint32_t m, uint32_t n) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns -> 16 registers per thread (lane = TMEM lane)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// 32 lanes x 8 consecutive 32-bit columns (steps of at most eight token rows read half an accumulator)
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float* v) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

// The same load without the wait: issue several, then tmem_ld_wait() once, then read the registers.
__device__ __forceinline__ void tmem_ld16_nowait(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

// ----------------------------------------------------------------------------- fabric words
// A tagged word is 64 bits {tag:32, payload:32}; one store carries data and its own
// validity, so no fence or separate flag is needed.
__device__ __forceinline__ void st_tagged(uint64_t* dst, uint32_t tag, uint32_t payload) {
  asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(dst), "r"(payload), "r"(tag) : "memory");
}
__device__ __forceinline__ void ld_tagged(const uint64_t* src, uint32_t& tag, uint32_t& payload) {
  asm volatile("ld.relaxed.sys.global.v2.b32 {%0, %1}, [%2];" : "=r"(payload), "=r"(tag) : "l"(src) : "memory");
}
// Poll until the word carries `tag`; bounded by a poll count and a wall-clock deadline.
static __device__ __noinline__ bool wait_tagged(const uint64_t* src, uint32_t tag, uint32_t& payload, uint64_t deadline_ns,
                                         uint32_t* status, uint32_t site) {
  uint32_t t;
#pragma unroll 1
  for (uint32_t i = 0;; ++i) {
    ld_tagged(src, t, payload);
    if (t == tag) return true;
    if ((i & 1023u) == 1023u) {
      if (status && *reinterpret_cast<volatile uint32_t*>(status) != 0u) return false;   // someone already failed
      if (globaltimer() > deadline_ns) break;
    }
  }
  report(status, site);
  return false;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

}  // namespace nrt

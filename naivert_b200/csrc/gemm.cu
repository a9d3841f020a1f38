// C ABI of the skinny tcgen05 GEMM engine: tensor-map encoding and kernel launch.
#include "gemm.cuh"
#include "launch.hpp"

#include <cudaTypedefs.h>
#include <string.h>

using namespace nrt;

namespace {

PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

template <bool FP8, bool DUAL, int EPI, int GROUP, int BSRC = kBTma>
int launch_variant(const CUtensorMap& a0, const CUtensorMap& a1, const CUtensorMap& b, const GemmArgs& args, int gx,
                   int gy, cudaStream_t stream, int pdl) {
  using Cfg = GemmCfg<FP8, DUAL, BSRC>;
  auto* kern = skinny_gemm_kernel<FP8, DUAL, EPI, GROUP, BSRC>;
  constexpr int kMaxSmem = 227 * 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxSmem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if ((EPI == kEpiAllReduce || (GROUP != kGroupItem && gy > 1)) && args.rows > kArRows) return -5;
  const bool clustered = GROUP != kGroupItem && gy > 1;
  if (clustered && gy > kMaxSplit) return -4;
  const int kb_total = args.k_total / (FP8 ? 128 : 64);
  const int ksplit = GROUP == kGroupNone && clustered ? gy : 1;
  if (kb_total % ksplit) return -6;
  if (BSRC != kBTma && (!args.nx || !args.ngamma || !args.nssq || args.k_total % 128)) return -6;
  const int smem = Cfg::smem_bytes(kb_total / ksplit, clustered ? gy : 1);
  if (smem > kMaxSmem) return -7;
  if (EPI == kEpiQkvPost) {
    const AttnPostArgs& q = args.post;
    // reductions over a head / the indexer key run over the 128 threads of one tile
    if (q.idx_heads > 0 && (q.idx_dim != kTileN || q.col_iq % kTileN || q.col_ik % kTileN || !q.iq_scale)) return -8;
    if ((q.q_norm || q.k_norm) && (q.head_dim != kTileN || q.col_q % kTileN || q.col_k % kTileN)) return -8;
    if ((q.col_q | q.col_k | q.col_v | q.head_dim | q.rope_dim) & 1) return -8;
  }
  if (clustered)
    return launch_cluster(kern, dim3(gx, gy, 1), dim3(192, 1, 1), dim3(1, gy, 1), smem, stream, pdl != 0, a0, a1, b, args);
  return launch_pdl(kern, dim3(gx, gy, 1), dim3(192, 1, 1), smem, stream, pdl != 0, a0, a1, b, args);
}

}  // namespace

// dtype: 0 = uint8 (e4m3 bytes), 1 = bf16, 2 = fp32.  dims/box innermost first; strides in bytes for
// dims 1..rank-1.  swizzle: 0 none, 1 = 32B, 2 = 64B, 3 = 128B.
extern "C" int nrt_tmap_encode(void* out128, int dtype, int rank, const uint64_t* dims, const uint64_t* strides,
                               const uint32_t* box, int swizzle, void* base) {
  auto fn = encode_fn();
  if (!fn) return -1;
  CUtensorMapDataType dt = dtype == 0 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                           : dtype == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                        : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) { gdim[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides[i];
  CUtensorMapSwizzle sw = swizzle == 3 ? CU_TENSOR_MAP_SWIZZLE_128B
                          : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                          : swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_32B
                                         : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUtensorMap m;
  CUresult r = fn(&m, dt, rank, base, gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return (int)r;
  memcpy(out128, &m, sizeof(m));
  return 0;
}

extern "C" int nrt_gemm_args_size() { return (int)sizeof(GemmArgs); }

// variant = fp8 | dual<<1 | epi<<2 | group<<5 | bsrc<<7
extern "C" int nrt_gemm_launch(int variant, const void* tmA0, const void* tmA1, const void* tmB, const void* args,
                               int grid_x, int grid_y, void* stream, int pdl) {
  CUtensorMap a0, a1, b;
  memcpy(&a0, tmA0, sizeof(a0));
  memcpy(&a1, tmA1 ? tmA1 : tmA0, sizeof(a1));
  memcpy(&b, tmB ? tmB : tmA0, sizeof(b));
  GemmArgs g;
  memcpy(&g, args, sizeof(g));
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define NRT_CASE(FP8, DUAL, EPI, GROUP)                                             \
  case ((FP8) | ((DUAL) << 1) | ((EPI) << 2) | ((GROUP) << 5)):                      \
    return launch_variant<(FP8) != 0, (DUAL) != 0, EPI, GROUP>(a0, a1, b, g, grid_x, grid_y, s, pdl);
#define NRT_CASE_NORM(FP8, DUAL, EPI, GROUP)                                        \
  case ((FP8) | ((DUAL) << 1) | ((EPI) << 2) | ((GROUP) << 5) | (kBNorm << 7)):      \
    return launch_variant<(FP8) != 0, (DUAL) != 0, EPI, GROUP, kBNorm>(a0, a1, b, g, grid_x, grid_y, s, pdl);
  switch (variant) {
    NRT_CASE(1, 0, kEpiStoreF32, kGroupNone)
    NRT_CASE(1, 0, kEpiAllReduce, kGroupNone)
    NRT_CASE(1, 1, kEpiSiluQuant, kGroupNone)
    NRT_CASE(1, 1, kEpiSiluQuant, kGroupItem)
    NRT_CASE(1, 0, kEpiAllReduce, kGroupLoop)
    NRT_CASE(1, 0, kEpiReturn, kGroupItem)
    NRT_CASE(1, 0, kEpiStoreBF16, kGroupItem)
    NRT_CASE(0, 0, kEpiStoreF32, kGroupItem)
    NRT_CASE(0, 0, kEpiStoreBF16, kGroupItem)
    NRT_CASE(0, 0, kEpiStoreF32, kGroupNone)
    NRT_CASE(0, 0, kEpiStoreBF16, kGroupNone)
    NRT_CASE(0, 0, kEpiAllReduce, kGroupNone)
    NRT_CASE(0, 1, kEpiSiluBF16, kGroupNone)
    // token operand normalised inside the kernel (fused RMSNorm)
    NRT_CASE_NORM(0, 0, kEpiQkvPost, kGroupNone)
    NRT_CASE_NORM(0, 0, kEpiStoreF32, kGroupNone)
    NRT_CASE_NORM(0, 1, kEpiSiluBF16, kGroupNone)
    NRT_CASE_NORM(1, 1, kEpiSiluQuant, kGroupNone)
    NRT_CASE_NORM(1, 1, kEpiSiluQuant, kGroupItem)
    default:
      return -2;
  }
#undef NRT_CASE
#undef NRT_CASE_NORM
}

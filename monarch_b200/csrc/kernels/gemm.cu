// Host launchers for the tcgen05 GEMM (see gemm_tcgen05.cuh).
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>

#include "gemm2_tcgen05.cuh"
#include "gemm_tcgen05.cuh"
#include "mb200.h"

namespace mb200 {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                              const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn get_encode() {
  static EncodeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeFn>(p);
  }
  return fn;
}

// 2-D bf16 tensor map: inner extent `inner` (contiguous), outer extent `outer` with
// leading dimension `ld` elements; box = {box_inner, box_outer}; 128-byte swizzle.
int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t ld, uint32_t box_inner, uint32_t box_outer) {
  EncodeFn enc = get_encode();
  if (!enc) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (ld & 7)) return -2;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                   strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA,
                     const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  gemm_cta_body<A_MN, B_MN>(&tmA, &tmB, p, blockIdx.x, gridDim.x, smem_raw);
}

template <bool A_MN, bool B_MN>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
                  cudaStream_t st) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<A_MN, B_MN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         GEMM_SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  gemm_bf16_kernel<A_MN, B_MN><<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, st>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

int make_gemm_tmaps(CUtensorMap* ta, CUtensorMap* tb, const void* A, const void* B, int M, int N,
                    int K, int lda, int ldb, int a_mn, int b_mn) {
  int r;
  if (a_mn)
    r = make_tmap_bf16_2d(ta, A, M, K, lda, 64, 64);
  else
    r = make_tmap_bf16_2d(ta, A, K, M, lda, 64, GEMM_BM);
  if (r) return r;
  if (b_mn)
    r = make_tmap_bf16_2d(tb, B, N, K, ldb, 64, 64);
  else
    r = make_tmap_bf16_2d(tb, B, K, N, ldb, 64, GEMM_BN);
  return r;
}

int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int a_mn,
                int b_mn, int grid, cudaStream_t st) {
  if (a_mn && b_mn) return launch<true, true>(ta, tb, p, grid, st);
  if (a_mn) return launch<true, false>(ta, tb, p, grid, st);
  if (b_mn) return launch<false, true>(ta, tb, p, grid, st);
  return launch<false, false>(ta, tb, p, grid, st);
}

// ------------------------------------------------------------------ CTA-pair variant
template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
    gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA,
                      const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  gemm2_cta_body<A_MN, B_MN>(&tmA, &tmB, p, blockIdx.x >> 1, gridDim.x >> 1, smem_raw);
}

// Number of CTA pairs that can be resident at once (<= SMs / 2; fewer when a GPC has an
// odd number of usable SMs).  Queried once per operand-layout variant.
template <bool A_MN, bool B_MN>
static int pair_capacity() {
  static int cap = 0;
  if (cap) return cap;
  if (cudaFuncSetAttribute(gemm2_bf16_kernel<A_MN, B_MN>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                           G2_SMEM_BYTES) != cudaSuccess)
    return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * (sm_count() / 2));
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = G2_SMEM_BYTES;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm2_bf16_kernel<A_MN, B_MN>, &cfg) != cudaSuccess ||
      n <= 0) {
    cudaGetLastError();
    n = sm_count() / 2;
  }
  if (n > sm_count() / 2) n = sm_count() / 2;
  cap = n;
  return cap;
}

template <bool A_MN, bool B_MN>
static int launch2(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                   cudaStream_t st) {
  const int cap = pair_capacity<A_MN, B_MN>();
  if (cap <= 0) return 1002;
  const int tiles = ((p.M + G2_BM - 1) / G2_BM) * ((p.N + G2_BN - 1) / G2_BN);
  const int pairs = tiles < cap ? tiles : cap;
  gemm2_bf16_kernel<A_MN, B_MN><<<2 * pairs, GEMM_THREADS, G2_SMEM_BYTES, st>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

int make_gemm2_tmaps(CUtensorMap* ta, CUtensorMap* tb, const void* A, const void* B, int M, int N,
                     int K, int lda, int ldb, int a_mn, int b_mn) {
  int r;
  if (a_mn)
    r = make_tmap_bf16_2d(ta, A, M, K, lda, 64, 64);
  else
    r = make_tmap_bf16_2d(ta, A, K, M, lda, 64, G2_HALF);
  if (r) return r;
  if (b_mn)
    r = make_tmap_bf16_2d(tb, B, N, K, ldb, 64, 64);
  else
    r = make_tmap_bf16_2d(tb, B, K, N, ldb, 64, G2_HALF);
  return r;
}

int launch_gemm2(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int a_mn,
                 int b_mn, cudaStream_t st) {
  if (a_mn && b_mn) return launch2<true, true>(ta, tb, p, st);
  if (a_mn) return launch2<true, false>(ta, tb, p, st);
  if (b_mn) return launch2<false, true>(ta, tb, p, st);
  return launch2<false, false>(ta, tb, p, st);
}

// 1: single-CTA 128x256 tiles; 2: CTA-pair 256x256 tiles.
static int g_gemm_impl = 2;

}  // namespace mb200

using namespace mb200;

extern "C" int mb200_gemm_bf16(const void* A, const void* B, void* C, const void* R, int M, int N,
                               int K, int lda, int ldb, int ldc, int ldr, int a_mn, int b_mn,
                               int accumulate, int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  CUtensorMap ta, tb;
  int r = make_gemm_tmaps(&ta, &tb, A, B, M, N, K, lda, ldb, a_mn, b_mn);
  if (r) return 1000 - r;
  GemmParams p{};
  p.C = reinterpret_cast<__nv_bfloat16*>(C);
  p.R = reinterpret_cast<const __nv_bfloat16*>(R);
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc; p.ldr = ldr;
  p.accumulate = accumulate;
  p.status = status;
  p.b_ready = nullptr;
  p.b_ready_target = 0;
  p.flag_chunk_elems = 1;
  p.b_flag_elem0 = 0;
  p.ldb = ldb;
  p.n_blk_rot = 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (g_gemm_impl == 2) {
    CUtensorMap ta2, tb2;
    r = make_gemm2_tmaps(&ta2, &tb2, A, B, M, N, K, lda, ldb, a_mn, b_mn);
    if (r) return 1000 - r;
    return launch_gemm2(ta2, tb2, p, a_mn, b_mn, st);
  }
  const int tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + GEMM_BN - 1) / GEMM_BN);
  int grid = sm_count();
  if (tiles < grid) grid = tiles;
  return launch_gemm(ta, tb, p, a_mn, b_mn, grid, st);
}

extern "C" int mb200_gemm_set_impl(int impl) {
  if (impl != 1 && impl != 2) return 1001;
  g_gemm_impl = impl;
  return 0;
}
extern "C" int mb200_gemm_get_impl() { return g_gemm_impl; }

// Fused all-gather -> GEMM over NVLink (FSDP parameter gather / tensor-parallel
// sequence-parallel gather feeding the first consuming GEMM).
//
//   C[M,N] = A[M,K] * W[N,K]^T (+R),  W = rows of a flat parameter buffer that is sharded
//   across ranks (rank r owns elements [r*S, (r+1)*S) of the buffer).
//
// One kernel, one launch: the first `n_comm` CTAs pull the needed element range of the
// buffer from every rank's shard with per-thread 16-byte peer loads (NVLink P2P), writing it
// to the local copy chunk by chunk and publishing a ready flag per chunk; all other CTAs run
// the persistent tcgen05 GEMM, whose TMA producer waits (bounded) for the chunks under each
// B tile before loading it from the *local* copy.  The transfer of later chunks overlaps
// the tensor-core work on earlier ones, and the gathered copy stays resident for the
// GEMMs that reuse the weight (recompute, input-gradient).
//
// No TMA touches peer memory and no load is multicast: peer data is read with plain
// ld.global by the copy CTAs only.
#include <cuda.h>
#include <cuda_runtime.h>

#include "gather.cuh"
#include "gemm2_tcgen05.cuh"
#include "gemm_tcgen05.cuh"
#include "mb200.h"

namespace mb200 {

int make_gemm_tmaps(CUtensorMap* ta, CUtensorMap* tb, const void* A, const void* B, int M, int N,
                    int K, int lda, int ldb, int a_mn, int b_mn);
int make_gemm2_tmaps(CUtensorMap* ta, CUtensorMap* tb, const void* A, const void* B, int M, int N,
                     int K, int lda, int ldb, int a_mn, int b_mn);
int sm_count();

template <bool A_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    ag_gemm_kernel(const __grid_constant__ CUtensorMap tmA,
                   const __grid_constant__ CUtensorMap tmB, const GemmParams p,
                   const GatherParams g, int n_comm) {
  extern __shared__ uint8_t smem_raw[];
  if ((int)blockIdx.x < n_comm) {
    gather_chunks_bulk(g, blockIdx.x, n_comm, smem_raw);
    return;
  }
  gemm_cta_body<A_MN, false>(&tmA, &tmB, p, blockIdx.x - n_comm, gridDim.x - n_comm, smem_raw);
}

// CTA-pair variant: the copy CTAs are the first n_comm/2 clusters, every other cluster is one
// 256x256-tile GEMM pair (cta_group::2).  n_comm is even, so no cluster mixes the two roles.
template <bool A_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
    ag_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA,
                        const __grid_constant__ CUtensorMap tmB, const GemmParams p,
                        const GatherParams g, int n_comm) {
  extern __shared__ uint8_t smem_raw[];
  if ((int)blockIdx.x < n_comm) {
    gather_chunks_bulk(g, blockIdx.x, n_comm, smem_raw);
    return;
  }
  gemm2_cta_body<A_MN, false>(&tmA, &tmB, p, ((int)blockIdx.x - n_comm) >> 1,
                              ((int)gridDim.x - n_comm) >> 1, smem_raw);
}

// Gather-only launch of the same copy loop (used for the chunks that hold 1-D parameters,
// which are needed before the first GEMM of a layer).
__global__ void __launch_bounds__(GEMM_THREADS) gather_only_kernel(const GatherParams g) {
  gather_chunks(g, blockIdx.x, gridDim.x);
}

}  // namespace mb200

using namespace mb200;

// C = A * W^T (+R) where W = unit_buf[w_elem_off : w_elem_off + N*K] is gathered by the same
// kernel.  Chunks [c_begin, c_end) of the unit are pulled and flagged with chunk_epoch.
extern "C" int mb200_ag_gemm(const void* A, int lda, int a_mn, int M, int K, void* unit_buf,
                             long long w_elem_off, int N, void* C, int ldc, const void* R, int ldr,
                             const void* const* shard_ptrs, long long shard_elems, int rank,
                             int world, long long c_begin, long long c_end, long long chunk_elems,
                             uint32_t* chunk_flags, uint32_t chunk_epoch, void* my_flags,
                             int wait_slot, uint32_t wait_epoch, int n_comm, int* status,
                             void* stream) {
  if (world > kMaxRanks || (shard_elems & 7) || (chunk_elems & 7) || (w_elem_off & 7)) return 1001;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const __nv_bfloat16* W = reinterpret_cast<const __nv_bfloat16*>(unit_buf) + w_elem_off;
  CUtensorMap ta, tb;
  int r = make_gemm_tmaps(&ta, &tb, A, W, M, N, K, lda, K, a_mn, 0);
  if (r) return 1000 - r;
  GemmParams p{};
  p.C = reinterpret_cast<__nv_bfloat16*>(C);
  p.R = reinterpret_cast<const __nv_bfloat16*>(R);
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc; p.ldr = ldr;
  p.accumulate = 0;
  p.status = status;
  p.b_ready = chunk_flags;
  p.b_ready_target = chunk_epoch;
  p.flag_chunk_elems = chunk_elems;
  p.b_flag_elem0 = w_elem_off;
  p.ldb = K;
  p.n_blk_rot = 0;
  GatherParams g = make_gather(unit_buf, shard_ptrs, shard_elems, rank, world, c_begin, c_end,
                               chunk_elems, chunk_flags, chunk_epoch, my_flags, wait_slot,
                               wait_epoch, status);
  const int sms = sm_count();
  if (n_comm <= 0) n_comm = 16;
  if (n_comm > sms / 2) n_comm = sms / 2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (mb200_gemm_get_impl() == 2) {
    n_comm &= ~1;
    if (n_comm < 2) n_comm = 2;
    CUtensorMap ta2, tb2;
    r = make_gemm2_tmaps(&ta2, &tb2, A, W, M, N, K, lda, K, a_mn, 0);
    if (r) return 1000 - r;
    const int tiles = ((M + G2_BM - 1) / G2_BM) * ((N + G2_BN - 1) / G2_BN);
    int pairs = sms / 2 - n_comm / 2;
    if (tiles < pairs) pairs = tiles;
    const int grid = n_comm + 2 * pairs;
    static bool configured2[2] = {false, false};
    if (!configured2[a_mn ? 1 : 0]) {
      cudaError_t e = a_mn ? cudaFuncSetAttribute(ag_gemm_pair_kernel<true>,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  G2_SMEM_BYTES)
                           : cudaFuncSetAttribute(ag_gemm_pair_kernel<false>,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  G2_SMEM_BYTES);
      if (e != cudaSuccess) return (int)e;
      configured2[a_mn ? 1 : 0] = true;
    }
    if (a_mn)
      ag_gemm_pair_kernel<true><<<grid, GEMM_THREADS, G2_SMEM_BYTES, st>>>(ta2, tb2, p, g, n_comm);
    else
      ag_gemm_pair_kernel<false><<<grid, GEMM_THREADS, G2_SMEM_BYTES, st>>>(ta2, tb2, p, g, n_comm);
    return (int)cudaGetLastError();
  }
  const int tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + GEMM_BN - 1) / GEMM_BN);
  int gemm_ctas = sms - n_comm;
  if (tiles < gemm_ctas) gemm_ctas = tiles;
  const int grid = n_comm + gemm_ctas;
  static bool configured[2] = {false, false};
  if (!configured[a_mn ? 1 : 0]) {
    cudaError_t e = a_mn ? cudaFuncSetAttribute(ag_gemm_kernel<true>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                GEMM_SMEM_BYTES)
                         : cudaFuncSetAttribute(ag_gemm_kernel<false>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                GEMM_SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured[a_mn ? 1 : 0] = true;
  }
  if (a_mn)
    ag_gemm_kernel<true><<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, st>>>(ta, tb, p, g, n_comm);
  else
    ag_gemm_kernel<false><<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, st>>>(ta, tb, p, g, n_comm);
  return (int)cudaGetLastError();
}

extern "C" int mb200_gather_chunks(void* unit_buf, const void* const* shard_ptrs,
                                   long long shard_elems, int rank, int world, long long c_begin,
                                   long long c_end, long long chunk_elems, uint32_t* chunk_flags,
                                   uint32_t chunk_epoch, void* my_flags, int wait_slot,
                                   uint32_t wait_epoch, int n_blocks, int* status, void* stream) {
  if (world > kMaxRanks || (shard_elems & 7) || (chunk_elems & 7)) return 1001;
  if (c_end <= c_begin) return 0;
  GatherParams g = make_gather(unit_buf, shard_ptrs, shard_elems, rank, world, c_begin, c_end,
                               chunk_elems, chunk_flags, chunk_epoch, my_flags, wait_slot,
                               wait_epoch, status);
  long long n = c_end - c_begin;
  int grid = n_blocks > 0 ? n_blocks : (int)(n < 64 ? n : 64);
  gather_only_kernel<<<grid, GEMM_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(g);
  return (int)cudaGetLastError();
}

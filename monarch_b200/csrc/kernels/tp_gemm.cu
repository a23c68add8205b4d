// Tensor-parallel (Megatron, sequence-parallel) GEMMs fused with their collectives.
//
// * ag_a_gemm: all-gather of the sequence-sharded activation (rank r owns rows
//   [r*M/W, (r+1)*M/W) of A) fused into the column-parallel GEMM that consumes it:
//   copy CTAs pull peer rows over NVLink into the local full A chunk by chunk while the
//   other CTAs run the tcgen05 GEMM, whose TMA producer waits (bounded) on the chunks under
//   each A tile.  The gathered A stays resident for the weight-gradient GEMM.
// * gemm_rs: row-parallel GEMM whose epilogue stores each bf16 partial tile straight into
//   the staging slot of the rank that owns those rows (plain 16-byte peer stores from the
//   epilogue warps, tile by tile, while later tiles are still on the tensor cores);
//   rs_finish sums the slots in fp32 (+ residual) on the owner after a flag barrier.
//
// No tensor-map TMA and no multicast on peer memory: peer data moves with plain loads and
// stores or with non-multicast bulk copies (cp.async.bulk) issued by the copy CTAs.
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
int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int a_mn,
                int b_mn, int grid, cudaStream_t st);
int launch_gemm2(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int a_mn,
                 int b_mn, cudaStream_t st);
int sm_count();

template <bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    ag_a_gemm_kernel(const __grid_constant__ CUtensorMap tmA,
                     const __grid_constant__ CUtensorMap tmB, const GemmParams p,
                     const GatherParams g, int n_comm) {
  extern __shared__ uint8_t smem_raw[];
  if ((int)blockIdx.x < n_comm) {
    gather_chunks_bulk(g, blockIdx.x, n_comm, smem_raw);
    return;
  }
  gemm_cta_body<false, B_MN>(&tmA, &tmB, p, blockIdx.x - n_comm, gridDim.x - n_comm, smem_raw);
}

template <bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
    ag_a_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA,
                          const __grid_constant__ CUtensorMap tmB, const GemmParams p,
                          const GatherParams g, int n_comm) {
  extern __shared__ uint8_t smem_raw[];
  if ((int)blockIdx.x < n_comm) {   // n_comm is even: whole clusters copy
    gather_chunks_bulk(g, blockIdx.x, n_comm, smem_raw);
    return;
  }
  gemm2_cta_body<false, B_MN>(&tmA, &tmB, p, ((int)blockIdx.x - n_comm) >> 1,
                              ((int)gridDim.x - n_comm) >> 1, smem_raw);
}

// out[r, c] = sum_s staging[s][r][c] (+ residual[r, c]); fp32 accumulation, bf16 out.
// With epoch != 0 the kernel is also the barrier between the GEMMs that filled the staging
// slots and this sum: block 0 tells every peer that this rank's GEMM has finished (true by
// stream order), every block waits (bounded) until all peers have said the same.
__global__ void __launch_bounds__(256)
    rs_finish_kernel(const __nv_bfloat16* __restrict__ staging, int world, int rows, int N, int ld,
                     const __nv_bfloat16* __restrict__ residual, int ldr,
                     __nv_bfloat16* __restrict__ out, int ldo, Peers flags, int rank, int slot,
                     uint32_t epoch, int* status) {
  if (epoch != 0) {
    __shared__ int sh_ok;
    if (blockIdx.x == 0) signal_all(flags, world, rank, slot, epoch, threadIdx.x);
    if (!block_wait_all(flags.p[rank], world, slot, epoch, status, &sh_ok)) return;
  }
  const int vec_per_row = N >> 3;
  const long long total = (long long)rows * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / vec_per_row);
    const int c = (int)(i - (long long)r * vec_per_row) << 3;
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int s = 0; s < world; ++s)
      acc8(a, *reinterpret_cast<const uint4*>(staging + ((size_t)s * rows + r) * ld + c));
    if (residual) acc8(a, *reinterpret_cast<const uint4*>(residual + (size_t)r * ldr + c));
    uint4 o;
    o.x = pack_bf16x2(a[0], a[1]);
    o.y = pack_bf16x2(a[2], a[3]);
    o.z = pack_bf16x2(a[4], a[5]);
    o.w = pack_bf16x2(a[6], a[7]);
    *reinterpret_cast<uint4*>(out + (size_t)r * ldo + c) = o;
  }
}

}  // namespace mb200

using namespace mb200;

// C[M,N] = AG(A)[M,K] * op(B) (+R).  a_full is the local [M,K] buffer (leading dimension K)
// that receives every rank's rows; shard_ptrs[r] points at rank r's M/world rows.
// b_mn=0: B is [N,K] row-major (ldb), b_mn=1: B is [K,N] row-major (ldb).
extern "C" int mb200_ag_a_gemm(void* a_full, const void* const* shard_ptrs, long long shard_elems,
                               int rank, int world, int M, int K, const void* B, int ldb, int b_mn,
                               int N, void* C, int ldc, const void* R, int ldr,
                               long long chunk_elems, uint32_t* chunk_flags, uint32_t chunk_epoch,
                               void* my_flags, int wait_slot, uint32_t wait_epoch, int n_comm,
                               int* status, void* stream) {
  if (world > kMaxRanks || (shard_elems & 7) || (chunk_elems & 7) || (K & 7)) return 1001;
  if ((long long)M * K != shard_elems * world) return 1001;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  CUtensorMap ta, tb;
  int r = make_gemm_tmaps(&ta, &tb, a_full, B, M, N, K, K, ldb, 0, b_mn);
  if (r) return 1000 - r;
  GemmParams p{};
  p.C = reinterpret_cast<__nv_bfloat16*>(C);
  p.R = reinterpret_cast<const __nv_bfloat16*>(R);
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc; p.ldr = ldr;
  p.status = status;
  p.flag_chunk_elems = 1;
  p.ldb = ldb;
  p.a_ready = chunk_flags;
  p.a_ready_target = chunk_epoch;
  p.a_flag_chunk_elems = chunk_elems;
  p.a_flag_elem0 = 0;
  p.lda = K;
  const long long n_chunks = ((long long)M * K + chunk_elems - 1) / chunk_elems;
  GatherParams g = make_gather(a_full, shard_ptrs, shard_elems, rank, world, 0, n_chunks,
                               chunk_elems, chunk_flags, chunk_epoch, my_flags, wait_slot,
                               wait_epoch, status);
  // own rows first, then the peers in ring order -- for the copies (every rank reads a
  // different peer at any time) and for the GEMM's tiles (the rows already here are
  // multiplied while the others travel); one rank's rows form one group of the tile order
  g.c_rot = ((long long)rank * shard_elems) / chunk_elems;
  const int rows_per_rank = M / world;
  p.m_rot = (int)(((long long)rank * rows_per_rank) / G2_BM);
  p.m_group = rows_per_rank / G2_BM;
  if (p.m_group < 1) p.m_group = 1;
  if (p.m_group > 8) p.m_group = 8;
  const int sms = sm_count();
  // n_comm < 0: the rows are brought in from outside the kernel (copy engines on another
  // stream, which raise the same chunk flags): no copy CTAs, every SM multiplies
  const bool external = n_comm < 0;
  if (n_comm == 0) n_comm = 16;
  if (n_comm > sms / 2) n_comm = sms / 2;
  if (external) n_comm = 0;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (mb200_gemm_get_impl() == 2) {
    n_comm &= ~1;
    if (n_comm < 2 && !external) n_comm = 2;
    CUtensorMap ta2, tb2;
    r = make_gemm2_tmaps(&ta2, &tb2, a_full, B, M, N, K, K, ldb, 0, b_mn);
    if (r) return 1000 - r;
    const int tiles = ((M + G2_BM - 1) / G2_BM) * ((N + G2_BN - 1) / G2_BN);
    int pairs = sms / 2 - n_comm / 2;
    if (tiles < pairs) pairs = tiles;
    const int grid = n_comm + 2 * pairs;
    static bool configured2[2] = {false, false};
    if (!configured2[b_mn ? 1 : 0]) {
      cudaError_t e = b_mn ? cudaFuncSetAttribute(ag_a_gemm_pair_kernel<true>,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  G2_SMEM_BYTES)
                           : cudaFuncSetAttribute(ag_a_gemm_pair_kernel<false>,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  G2_SMEM_BYTES);
      if (e != cudaSuccess) return (int)e;
      configured2[b_mn ? 1 : 0] = true;
    }
    if (b_mn)
      ag_a_gemm_pair_kernel<true><<<grid, GEMM_THREADS, G2_SMEM_BYTES, st>>>(ta2, tb2, p, g, n_comm);
    else
      ag_a_gemm_pair_kernel<false><<<grid, GEMM_THREADS, G2_SMEM_BYTES, st>>>(ta2, tb2, p, g, n_comm);
    return (int)cudaGetLastError();
  }
  const int tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + GEMM_BN - 1) / GEMM_BN);
  int gemm_ctas = sms - n_comm;
  if (tiles < gemm_ctas) gemm_ctas = tiles;
  const int grid = n_comm + gemm_ctas;
  static bool configured[2] = {false, false};
  if (!configured[b_mn ? 1 : 0]) {
    cudaError_t e = b_mn ? cudaFuncSetAttribute(ag_a_gemm_kernel<true>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                GEMM_SMEM_BYTES)
                         : cudaFuncSetAttribute(ag_a_gemm_kernel<false>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                GEMM_SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured[b_mn ? 1 : 0] = true;
  }
  if (b_mn)
    ag_a_gemm_kernel<true><<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, st>>>(ta, tb, p, g, n_comm);
  else
    ag_a_gemm_kernel<false><<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, st>>>(ta, tb, p, g, n_comm);
  return (int)cudaGetLastError();
}

// Partial[M,N] = op(A) op(B) on this rank's K slice; rows [o*rpr, (o+1)*rpr) are stored (bf16)
// into staging_ptrs[o] + (src_rank*rpr + row % rpr) * rs_ld.  N must be a multiple of 32.
extern "C" int mb200_gemm_rs(const void* A, const void* B, int M, int N, int K, int lda, int ldb,
                             int a_mn, int b_mn, const void* const* staging_ptrs, int world,
                             int rows_per_rank, int rs_ld, int src_rank, int impl, int* status,
                             void* stream) {
  if (world > kMaxRanks || (N & 31) || (rs_ld & 7) || rows_per_rank <= 0 ||
      (long long)rows_per_rank * world < M)
    return 1001;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.status = status;
  p.flag_chunk_elems = 1;
  p.a_flag_chunk_elems = 1;
  p.ldb = ldb;
  p.lda = lda;
  for (int i = 0; i < world; ++i) p.rs_out[i] = const_cast<void*>(staging_ptrs[i]);
  p.rs_rows_per_rank = rows_per_rank;
  p.rs_ld = rs_ld;
  p.rs_src_rank = src_rank;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  CUtensorMap ta, tb;
  if (impl == 2) {
    int r = make_gemm2_tmaps(&ta, &tb, A, B, M, N, K, lda, ldb, a_mn, b_mn);
    if (r) return 1000 - r;
    return launch_gemm2(ta, tb, p, a_mn, b_mn, st);
  }
  int r = make_gemm_tmaps(&ta, &tb, A, B, M, N, K, lda, ldb, a_mn, b_mn);
  if (r) return 1000 - r;
  const int tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + GEMM_BN - 1) / GEMM_BN);
  int grid = sm_count();
  if (tiles < grid) grid = tiles;
  return launch_gemm(ta, tb, p, a_mn, b_mn, grid, st);
}

static int rs_finish_launch(const void* staging, int world, int rows, int N, int ld,
                            const void* residual, int ldr, void* out, int ldo,
                            const void* const* flag_ptrs, int rank, int slot, uint32_t epoch,
                            int* status, void* stream);

static Peers tp_peers(const void* const* ptrs, int world) {
  Peers p{};
  if (ptrs != nullptr)
    for (int i = 0; i < world && i < kMaxRanks; ++i) p.p[i] = const_cast<void*>(ptrs[i]);
  return p;
}

extern "C" int mb200_rs_finish(const void* staging, int world, int rows, int N, int ld,
                               const void* residual, int ldr, void* out, int ldo, void* stream) {
  return rs_finish_launch(staging, world, rows, N, ld, residual, ldr, out, ldo, nullptr, 0, 0, 0,
                          nullptr, stream);
}

// The sum, preceded inside the same launch by the cross-rank barrier that orders it after
// every rank's mb200_gemm_rs (flag slot `slot`, a fresh `epoch` per call).
extern "C" int mb200_rs_finish_sync(const void* staging, int world, int rows, int N, int ld,
                                    const void* residual, int ldr, void* out, int ldo,
                                    const void* const* flag_ptrs, int rank, int slot,
                                    uint32_t epoch, int* status, void* stream) {
  if (flag_ptrs == nullptr || epoch == 0 || world > kMaxRanks) return 1001;
  return rs_finish_launch(staging, world, rows, N, ld, residual, ldr, out, ldo, flag_ptrs, rank,
                          slot, epoch, status, stream);
}

static int rs_finish_launch(const void* staging, int world, int rows, int N, int ld,
                            const void* residual, int ldr, void* out, int ldo,
                            const void* const* flag_ptrs, int rank, int slot, uint32_t epoch,
                            int* status, void* stream) {
  if ((N & 7) || (ld & 7) || (ldo & 7) || (residual && (ldr & 7))) return 1001;
  if (rows <= 0 || N <= 0) return 0;
  const long long total = (long long)rows * (N >> 3);
  int blocks = (int)((total + 255) / 256);
  const int cap = sm_count() * 8;
  if (blocks > cap) blocks = cap;
  rs_finish_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(staging), world, rows, N, ld,
      reinterpret_cast<const __nv_bfloat16*>(residual), ldr,
      reinterpret_cast<__nv_bfloat16*>(out), ldo,
      tp_peers(flag_ptrs, world), rank, slot, epoch, status);
  return (int)cudaGetLastError();
}

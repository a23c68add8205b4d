// Expert-parallel mixture-of-experts kernels: token dispatch and combine over NVLink fused
// with the expert GEMMs (one expert per rank, top-k routing).
//
// Every rank publishes, in peer-mapped memory, per expert e: counts[e] and lists[e][*]
// (entries token*K + k of the tokens it routes to e), next to its token rows and router
// weights.  The rank that holds expert e then runs
//
//   moe_gather_gemm   dispatch fused with the first GEMM: copy CTAs walk the ranks' lists,
//                     pull the routed token rows over NVLink into a local [capacity, d]
//                     buffer (16 rows per readiness flag) and record, per gathered row, its
//                     home rank, slot and router weight; the tcgen05 GEMM CTAs of the same
//                     launch consume row blocks as they land.  The number of rows is only
//                     known on the device: the GEMM reads the ranks' counts itself.
//   gemm (scatter)    combine fused with the second GEMM: the epilogue stores each output
//                     row straight into slot (token, k) of its home rank's combine buffer.
//   moe_combine       y[t] = sum_k slot[t][k] (+ residual) on the home rank.
//
// The backward pass reuses the same two fused kernels with the roles of activations and
// gradients swapped.  No TMA touches peer memory; nothing is multicast; waits are bounded.
#include <cuda.h>
#include <cuda_runtime.h>

#include "comm.cuh"
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

constexpr int kMoeRowsPerFlag = 16;

// ------------------------------------------------------------------------------ routing
// counts[e] (zeroed by the caller) and lists[e*T + pos] = t*topk + k.
__global__ void moe_route_kernel(const int* __restrict__ top_idx, int T, int topk, int E,
                                 int* counts, int* lists) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * topk) return;
  const int e = top_idx[i];
  if (e < 0 || e >= E) return;
  const int pos = atomicAdd(&counts[e], 1);
  lists[(size_t)e * T + pos] = i;
}

struct MoeGather {
  Peers counts;   // int[E] per rank
  Peers lists;    // int[E*T] per rank
  Peers rows;     // bf16 [T, d] per rank (token rows to pull)
  Peers wts;      // float [T*topk] per rank (router weights), may be null
  int world, expert, T, topk, d, cap;
  __nv_bfloat16* dst;   // [cap, d]
  int* row_rank;        // [cap]
  int* row_slot;        // [cap]
  float* row_w;         // [cap]
  int* m_count;         // [1] rows gathered (clamped to cap)
  uint32_t* flags;      // one per kMoeRowsPerFlag rows
  uint32_t epoch;
  int* status;
};

__device__ __forceinline__ void moe_gather_rows(const MoeGather& g, int cta, int n_cta) {
  __shared__ int s_off[kMaxRanks + 1];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int s = 0; s < g.world; ++s) {
      s_off[s] = acc;
      acc += *reinterpret_cast<const volatile int*>(
          reinterpret_cast<const int*>(g.counts.p[s]) + g.expert);
    }
    s_off[g.world] = acc;
    if (cta == 0) *g.m_count = acc < g.cap ? acc : g.cap;
  }
  __syncthreads();
  const int total = s_off[g.world] < g.cap ? s_off[g.world] : g.cap;
  const int padded = ((total + 63) / 64) * 64 < g.cap ? ((total + 63) / 64) * 64 : g.cap;
  const int n_groups = (padded + kMoeRowsPerFlag - 1) / kMoeRowsPerFlag;
  const int vec_per_row = g.d >> 3;
  for (int grp = cta; grp < n_groups; grp += n_cta) {
    const int r0 = grp * kMoeRowsPerFlag;
    for (int rr = 0; rr < kMoeRowsPerFlag; ++rr) {
      const int i = r0 + rr;
      if (i >= padded) break;
      uint4* drow = reinterpret_cast<uint4*>(g.dst + (size_t)i * g.d);
      if (i >= total) {  // zero tail up to a multiple of 64 rows: a later reduction over
                         // the row dimension reads whole 64-row blocks
        for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) drow[v] = make_uint4(0, 0, 0, 0);
        if (threadIdx.x == 0) {
          g.row_rank[i] = 0;
          g.row_slot[i] = 0;
          g.row_w[i] = 0.f;
        }
        continue;
      }
      int s = 0;
      while (s + 1 < g.world && i >= s_off[s + 1]) ++s;
      const int slot = reinterpret_cast<const int*>(g.lists.p[s])[(size_t)g.expert * g.T +
                                                                  (i - s_off[s])];
      const int tok = slot / g.topk;
      const uint4* srow = reinterpret_cast<const uint4*>(
          reinterpret_cast<const __nv_bfloat16*>(g.rows.p[s]) + (size_t)tok * g.d);
      for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) drow[v] = ld_nc_v4(srow + v);
      if (threadIdx.x == 0) {
        g.row_rank[i] = s;
        g.row_slot[i] = slot;
        g.row_w[i] = g.wts.p[s] ? reinterpret_cast<const float*>(g.wts.p[s])[slot] : 1.f;
      }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) st_release_gpu(g.flags + grp, g.epoch);
  }
}

template <bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    moe_gather_gemm_kernel(const __grid_constant__ CUtensorMap tmA,
                           const __grid_constant__ CUtensorMap tmB, const GemmParams p,
                           const MoeGather g, int n_comm) {
  extern __shared__ uint8_t smem_raw[];
  if ((int)blockIdx.x < n_comm) {
    moe_gather_rows(g, blockIdx.x, n_comm);
    return;
  }
  gemm_cta_body<false, B_MN>(&tmA, &tmB, p, blockIdx.x - n_comm, gridDim.x - n_comm, smem_raw);
}

template <bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
    moe_gather_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA,
                                const __grid_constant__ CUtensorMap tmB, const GemmParams p,
                                const MoeGather g, int n_comm) {
  extern __shared__ uint8_t smem_raw[];
  if ((int)blockIdx.x < n_comm) {   // n_comm is even: whole clusters gather
    moe_gather_rows(g, blockIdx.x, n_comm);
    return;
  }
  gemm2_cta_body<false, B_MN>(&tmA, &tmB, p, ((int)blockIdx.x - n_comm) >> 1,
                              ((int)gridDim.x - n_comm) >> 1, smem_raw);
}

// ------------------------------------------------------------------- expert SwiGLU
// h[i] = w[i] * silu(gate[i]) * up[i] for rows i < *m; rows up to the next multiple of 64
// (bounded by cap) are zeroed.
__global__ void __launch_bounds__(256)
    moe_swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, const float* __restrict__ w,
                          const int* __restrict__ m_dev, __nv_bfloat16* __restrict__ h, int cap,
                          int F) {
  const int M = min(*m_dev, cap);
  const int padded = min(((M + 63) / 64) * 64, cap);
  const int vec_per_row = F >> 3;
  const long long total = (long long)padded * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / vec_per_row);
    const int c = (int)(i - (long long)r * vec_per_row) << 3;
    uint4 o = make_uint4(0, 0, 0, 0);
    if (r < M) {
      const float wr = w[r];
      const uint4 g4 = *reinterpret_cast<const uint4*>(gu + (size_t)r * 2 * F + c);
      const uint4 u4 = *reinterpret_cast<const uint4*>(gu + (size_t)r * 2 * F + F + c);
      const uint32_t* gp = &g4.x;
      const uint32_t* up = &u4.x;
      uint32_t* op = &o.x;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 gg = unpack_bf16x2(gp[q]), uu = unpack_bf16x2(up[q]);
        const float a = gg.x / (1.f + __expf(-gg.x)) * uu.x * wr;
        const float b = gg.y / (1.f + __expf(-gg.y)) * uu.y * wr;
        op[q] = pack_bf16x2(a, b);
      }
    }
    *reinterpret_cast<uint4*>(h + (size_t)r * F + c) = o;
  }
}

// One block per row: d_gu = w * d_h * d(silu(g) u); dw[i] = sum_f d_h * silu(g) * u, stored
// into the home rank's router-weight gradient slot.
__global__ void __launch_bounds__(256)
    moe_swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dh,
                          const float* __restrict__ w, const int* __restrict__ m_dev,
                          const int* __restrict__ row_rank, const int* __restrict__ row_slot,
                          __nv_bfloat16* __restrict__ dgu, Peers dw_out, int cap, int F) {
  const int M = min(*m_dev, cap);
  const int padded = min(((M + 63) / 64) * 64, cap);
  __shared__ float red[8];
  for (int r = blockIdx.x; r < padded; r += gridDim.x) {
    __nv_bfloat16* orow = dgu + (size_t)r * 2 * F;
    if (r >= M) {
      for (int c = threadIdx.x * 8; c < 2 * F; c += blockDim.x * 8)
        *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
      continue;
    }
    const float wr = w[r];
    float acc = 0.f;
    for (int c = threadIdx.x * 8; c < F; c += blockDim.x * 8) {
      const uint4 g4 = *reinterpret_cast<const uint4*>(gu + (size_t)r * 2 * F + c);
      const uint4 u4 = *reinterpret_cast<const uint4*>(gu + (size_t)r * 2 * F + F + c);
      const uint4 d4 = *reinterpret_cast<const uint4*>(dh + (size_t)r * F + c);
      const uint32_t* gp = &g4.x;
      const uint32_t* up = &u4.x;
      const uint32_t* dp = &d4.x;
      uint4 og, ou;
      uint32_t* ogp = &og.x;
      uint32_t* oup = &ou.x;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 gg = unpack_bf16x2(gp[q]), uu = unpack_bf16x2(up[q]), dd = unpack_bf16x2(dp[q]);
        float rg[2], ru[2];
        const float gv[2] = {gg.x, gg.y}, uv[2] = {uu.x, uu.y}, dv[2] = {dd.x, dd.y};
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const float sg = 1.f / (1.f + __expf(-gv[j]));
          const float silu = gv[j] * sg;
          acc += dv[j] * silu * uv[j];
          const float dhw = dv[j] * wr;
          rg[j] = dhw * uv[j] * (sg * (1.f + gv[j] * (1.f - sg)));
          ru[j] = dhw * silu;
        }
        ogp[q] = pack_bf16x2(rg[0], rg[1]);
        oup[q] = pack_bf16x2(ru[0], ru[1]);
      }
      *reinterpret_cast<uint4*>(orow + c) = og;
      *reinterpret_cast<uint4*>(orow + F + c) = ou;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
      reinterpret_cast<float*>(dw_out.p[row_rank[r]])[row_slot[r]] = t;
    }
    __syncthreads();
  }
}

// y[t] = sum_k comb[t][k] (+ residual[t]); bf16 in/out, fp32 sum.
__global__ void __launch_bounds__(256)
    moe_combine_kernel(const __nv_bfloat16* __restrict__ comb, int T, int topk, int d,
                       const __nv_bfloat16* __restrict__ residual, int ldr,
                       __nv_bfloat16* __restrict__ out, int ldo) {
  const int vec_per_row = d >> 3;
  const long long total = (long long)T * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / vec_per_row);
    const int c = (int)(i - (long long)t * vec_per_row) << 3;
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k = 0; k < topk; ++k)
      acc8(a, *reinterpret_cast<const uint4*>(comb + ((size_t)t * topk + k) * d + c));
    if (residual) acc8(a, *reinterpret_cast<const uint4*>(residual + (size_t)t * ldr + c));
    uint4 o;
    o.x = pack_bf16x2(a[0], a[1]);
    o.y = pack_bf16x2(a[2], a[3]);
    o.z = pack_bf16x2(a[4], a[5]);
    o.w = pack_bf16x2(a[6], a[7]);
    *reinterpret_cast<uint4*>(out + (size_t)t * ldo + c) = o;
  }
}

}  // namespace mb200

using namespace mb200;

extern "C" int mb200_moe_route(const int* top_idx, int T, int topk, int E, int* counts, int* lists,
                               void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(counts, 0, sizeof(int) * E, st);
  if (e != cudaSuccess) return (int)e;
  const int n = T * topk;
  moe_route_kernel<<<(n + 255) / 256, 256, 0, st>>>(top_idx, T, topk, E, counts, lists);
  return (int)cudaGetLastError();
}

// out[cap, N] = gathered[cap, d] @ op(W); gathers the rows routed to `expert` from all ranks.
extern "C" int mb200_moe_gather_gemm(const void* const* counts_ptrs, const void* const* lists_ptrs,
                                     const void* const* rows_ptrs, const void* const* wts_ptrs,
                                     int world, int expert, int T, int topk, int d, int cap,
                                     void* gathered, int* row_rank, int* row_slot, float* row_w,
                                     int* m_count, uint32_t* flags, uint32_t epoch, const void* W,
                                     int ldw, int b_mn, int N, void* out, int ldo, int n_comm,
                                     int* status, void* stream) {
  if (world > kMaxRanks || (d & 7) || cap <= 0) return 1001;
  CUtensorMap ta, tb;
  int r = make_gemm_tmaps(&ta, &tb, gathered, W, cap, N, d, d, ldw, 0, b_mn);
  if (r) return 1000 - r;
  GemmParams p{};
  p.C = reinterpret_cast<__nv_bfloat16*>(out);
  p.M = cap; p.N = N; p.K = d;
  p.ldc = ldo;
  p.status = status;
  p.flag_chunk_elems = 1;
  p.ldb = ldw;
  p.a_ready = flags;
  p.a_ready_target = epoch;
  p.a_flag_chunk_elems = (long long)kMoeRowsPerFlag * d;
  p.a_flag_elem0 = 0;
  p.lda = d;
  for (int i = 0; i < world; ++i)
    p.dyn_m_parts[i] = reinterpret_cast<const int*>(counts_ptrs[i]) + expert;
  p.dyn_m_nparts = world;
  MoeGather g{};
  for (int i = 0; i < world; ++i) {
    g.counts.p[i] = const_cast<void*>(counts_ptrs[i]);
    g.lists.p[i] = const_cast<void*>(lists_ptrs[i]);
    g.rows.p[i] = const_cast<void*>(rows_ptrs[i]);
    g.wts.p[i] = wts_ptrs ? const_cast<void*>(wts_ptrs[i]) : nullptr;
  }
  g.world = world; g.expert = expert; g.T = T; g.topk = topk; g.d = d; g.cap = cap;
  g.dst = reinterpret_cast<__nv_bfloat16*>(gathered);
  g.row_rank = row_rank; g.row_slot = row_slot; g.row_w = row_w; g.m_count = m_count;
  g.flags = flags; g.epoch = epoch; g.status = status;
  const int sms = sm_count();
  if (n_comm <= 0) n_comm = 24;
  if (n_comm > sms / 2) n_comm = sms / 2;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (mb200_gemm_get_impl() == 2) {
    n_comm &= ~1;
    if (n_comm < 2) n_comm = 2;
    CUtensorMap ta2, tb2;
    r = make_gemm2_tmaps(&ta2, &tb2, gathered, W, cap, N, d, d, ldw, 0, b_mn);
    if (r) return 1000 - r;
    const int tiles = ((cap + G2_BM - 1) / G2_BM) * ((N + G2_BN - 1) / G2_BN);
    int pairs = sms / 2 - n_comm / 2;
    if (tiles < pairs) pairs = tiles;
    const int grid = n_comm + 2 * pairs;
    static bool configured2[2] = {false, false};
    if (!configured2[b_mn ? 1 : 0]) {
      cudaError_t e = b_mn ? cudaFuncSetAttribute(moe_gather_gemm_pair_kernel<true>,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  G2_SMEM_BYTES)
                           : cudaFuncSetAttribute(moe_gather_gemm_pair_kernel<false>,
                                                  cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                  G2_SMEM_BYTES);
      if (e != cudaSuccess) return (int)e;
      configured2[b_mn ? 1 : 0] = true;
    }
    if (b_mn)
      moe_gather_gemm_pair_kernel<true><<<grid, GEMM_THREADS, G2_SMEM_BYTES, st>>>(ta2, tb2, p, g,
                                                                                  n_comm);
    else
      moe_gather_gemm_pair_kernel<false><<<grid, GEMM_THREADS, G2_SMEM_BYTES, st>>>(ta2, tb2, p, g,
                                                                                   n_comm);
    return (int)cudaGetLastError();
  }
  const int tiles = ((cap + GEMM_BM - 1) / GEMM_BM) * ((N + GEMM_BN - 1) / GEMM_BN);
  int gemm_ctas = sms - n_comm;
  if (tiles < gemm_ctas) gemm_ctas = tiles;
  static bool configured[2] = {false, false};
  if (!configured[b_mn ? 1 : 0]) {
    cudaError_t e = b_mn ? cudaFuncSetAttribute(moe_gather_gemm_kernel<true>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                GEMM_SMEM_BYTES)
                         : cudaFuncSetAttribute(moe_gather_gemm_kernel<false>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                GEMM_SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured[b_mn ? 1 : 0] = true;
  }
  const int grid = n_comm + gemm_ctas;
  if (b_mn)
    moe_gather_gemm_kernel<true><<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, st>>>(ta, tb, p, g, n_comm);
  else
    moe_gather_gemm_kernel<false><<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, st>>>(ta, tb, p, g, n_comm);
  return (int)cudaGetLastError();
}

// General GEMM with device-side row counts and the optional scatter epilogue.
// dyn_m / dyn_k: device int pointers (or null); sc_*: scatter epilogue (or null).
extern "C" int mb200_gemm_bf16_ex(const void* A, const void* B, void* C, int M, int N, int K,
                                  int lda, int ldb, int ldc, int a_mn, int b_mn, int accumulate,
                                  const int* dyn_m, const int* dyn_k, const int* sc_rank,
                                  const int* sc_slot, const void* const* sc_out, int world,
                                  int sc_ld, int impl, int* status, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (sc_rank && ((N & 31) || (sc_ld & 7) || world > kMaxRanks)) return 1001;
  GemmParams p{};
  p.C = reinterpret_cast<__nv_bfloat16*>(C);
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc;
  p.accumulate = accumulate;
  p.status = status;
  p.flag_chunk_elems = 1;
  p.a_flag_chunk_elems = 1;
  p.ldb = ldb;
  p.lda = lda;
  if (dyn_m) {
    p.dyn_m_parts[0] = dyn_m;
    p.dyn_m_nparts = 1;
  }
  p.dyn_k = dyn_k;
  if (sc_rank) {
    p.sc_rank = sc_rank;
    p.sc_slot = sc_slot;
    for (int i = 0; i < world; ++i) p.sc_out[i] = const_cast<void*>(sc_out[i]);
    p.sc_ld = sc_ld;
  }
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

extern "C" int mb200_moe_swiglu_fwd(const void* gu, const float* w, const int* m_dev, void* h,
                                    int cap, int F, void* stream) {
  if (F & 7) return 1001;
  const int blocks = sm_count() * 8;
  moe_swiglu_fwd_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(gu), w, m_dev, reinterpret_cast<__nv_bfloat16*>(h),
      cap, F);
  return (int)cudaGetLastError();
}

extern "C" int mb200_moe_swiglu_bwd(const void* gu, const void* dh, const float* w,
                                    const int* m_dev, const int* row_rank, const int* row_slot,
                                    void* dgu, const void* const* dw_ptrs, int world, int cap,
                                    int F, void* stream) {
  if ((F & 7) || world > kMaxRanks) return 1001;
  Peers dw{};
  for (int i = 0; i < world; ++i) dw.p[i] = const_cast<void*>(dw_ptrs[i]);
  int blocks = cap < sm_count() * 8 ? cap : sm_count() * 8;
  moe_swiglu_bwd_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(gu), reinterpret_cast<const __nv_bfloat16*>(dh), w,
      m_dev, row_rank, row_slot, reinterpret_cast<__nv_bfloat16*>(dgu), dw, cap, F);
  return (int)cudaGetLastError();
}

extern "C" int mb200_moe_combine(const void* comb, int T, int topk, int d, const void* residual,
                                 int ldr, void* out, int ldo, void* stream) {
  if ((d & 7) || (ldo & 7) || (residual && (ldr & 7))) return 1001;
  const long long total = (long long)T * (d >> 3);
  int blocks = (int)((total + 255) / 256);
  if (blocks > sm_count() * 8) blocks = sm_count() * 8;
  moe_combine_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(comb), T, topk, d,
      reinterpret_cast<const __nv_bfloat16*>(residual), ldr,
      reinterpret_cast<__nv_bfloat16*>(out), ldo);
  return (int)cudaGetLastError();
}

// Causal grouped-query flash attention, backward, for sm_100a (tcgen05 + TMEM + TMA).
//
// Three launches:
//   1. delta[b,h,s] = sum_d dO * O                       (one warp per row and head)
//   2. dK, dV: one CTA per (kv block of 128 rows, kv head, batch); it keeps K and V in
//      shared memory, walks over every query block at or below the diagonal of every
//      query head of the group, and accumulates dV += P^T dO and dK += dS^T Q in TMEM:
//        S^T = K Q^T, dP^T = V dO^T      (tcgen05.mma, operands in shared memory)
//        P^T = exp2(S^T c - lse), dS^T = P^T (dP^T - delta)   (8 warps, one kv row per
//                                         thread, written back as bf16 over S^T / dP^T)
//        dV += P^T dO, dK += dS^T Q      (A operand from TMEM, dO / Q MN-major from smem)
//   3. dQ: one CTA per (query block, query head, batch), walks over the kv blocks up to
//      the diagonal:  S = Q K^T, dP = dO V^T, dS = P (dP - delta), dQ += dS K.
// Splitting dQ off costs two extra MMAs per block pair but needs no atomics, no fp32 dQ
// buffer and no transposed copy of dS in shared memory: every operand is either a TMA tile
// or lives in TMEM.  Accumulators never leave TMEM until the epilogue.
//
// Warp roles (320 threads): 0 TMA producer, 1 MMA issuer, 2-9 compute/epilogue; warps w and
// w+4 share a TMEM lane quadrant and split the 128 columns of a tile in halves.  The bf16
// operand of half h is written at columns [64h, 64h+32) of the fp32 tile it replaces, so
// neither half overwrites columns the other half still has to read.
#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>

#include "mb200.h"
#include "ptx.cuh"

namespace mb200 {

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t ld, uint32_t box_inner, uint32_t box_outer);

constexpr int AB_T = 128;        // tile rows (queries and keys)
constexpr int AB_THREADS = 320;
constexpr float kLog2e = 1.4426950408889634f;

struct AttBwdParams {
  const float* lse;    // [B, Hq, S]
  const float* delta;  // [B, Hq, S]
  __nv_bfloat16* dq;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  int ld_d;            // row stride of dq/dk/dv
  int B, S, Hq, Hkv;
  float scale, scale_log2;
  int* status;
};

// ------------------------------------------------------------------------- delta
__global__ void __launch_bounds__(256)
    attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                      float* __restrict__ delta, int B, int S, int Hq, int hd, int ld_o,
                      int ld_do) {
  const long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = (long long)B * S * Hq;
  if (w >= total) return;
  const long long t = w / Hq;
  const int h = (int)(w - t * Hq);
  const __nv_bfloat16* op = o + t * ld_o + h * hd;
  const __nv_bfloat16* dp = dout + t * ld_do + h * hd;
  float acc = 0.f;
  for (int d = lane * 2; d < hd; d += 64) {
    float2 a = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(op + d));
    float2 g = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(dp + d));
    acc += a.x * g.x + a.y * g.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    const long long b = t / S;
    const long long s = t - b * S;
    delta[(b * Hq + h) * S + s] = acc;
  }
}

// ------------------------------------------------------------------------ dK, dV
template <int HD>
struct DkvSmem {
  static constexpr int kTile = AB_T * HD * 2;
  static constexpr int kStage = 2 * kTile + 1024;  // Q tile, dO tile, lse[128], delta[128]
  static constexpr int kData = 2 * kTile + 2 * kStage;
  static constexpr int kTotal = kData + 1024 + 256;
};

struct DkvBars {
  uint64_t kv_full;
  uint64_t qdo_full[2], qdo_empty[2];
  uint64_t sdp_full, pds_ready, acc_done;
  uint32_t tmem_base;
  volatile int abort_word;
};

__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes,
                                             uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

template <int HD>
__global__ void __launch_bounds__(AB_THREADS, 1)
    attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ,
                        const __grid_constant__ CUtensorMap tmK,
                        const __grid_constant__ CUtensorMap tmV,
                        const __grid_constant__ CUtensorMap tmDO, const AttBwdParams p) {
  using SM = DkvSmem<HD>;
  constexpr int NCH = HD / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + SM::kTile;
  uint8_t* sStage = sV + SM::kTile;  // [2] x {Q, dO, lse, delta}
  DkvBars* bars = reinterpret_cast<DkvBars*>(smem + SM::kData);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_blk = p.S / AB_T;
  const int j = blockIdx.x;  // kv block; low j = most work, scheduled first
  const int kv_head = blockIdx.y;
  const int b = blockIdx.z;
  const int group = p.Hq / p.Hkv;
  const int nq = n_blk - j;          // query blocks at or below the diagonal
  const int nsteps = group * nq;
  const int row_base = b * p.S;

  if (threadIdx.x == 0) {
    mbar_init(&bars->kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->qdo_full[s], 1);
      mbar_init(&bars->qdo_empty[s], 1);
    }
    mbar_init(&bars->sdp_full, 1);
    mbar_init(&bars->pds_ready, 8);
    mbar_init(&bars->acc_done, 1);
    bars->abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  volatile int* abort_word = &bars->abort_word;
  // TMEM columns: S^T/P^T at 0, dP^T/dS^T at 128, dV at 256, dK at 256 + HD
  constexpr uint32_t kColST = 0, kColDP = 128, kColDV = 256, kColDK = 256 + HD;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      tma_prefetch_desc(&tmDO);
      mbar_expect_tx(&bars->kv_full, 2 * SM::kTile);
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        tma_load_2d(sK + c * (AB_T * 128), &tmK, &bars->kv_full, kv_head * HD + c * 64,
                    row_base + j * AB_T);
        tma_load_2d(sV + c * (AB_T * 128), &tmV, &bars->kv_full, kv_head * HD + c * 64,
                    row_base + j * AB_T);
      }
      for (int t = 0; t < nsteps; ++t) {
        const int st = t & 1;
        if (!mbar_wait(&bars->qdo_empty[st], ((uint32_t)(t >> 1) & 1) ^ 1, abort_word, p.status))
          break;
        const int h = kv_head * group + t / nq;
        const int i = j + t % nq;
        uint8_t* sq = sStage + st * SM::kStage;
        uint8_t* sdo = sq + SM::kTile;
        float* sl = reinterpret_cast<float*>(sdo + SM::kTile);
        mbar_expect_tx(&bars->qdo_full[st], 2 * SM::kTile + 1024);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          tma_load_2d(sq + c * (AB_T * 128), &tmQ, &bars->qdo_full[st], h * HD + c * 64,
                      row_base + i * AB_T);
          tma_load_2d(sdo + c * (AB_T * 128), &tmDO, &bars->qdo_full[st], h * HD + c * 64,
                      row_base + i * AB_T);
        }
        const size_t lrow = ((size_t)b * p.Hq + h) * p.S + (size_t)i * AB_T;
        bulk_load_1d(sl, p.lse + lrow, 512, &bars->qdo_full[st]);
        bulk_load_1d(sl + 128, p.delta + lrow, 512, &bars->qdo_full[st]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_ss = umma_idesc_bf16(AB_T, AB_T, 0, 0);
      constexpr uint32_t idesc_ts = umma_idesc_bf16(AB_T, HD, 0, 1);
      bool ok = mbar_wait(&bars->kv_full, 0, abort_word, p.status);
      tc_fence_after();
      const uint32_t sk = smem_u32(sK), sv = smem_u32(sV);
      for (int t = 0; ok && t < nsteps; ++t) {
        const int st = t & 1;
        ok = mbar_wait(&bars->qdo_full[st], (uint32_t)(t >> 1) & 1, abort_word, p.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sq = smem_u32(sStage + st * SM::kStage);
        const uint32_t sdo = sq + SM::kTile;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk / 4) * (AB_T * 128) + (kk % 4) * 32;
          umma_f16(tmem_base + kColST, umma_smem_desc_sw128(sk + off, 16, 1024),
                   umma_smem_desc_sw128(sq + off, 16, 1024), idesc_ss, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk / 4) * (AB_T * 128) + (kk % 4) * 32;
          umma_f16(tmem_base + kColDP, umma_smem_desc_sw128(sv + off, 16, 1024),
                   umma_smem_desc_sw128(sdo + off, 16, 1024), idesc_ss, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bars->sdp_full);
        ok = mbar_wait(&bars->pds_ready, (uint32_t)t & 1, abort_word, p.status);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < AB_T / 16; ++kk) {
          const uint32_t a_col = (kk / 4) * 64 + (kk % 4) * 8;  // bf16 halves at 0 and 64
          umma_f16_ts(tmem_base + kColDV, tmem_base + kColST + a_col,
                      umma_smem_desc_sw128(sdo + kk * 2048, AB_T * 128, 1024), idesc_ts,
                      (t > 0 || kk > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < AB_T / 16; ++kk) {
          const uint32_t a_col = (kk / 4) * 64 + (kk % 4) * 8;
          umma_f16_ts(tmem_base + kColDK, tmem_base + kColDP + a_col,
                      umma_smem_desc_sw128(sq + kk * 2048, AB_T * 128, 1024), idesc_ts,
                      (t > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&bars->qdo_empty[st]);
      }
      if (ok) umma_commit(&bars->acc_done);
    }
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quad * 32 + lane;  // kv row inside the block
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const uint32_t t_st = tmem_base + kColST + lane_off + half * 64;
    const uint32_t t_dp = tmem_base + kColDP + lane_off + half * 64;
    bool ok = true;
    for (int t = 0; t < nsteps; ++t) {
      ok = mbar_wait(&bars->sdp_full, (uint32_t)t & 1, abort_word, p.status);
      if (!ok) break;
      tc_fence_after();
      const int st = t & 1;
      const float* sl = reinterpret_cast<const float*>(sStage + st * SM::kStage + 2 * SM::kTile);
      const bool diag = (t % nq) == 0;  // query block == kv block
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t sv[32], dv[32];
        tmem_ld_32x32b_x32(t_st + c * 32, sv);
        tmem_ld_32x32b_x32(t_dp + c * 32, dv);
        tmem_ld_wait();
        const int q0 = half * 64 + c * 32;
        uint32_t pp[16], ds[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float2 l2 = *reinterpret_cast<const float2*>(sl + q0 + 2 * i);
          const float2 d2 = *reinterpret_cast<const float2*>(sl + 128 + q0 + 2 * i);
          float p0 = ex2_approx(__uint_as_float(sv[2 * i]) * p.scale_log2 - l2.x * kLog2e);
          float p1 = ex2_approx(__uint_as_float(sv[2 * i + 1]) * p.scale_log2 - l2.y * kLog2e);
          if (diag) {
            if (q0 + 2 * i < r) p0 = 0.f;      // query position before the key position
            if (q0 + 2 * i + 1 < r) p1 = 0.f;
          }
          const float s0 = p0 * (__uint_as_float(dv[2 * i]) - d2.x);
          const float s1 = p1 * (__uint_as_float(dv[2 * i + 1]) - d2.y);
          pp[i] = pack_bf16x2(p0, p1);
          ds[i] = pack_bf16x2(s0, s1);
        }
        tmem_st_32x32b_x16(t_st + c * 16, pp);
        tmem_st_32x32b_x16(t_dp + c * 16, ds);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->pds_ready);
    }
    if (ok) ok = mbar_wait(&bars->acc_done, 0, abort_word, p.status);
    if (ok) {
      tc_fence_after();
      const size_t grow = (size_t)(row_base + j * AB_T + r);
      constexpr int kHalfCols = HD / 2;
      __nv_bfloat16* dvrow = p.dv + grow * p.ld_d + kv_head * HD + half * kHalfCols;
      __nv_bfloat16* dkrow = p.dk + grow * p.ld_d + kv_head * HD + half * kHalfCols;
#pragma unroll 1
      for (int c = 0; c < kHalfCols / 32; ++c) {
        uint32_t a[32], bq[32];
        tmem_ld_32x32b_x32(tmem_base + kColDV + lane_off + half * kHalfCols + c * 32, a);
        tmem_ld_32x32b_x32(tmem_base + kColDK + lane_off + half * kHalfCols + c * 32, bq);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 x, y;
          x.x = pack_bf16x2(__uint_as_float(a[q * 8 + 0]), __uint_as_float(a[q * 8 + 1]));
          x.y = pack_bf16x2(__uint_as_float(a[q * 8 + 2]), __uint_as_float(a[q * 8 + 3]));
          x.z = pack_bf16x2(__uint_as_float(a[q * 8 + 4]), __uint_as_float(a[q * 8 + 5]));
          x.w = pack_bf16x2(__uint_as_float(a[q * 8 + 6]), __uint_as_float(a[q * 8 + 7]));
          y.x = pack_bf16x2(__uint_as_float(bq[q * 8 + 0]) * p.scale,
                            __uint_as_float(bq[q * 8 + 1]) * p.scale);
          y.y = pack_bf16x2(__uint_as_float(bq[q * 8 + 2]) * p.scale,
                            __uint_as_float(bq[q * 8 + 3]) * p.scale);
          y.z = pack_bf16x2(__uint_as_float(bq[q * 8 + 4]) * p.scale,
                            __uint_as_float(bq[q * 8 + 5]) * p.scale);
          y.w = pack_bf16x2(__uint_as_float(bq[q * 8 + 6]) * p.scale,
                            __uint_as_float(bq[q * 8 + 7]) * p.scale);
          *reinterpret_cast<uint4*>(dvrow + c * 32 + q * 8) = x;
          *reinterpret_cast<uint4*>(dkrow + c * 32 + q * 8) = y;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ----------------------------------------------------------------------------- dQ
template <int HD>
struct DqSmem {
  static constexpr int kTile = AB_T * HD * 2;
  static constexpr int kData = 2 * kTile + 2 * 2 * kTile;  // Q, dO, 2 stages of {K, V}
  static constexpr int kTotal = kData + 1024 + 256;
};

struct DqBars {
  uint64_t qdo_full;
  uint64_t kv_full[2], kv_empty[2];
  uint64_t sdp_full, ds_ready, acc_done;
  uint32_t tmem_base;
  volatile int abort_word;
};

template <int HD>
__global__ void __launch_bounds__(AB_THREADS, 1)
    attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ,
                       const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV,
                       const __grid_constant__ CUtensorMap tmDO, const AttBwdParams p) {
  using SM = DqSmem<HD>;
  constexpr int NCH = HD / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + SM::kTile;
  uint8_t* sKV = sDO + SM::kTile;  // [2] x {K, V}
  DqBars* bars = reinterpret_cast<DqBars*>(smem + SM::kData);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_blk = p.S / AB_T;
  const int i = n_blk - 1 - (int)blockIdx.x;  // query block; heavy blocks first
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int kv_head = h / (p.Hq / p.Hkv);
  const int row_base = b * p.S;
  const int nsteps = i + 1;

  if (threadIdx.x == 0) {
    mbar_init(&bars->qdo_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      mbar_init(&bars->kv_empty[s], 1);
    }
    mbar_init(&bars->sdp_full, 1);
    mbar_init(&bars->ds_ready, 8);
    mbar_init(&bars->acc_done, 1);
    bars->abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  volatile int* abort_word = &bars->abort_word;
  constexpr uint32_t kColS = 0, kColDP = 128, kColDQ = 256;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      tma_prefetch_desc(&tmDO);
      mbar_expect_tx(&bars->qdo_full, 2 * SM::kTile);
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        tma_load_2d(sQ + c * (AB_T * 128), &tmQ, &bars->qdo_full, h * HD + c * 64,
                    row_base + i * AB_T);
        tma_load_2d(sDO + c * (AB_T * 128), &tmDO, &bars->qdo_full, h * HD + c * 64,
                    row_base + i * AB_T);
      }
      for (int t = 0; t < nsteps; ++t) {
        const int st = t & 1;
        if (!mbar_wait(&bars->kv_empty[st], ((uint32_t)(t >> 1) & 1) ^ 1, abort_word, p.status))
          break;
        uint8_t* sk = sKV + st * 2 * SM::kTile;
        uint8_t* sv = sk + SM::kTile;
        mbar_expect_tx(&bars->kv_full[st], 2 * SM::kTile);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          tma_load_2d(sk + c * (AB_T * 128), &tmK, &bars->kv_full[st], kv_head * HD + c * 64,
                      row_base + t * AB_T);
          tma_load_2d(sv + c * (AB_T * 128), &tmV, &bars->kv_full[st], kv_head * HD + c * 64,
                      row_base + t * AB_T);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_ss = umma_idesc_bf16(AB_T, AB_T, 0, 0);
      constexpr uint32_t idesc_ts = umma_idesc_bf16(AB_T, HD, 0, 1);
      bool ok = mbar_wait(&bars->qdo_full, 0, abort_word, p.status);
      tc_fence_after();
      const uint32_t sq = smem_u32(sQ), sdo = smem_u32(sDO);
      for (int t = 0; ok && t < nsteps; ++t) {
        const int st = t & 1;
        ok = mbar_wait(&bars->kv_full[st], (uint32_t)(t >> 1) & 1, abort_word, p.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sk = smem_u32(sKV + st * 2 * SM::kTile);
        const uint32_t sv = sk + SM::kTile;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk / 4) * (AB_T * 128) + (kk % 4) * 32;
          umma_f16(tmem_base + kColS, umma_smem_desc_sw128(sq + off, 16, 1024),
                   umma_smem_desc_sw128(sk + off, 16, 1024), idesc_ss, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk / 4) * (AB_T * 128) + (kk % 4) * 32;
          umma_f16(tmem_base + kColDP, umma_smem_desc_sw128(sdo + off, 16, 1024),
                   umma_smem_desc_sw128(sv + off, 16, 1024), idesc_ss, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bars->sdp_full);
        ok = mbar_wait(&bars->ds_ready, (uint32_t)t & 1, abort_word, p.status);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < AB_T / 16; ++kk) {
          const uint32_t a_col = (kk / 4) * 64 + (kk % 4) * 8;
          umma_f16_ts(tmem_base + kColDQ, tmem_base + kColDP + a_col,
                      umma_smem_desc_sw128(sk + kk * 2048, AB_T * 128, 1024), idesc_ts,
                      (t > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&bars->kv_empty[st]);
      }
      if (ok) umma_commit(&bars->acc_done);
    }
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quad * 32 + lane;  // query row inside the block
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const uint32_t t_s = tmem_base + kColS + lane_off + half * 64;
    const uint32_t t_dp = tmem_base + kColDP + lane_off + half * 64;
    const size_t lrow = ((size_t)b * p.Hq + h) * p.S + (size_t)i * AB_T + r;
    const float lse2 = p.lse[lrow] * kLog2e;
    const float dl = p.delta[lrow];
    bool ok = true;
    for (int t = 0; t < nsteps; ++t) {
      ok = mbar_wait(&bars->sdp_full, (uint32_t)t & 1, abort_word, p.status);
      if (!ok) break;
      tc_fence_after();
      const bool diag = (t == i);
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t sv[32], dv[32];
        tmem_ld_32x32b_x32(t_s + c * 32, sv);
        tmem_ld_32x32b_x32(t_dp + c * 32, dv);
        tmem_ld_wait();
        const int k0 = half * 64 + c * 32;
        uint32_t ds[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          float p0 = ex2_approx(__uint_as_float(sv[2 * e]) * p.scale_log2 - lse2);
          float p1 = ex2_approx(__uint_as_float(sv[2 * e + 1]) * p.scale_log2 - lse2);
          if (diag) {
            if (k0 + 2 * e > r) p0 = 0.f;
            if (k0 + 2 * e + 1 > r) p1 = 0.f;
          }
          ds[e] = pack_bf16x2(p0 * (__uint_as_float(dv[2 * e]) - dl),
                              p1 * (__uint_as_float(dv[2 * e + 1]) - dl));
        }
        tmem_st_32x32b_x16(t_dp + c * 16, ds);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->ds_ready);
    }
    if (ok) ok = mbar_wait(&bars->acc_done, 0, abort_word, p.status);
    if (ok) {
      tc_fence_after();
      constexpr int kHalfCols = HD / 2;
      const size_t grow = (size_t)(row_base + i * AB_T + r);
      __nv_bfloat16* dqrow = p.dq + grow * p.ld_d + h * HD + half * kHalfCols;
#pragma unroll 1
      for (int c = 0; c < kHalfCols / 32; ++c) {
        uint32_t a[32];
        tmem_ld_32x32b_x32(tmem_base + kColDQ + lane_off + half * kHalfCols + c * 32, a);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 x;
          x.x = pack_bf16x2(__uint_as_float(a[q * 8 + 0]) * p.scale,
                            __uint_as_float(a[q * 8 + 1]) * p.scale);
          x.y = pack_bf16x2(__uint_as_float(a[q * 8 + 2]) * p.scale,
                            __uint_as_float(a[q * 8 + 3]) * p.scale);
          x.z = pack_bf16x2(__uint_as_float(a[q * 8 + 4]) * p.scale,
                            __uint_as_float(a[q * 8 + 5]) * p.scale);
          x.w = pack_bf16x2(__uint_as_float(a[q * 8 + 6]) * p.scale,
                            __uint_as_float(a[q * 8 + 7]) * p.scale);
          *reinterpret_cast<uint4*>(dqrow + c * 32 + q * 8) = x;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int HD>
static int launch_attn_bwd(const void* q, const void* k, const void* v, const void* dout,
                           int ld_qkv, int ld_do, const AttBwdParams& p, cudaStream_t st) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_dkv_kernel<HD>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         DkvSmem<HD>::kTotal);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_bwd_dq_kernel<HD>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, DqSmem<HD>::kTotal);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const uint64_t T = (uint64_t)p.B * p.S;
  CUtensorMap tq, tk, tv, tdo;
  int r = make_tmap_bf16_2d(&tq, q, (uint64_t)p.Hq * HD, T, ld_qkv, 64, AB_T);
  if (!r) r = make_tmap_bf16_2d(&tk, k, (uint64_t)p.Hkv * HD, T, ld_qkv, 64, AB_T);
  if (!r) r = make_tmap_bf16_2d(&tv, v, (uint64_t)p.Hkv * HD, T, ld_qkv, 64, AB_T);
  if (!r) r = make_tmap_bf16_2d(&tdo, dout, (uint64_t)p.Hq * HD, T, ld_do, 64, AB_T);
  if (r) return 1000 - r;
  const int n_blk = p.S / AB_T;
  attn_bwd_dkv_kernel<HD><<<dim3(n_blk, p.Hkv, p.B), AB_THREADS, DkvSmem<HD>::kTotal, st>>>(
      tq, tk, tv, tdo, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  attn_bwd_dq_kernel<HD><<<dim3(n_blk, p.Hq, p.B), AB_THREADS, DqSmem<HD>::kTotal, st>>>(
      tq, tk, tv, tdo, p);
  return (int)cudaGetLastError();
}

}  // namespace mb200

using namespace mb200;

// dout must have the layout of o ([B*S, Hq*hd], row stride ld_o).
extern "C" int mb200_attn_bwd(const void* q, const void* k, const void* v, const void* o,
                              const void* dout, const float* lse, float* delta, void* dq, void* dk,
                              void* dv, int B, int S, int Hq, int Hkv, int hd, int ld_qkv,
                              int ld_o, int ld_dqkv, float scale, int* status, void* stream) {
  if (B <= 0 || S <= 0) return 0;
  if ((S % AB_T) || (hd != 64 && hd != 128) || Hkv <= 0 || (Hq % Hkv) || (ld_dqkv & 7) ||
      (ld_o & 7) || (reinterpret_cast<uintptr_t>(dq) & 15) ||
      (reinterpret_cast<uintptr_t>(dk) & 15) || (reinterpret_cast<uintptr_t>(dv) & 15) ||
      (reinterpret_cast<uintptr_t>(lse) & 15) || (reinterpret_cast<uintptr_t>(delta) & 15))
    return 1001;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long rows = (long long)B * S * Hq;
  const int blocks = (int)((rows * 32 + 255) / 256);
  attn_delta_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(o),
                                            reinterpret_cast<const __nv_bfloat16*>(dout), delta, B,
                                            S, Hq, hd, ld_o, ld_o);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  AttBwdParams p{};
  p.lse = lse;
  p.delta = delta;
  p.dq = reinterpret_cast<__nv_bfloat16*>(dq);
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk);
  p.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  p.ld_d = ld_dqkv;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.scale = scale;
  p.scale_log2 = scale * kLog2e;
  p.status = status;
  if (hd == 128) return launch_attn_bwd<128>(q, k, v, dout, ld_qkv, ld_o, p, st);
  return launch_attn_bwd<64>(q, k, v, dout, ld_qkv, ld_o, p, st);
}

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
// Both kernels step through their inner dimension 64 rows at a time with two sets of
// (S, dP) accumulator columns: while the eight compute warps turn set t&1 into bf16
// operands, the tensor pipe already runs S and dP of step t+1 into the other set, and the
// accumulating MMAs of step t follow as soon as its operands are written.
//
// Warp roles (576 threads): 0 TMA producer, 1 MMA issuer, 2-17 compute/epilogue; warps w,
// w+4, w+8, w+12 share a TMEM lane quadrant and split the 64 columns of a set in quarters
// (four warps per scheduler hide the TMEM load latency of each other).  The bf16 operand of
// quarter c is written at columns [16c, 16c+8) of the fp32 columns it replaces, so no warp
// overwrites columns another warp still has to read.
#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>

#include "mb200.h"
#include "ptx.cuh"

namespace mb200 {

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t ld, uint32_t box_inner, uint32_t box_outer);

constexpr int AB_T = 128;        // tile rows (queries and keys)
constexpr int AB_THREADS = 576;   // TMA warp, MMA warp, 16 compute warps
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
constexpr int AB_SUB = 64;       // rows of the streamed operand per step
constexpr int AB_STAGES = 4;

template <int HD>
struct DkvSmem {
  static constexpr int kTile = AB_T * HD * 2;          // K, V (resident)
  static constexpr int kSub = AB_SUB * HD * 2;         // Q or dO sub-tile
  static constexpr int kStage = 2 * kSub + 1024;       // Q, dO, lse[64], delta[64] (+pad)
  static constexpr int kData = 2 * kTile + AB_STAGES * kStage;
  static constexpr int kTotal = kData + 1024 + 256;
};

struct DkvBars {
  uint64_t kv_full;
  uint64_t qdo_full[AB_STAGES], qdo_empty[AB_STAGES];
  uint64_t sdp_full[2], pds_ready[2], acc_done;
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
    attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ,    // box 64 x 64 rows
                        const __grid_constant__ CUtensorMap tmK,    // box 64 x 128 rows
                        const __grid_constant__ CUtensorMap tmV,
                        const __grid_constant__ CUtensorMap tmDO,   // box 64 x 64 rows
                        const AttBwdParams p) {
  using SM = DkvSmem<HD>;
  constexpr int NCH = HD / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + SM::kTile;
  uint8_t* sStage = sV + SM::kTile;
  DkvBars* bars = reinterpret_cast<DkvBars*>(smem + SM::kData);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_blk = p.S / AB_T;
  // linear block id: all (head, batch) pairs of kv block 0 first, then block 1, ...: low j
  // = most work, so the heaviest CTAs of every head start first
  const int heads_x_batch = p.Hkv * p.B;
  const int j = (int)blockIdx.x / heads_x_batch;
  const int hb = (int)blockIdx.x % heads_x_batch;
  const int kv_head = hb % p.Hkv;
  const int b = hb / p.Hkv;
  const int group = p.Hq / p.Hkv;
  const int nq = 2 * (n_blk - j);    // 64-row query sub-blocks at or below the diagonal
  const int nsteps = group * nq;
  const int row_base = b * p.S;

  if (threadIdx.x == 0) {
    mbar_init(&bars->kv_full, 1);
    for (int s = 0; s < AB_STAGES; ++s) {
      mbar_init(&bars->qdo_full[s], 1);
      mbar_init(&bars->qdo_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->sdp_full[s], 1);
      mbar_init(&bars->pds_ready[s], 16);
    }
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
  // TMEM columns: set s: S^T/P^T at s*128, dP^T/dS^T at s*128 + 64; dV at 256, dK at 256 + HD
  constexpr uint32_t kColDV = 256, kColDK = 256 + HD;

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
        const int st = t % AB_STAGES;
        if (!mbar_wait(&bars->qdo_empty[st], ((uint32_t)(t / AB_STAGES) & 1) ^ 1, abort_word,
                       p.status))
          break;
        const int h = kv_head * group + t / nq;
        const int q0 = (2 * j + t % nq) * AB_SUB;   // first query row of this sub-block
        uint8_t* sq = sStage + st * SM::kStage;
        uint8_t* sdo = sq + SM::kSub;
        float* sl = reinterpret_cast<float*>(sdo + SM::kSub);
        mbar_expect_tx(&bars->qdo_full[st], 2 * SM::kSub + 512);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          tma_load_2d(sq + c * (AB_SUB * 128), &tmQ, &bars->qdo_full[st], h * HD + c * 64,
                      row_base + q0);
          tma_load_2d(sdo + c * (AB_SUB * 128), &tmDO, &bars->qdo_full[st], h * HD + c * 64,
                      row_base + q0);
        }
        const size_t lrow = ((size_t)b * p.Hq + h) * p.S + (size_t)q0;
        bulk_load_1d(sl, p.lse + lrow, 256, &bars->qdo_full[st]);
        bulk_load_1d(sl + 64, p.delta + lrow, 256, &bars->qdo_full[st]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_ss = umma_idesc_bf16(AB_T, AB_SUB, 0, 0);
      constexpr uint32_t idesc_ts = umma_idesc_bf16(AB_T, HD, 0, 1);
      bool ok = mbar_wait(&bars->kv_full, 0, abort_word, p.status);
      tc_fence_after();
      const uint32_t sk = smem_u32(sK), sv = smem_u32(sV);
      // S^T and dP^T of step t into accumulator set t&1
      auto issue_sdp = [&](int t) -> bool {
        const int st = t % AB_STAGES;
        if (!mbar_wait(&bars->qdo_full[st], (uint32_t)(t / AB_STAGES) & 1, abort_word, p.status))
          return false;
        tc_fence_after();
        const uint32_t sq = smem_u32(sStage + st * SM::kStage);
        const uint32_t sdo = sq + SM::kSub;
        const uint32_t c_st = tmem_base + (t & 1) * 128, c_dp = c_st + 64;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t offk = (kk / 4) * (AB_T * 128) + (kk % 4) * 32;
          const uint32_t offq = (kk / 4) * (AB_SUB * 128) + (kk % 4) * 32;
          umma_f16(c_st, umma_smem_desc_sw128(sk + offk, 16, 1024),
                   umma_smem_desc_sw128(sq + offq, 16, 1024), idesc_ss, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t offk = (kk / 4) * (AB_T * 128) + (kk % 4) * 32;
          const uint32_t offq = (kk / 4) * (AB_SUB * 128) + (kk % 4) * 32;
          umma_f16(c_dp, umma_smem_desc_sw128(sv + offk, 16, 1024),
                   umma_smem_desc_sw128(sdo + offq, 16, 1024), idesc_ss, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bars->sdp_full[t & 1]);
        return true;
      };
      if (ok && nsteps > 0) ok = issue_sdp(0);
      for (int t = 0; ok && t < nsteps; ++t) {
        if (t + 1 < nsteps) {
          ok = issue_sdp(t + 1);   // runs on the tensor pipe while the warps work on step t
          if (!ok) break;
        }
        ok = mbar_wait(&bars->pds_ready[t & 1], (uint32_t)(t >> 1) & 1, abort_word, p.status);
        if (!ok) break;
        tc_fence_after();
        const int st = t % AB_STAGES;
        const uint32_t sq = smem_u32(sStage + st * SM::kStage);
        const uint32_t sdo = sq + SM::kSub;
        const uint32_t c_st = tmem_base + (t & 1) * 128, c_dp = c_st + 64;
#pragma unroll
        for (int kk = 0; kk < AB_SUB / 16; ++kk) {
          const uint32_t a_col = kk * 16;  // bf16 quarter kk sits at columns [16kk, 16kk+8)
          umma_f16_ts(tmem_base + kColDV, c_st + a_col,
                      umma_smem_desc_sw128(sdo + kk * 2048, AB_SUB * 128, 1024), idesc_ts,
                      (t > 0 || kk > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < AB_SUB / 16; ++kk) {
          const uint32_t a_col = kk * 16;
          umma_f16_ts(tmem_base + kColDK, c_dp + a_col,
                      umma_smem_desc_sw128(sq + kk * 2048, AB_SUB * 128, 1024), idesc_ts,
                      (t > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&bars->qdo_empty[st]);
      }
      if (ok) umma_commit(&bars->acc_done);
    }
  } else {
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;  // quarter of the 64 columns this warp converts
    const int r = quad * 32 + lane;    // kv row inside the block
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    bool ok = true;
    for (int t = 0; t < nsteps; ++t) {
      ok = mbar_wait(&bars->sdp_full[t & 1], (uint32_t)(t >> 1) & 1, abort_word, p.status);
      if (!ok) break;
      tc_fence_after();
      const int st = t % AB_STAGES;
      const float* sl = reinterpret_cast<const float*>(sStage + st * SM::kStage + 2 * SM::kSub);
      const uint32_t t_st = tmem_base + (t & 1) * 128 + lane_off + part * 16;
      const uint32_t t_dp = t_st + 64;
      // query sub-blocks 2j and 2j+1 overlap the diagonal of kv block j
      const int sub = t % nq;
      const int q_rel = sub * AB_SUB + part * 16;  // first query of this warp, rel. to kv row 0
      uint32_t sv[16], dv[16];
      tmem_ld_32x32b_x16(t_st, sv);
      tmem_ld_32x32b_x16(t_dp, dv);
      tmem_ld_wait();
      uint32_t pp[8], ds[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float2 l2 = *reinterpret_cast<const float2*>(sl + part * 16 + 2 * i);
        const float2 d2 = *reinterpret_cast<const float2*>(sl + 64 + part * 16 + 2 * i);
        float p0 = ex2_approx(fmaf(__uint_as_float(sv[2 * i]), p.scale_log2, -l2.x * kLog2e));
        float p1 = ex2_approx(fmaf(__uint_as_float(sv[2 * i + 1]), p.scale_log2, -l2.y * kLog2e));
        if (sub < 2) {
          if (q_rel + 2 * i < r) p0 = 0.f;      // query position before the key position
          if (q_rel + 2 * i + 1 < r) p1 = 0.f;
        }
        const float s0 = p0 * (__uint_as_float(dv[2 * i]) - d2.x);
        const float s1 = p1 * (__uint_as_float(dv[2 * i + 1]) - d2.y);
        pp[i] = pack_bf16x2(p0, p1);
        ds[i] = pack_bf16x2(s0, s1);
      }
      tmem_st_32x32b_x8(t_st, pp);
      tmem_st_32x32b_x8(t_dp, ds);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->pds_ready[t & 1]);
    }
    if (ok) ok = mbar_wait(&bars->acc_done, 0, abort_word, p.status);
    if (ok) {
      tc_fence_after();
      const size_t grow = (size_t)(row_base + j * AB_T + r);
      constexpr int kCols = HD / 4;   // columns of dV and dK this warp writes (32 or 16)
      __nv_bfloat16* dvrow = p.dv + grow * p.ld_d + kv_head * HD + part * kCols;
      __nv_bfloat16* dkrow = p.dk + grow * p.ld_d + kv_head * HD + part * kCols;
      uint32_t a[kCols], bq[kCols];
      if constexpr (kCols == 32) {
        tmem_ld_32x32b_x32(tmem_base + kColDV + lane_off + part * kCols, a);
        tmem_ld_32x32b_x32(tmem_base + kColDK + lane_off + part * kCols, bq);
      } else {
        tmem_ld_32x32b_x16(tmem_base + kColDV + lane_off + part * kCols, a);
        tmem_ld_32x32b_x16(tmem_base + kColDK + lane_off + part * kCols, bq);
      }
      tmem_ld_wait();
#pragma unroll
      for (int q = 0; q < kCols / 8; ++q) {
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
        *reinterpret_cast<uint4*>(dvrow + q * 8) = x;
        *reinterpret_cast<uint4*>(dkrow + q * 8) = y;
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
  static constexpr int kTile = AB_T * HD * 2;      // Q, dO (resident)
  static constexpr int kSub = AB_SUB * HD * 2;     // K or V sub-tile
  static constexpr int kStage = 2 * kSub;
  static constexpr int kData = 2 * kTile + AB_STAGES * kStage;
  static constexpr int kTotal = kData + 1024 + 256;
};

struct DqBars {
  uint64_t qdo_full;
  uint64_t kv_full[AB_STAGES], kv_empty[AB_STAGES];
  uint64_t sdp_full[2], ds_ready[2], acc_done;
  uint32_t tmem_base;
  volatile int abort_word;
};

template <int HD>
__global__ void __launch_bounds__(AB_THREADS, 1)
    attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ,    // box 64 x 128 rows
                       const __grid_constant__ CUtensorMap tmK,    // box 64 x 64 rows
                       const __grid_constant__ CUtensorMap tmV,
                       const __grid_constant__ CUtensorMap tmDO,   // box 64 x 128 rows
                       const AttBwdParams p) {
  using SM = DqSmem<HD>;
  constexpr int NCH = HD / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + SM::kTile;
  uint8_t* sKV = sDO + SM::kTile;  // [stages] x {K sub-tile, V sub-tile}
  DqBars* bars = reinterpret_cast<DqBars*>(smem + SM::kData);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_blk = p.S / AB_T;
  const int i = n_blk - 1 - (int)blockIdx.x;  // query block; heavy blocks first
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int kv_head = h / (p.Hq / p.Hkv);
  const int row_base = b * p.S;
  const int nsteps = 2 * (i + 1);             // 64-row kv sub-blocks up to the diagonal

  if (threadIdx.x == 0) {
    mbar_init(&bars->qdo_full, 1);
    for (int s = 0; s < AB_STAGES; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      mbar_init(&bars->kv_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->sdp_full[s], 1);
      mbar_init(&bars->ds_ready[s], 16);
    }
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
  // TMEM columns: set s: S at s*128, dP/dS at s*128 + 64; dQ at 256
  constexpr uint32_t kColDQ = 256;

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
        const int st = t % AB_STAGES;
        if (!mbar_wait(&bars->kv_empty[st], ((uint32_t)(t / AB_STAGES) & 1) ^ 1, abort_word,
                       p.status))
          break;
        uint8_t* sk = sKV + st * SM::kStage;
        uint8_t* sv = sk + SM::kSub;
        mbar_expect_tx(&bars->kv_full[st], 2 * SM::kSub);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          tma_load_2d(sk + c * (AB_SUB * 128), &tmK, &bars->kv_full[st], kv_head * HD + c * 64,
                      row_base + t * AB_SUB);
          tma_load_2d(sv + c * (AB_SUB * 128), &tmV, &bars->kv_full[st], kv_head * HD + c * 64,
                      row_base + t * AB_SUB);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_ss = umma_idesc_bf16(AB_T, AB_SUB, 0, 0);
      constexpr uint32_t idesc_ts = umma_idesc_bf16(AB_T, HD, 0, 1);
      bool ok = mbar_wait(&bars->qdo_full, 0, abort_word, p.status);
      tc_fence_after();
      const uint32_t sq = smem_u32(sQ), sdo = smem_u32(sDO);
      auto issue_sdp = [&](int t) -> bool {
        const int st = t % AB_STAGES;
        if (!mbar_wait(&bars->kv_full[st], (uint32_t)(t / AB_STAGES) & 1, abort_word, p.status))
          return false;
        tc_fence_after();
        const uint32_t sk = smem_u32(sKV + st * SM::kStage);
        const uint32_t sv = sk + SM::kSub;
        const uint32_t c_s = tmem_base + (t & 1) * 128, c_dp = c_s + 64;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t offq = (kk / 4) * (AB_T * 128) + (kk % 4) * 32;
          const uint32_t offk = (kk / 4) * (AB_SUB * 128) + (kk % 4) * 32;
          umma_f16(c_s, umma_smem_desc_sw128(sq + offq, 16, 1024),
                   umma_smem_desc_sw128(sk + offk, 16, 1024), idesc_ss, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t offq = (kk / 4) * (AB_T * 128) + (kk % 4) * 32;
          const uint32_t offk = (kk / 4) * (AB_SUB * 128) + (kk % 4) * 32;
          umma_f16(c_dp, umma_smem_desc_sw128(sdo + offq, 16, 1024),
                   umma_smem_desc_sw128(sv + offk, 16, 1024), idesc_ss, kk > 0 ? 1u : 0u);
        }
        umma_commit(&bars->sdp_full[t & 1]);
        return true;
      };
      if (ok) ok = issue_sdp(0);
      for (int t = 0; ok && t < nsteps; ++t) {
        if (t + 1 < nsteps) {
          ok = issue_sdp(t + 1);
          if (!ok) break;
        }
        ok = mbar_wait(&bars->ds_ready[t & 1], (uint32_t)(t >> 1) & 1, abort_word, p.status);
        if (!ok) break;
        tc_fence_after();
        const int st = t % AB_STAGES;
        const uint32_t sk = smem_u32(sKV + st * SM::kStage);
        const uint32_t c_dp = tmem_base + (t & 1) * 128 + 64;
#pragma unroll
        for (int kk = 0; kk < AB_SUB / 16; ++kk) {
          const uint32_t a_col = kk * 16;
          umma_f16_ts(tmem_base + kColDQ, c_dp + a_col,
                      umma_smem_desc_sw128(sk + kk * 2048, AB_SUB * 128, 1024), idesc_ts,
                      (t > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&bars->kv_empty[st]);
      }
      if (ok) umma_commit(&bars->acc_done);
    }
  } else {
    const int quad = warp & 3;
    const int part = (warp - 2) >> 2;  // quarter of the 64 columns this warp converts
    const int r = quad * 32 + lane;    // query row inside the block
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    const size_t lrow = ((size_t)b * p.Hq + h) * p.S + (size_t)i * AB_T + r;
    const float neg_lse2 = -p.lse[lrow] * kLog2e;
    const float dl = p.delta[lrow];
    bool ok = true;
    for (int t = 0; t < nsteps; ++t) {
      ok = mbar_wait(&bars->sdp_full[t & 1], (uint32_t)(t >> 1) & 1, abort_word, p.status);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_s = tmem_base + (t & 1) * 128 + lane_off + part * 16;
      const uint32_t t_dp = t_s + 64;
      // kv sub-blocks 2i and 2i+1 overlap the diagonal of query block i
      const bool diag = t >= 2 * i;
      const int k_rel = (t - 2 * i) * AB_SUB + part * 16;  // first key of this warp rel. to q row 0
      uint32_t sv[16], dv[16];
      tmem_ld_32x32b_x16(t_s, sv);
      tmem_ld_32x32b_x16(t_dp, dv);
      tmem_ld_wait();
      uint32_t ds[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float p0 = ex2_approx(fmaf(__uint_as_float(sv[2 * e]), p.scale_log2, neg_lse2));
        float p1 = ex2_approx(fmaf(__uint_as_float(sv[2 * e + 1]), p.scale_log2, neg_lse2));
        if (diag) {
          if (k_rel + 2 * e > r) p0 = 0.f;
          if (k_rel + 2 * e + 1 > r) p1 = 0.f;
        }
        ds[e] = pack_bf16x2(p0 * (__uint_as_float(dv[2 * e]) - dl),
                            p1 * (__uint_as_float(dv[2 * e + 1]) - dl));
      }
      tmem_st_32x32b_x8(t_dp, ds);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->ds_ready[t & 1]);
    }
    if (ok) ok = mbar_wait(&bars->acc_done, 0, abort_word, p.status);
    if (ok) {
      tc_fence_after();
      constexpr int kCols = HD / 4;
      const size_t grow = (size_t)(row_base + i * AB_T + r);
      __nv_bfloat16* dqrow = p.dq + grow * p.ld_d + h * HD + part * kCols;
      uint32_t a[kCols];
      if constexpr (kCols == 32)
        tmem_ld_32x32b_x32(tmem_base + kColDQ + lane_off + part * kCols, a);
      else
        tmem_ld_32x32b_x16(tmem_base + kColDQ + lane_off + part * kCols, a);
      tmem_ld_wait();
#pragma unroll
      for (int q = 0; q < kCols / 8; ++q) {
        uint4 x;
        x.x = pack_bf16x2(__uint_as_float(a[q * 8 + 0]) * p.scale,
                          __uint_as_float(a[q * 8 + 1]) * p.scale);
        x.y = pack_bf16x2(__uint_as_float(a[q * 8 + 2]) * p.scale,
                          __uint_as_float(a[q * 8 + 3]) * p.scale);
        x.z = pack_bf16x2(__uint_as_float(a[q * 8 + 4]) * p.scale,
                          __uint_as_float(a[q * 8 + 5]) * p.scale);
        x.w = pack_bf16x2(__uint_as_float(a[q * 8 + 6]) * p.scale,
                          __uint_as_float(a[q * 8 + 7]) * p.scale);
        *reinterpret_cast<uint4*>(dqrow + q * 8) = x;
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
  // 128-row boxes for the resident tiles, 64-row boxes for the streamed ones
  CUtensorMap tq, tk, tv, tdo, tq64, tk64, tv64, tdo64;
  int r = make_tmap_bf16_2d(&tq, q, (uint64_t)p.Hq * HD, T, ld_qkv, 64, AB_T);
  if (!r) r = make_tmap_bf16_2d(&tk, k, (uint64_t)p.Hkv * HD, T, ld_qkv, 64, AB_T);
  if (!r) r = make_tmap_bf16_2d(&tv, v, (uint64_t)p.Hkv * HD, T, ld_qkv, 64, AB_T);
  if (!r) r = make_tmap_bf16_2d(&tdo, dout, (uint64_t)p.Hq * HD, T, ld_do, 64, AB_T);
  if (!r) r = make_tmap_bf16_2d(&tq64, q, (uint64_t)p.Hq * HD, T, ld_qkv, 64, AB_SUB);
  if (!r) r = make_tmap_bf16_2d(&tk64, k, (uint64_t)p.Hkv * HD, T, ld_qkv, 64, AB_SUB);
  if (!r) r = make_tmap_bf16_2d(&tv64, v, (uint64_t)p.Hkv * HD, T, ld_qkv, 64, AB_SUB);
  if (!r) r = make_tmap_bf16_2d(&tdo64, dout, (uint64_t)p.Hq * HD, T, ld_do, 64, AB_SUB);
  if (r) return 1000 - r;
  const int n_blk = p.S / AB_T;
  attn_bwd_dkv_kernel<HD><<<dim3(n_blk * p.Hkv * p.B), AB_THREADS, DkvSmem<HD>::kTotal, st>>>(
      tq64, tk, tv, tdo64, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  attn_bwd_dq_kernel<HD><<<dim3(n_blk, p.Hq, p.B), AB_THREADS, DqSmem<HD>::kTotal, st>>>(
      tq, tk64, tv64, tdo, p);
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

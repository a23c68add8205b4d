// Causal grouped-query flash attention, forward, for sm_100a (tcgen05 + TMEM + TMA).
//
// One CTA works on two 128-row query tiles that share their K/V stream ("slots"): two query
// heads of one KV group at the same rows (grouped-query models), or two consecutive row
// blocks of one head (multi-head models).  Per KV block of 128 rows and per slot:
//
//   S = Q K^T      tcgen05.mma, both operands in shared memory (TMA, 128-byte swizzle),
//                  fp32 result in TMEM (128 columns)
//   P = exp2(S*c - m)   four softmax warps per slot, one thread per query row, read S from
//                  TMEM, keep the running max / sum in registers and write P back as bf16
//                  into the same TMEM columns
//   O += P V       tcgen05.mma with the A operand read from TMEM and V (MN-major) from
//                  shared memory; O stays in TMEM (hd columns) for the whole KV loop
//
// The MMA warp alternates between the slots (PV of one slot, then QK^T of its next block),
// so the tensor pipe works on one slot while the other slot's warps are in the exponentials.
// The running max is updated lazily: O and the running sum are rescaled only when the new
// row max exceeds the one in use by more than 2^8, which keeps P in range and makes the
// TMEM read-modify-write of O rare.  TMEM: S0 S1 O0 O1 = 4 x 128 columns.
//
// Warp roles (320 threads): 0 TMA producer, 1 MMA issuer, 2-5 softmax slot 0, 6-9 softmax
// slot 1.  Every wait is bounded and unwinds through a common exit that frees TMEM.
#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>

#include "mb200.h"
#include "ptx.cuh"

namespace mb200 {

int make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                      uint64_t ld, uint32_t box_inner, uint32_t box_outer);

constexpr int ATT_BM = 128;  // query rows per slot
constexpr int ATT_BN = 128;  // kv rows per block
constexpr int ATT_THREADS = 320;
constexpr int ATT_KV_STAGES = 2;

template <int HD>
struct AttFwdSmem {
  static constexpr int kQBytes = ATT_BM * HD * 2;
  static constexpr int kKVBytes = ATT_BN * HD * 2;
  static constexpr int kDataBytes = 2 * kQBytes + 2 * ATT_KV_STAGES * kKVBytes;
  static constexpr int kTotal = kDataBytes + 1024 + 256;
};

struct AttBars {
  uint64_t q_full;
  uint64_t k_full[ATT_KV_STAGES], k_empty[ATT_KV_STAGES];
  uint64_t v_full[ATT_KV_STAGES], v_empty[ATT_KV_STAGES];
  uint64_t s_full[2], p_ready[2], o_done[2];
  uint32_t tmem_base;
  volatile int abort_word;
};

struct AttFwdParams {
  __nv_bfloat16* o;
  float* lse;
  int B, S, Hq, Hkv;
  int ld_o;
  float scale_log2;  // softmax scale * log2(e)
  int pair_heads;    // 1: slots are two heads of one KV group; 0: two row blocks of one head
  int* status;
};

template <int HD>
__global__ void __launch_bounds__(ATT_THREADS, 1)
    attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const AttFwdParams p) {
  using SM = AttFwdSmem<HD>;
  constexpr int NCH = HD / 64;  // 64-column (128-byte) slices per row
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;                                  // [2 slots][NCH][128 rows x 128 B]
  uint8_t* sK = sQ + 2 * SM::kQBytes;                  // [stages][NCH][128 x 128 B]
  uint8_t* sV = sK + ATT_KV_STAGES * SM::kKVBytes;     // [stages][NCH][128 x 128 B]
  AttBars* bars = reinterpret_cast<AttBars*>(smem + SM::kDataBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_qblk = p.S / ATT_BM;

  // ---- which two query tiles this CTA owns (heaviest tiles are scheduled first)
  const int b = blockIdx.z;
  int head[2], qblk[2];
  bool valid[2] = {true, true};
  if (p.pair_heads) {
    const int qb = n_qblk - 1 - (int)blockIdx.x;
    head[0] = 2 * blockIdx.y;
    head[1] = 2 * blockIdx.y + 1;
    qblk[0] = qblk[1] = qb;
  } else {
    const int n_pairs = (n_qblk + 1) / 2;
    const int pr = n_pairs - 1 - (int)blockIdx.x;
    head[0] = head[1] = blockIdx.y;
    qblk[0] = 2 * pr;
    qblk[1] = 2 * pr + 1;
    valid[1] = qblk[1] < n_qblk;
  }
  const int kv_head = head[0] / (p.Hq / p.Hkv);
  int last[2];
  last[0] = qblk[0];
  last[1] = valid[1] ? qblk[1] : -1;
  const int jmax = last[1] > last[0] ? last[1] : last[0];
  const int row_base = b * p.S;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < ATT_KV_STAGES; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->s_full[s], 1);
      mbar_init(&bars->p_ready[s], 4);
      mbar_init(&bars->o_done[s], 1);
    }
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
  // TMEM columns: S/P of slot s at s*128, O of slot s at 256 + s*128
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      const int n_valid = valid[1] ? 2 : 1;
      mbar_expect_tx(&bars->q_full, n_valid * SM::kQBytes);
      for (int s = 0; s < n_valid; ++s)
#pragma unroll
        for (int c = 0; c < NCH; ++c)
          tma_load_2d(sQ + s * SM::kQBytes + c * (ATT_BM * 128), &tmQ, &bars->q_full,
                      head[s] * HD + c * 64, row_base + qblk[s] * ATT_BM);
      for (int j = 0; j <= jmax; ++j) {
        const int st = j % ATT_KV_STAGES;
        const uint32_t ph = (uint32_t)(j / ATT_KV_STAGES) & 1;
        if (!mbar_wait(&bars->k_empty[st], ph ^ 1, abort_word, p.status)) break;
        mbar_expect_tx(&bars->k_full[st], SM::kKVBytes);
#pragma unroll
        for (int c = 0; c < NCH; ++c)
          tma_load_2d(sK + st * SM::kKVBytes + c * (ATT_BN * 128), &tmK, &bars->k_full[st],
                      kv_head * HD + c * 64, row_base + j * ATT_BN);
        if (!mbar_wait(&bars->v_empty[st], ph ^ 1, abort_word, p.status)) break;
        mbar_expect_tx(&bars->v_full[st], SM::kKVBytes);
#pragma unroll
        for (int c = 0; c < NCH; ++c)
          tma_load_2d(sV + st * SM::kKVBytes + c * (ATT_BN * 128), &tmV, &bars->v_full[st],
                      kv_head * HD + c * 64, row_base + j * ATT_BN);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(ATT_BM, ATT_BN, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(ATT_BM, HD, 0, 1);
      bool ok = mbar_wait(&bars->q_full, 0, abort_word, p.status);
      tc_fence_after();
      for (int j = 0; ok && j <= jmax + 1; ++j) {
        const int st = j % ATT_KV_STAGES;
        if (j <= jmax) {
          ok = mbar_wait(&bars->k_full[st], (uint32_t)(j / ATT_KV_STAGES) & 1, abort_word,
                         p.status);
          if (!ok) break;
          tc_fence_after();
        }
        bool v_waited = false;
        for (int s = 0; s < 2 && ok; ++s) {
          if (j >= 1 && j - 1 <= last[s]) {
            const int jp = j - 1, stp = jp % ATT_KV_STAGES;
            if (!v_waited) {
              ok = mbar_wait(&bars->v_full[stp], (uint32_t)(jp / ATT_KV_STAGES) & 1, abort_word,
                             p.status);
              v_waited = true;
              if (!ok) break;
            }
            ok = mbar_wait(&bars->p_ready[s], (uint32_t)jp & 1, abort_word, p.status);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sv = smem_u32(sV + stp * SM::kKVBytes);
            const uint32_t p_tmem = tmem_base + s * 128;
            const uint32_t o_tmem = tmem_base + 256 + s * 128;
#pragma unroll
            for (int kk = 0; kk < ATT_BN / 16; ++kk) {
              const uint64_t dv = umma_smem_desc_sw128(sv + kk * 2048, ATT_BN * 128, 1024);
              umma_f16_ts(o_tmem, p_tmem + kk * 8, dv, idesc_pv, (jp > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit(&bars->o_done[s]);
          }
          if (j <= last[s]) {
            const uint32_t sq = smem_u32(sQ + s * SM::kQBytes);
            const uint32_t sk = smem_u32(sK + st * SM::kKVBytes);
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
              const uint32_t off = (kk / 4) * (ATT_BM * 128) + (kk % 4) * 32;
              const uint64_t dq = umma_smem_desc_sw128(sq + off, 16, 1024);
              const uint64_t dk = umma_smem_desc_sw128(sk + off, 16, 1024);
              umma_f16(tmem_base + s * 128, dq, dk, idesc_qk, kk > 0 ? 1u : 0u);
            }
            umma_commit(&bars->s_full[s]);
          }
        }
        if (!ok) break;
        if (j >= 1) umma_commit(&bars->v_empty[(j - 1) % ATT_KV_STAGES]);
        if (j <= jmax) umma_commit(&bars->k_empty[st]);
      }
    }
  } else {
    // ---------------------------------------------------------- softmax + epilogue warps
    const int s = (warp - 2) >> 2;     // slot
    const int quad = warp & 3;         // TMEM lane quadrant this warp may access
    const int r = quad * 32 + lane;    // query row inside the tile
    if (valid[s]) {
      const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
      const uint32_t s_tmem = tmem_base + s * 128 + lane_off;
      const uint32_t o_tmem = tmem_base + 256 + s * 128 + lane_off;
      const int q_row = qblk[s] * ATT_BM + r;  // position inside the sequence
      float m_used = -INFINITY, l = 0.f;
      bool ok = true;
      for (int j = 0; j <= last[s]; ++j) {
        ok = mbar_wait(&bars->s_full[s], (uint32_t)j & 1, abort_word, p.status);
        if (!ok) break;
        tc_fence_after();
        const bool diag = (j == qblk[s]);
        // the whole S row (128 fp32) goes to registers with one wait
        uint32_t v[128];
#pragma unroll
        for (int c = 0; c < 4; ++c)
          tmem_ld_32x32b_x32(s_tmem + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[c * 32]));
        tmem_ld_wait();
        if (diag) {
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (i > r) v[i] = 0xff800000u;  // -inf: key position after the query position
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 128; i += 4) {
          mx4[0] = fmaxf(mx4[0], __uint_as_float(v[i]));
          mx4[1] = fmaxf(mx4[1], __uint_as_float(v[i + 1]));
          mx4[2] = fmaxf(mx4[2], __uint_as_float(v[i + 2]));
          mx4[3] = fmaxf(mx4[3], __uint_as_float(v[i + 3]));
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
        // PV of the previous block must have retired before O may be touched, and before
        // P of this block goes on top of the S columns the tensor pipe was reading
        if (j > 0) {
          ok = mbar_wait(&bars->o_done[s], (uint32_t)(j - 1) & 1, abort_word, p.status);
          if (!ok) break;
          tc_fence_after();
        }
        float alpha = 1.f;
        if (j == 0) {
          m_used = mx;
        } else if (mx > m_used + 8.f) {
          alpha = ex2_approx(m_used - mx);
          m_used = mx;
        }
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
          l *= alpha;
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t ov[32];
            tmem_ld_32x32b_x32(o_tmem + c * 32, ov);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            tmem_st_32x32b_x32(o_tmem + c * 32, ov);
          }
          tmem_st_wait();
        }
        // P = exp2(S*c - m) as packed bf16 pairs, written over the S columns
        float l4[4] = {0.f, 0.f, 0.f, 0.f};
        const float neg_m = -m_used;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float x0 =
                ex2_approx(fmaf(__uint_as_float(v[c * 32 + 2 * i]), p.scale_log2, neg_m));
            const float x1 =
                ex2_approx(fmaf(__uint_as_float(v[c * 32 + 2 * i + 1]), p.scale_log2, neg_m));
            l4[(i & 1) * 2] += x0;
            l4[(i & 1) * 2 + 1] += x1;
            pk[i] = pack_bf16x2(x0, x1);
          }
          tmem_st_32x32b_x16(s_tmem + c * 16, pk);
        }
        l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_ready[s]);
      }
      // ---- epilogue: O / l -> bf16, lse
      if (ok) ok = mbar_wait(&bars->o_done[s], (uint32_t)last[s] & 1, abort_word, p.status);
      if (ok) {
        tc_fence_after();
        const float inv_l = 1.f / l;
        const size_t grow = (size_t)(row_base + q_row);
        __nv_bfloat16* orow = p.o + grow * p.ld_o + head[s] * HD;
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(o_tmem + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 o4;
            o4.x = pack_bf16x2(__uint_as_float(v[q * 8 + 0]) * inv_l,
                               __uint_as_float(v[q * 8 + 1]) * inv_l);
            o4.y = pack_bf16x2(__uint_as_float(v[q * 8 + 2]) * inv_l,
                               __uint_as_float(v[q * 8 + 3]) * inv_l);
            o4.z = pack_bf16x2(__uint_as_float(v[q * 8 + 4]) * inv_l,
                               __uint_as_float(v[q * 8 + 5]) * inv_l);
            o4.w = pack_bf16x2(__uint_as_float(v[q * 8 + 6]) * inv_l,
                               __uint_as_float(v[q * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = o4;
          }
        }
        p.lse[((size_t)b * p.Hq + head[s]) * p.S + q_row] =
            (m_used + log2f(l)) * 0.6931471805599453f;
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
static int launch_attn_fwd(const void* q, const void* k, const void* v, const AttFwdParams& p,
                           int ld_qkv, cudaStream_t st) {
  using SM = AttFwdSmem<HD>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<HD>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, SM::kTotal);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const uint64_t T = (uint64_t)p.B * p.S;
  CUtensorMap tq, tk, tv;
  int r = make_tmap_bf16_2d(&tq, q, (uint64_t)p.Hq * HD, T, ld_qkv, 64, ATT_BM);
  if (!r) r = make_tmap_bf16_2d(&tk, k, (uint64_t)p.Hkv * HD, T, ld_qkv, 64, ATT_BN);
  if (!r) r = make_tmap_bf16_2d(&tv, v, (uint64_t)p.Hkv * HD, T, ld_qkv, 64, ATT_BN);
  if (r) return 1000 - r;
  const int n_qblk = p.S / ATT_BM;
  dim3 grid;
  if (p.pair_heads)
    grid = dim3(n_qblk, p.Hq / 2, p.B);
  else
    grid = dim3((n_qblk + 1) / 2, p.Hq, p.B);
  attn_fwd_kernel<HD><<<grid, ATT_THREADS, SM::kTotal, st>>>(tq, tk, tv, p);
  return (int)cudaGetLastError();
}

}  // namespace mb200

using namespace mb200;

extern "C" int mb200_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                              int B, int S, int Hq, int Hkv, int hd, int ld_qkv, int ld_o,
                              float scale, int* status, void* stream) {
  if (B <= 0 || S <= 0) return 0;
  if ((S % ATT_BM) || (hd != 64 && hd != 128) || Hkv <= 0 || (Hq % Hkv) || (ld_o & 7) ||
      (reinterpret_cast<uintptr_t>(o) & 15))
    return 1001;
  AttFwdParams p{};
  p.o = reinterpret_cast<__nv_bfloat16*>(o);
  p.lse = lse;
  p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv;
  p.ld_o = ld_o;
  p.scale_log2 = scale * 1.4426950408889634f;
  const int group = Hq / Hkv;
  p.pair_heads = (group % 2 == 0) ? 1 : 0;
  p.status = status;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (hd == 128) return launch_attn_fwd<128>(q, k, v, p, ld_qkv, st);
  return launch_attn_fwd<64>(q, k, v, p, ld_qkv, st);
}

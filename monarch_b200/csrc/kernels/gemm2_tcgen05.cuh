// CTA-pair variant of the persistent bf16 GEMM: tcgen05.mma.cta_group::2, 256x256 tiles.
//
// A cluster of two CTAs (neighbouring SMs) computes one 256x256 output tile per step:
//   * CTA r of the pair stages rows [r*128, r*128+128) of the A tile and rows
//     [r*128, r*128+128) of the B tile (32 KB per stage instead of 48 KB for a 128x256
//     single-CTA tile), so the tensor pipe reads 64 B/clk of shared memory per SM where
//     the single-CTA kernel needs 96 B/clk on top of the TMA writes; that shared-memory
//     port pressure is what holds the single-CTA kernel at ~75 % tensor-pipe activity;
//   * the even CTA issues the MMA for the pair; the hardware reads each CTA's operand
//     halves from that CTA's shared memory and writes each CTA's 128 accumulator rows
//     (all 256 columns) to that CTA's TMEM;
//   * both CTAs' TMA loads complete on the even CTA's "full" barrier; the MMA's commit
//     arrives on both CTAs' "empty" and "accumulator full" barriers (commit multicast,
//     not a data multicast: every load here writes the issuing CTA's shared memory only);
//   * epilogue warps of both CTAs drain their own TMEM and arrive (remotely for the odd
//     CTA) on the even CTA's "accumulator empty" barrier.
//
// Same operand-layout support (K-major / MN-major A and B), same optional readiness
// gating and reduce-scatter epilogue as the single-CTA body.  Every wait is bounded.
#pragma once
#include "gemm_tcgen05.cuh"

namespace mb200 {

constexpr int G2_BM = 256;       // per pair
constexpr int G2_BN = 256;       // per pair
constexpr int G2_HALF = 128;     // rows of A and of B staged by one CTA
constexpr int G2_BK = 64;
constexpr int G2_STAGES = 6;
constexpr int G2_A_BYTES = G2_HALF * G2_BK * 2;
constexpr int G2_B_BYTES = G2_HALF * G2_BK * 2;
constexpr int G2_STAGE_BYTES = G2_A_BYTES + G2_B_BYTES;
constexpr int G2_SMEM_BYTES = G2_STAGES * G2_STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;

// Tile t of the persistent schedule -> (m block, n block).  Tiles are walked in groups of
// G2_GROUP_M m-blocks across all n-blocks: the CTA pairs that run at the same time then
// share about G2_GROUP_M A panels and npairs / G2_GROUP_M B panels (instead of every A
// panel and two or three B panels with a plain m-fastest walk), and the next wave reuses
// the same B panels while they are still in L2.  Kernels whose B operand arrives chunk by
// chunk (`ordered`: a gather fused into the GEMM) keep the n-major walk that follows the
// order in which the chunks land, rotated by `rot`.
constexpr int G2_GROUP_M = 8;
__device__ __forceinline__ void tile_coords(int t, int m_blocks, int n_blocks, int rot,
                                            bool ordered, int m_group, int m_rot, int& m_blk,
                                            int& n_blk) {
  if (ordered) {
    m_blk = t % m_blocks;
    n_blk = t / m_blocks + rot;
    if (n_blk >= n_blocks) n_blk -= n_blocks;
    return;
  }
  const int group_m = m_group > 0 ? m_group : G2_GROUP_M;
  const int per_group = group_m * n_blocks;
  const int group = t / per_group;
  const int first_m = group * group_m;
  const int gm = (m_blocks - first_m) < group_m ? (m_blocks - first_m) : group_m;
  const int in_group = t - group * per_group;
  m_blk = first_m + in_group % gm + m_rot;
  if (m_blk >= m_blocks) m_blk -= m_blocks;
  n_blk = in_group / gm;
}

struct Gemm2Shared {
  uint64_t full[G2_STAGES];    // used in the even CTA: loads of both CTAs complete here
  uint64_t empty[G2_STAGES];   // per CTA, signalled by the pair's MMA commit
  uint64_t tmem_full[2];       // per CTA, signalled by the pair's MMA commit
  uint64_t tmem_empty[2];      // used in the even CTA: 4 epilogue warps x 2 CTAs arrive
  uint32_t tmem_base;
  volatile int abort_word;
};

template <bool A_MN, bool B_MN>
__device__ __forceinline__ void gemm2_cta_body(const CUtensorMap* tmA, const CUtensorMap* tmB,
                                               const GemmParams& p, int vpair, int npairs,
                                               uint8_t* smem_raw) {
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  Gemm2Shared* sh = reinterpret_cast<Gemm2Shared*>(smem + G2_STAGES * G2_STAGE_BYTES);

  const uint32_t cta = cluster_ctarank();  // 0: issues the MMAs; 1: partner
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int M = gemm_dyn_m(p);
  const int Kd = gemm_dyn_k(p);
  const int m_blocks = (M + G2_BM - 1) / G2_BM;
  const int n_blocks = (p.N + G2_BN - 1) / G2_BN;
  const int k_iters = (Kd + G2_BK - 1) / G2_BK;
  const int num_tiles = m_blocks * n_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < G2_STAGES; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sh->tmem_full[s], 1);
      mbar_init(&sh->tmem_empty[s], 8);
    }
    sh->abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(&sh->tmem_base, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the partner's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_word = &sh->abort_word;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(tmA);
      tma_prefetch_desc(tmB);
      const uint32_t full0 = mapa_u32(smem_u32(&sh->full[0]), 0);  // even CTA's barriers
      int stage = 0;
      uint32_t phase = 0;
      for (int t = vpair; t < num_tiles; t += npairs) {
        int m_blk, n_blk;
        tile_coords(t, m_blocks, n_blocks, p.n_blk_rot, p.b_ready != nullptr, p.m_group, p.m_rot,
                    m_blk, n_blk);
        const int m0 = m_blk * G2_BM + (int)cta * G2_HALF;
        const int n0 = n_blk * G2_BN + (int)cta * G2_HALF;
        bool ok = true;
        if (p.b_ready && n0 < p.N) {
          int last = n0 + G2_HALF - 1;
          if (last >= p.N) last = p.N - 1;
          ok = gemm_wait_rows(p.b_ready, p.b_ready_target, p.flag_chunk_elems, p.b_flag_elem0,
                              p.ldb, n0, last, p.K, p.status);
        }
        if (ok && p.a_ready && m0 < M) {
          int last = m0 + G2_HALF - 1;
          if (last >= M) last = M - 1;
          ok = gemm_wait_rows(p.a_ready, p.a_ready_target, p.a_flag_chunk_elems, p.a_flag_elem0,
                              p.lda, m0, last, p.K, p.status);
        }
        if (!ok) {
          *abort_word = 1;
          break;
        }
        bool failed = false;
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(&sh->empty[stage], phase ^ 1, abort_word, p.status)) {
            failed = true;
            break;
          }
          uint8_t* sa = smem + stage * G2_STAGE_BYTES;
          uint8_t* sb = sa + G2_A_BYTES;
          if (cta == 0) mbar_expect_tx(&sh->full[stage], 2 * G2_STAGE_BYTES);
          const uint32_t bar = full0 + stage * 8;
          const int k0 = k * G2_BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < G2_HALF / 64; ++j)
              tma_load_2d_pair(sa + j * 8192, tmA, bar, m0 + j * 64, k0);
          } else {
            tma_load_2d_pair(sa, tmA, bar, k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < G2_HALF / 64; ++j)
              tma_load_2d_pair(sb + j * 8192, tmB, bar, n0 + j * 64, k0);
          } else {
            tma_load_2d_pair(sb, tmB, bar, k0, n0);
          }
          if (++stage == G2_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (failed) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------- MMA issuer (even CTA only)
    if (cta == 0 && lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(G2_BM, G2_BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = vpair; t < num_tiles; t += npairs) {
        if (!mbar_wait(&sh->tmem_empty[acc], acc_phase ^ 1, abort_word, p.status)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * G2_BN;
        bool failed = false;
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(&sh->full[stage], phase, abort_word, p.status)) {
            failed = true;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * G2_STAGE_BYTES);
          const uint32_t sb = sa + G2_A_BYTES;
#pragma unroll
          for (int kk = 0; kk < G2_BK / 16; ++kk) {
            const uint64_t da = A_MN ? umma_smem_desc_sw128(sa + kk * 2048, 8192, 1024)
                                     : umma_smem_desc_sw128(sa + kk * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc_sw128(sb + kk * 2048, 8192, 1024)
                                     : umma_smem_desc_sw128(sb + kk * 32, 16, 1024);
            umma_f16_pair(d_tmem, da, db, idesc, (k > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit_pair(&sh->empty[stage], 3);  // both CTAs may refill this stage
          if (++stage == G2_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (failed) break;
        umma_commit_pair(&sh->tmem_full[acc], 3);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quad = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool vec_ok = ((p.ldc & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) &&
                        (!p.R || (((p.ldr & 7) == 0) &&
                                  ((reinterpret_cast<uintptr_t>(p.R) & 15) == 0)));
    const uint32_t empty0 = mapa_u32(smem_u32(&sh->tmem_empty[0]), 0);
    for (int t = vpair; t < num_tiles; t += npairs) {
      int m_blk, n_blk;
      tile_coords(t, m_blocks, n_blocks, p.n_blk_rot, p.b_ready != nullptr, p.m_group, p.m_rot,
                    m_blk, n_blk);
      const int row = m_blk * G2_BM + (int)cta * G2_HALF + quad * 32 + lane;
      const int n0 = n_blk * G2_BN;
      if (!mbar_wait(&sh->tmem_full[acc], acc_phase, abort_word, p.status)) break;
      tc_fence_after();
      const uint32_t t_base = tmem_base + acc * G2_BN + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < G2_BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(t_base + c * 32, v);
        tmem_ld_wait();
        if (k_iters == 0) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        gemm_store_strip(p, v, row, n0 + c * 32, vec_ok, M);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(empty0 + acc * 8);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  // Common exit: every role of both CTAs reaches this point (all waits are bounded).  The
  // cluster barrier keeps each CTA's shared memory and TMEM alive until its partner is done.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

}  // namespace mb200

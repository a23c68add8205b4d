// Persistent warp-specialised bf16 GEMM for sm_100a.
//
//   C[M,N] (bf16) = opA(A) * opB(B) (+ R) (+ C)        fp32 accumulation in TMEM
//
// * operands are staged by TMA (cp.async.bulk.tensor.2d, 128-byte swizzle) through a
//   4-deep mbarrier ring; one elected thread issues tcgen05.mma (128x256x16 per
//   instruction); the fp32 accumulator lives in TMEM and is double-buffered
//   (2 x 256 columns) so the epilogue of tile i overlaps the main loop of tile i+1.
// * either operand may be K-major (row-major [rows,K]) or MN-major (row-major [K,rows]),
//   which covers forward (X W^T), input-gradient (dY W) and weight-gradient (dY^T X)
//   products of a linear layer without any transpose pass.
// * the body is a __device__ function over a *virtual* CTA id so that fused
//   compute+collective kernels can run it on a subset of the grid while other CTAs
//   move peer data; the TMA producer can be gated on global "ready" flags per block
//   of B rows (bounded wait).
#pragma once
#include "ptx.cuh"

namespace mb200 {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BN = 256;
constexpr int GEMM_BK = 64;
constexpr int GEMM_STAGES = 4;
constexpr int GEMM_THREADS = 192;  // warp0: TMA, warp1: MMA, warps 2-5: epilogue
constexpr int GEMM_A_BYTES = GEMM_BM * GEMM_BK * 2;
constexpr int GEMM_B_BYTES = GEMM_BN * GEMM_BK * 2;
constexpr int GEMM_STAGE_BYTES = GEMM_A_BYTES + GEMM_B_BYTES;
constexpr int GEMM_SMEM_BYTES = GEMM_STAGES * GEMM_STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;

struct GemmParams {
  __nv_bfloat16* C;
  const __nv_bfloat16* R;  // optional residual, same shape as C
  int M, N, K;
  int ldc, ldr;
  int accumulate;  // C += result
  int* status;
  // Optional gating of B tiles on readiness flags (fused all-gather -> GEMM).  B (K-major,
  // rows of K elements, leading dimension ldb) lives inside a buffer that is being filled
  // chunk by chunk: elements [f*flag_chunk_elems, (f+1)*flag_chunk_elems) of that buffer
  // are usable once b_ready[f] >= b_ready_target; B[0,0] is element b_flag_elem0 of it.
  const uint32_t* b_ready;
  uint32_t b_ready_target;
  long long flag_chunk_elems;
  long long b_flag_elem0;
  int ldb;
  int n_blk_rot;  // rotate the N-block order so locally-owned blocks come first
  // Same gating for the A operand (K-major rows, leading dimension lda): tensor-parallel
  // sequence-parallel all-gather of activations feeding a column-parallel GEMM.
  const uint32_t* a_ready;
  uint32_t a_ready_target;
  long long a_flag_chunk_elems;
  long long a_flag_elem0;
  int lda;
  // Tile order of the CTA-pair kernel when A arrives rank by rank: groups of m_group
  // m-blocks (0: the default group size), the whole order rotated by m_rot m-blocks so
  // that the rows this rank already holds are multiplied first.
  int m_group;
  int m_rot;
  // Reduce-scatter epilogue (row-parallel GEMM -> sequence-parallel output): when
  // rs_rows_per_rank > 0 the bf16 partial tile is stored over NVLink into the staging
  // buffer of the rank that owns the row, in the slot of the producing rank:
  //   rs_out[row / rs_rows_per_rank][rs_src_rank][row % rs_rows_per_rank, col]
  // (leading dimension rs_ld).  The owner sums the slots in fp32 afterwards.  C/R unused.
  void* rs_out[8];
  int rs_rows_per_rank;
  int rs_ld;
  int rs_src_rank;
  // Row counts known only on the device (mixture-of-experts token counts): when
  // dyn_m_nparts > 0 the number of valid rows is min(M, sum of *dyn_m_parts[i]) (the parts
  // may live on peer GPUs); when dyn_k is set the reduction length is min(K, *dyn_k).  M and
  // K are then capacities; operand rows beyond the dynamic K must be zero.
  const int* dyn_m_parts[8];
  int dyn_m_nparts;
  const int* dyn_k;
  // Scatter epilogue (expert output -> the token's home rank): row i of the result is
  // stored (bf16) at sc_out[sc_rank[i]] + sc_slot[i] * sc_ld + col.  C/R unused.
  const int* sc_rank;
  const int* sc_slot;
  void* sc_out[8];
  int sc_ld;
};

__device__ __forceinline__ int gemm_dyn_m(const GemmParams& p) {
  if (p.dyn_m_nparts <= 0) return p.M;
  int m = 0;
  for (int i = 0; i < p.dyn_m_nparts; ++i)
    m += *reinterpret_cast<const volatile int*>(p.dyn_m_parts[i]);
  return m < p.M ? m : p.M;
}
__device__ __forceinline__ int gemm_dyn_k(const GemmParams& p) {
  if (!p.dyn_k) return p.K;
  const int k = *reinterpret_cast<const volatile int*>(p.dyn_k);
  return k < p.K ? k : p.K;
}

// Shared by both bodies: write one 32-column strip of an accumulator row.
__device__ __forceinline__ void gemm_store_strip(const GemmParams& p, const uint32_t (&v)[32],
                                                 int row, int col, bool vec_ok, int M) {
  if (p.sc_rank) {
    if (row < M && col + 32 <= p.N) {
      __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.sc_out[p.sc_rank[row]]) +
                          (size_t)p.sc_slot[row] * p.sc_ld + col;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 o;
        o.x = pack_bf16x2(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]));
        o.y = pack_bf16x2(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]));
        o.z = pack_bf16x2(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]));
        o.w = pack_bf16x2(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]));
        *reinterpret_cast<uint4*>(op + q * 8) = o;
      }
    }
    return;
  }
  if (p.rs_rows_per_rank > 0) {
    // reduce-scatter epilogue: bf16 partial strip into the owner rank's staging slot
    if (row < M && col + 32 <= p.N) {
      const int owner = row / p.rs_rows_per_rank;
      __nv_bfloat16* op = reinterpret_cast<__nv_bfloat16*>(p.rs_out[owner]) +
                          ((size_t)p.rs_src_rank * p.rs_rows_per_rank +
                           (row - owner * p.rs_rows_per_rank)) * p.rs_ld + col;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 o;
        o.x = pack_bf16x2(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]));
        o.y = pack_bf16x2(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]));
        o.z = pack_bf16x2(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]));
        o.w = pack_bf16x2(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]));
        *reinterpret_cast<uint4*>(op + q * 8) = o;
      }
    }
    return;
  }
  if (row >= M || col >= p.N) return;
  __nv_bfloat16* cp = p.C + (size_t)row * p.ldc + col;
  const __nv_bfloat16* rp = p.R ? p.R + (size_t)row * p.ldr + col : nullptr;
  if (vec_ok && col + 32 <= p.N) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float f[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(v[q * 8 + i]);
      if (rp) {
        uint4 r4 = *reinterpret_cast<const uint4*>(rp + q * 8);
        float2 a = unpack_bf16x2(r4.x), b = unpack_bf16x2(r4.y), c2 = unpack_bf16x2(r4.z),
               d = unpack_bf16x2(r4.w);
        f[0] += a.x; f[1] += a.y; f[2] += b.x; f[3] += b.y;
        f[4] += c2.x; f[5] += c2.y; f[6] += d.x; f[7] += d.y;
      }
      if (p.accumulate) {
        uint4 r4 = *reinterpret_cast<const uint4*>(cp + q * 8);
        float2 a = unpack_bf16x2(r4.x), b = unpack_bf16x2(r4.y), c2 = unpack_bf16x2(r4.z),
               d = unpack_bf16x2(r4.w);
        f[0] += a.x; f[1] += a.y; f[2] += b.x; f[3] += b.y;
        f[4] += c2.x; f[5] += c2.y; f[6] += d.x; f[7] += d.y;
      }
      uint4 o;
      o.x = pack_bf16x2(f[0], f[1]);
      o.y = pack_bf16x2(f[2], f[3]);
      o.z = pack_bf16x2(f[4], f[5]);
      o.w = pack_bf16x2(f[6], f[7]);
      *reinterpret_cast<uint4*>(cp + q * 8) = o;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if (col + i < p.N) {
        float f = __uint_as_float(v[i]);
        if (rp) f += __bfloat162float(rp[i]);
        if (p.accumulate) f += __bfloat162float(cp[i]);
        cp[i] = __float2bfloat16(f);
      }
    }
  }
}

// Bounded wait for the readiness flags that cover rows [r0, r1] (leading dimension ld,
// K elements per row) of an operand living at element `elem0` of a chunk-flagged buffer.
__device__ __forceinline__ bool gemm_wait_rows(const uint32_t* ready, uint32_t target,
                                               long long chunk_elems, long long elem0, int ld,
                                               int r0, int r1, int K, int* status) {
  const long long f0 = (elem0 + (long long)r0 * ld) / chunk_elems;
  const long long f1 = (elem0 + (long long)r1 * ld + K - 1) / chunk_elems;
  bool ok = true;
  for (long long f = f0; f <= f1 && ok; ++f) ok = flag_wait_ge<false>(ready + f, target, status);
  // the chunks were written through the generic proxy by other CTAs; order those writes
  // (observed via the acquire above) before this thread's TMA reads
  asm volatile("fence.proxy.async;" ::: "memory");
  return ok;
}

struct GemmShared {
  uint64_t full[GEMM_STAGES];
  uint64_t empty[GEMM_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  volatile int abort_word;
};

template <bool A_MN, bool B_MN>
__device__ __forceinline__ void gemm_cta_body(const CUtensorMap* tmA, const CUtensorMap* tmB,
                                              const GemmParams& p, int vcta, int nvcta,
                                              uint8_t* smem_raw) {
  // 1024-byte aligned stage buffers (required by the 128-byte swizzle atoms).
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  GemmShared* sh = reinterpret_cast<GemmShared*>(smem + GEMM_STAGES * GEMM_STAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int M = gemm_dyn_m(p);
  const int Kd = gemm_dyn_k(p);
  const int m_blocks = (M + GEMM_BM - 1) / GEMM_BM;
  const int n_blocks = (p.N + GEMM_BN - 1) / GEMM_BN;
  const int k_iters = (Kd + GEMM_BK - 1) / GEMM_BK;
  const int num_tiles = m_blocks * n_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < GEMM_STAGES; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sh->tmem_full[s], 1);
      mbar_init(&sh->tmem_empty[s], 4);
    }
    sh->abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  volatile int* abort_word = &sh->abort_word;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(tmA);
      tma_prefetch_desc(tmB);
      int stage = 0;
      uint32_t phase = 0;
      for (int t = vcta; t < num_tiles; t += nvcta) {
        const int m_blk = t % m_blocks;
        int n_blk = t / m_blocks + p.n_blk_rot;
        if (n_blk >= n_blocks) n_blk -= n_blocks;
        const int m0 = m_blk * GEMM_BM, n0 = n_blk * GEMM_BN;
        bool ok = true;
        if (p.b_ready) {
          // both ends of the block: a 256-row block may straddle several flag ranges
          int last_row = n0 + GEMM_BN - 1;
          if (last_row >= p.N) last_row = p.N - 1;
          ok = gemm_wait_rows(p.b_ready, p.b_ready_target, p.flag_chunk_elems, p.b_flag_elem0,
                              p.ldb, n0, last_row, p.K, p.status);
        }
        if (ok && p.a_ready) {
          int last_row = m0 + GEMM_BM - 1;
          if (last_row >= M) last_row = M - 1;
          ok = gemm_wait_rows(p.a_ready, p.a_ready_target, p.a_flag_chunk_elems, p.a_flag_elem0,
                              p.lda, m0, last_row, p.K, p.status);
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
          uint8_t* sa = smem + stage * GEMM_STAGE_BYTES;
          uint8_t* sb = sa + GEMM_A_BYTES;
          mbar_expect_tx(&sh->full[stage], GEMM_STAGE_BYTES);
          const int k0 = k * GEMM_BK;
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < GEMM_BM / 64; ++j)
              tma_load_2d(sa + j * 8192, tmA, &sh->full[stage], m0 + j * 64, k0);
          } else {
            tma_load_2d(sa, tmA, &sh->full[stage], k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < GEMM_BN / 64; ++j)
              tma_load_2d(sb + j * 8192, tmB, &sh->full[stage], n0 + j * 64, k0);
          } else {
            tma_load_2d(sb, tmB, &sh->full[stage], k0, n0);
          }
          if (++stage == GEMM_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (failed) break;
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(GEMM_BM, GEMM_BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      for (int t = vcta; t < num_tiles; t += nvcta) {
        if (!mbar_wait(&sh->tmem_empty[acc], acc_phase ^ 1, abort_word, p.status)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * GEMM_BN;
        bool failed = false;
        for (int k = 0; k < k_iters; ++k) {
          if (!mbar_wait(&sh->full[stage], phase, abort_word, p.status)) {
            failed = true;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * GEMM_STAGE_BYTES);
          const uint32_t sb = sa + GEMM_A_BYTES;
#pragma unroll
          for (int kk = 0; kk < GEMM_BK / 16; ++kk) {
            const uint64_t da = A_MN ? umma_smem_desc_sw128(sa + kk * 2048, 8192, 1024)
                                     : umma_smem_desc_sw128(sa + kk * 32, 16, 1024);
            const uint64_t db = B_MN ? umma_smem_desc_sw128(sb + kk * 2048, 8192, 1024)
                                     : umma_smem_desc_sw128(sb + kk * 32, 16, 1024);
            umma_f16(d_tmem, da, db, idesc, (k > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&sh->empty[stage]);  // stage reusable once these MMAs retire
          if (++stage == GEMM_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (failed) break;
        umma_commit(&sh->tmem_full[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool vec_ok = ((p.ldc & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) &&
                        (!p.R || (((p.ldr & 7) == 0) &&
                                  ((reinterpret_cast<uintptr_t>(p.R) & 15) == 0)));
    for (int t = vcta; t < num_tiles; t += nvcta) {
      const int m_blk = t % m_blocks;
      int n_blk = t / m_blocks + p.n_blk_rot;
      if (n_blk >= n_blocks) n_blk -= n_blocks;
      const int row = m_blk * GEMM_BM + quad * 32 + lane;
      const int n0 = n_blk * GEMM_BN;
      if (!mbar_wait(&sh->tmem_full[acc], acc_phase, abort_word, p.status)) break;
      tc_fence_after();
      const uint32_t t_base = tmem_base + acc * GEMM_BN + ((uint32_t)(quad * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < GEMM_BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(t_base + c * 32, v);
        tmem_ld_wait();
        if (k_iters == 0) {  // empty reduction (no tokens): the accumulator was never written
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        gemm_store_strip(p, v, row, n0 + c * 32, vec_ok, M);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->tmem_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  // Common exit: every role reaches this point (all waits are bounded).
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace mb200

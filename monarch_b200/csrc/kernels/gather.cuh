// Chunked pull all-gather of a flat bf16 buffer that is sharded across ranks (rank r owns
// elements [r*S, (r+1)*S)): copy CTAs read every rank's shard over NVLink (plain loads or
// non-multicast bulk copies staged through shared memory), write the local full copy chunk
// by chunk and publish one ready flag per chunk.  Shared by the fused all-gather->GEMM
// kernels (FSDP parameter gather, tensor-parallel activation gather).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "comm.cuh"

namespace mb200 {

struct GatherParams {
  __nv_bfloat16* dst;       // local copy of the whole sharded buffer
  Peers src;                // every rank's shard base
  long long shard_elems;
  int rank, world;
  long long c_begin, c_end;  // chunk range to gather
  long long chunk_elems;
  long long total_elems;
  uint32_t* chunk_flags;
  uint32_t chunk_epoch;
  void* my_flags;           // cross-rank epoch flags ("shard updated")
  int wait_slot;
  uint32_t wait_epoch;
  int* status;
  // Visit the chunks of [c_begin, c_end) starting c_rot chunks into the range and wrapping
  // around: every rank then starts with its own rows and reads a different peer at any time.
  long long c_rot;
};

__device__ __forceinline__ void gather_chunks(const GatherParams& g, int cta, int n_cta) {
  __shared__ int sh_ok;
  if (g.wait_epoch) {
    if (!block_wait_all(g.my_flags, g.world, g.wait_slot, g.wait_epoch, g.status, &sh_ok)) return;
  }
  const int nthr = blockDim.x;
  for (long long c = g.c_begin + cta; c < g.c_end; c += n_cta) {
    const long long e0 = c * g.chunk_elems;
    long long e1 = e0 + g.chunk_elems;
    if (e1 > g.total_elems) e1 = g.total_elems;
    // 4 independent 16-byte loads in flight per thread
    for (long long e = e0 + (long long)threadIdx.x * 8; e < e1; e += (long long)nthr * 32) {
      uint4 v[4];
      bool ok[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const long long ej = e + (long long)j * nthr * 8;
        ok[j] = ej < e1;
        if (ok[j]) {
          const int p = (int)(ej / g.shard_elems);
          const long long off = ej - (long long)p * g.shard_elems;
          v[j] = ld_nc_v4(reinterpret_cast<const __nv_bfloat16*>(g.src.p[p]) + off);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (ok[j]) *reinterpret_cast<uint4*>(g.dst + e + (long long)j * nthr * 8) = v[j];
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) st_release_gpu(g.chunk_flags + c, g.chunk_epoch);
  }
}

// Bulk-copy variant used inside the fused kernel: one thread per copy CTA drives a ring of
// 16 KB shared-memory stages with cp.async.bulk (peer/global -> smem -> local global), so
// a handful of CTAs keep more than a megabyte in flight over NVLink.
constexpr int kBulkPiece = 16384;   // bytes per bulk copy
constexpr int kBulkStages = 10;
constexpr int kBulkLag = 3;         // a stage is reused once its store is 3 groups old

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
               "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}

struct BulkPiece {
  long long elem;   // first element (in the gathered buffer)
  uint32_t bytes;
  long long chunk;  // chunk this piece belongs to
  bool last;        // last piece of its chunk
};

// Enumerates the pieces of this CTA's chunks in order.
struct PieceIter {
  const GatherParams& g;
  int cta, n_cta;
  long long k, c, e, e1;   // k: position in the visiting order, c: the chunk visited there
  __device__ PieceIter(const GatherParams& gp, int cta_, int n) : g(gp), cta(cta_), n_cta(n) {
    k = g.c_begin + cta;
    start_chunk();
  }
  __device__ void start_chunk() {
    c = k;
    if (k < g.c_end) {
      if (g.c_rot > 0) {
        c = k + g.c_rot;
        if (c >= g.c_end) c -= (g.c_end - g.c_begin);
      }
      e = c * g.chunk_elems;
      e1 = e + g.chunk_elems;
      if (e1 > g.total_elems) e1 = g.total_elems;
    }
  }
  __device__ bool next(BulkPiece& out) {
    if (k >= g.c_end) return false;
    long long n = kBulkPiece / 2;
    if (e + n > e1) n = e1 - e;
    const long long p = e / g.shard_elems;
    const long long shard_end = (p + 1) * g.shard_elems;
    if (e + n > shard_end) n = shard_end - e;  // never straddle two ranks' shards
    out.elem = e;
    out.bytes = (uint32_t)(n * 2);
    out.chunk = c;
    e += n;
    out.last = (e >= e1);
    if (out.last) {
      k += n_cta;
      start_chunk();
    }
    return true;
  }
};

__device__ __forceinline__ void gather_chunks_bulk(const GatherParams& g, int cta, int n_cta,
                                                   uint8_t* smem_raw) {
  __shared__ int sh_ok;
  if (g.wait_epoch) {
    if (!block_wait_all(g.my_flags, g.world, g.wait_slot, g.wait_epoch, g.status, &sh_ok)) return;
  }
  if (threadIdx.x != 0) return;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) &
                                             ~static_cast<uintptr_t>(127));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kBulkStages * kBulkPiece);
  volatile int* abort_word = reinterpret_cast<volatile int*>(bars + kBulkStages);
  for (int s = 0; s < kBulkStages; ++s) mbar_init(&bars[s], 1);
  *abort_word = 0;
  mbar_fence_init();

  PieceIter load_it(g, cta, n_cta), store_it(g, cta, n_cta);
  long long issued = 0, stored = 0;
  // chunks whose last store has been issued but whose flag is not yet published
  long long pend_chunk[kBulkLag + 2];
  long long pend_at[kBulkLag + 2];
  int n_pend = 0;
  auto issue_load = [&]() -> bool {
    BulkPiece p;
    if (!load_it.next(p)) return false;
    const int s = (int)(issued % kBulkStages);
    const long long r = p.elem / g.shard_elems;
    const long long off = p.elem - r * g.shard_elems;
    mbar_expect_tx(&bars[s], p.bytes);
    bulk_load(smem + s * kBulkPiece,
              reinterpret_cast<const __nv_bfloat16*>(g.src.p[(int)r]) + off, p.bytes, &bars[s]);
    ++issued;
    return true;
  };
  auto publish_upto = [&](long long done_stores) {
    // stores with index < done_stores are complete
    int w = 0;
    for (int i = 0; i < n_pend; ++i) {
      if (pend_at[i] < done_stores) {
        asm volatile("fence.proxy.async;" ::: "memory");
        __threadfence();
        st_release_gpu(g.chunk_flags + pend_chunk[i], g.chunk_epoch);
      } else {
        pend_chunk[w] = pend_chunk[i];
        pend_at[w] = pend_at[i];
        ++w;
      }
    }
    n_pend = w;
  };
  for (int i = 0; i < kBulkStages - kBulkLag; ++i)
    if (!issue_load()) break;
  BulkPiece p;
  while (store_it.next(p)) {
    const int s = (int)(stored % kBulkStages);
    const uint32_t parity = (uint32_t)((stored / kBulkStages) & 1);
    if (!mbar_wait(&bars[s], parity, abort_word, g.status)) break;
    bulk_store(g.dst + p.elem, smem + s * kBulkPiece, p.bytes);
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    if (p.last) {
      pend_chunk[n_pend] = p.chunk;
      pend_at[n_pend] = stored;
      ++n_pend;
    }
    ++stored;
    // all but the newest kBulkLag groups are complete: their stages are free, their
    // chunks can be announced
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(kBulkLag) : "memory");
    publish_upto(stored - kBulkLag);
    issue_load();
  }
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  publish_upto(stored);
}

inline GatherParams make_gather(void* unit_buf, const void* const* shard_ptrs,
                                long long shard_elems, int rank, int world, long long c_begin,
                         long long c_end, long long chunk_elems, uint32_t* chunk_flags,
                                uint32_t chunk_epoch, void* my_flags, int wait_slot,
                                uint32_t wait_epoch, int* status) {
  GatherParams g{};
  g.dst = reinterpret_cast<__nv_bfloat16*>(unit_buf);
  for (int i = 0; i < world && i < kMaxRanks; ++i) g.src.p[i] = const_cast<void*>(shard_ptrs[i]);
  g.shard_elems = shard_elems;
  g.rank = rank;
  g.world = world;
  g.c_begin = c_begin;
  g.c_end = c_end;
  g.chunk_elems = chunk_elems;
  g.total_elems = shard_elems * world;
  g.chunk_flags = chunk_flags;
  g.chunk_epoch = chunk_epoch;
  g.my_flags = my_flags;
  g.wait_slot = wait_slot;
  g.wait_epoch = wait_epoch;
  g.status = status;
  return g;
}

}  // namespace mb200

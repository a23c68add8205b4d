// NVLink / NVSwitch collectives written as plain CUDA kernels over peer-mapped
// ("symmetric") memory: every rank passes the base pointers of all ranks' buffers and the
// kernels issue ordinary ld/st.global on peer addresses.  Each collective is fused with
// the compute that follows it:
//
//   * rs_adamw      reduce-scatter of bf16 gradients (fp32 accumulation) + AdamW on the
//                   rank's fp32 master/moment shard + bf16 cast of the updated shard
//   * allreduce     two-shot in-place all-reduce fused with the 1/N scale and the bf16
//                   cast (fp32 or bf16 in, bf16 out)
//   * allgather     pull of every rank's shard into a local buffer, optionally
//                   publishing per-chunk ready flags that a GEMM's TMA producer waits on
//   * peer_copy     one-sided put/get between two GPUs with a completion flag
//   * barrier       flag barrier
//
// Cross-rank ordering uses monotonically increasing epochs in per-rank flag arrays
// (flags[slot * kMaxRanks + source_rank]); every wait is bounded and reports through the
// status word instead of hanging.  No tensor-map TMA and no multicast loads: peer data
// moves with per-thread 16-byte loads and stores.
#include <cuda_bf16.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <string.h>
#include <stdint.h>

#define MB200_BOUNDS_TU 1
#include "comm.cuh"
#include "mb200.h"

namespace mb200 {

// ------------------------------------------------------------------------ barrier --
__global__ void barrier_kernel(Peers flags, int rank, int world, int slot, uint32_t epoch,
                               int* status) {
  signal_all(flags, world, rank, slot, epoch, threadIdx.x);
  __syncthreads();
  if (threadIdx.x == 0) wait_all(flags.p[rank], world, slot, epoch, status);
}

__global__ void wait_kernel(void* my_flags, int world, int slot, uint32_t epoch, int* status) {
  if (threadIdx.x == 0) wait_all(my_flags, world, slot, epoch, status);
}

// ---------------------------------------------------------------------- all-gather --
// dst[p * shard_elems + i] = src_p[i] for every rank p; 16-byte vectors of bf16.
// If wait_epoch != 0 the kernel first waits until every rank published wait_epoch in
// wait_slot ("my shard is up to date").  If chunk_flags != nullptr, blocks copy whole
// chunks of `chunk_elems` and publish chunk_epoch in chunk_flags[chunk] when done.
__global__ void __launch_bounds__(256)
    allgather_pull_kernel(__nv_bfloat16* __restrict__ dst, Peers src, int64_t shard_elems,
                          int rank, int world, void* my_flags, int wait_slot,
                          uint32_t wait_epoch, uint32_t* chunk_flags, int64_t chunk_elems,
                          uint32_t chunk_epoch, int* status) {
  __shared__ int sh_ok;
  if (wait_epoch) {
    if (!block_wait_all(my_flags, world, wait_slot, wait_epoch, status, &sh_ok)) return;
  }
  if (chunk_flags == nullptr) {
    // Every thread keeps eight independent 16-byte loads in flight: a pull over NVLink is
    // bound by outstanding bytes (about 3 us of latency x 770 GB/s = 2.4 MB), not by issue
    // rate, so a modest grid (128 blocks = 4 MB in flight) saturates the link and leaves the
    // other SMs to the GEMMs that run beside it.
    const int64_t vps = shard_elems >> 3;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int k = 0; k < world; ++k) {
      const int p = (rank + k) % world;  // start with the local shard, stagger peers
      const uint4* s4 = reinterpret_cast<const uint4*>(src.p[p]);
      uint4* d4 = reinterpret_cast<uint4*>(dst + (int64_t)p * shard_elems);
      int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
      for (; i + 7 * stride < vps; i += 8 * stride) {
        uint4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = ld_nc_v4(s4 + i + j * stride);
#pragma unroll
        for (int j = 0; j < 8; ++j) d4[i + j * stride] = v[j];
      }
      for (; i < vps; i += stride) d4[i] = ld_nc_v4(s4 + i);
    }
    return;
  }
  // chunked mode: chunk c covers dst elements [c*chunk_elems, (c+1)*chunk_elems)
  const int64_t total_elems = shard_elems * world;
  const int64_t n_chunks = (total_elems + chunk_elems - 1) / chunk_elems;
  const int64_t my_first = ((int64_t)rank * shard_elems) / chunk_elems;
  for (int64_t cc = blockIdx.x; cc < n_chunks; cc += gridDim.x) {
    const int64_t c = (my_first + cc) % n_chunks;  // local chunks first
    const int64_t e0 = c * chunk_elems;
    int64_t e1 = e0 + chunk_elems;
    if (e1 > total_elems) e1 = total_elems;
    for (int64_t e = e0 + (int64_t)threadIdx.x * 8; e < e1; e += (int64_t)blockDim.x * 8) {
      const int p = (int)(e / shard_elems);
      const int64_t off = e - (int64_t)p * shard_elems;
      const uint4 val = ld_nc_v4(reinterpret_cast<const __nv_bfloat16*>(src.p[p]) + off);
      *reinterpret_cast<uint4*>(dst + e) = val;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) st_release_gpu(chunk_flags + c, chunk_epoch);
  }
}

// -------------------------------------------------------- reduce-scatter + AdamW ----
// grads.p[r] points at rank r's gradient buffer for this unit (bf16, `unit_elems` long,
// unit_elems = world * shard_elems).  This rank owns elements [rank*shard, (rank+1)*shard).
__global__ void __launch_bounds__(256)
    rs_adamw_kernel(Peers grads, const void* mc_grads, Peers flags, float* __restrict__ master,
                    float* __restrict__ m,
                    float* __restrict__ v, __nv_bfloat16* __restrict__ param_shard,
                    int64_t shard_elems, int rank, int world, int grad_slot, int param_slot,
                    uint32_t epoch, float lr, float beta1, float beta2, float eps, float wd,
                    float inv_bc1, float inv_sqrt_bc2, float grad_scale, unsigned int* counter,
                    int* status) {
  __shared__ int sh_ok;
  // My gradients for this unit are complete (stream order): tell everyone, then wait for
  // everyone else's.
  if (blockIdx.x == 0) signal_all(flags, world, rank, grad_slot, epoch, threadIdx.x);
  if (!block_wait_all(flags.p[rank], world, grad_slot, epoch, status, &sh_ok)) {
    // gave up: still take part in the block count, so that the counter is back at zero
    // for the next launch even when only some blocks of this one timed out
    last_block_done(counter);
    return;
  }

  const int64_t base = (int64_t)rank * shard_elems;
  const int64_t nvec = shard_elems >> 3;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const float decay = 1.f - lr * wd;
  // AdamW on vector i (8 elements) of the shard given the summed gradient g
  auto update = [&](int64_t i, const float (&g)[8]) {
    float4 p0 = reinterpret_cast<float4*>(master)[i * 2], p1 = reinterpret_cast<float4*>(master)[i * 2 + 1];
    float4 m0 = reinterpret_cast<float4*>(m)[i * 2], m1 = reinterpret_cast<float4*>(m)[i * 2 + 1];
    float4 v0 = reinterpret_cast<float4*>(v)[i * 2], v1 = reinterpret_cast<float4*>(v)[i * 2 + 1];
    float pv[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
    float mv[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
    float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gg = g[k] * grad_scale;
      pv[k] *= decay;
      mv[k] = beta1 * mv[k] + (1.f - beta1) * gg;
      vv[k] = beta2 * vv[k] + (1.f - beta2) * gg * gg;
      pv[k] -= lr * inv_bc1 * mv[k] / (sqrtf(vv[k]) * inv_sqrt_bc2 + eps);
    }
    reinterpret_cast<float4*>(master)[i * 2] = make_float4(pv[0], pv[1], pv[2], pv[3]);
    reinterpret_cast<float4*>(master)[i * 2 + 1] = make_float4(pv[4], pv[5], pv[6], pv[7]);
    reinterpret_cast<float4*>(m)[i * 2] = make_float4(mv[0], mv[1], mv[2], mv[3]);
    reinterpret_cast<float4*>(m)[i * 2 + 1] = make_float4(mv[4], mv[5], mv[6], mv[7]);
    reinterpret_cast<float4*>(v)[i * 2] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    reinterpret_cast<float4*>(v)[i * 2 + 1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
    uint4 o;
    o.x = pack_bf16x2(pv[0], pv[1]);
    o.y = pack_bf16x2(pv[2], pv[3]);
    o.z = pack_bf16x2(pv[4], pv[5]);
    o.w = pack_bf16x2(pv[6], pv[7]);
    reinterpret_cast<uint4*>(param_shard)[i] = o;
  };
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (mc_grads) {
    // In-switch reduction: one load returns the fp32-accumulated sum of every rank's copy.
    // Four of them in flight per thread keep the link busy with a grid that leaves most SMs
    // to the backward pass running beside this kernel.
    const __nv_bfloat16* mc = reinterpret_cast<const __nv_bfloat16*>(mc_grads) + base;
    for (; i + 3 * stride < nvec; i += 4 * stride) {
      uint4 r[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) r[j] = multimem_ld_sum<__nv_bfloat16>(mc + (i + j * stride) * 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        acc8(g, r[j]);
        update(i + j * stride, g);
      }
    }
    for (; i < nvec; i += stride) {
      float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      acc8(g, multimem_ld_sum<__nv_bfloat16>(mc + i * 8));
      update(i, g);
    }
  } else {
    for (; i < nvec; i += stride) {
      float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      uint4 raw[kMaxRanks];
#pragma unroll
      for (int k = 0; k < kMaxRanks; ++k) {
        if (k < world) {
          const int p = (rank + k) % world;
          raw[k] = ld_nc_v4(reinterpret_cast<const __nv_bfloat16*>(grads.p[p]) + base + i * 8);
        }
      }
#pragma unroll
      for (int k = 0; k < kMaxRanks; ++k)
        if (k < world) acc8(g, raw[k]);
      update(i, g);
    }
  }
  // The updated bf16 shard is what peers gather next step: announce it once every block
  // of this launch has finished.
  if (last_block_done(counter)) signal_all(flags, world, rank, param_slot, epoch, threadIdx.x);
}

// -------------------------------------------- all-reduce + scale + cast (two-shot) ----
// in.p[r] / out.p[r]: rank r's input / output buffers (may alias for bf16 in place).
// Rank r reduces elements [r*n/world, (r+1)*n/world) over all ranks and stores the scaled
// bf16 result into every rank's output.
template <bool kInFp32>
__global__ void __launch_bounds__(256)
    allreduce_kernel(Peers in, Peers out, const void* mc_in, void* mc_out, Peers flags, int64_t n,
                     int rank, int world, float scale, int slot, uint32_t epoch,
                     unsigned int* counter, int* status) {
  __shared__ int sh_ok;
  if (blockIdx.x == 0) signal_all(flags, world, rank, slot, epoch, threadIdx.x);
  if (!block_wait_all(flags.p[rank], world, slot, epoch, status, &sh_ok)) {
    last_block_done(counter);  // keep the block count consistent for the next launch
    return;
  }
  const int64_t nvec = n >> 3;
  const int64_t per = (nvec + world - 1) / world;
  const int64_t v0 = per * rank;
  int64_t v1 = v0 + per;
  if (v1 > nvec) v1 = nvec;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = v0 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (mc_in && mc_out && !kInFp32) {
    // both halves through the switch: four reductions in flight per thread, each result
    // scaled and written to every rank with one multicast store
    const __nv_bfloat16* mi = reinterpret_cast<const __nv_bfloat16*>(mc_in);
    for (; i + 3 * stride < v1; i += 4 * stride) {
      uint4 r[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) r[j] = multimem_ld_sum<__nv_bfloat16>(mi + (i + j * stride) * 8);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        acc8(g, r[j]);
        uint4 o;
        o.x = pack_bf16x2(g[0] * scale, g[1] * scale);
        o.y = pack_bf16x2(g[2] * scale, g[3] * scale);
        o.z = pack_bf16x2(g[4] * scale, g[5] * scale);
        o.w = pack_bf16x2(g[6] * scale, g[7] * scale);
        multimem_st_v4(reinterpret_cast<uint4*>(mc_out) + i + j * stride, o);
      }
    }
  }
  for (; i < v1; i += stride) {
    float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (mc_in) {
      if (kInFp32) {
        const uint4 a = multimem_ld_sum<float>(reinterpret_cast<const float*>(mc_in) + i * 8);
        const uint4 b = multimem_ld_sum<float>(reinterpret_cast<const float*>(mc_in) + i * 8 + 4);
        g[0] = __uint_as_float(a.x); g[1] = __uint_as_float(a.y);
        g[2] = __uint_as_float(a.z); g[3] = __uint_as_float(a.w);
        g[4] = __uint_as_float(b.x); g[5] = __uint_as_float(b.y);
        g[6] = __uint_as_float(b.z); g[7] = __uint_as_float(b.w);
      } else {
        acc8(g, multimem_ld_sum<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(mc_in) +
                                               i * 8));
      }
    } else if (kInFp32) {
#pragma unroll
      for (int k = 0; k < kMaxRanks; ++k) {
        if (k < world) {
          const int p = (rank + k) % world;
          const uint4 a = ld_nc_v4(reinterpret_cast<const float*>(in.p[p]) + i * 8);
          const uint4 b = ld_nc_v4(reinterpret_cast<const float*>(in.p[p]) + i * 8 + 4);
          g[0] += __uint_as_float(a.x); g[1] += __uint_as_float(a.y);
          g[2] += __uint_as_float(a.z); g[3] += __uint_as_float(a.w);
          g[4] += __uint_as_float(b.x); g[5] += __uint_as_float(b.y);
          g[6] += __uint_as_float(b.z); g[7] += __uint_as_float(b.w);
        }
      }
    } else {
      uint4 raw[kMaxRanks];
#pragma unroll
      for (int k = 0; k < kMaxRanks; ++k)
        if (k < world)
          raw[k] = ld_nc_v4(reinterpret_cast<const __nv_bfloat16*>(in.p[(rank + k) % world]) + i * 8);
#pragma unroll
      for (int k = 0; k < kMaxRanks; ++k)
        if (k < world) acc8(g, raw[k]);
    }
    uint4 o;
    o.x = pack_bf16x2(g[0] * scale, g[1] * scale);
    o.y = pack_bf16x2(g[2] * scale, g[3] * scale);
    o.z = pack_bf16x2(g[4] * scale, g[5] * scale);
    o.w = pack_bf16x2(g[6] * scale, g[7] * scale);
    if (mc_out) {
      multimem_st_v4(reinterpret_cast<uint4*>(mc_out) + i, o);  // one store reaches every rank
    } else {
#pragma unroll
      for (int k = 0; k < kMaxRanks; ++k)
        if (k < world)
          st_v4(reinterpret_cast<uint4*>(out.p[(rank + k) % world]) + i, o);
    }
  }
  if (last_block_done(counter)) {
    signal_all(flags, world, rank, slot + 1, epoch, threadIdx.x);
    // every rank's share of the result must have landed here before a consumer on this
    // stream reads it: the last block stays until all ranks have said so (bounded wait)
    block_wait_all(flags.p[rank], world, slot + 1, epoch, status, &sh_ok);
  }
}

// ----------------------------------------------------------------------- peer copy ----
// One-sided transfer: either pointer may be a peer mapping.  After the data is written a
// completion word is published (system scope) at `done_flag` (may live on the peer).
__global__ void __launch_bounds__(256)
    peer_copy_kernel(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src, int64_t nbytes,
                     uint32_t* done_flag, uint32_t done_value, unsigned int* counter) {
  const int64_t nvec = nbytes >> 4;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const bool aligned = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0;
  if (aligned) {
    // four independent 16-byte loads in flight per thread: a pull over NVLink is bound by
    // the number of outstanding loads, not by issue rate
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < nvec; i += 4 * stride) {
      uint4 v0 = ld_nc_v4(reinterpret_cast<const uint4*>(src) + i);
      uint4 v1 = ld_nc_v4(reinterpret_cast<const uint4*>(src) + i + stride);
      uint4 v2 = ld_nc_v4(reinterpret_cast<const uint4*>(src) + i + 2 * stride);
      uint4 v3 = ld_nc_v4(reinterpret_cast<const uint4*>(src) + i + 3 * stride);
      reinterpret_cast<uint4*>(dst)[i] = v0;
      reinterpret_cast<uint4*>(dst)[i + stride] = v1;
      reinterpret_cast<uint4*>(dst)[i + 2 * stride] = v2;
      reinterpret_cast<uint4*>(dst)[i + 3 * stride] = v3;
    }
    for (; i < nvec; i += stride)
      reinterpret_cast<uint4*>(dst)[i] = ld_nc_v4(reinterpret_cast<const uint4*>(src) + i);
    for (int64_t b = (nvec << 4) + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < nbytes;
         b += stride)
      dst[b] = src[b];
  } else {
    for (int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; b < nbytes; b += stride)
      dst[b] = src[b];
  }
  if (done_flag && last_block_done(counter)) {
    if (threadIdx.x == 0) {
      __threadfence_system();
      st_release_sys(done_flag, done_value);
    }
  }
}

// Bounded wait for a completion word (used by the receiver of a put, or by tests that
// withhold the signal to exercise the timeout path).  limit_ms bounds the spin.
__global__ void wait_flag_kernel(const uint32_t* flag, uint32_t value, int limit_ms, int* status) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    // ~2e6 cycles per ms at the upper end of the SM clock range
    flag_wait_ge<true>(flag, value, status, (long long)limit_ms * 2000000LL);
  }
}

static Peers make_peers(const void* const* ptrs, int world) {
  Peers p{};
  for (int i = 0; i < world && i < kMaxRanks; ++i) p.p[i] = const_cast<void*>(ptrs[i]);
  return p;
}

static int comm_grid(int64_t work_items, int per_block, int cap) {
  int64_t b = (work_items + per_block - 1) / per_block;
  if (b < 1) b = 1;
  return (int)(b < cap ? b : cap);
}

}  // namespace mb200

using namespace mb200;
#define ST(s) reinterpret_cast<cudaStream_t>(s)

extern "C" int mb200_comm_max_ranks() { return kMaxRanks; }

extern "C" int mb200_barrier(const void* const* flag_ptrs, int rank, int world, int slot,
                             uint32_t epoch, int* status, void* stream) {
  if (world > kMaxRanks) return 1001;
  barrier_kernel<<<1, 32, 0, ST(stream)>>>(make_peers(flag_ptrs, world), rank, world, slot, epoch,
                                            status);
  return (int)cudaGetLastError();
}

extern "C" int mb200_wait_flags(void* my_flags, int world, int slot, uint32_t epoch, int* status,
                                void* stream) {
  wait_kernel<<<1, 32, 0, ST(stream)>>>(my_flags, world, slot, epoch, status);
  return (int)cudaGetLastError();
}

extern "C" int mb200_allgather_pull(void* dst, const void* const* src_ptrs, int64_t shard_elems,
                                    int rank, int world, void* my_flags, int wait_slot,
                                    uint32_t wait_epoch, uint32_t* chunk_flags,
                                    int64_t chunk_elems, uint32_t chunk_epoch, int n_blocks,
                                    int* status, void* stream) {
  if (world > kMaxRanks || (shard_elems & 7)) return 1001;
  if (chunk_flags && (chunk_elems & 7)) return 1001;
  const int grid = n_blocks > 0 ? n_blocks
                   : chunk_flags ? comm_grid(shard_elems * world / 8, 256 * 8, 296)
                                 : comm_grid(shard_elems / 8, 256 * 8, 128);
  allgather_pull_kernel<<<grid, 256, 0, ST(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(dst), make_peers(src_ptrs, world), shard_elems, rank, world,
      my_flags, wait_slot, wait_epoch, chunk_flags, chunk_elems, chunk_epoch, status);
  return (int)cudaGetLastError();
}

// mc_grads: multicast mapping of the gradient buffers at the same offset as grad_ptrs (the
// reduction then happens in the switch), or null for plain peer loads.
extern "C" int mb200_rs_adamw(const void* const* grad_ptrs, const void* mc_grads,
                              const void* const* flag_ptrs,
                              float* master, float* m, float* v, void* param_shard,
                              int64_t shard_elems, int rank, int world, int grad_slot,
                              int param_slot, uint32_t epoch, float lr, float beta1, float beta2,
                              float eps, float wd, int step, float grad_scale,
                              unsigned int* counter, int n_blocks, int* status, void* stream) {
  if (world > kMaxRanks || (shard_elems & 7)) return 1001;
  const double bc1 = 1.0 - pow((double)beta1, (double)step);
  const double bc2 = 1.0 - pow((double)beta2, (double)step);
  const int grid = n_blocks > 0 ? n_blocks
                                 : comm_grid(shard_elems / 8, 256 * 4, mc_grads ? 296 : 592);
  rs_adamw_kernel<<<grid, 256, 0, ST(stream)>>>(
      make_peers(grad_ptrs, world), mc_grads, make_peers(flag_ptrs, world), master, m, v,
      reinterpret_cast<__nv_bfloat16*>(param_shard), shard_elems, rank, world, grad_slot,
      param_slot, epoch, lr, beta1, beta2, eps, wd, (float)(1.0 / bc1), (float)(1.0 / sqrt(bc2)),
      grad_scale, counter, status);
  return (int)cudaGetLastError();
}

// mc_in / mc_out: multicast mappings of the input / output buffers (null: peer loads/stores).
extern "C" int mb200_allreduce_scale_cast(const void* const* in_ptrs, const void* const* out_ptrs,
                                          const void* mc_in, void* mc_out,
                                          const void* const* flag_ptrs, int64_t n, int in_fp32,
                                          int rank, int world, float scale, int slot,
                                          uint32_t epoch, unsigned int* counter, int n_blocks,
                                          int* status, void* stream) {
  if (world > kMaxRanks || (n & 7)) return 1001;
  const int grid = n_blocks > 0 ? n_blocks : comm_grid(n / 8 / world, 256 * 4, 296);
  Peers in = make_peers(in_ptrs, world), out = make_peers(out_ptrs, world),
        fl = make_peers(flag_ptrs, world);
  if (in_fp32)
    allreduce_kernel<true><<<grid, 256, 0, ST(stream)>>>(in, out, mc_in, mc_out, fl, n, rank,
                                                          world, scale, slot, epoch, counter,
                                                          status);
  else
    allreduce_kernel<false><<<grid, 256, 0, ST(stream)>>>(in, out, mc_in, mc_out, fl, n, rank,
                                                           world, scale, slot, epoch, counter,
                                                           status);
  return (int)cudaGetLastError();
}

extern "C" int mb200_peer_copy(void* dst, const void* src, int64_t nbytes, uint32_t* done_flag,
                               uint32_t done_value, unsigned int* counter, int n_blocks,
                               void* stream) {
  if (nbytes <= 0 && !done_flag) return 0;
  const int grid = n_blocks > 0 ? n_blocks : comm_grid(nbytes / 16 + 1, 256 * 8, 296);
  peer_copy_kernel<<<grid, 256, 0, ST(stream)>>>(reinterpret_cast<uint8_t*>(dst),
                                                 reinterpret_cast<const uint8_t*>(src), nbytes,
                                                 done_flag, done_value, counter);
  return (int)cudaGetLastError();
}

// The same, and wait for it: one call for a one-sided transfer whose caller blocks until the
// bytes have landed (RDMABuffer.read_into / write_from).  Waiting for the stream is waiting
// for the transfer; no completion flag is involved.
extern "C" int mb200_peer_copy_sync(void* dst, const void* src, int64_t nbytes, int n_blocks,
                                    void* stream) {
  if (nbytes <= 0) return 0;
  const int grid = n_blocks > 0 ? n_blocks : comm_grid(nbytes / 16 + 1, 256 * 8, 296);
  peer_copy_kernel<<<grid, 256, 0, ST(stream)>>>(reinterpret_cast<uint8_t*>(dst),
                                                 reinterpret_cast<const uint8_t*>(src), nbytes,
                                                 nullptr, 0, nullptr);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  return (int)cudaStreamSynchronize(ST(stream));
}

// One asynchronous device-to-device copy on the copy engines (either pointer may be a mapping
// of a peer's memory): the SM-free way to move a shard when GEMMs own the SMs.
extern "C" int mb200_memcpy_d2d_async(void* dst, const void* src, int64_t nbytes, void* stream) {
  if (nbytes <= 0) return 0;
  return (int)cudaMemcpyAsync(dst, src, (size_t)nbytes, cudaMemcpyDeviceToDevice, ST(stream));
}

// Asynchronous fill of `count` 32-bit words with `value` (the driver's cuMemsetD32Async): used
// to raise a range of readiness flags behind a copy-engine transfer on the same stream.
extern "C" int mb200_memset_d32_async(void* dst, uint32_t value, int64_t count, void* stream) {
  using Fn = CUresult (*)(CUdeviceptr, unsigned int, size_t, CUstream);
  static Fn fn = nullptr;
  if (!fn) {
    void* fp = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemsetD32Async", &fp, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return 1004;
    fn = reinterpret_cast<Fn>(fp);
  }
  if (count <= 0) return 0;
  const CUresult r = fn(reinterpret_cast<CUdeviceptr>(dst), value, (size_t)count,
                        reinterpret_cast<CUstream>(stream));
  return r == CUDA_SUCCESS ? 0 : 1007;
}

// Let kernels running on device `dev` dereference memory that lives on device `peer` (memory
// opened through CUDA IPC or allocated by this process).  Idempotent.  Returns 0, or 1003 when
// the two devices have no peer path.
extern "C" int mb200_enable_peer_access(int dev, int peer) {
  if (dev == peer) return 0;
  int can = 0;
  cudaError_t e = cudaDeviceCanAccessPeer(&can, dev, peer);
  if (e != cudaSuccess) return (int)e;
  if (!can) return 1003;
  int cur = 0;
  cudaGetDevice(&cur);
  cudaSetDevice(dev);
  e = cudaDeviceEnablePeerAccess(peer, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    e = cudaSuccess;
  }
  cudaSetDevice(cur);
  return (int)e;
}

// ---- CUDA IPC export / import of a device buffer (RDMABuffer between processes) -----------
// Export: the handle names the whole allocation that contains `ptr`; `offset` is ptr's
// distance from its base.  Import: must run with the READER's device current and with lazy
// peer access, so that the mapping is usable by kernels of that device even when the memory
// lives on another GPU (a mapping opened in the owner device's context is not reachable
// through peer access from a different device of the importing process).
extern "C" int mb200_ipc_export(const void* ptr, void* handle_out64, int64_t* offset_out,
                                int64_t* alloc_size_out) {
  using GetRange = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
  static GetRange get_range = nullptr;
  if (!get_range) {
    void* fp = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fp, cudaEnableDefault, &q) !=
            cudaSuccess || q != cudaDriverEntryPointSuccess)
      return 1004;
    get_range = reinterpret_cast<GetRange>(fp);
  }
  // the driver call needs the owning device's context current on this thread (the caller may
  // be a runtime thread that has never touched CUDA)
  cudaPointerAttributes attr;
  cudaError_t e = cudaPointerGetAttributes(&attr, ptr);
  if (e != cudaSuccess) return (int)e;
  if (attr.type != cudaMemoryTypeDevice) return 1006;
  int cur = 0;
  cudaGetDevice(&cur);
  cudaSetDevice(attr.device);
  cudaFree(nullptr);
  CUdeviceptr base = 0;
  size_t size = 0;
  const CUresult cr = get_range(&base, &size, reinterpret_cast<CUdeviceptr>(ptr));
  cudaIpcMemHandle_t h;
  if (cr == CUDA_SUCCESS) e = cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base));
  cudaSetDevice(cur);
  if (cr != CUDA_SUCCESS) return 1005;
  if (e != cudaSuccess) return (int)e;
  static_assert(sizeof(h) == 64, "cudaIpcMemHandle_t is 64 bytes");
  memcpy(handle_out64, &h, 64);
  *offset_out = (int64_t)(reinterpret_cast<CUdeviceptr>(ptr) - base);
  *alloc_size_out = (int64_t)size;
  return 0;
}

extern "C" int mb200_ipc_open(const void* handle64, int reader_device, void** base_out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  int cur = 0;
  cudaGetDevice(&cur);
  cudaSetDevice(reader_device);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  cudaSetDevice(cur);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return (int)e;
  }
  *base_out = p;
  return 0;
}

extern "C" int mb200_ipc_close(void* base) { return (int)cudaIpcCloseMemHandle(base); }

extern "C" int mb200_wait_flag(const uint32_t* flag, uint32_t value, int limit_ms, int* status,
                               void* stream) {
  wait_flag_kernel<<<1, 32, 0, ST(stream)>>>(flag, value, limit_ms, status);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ GPU-driven ping-pong --
// Two GPUs bounce a payload with no host in the loop: the leader stores `n_vec` 16-byte words
// into the follower's buffer over NVLink and raises the follower's flag; the follower waits for
// the flag, stores the payload back and raises the leader's flag.  One launch per rank does
// `iters` round trips.  Every wait is bounded: a peer that never launches costs the waiting
// side its time limit and an error status, not a hang.  (The reference's counterpart drives
// a NIC from the GPU and spins without a limit: monarch_rdma/examples/cuda_ping_pong.)
__global__ void __launch_bounds__(256)
    pingpong_kernel(uint4* __restrict__ my_buf, uint4* __restrict__ peer_buf, uint32_t* my_flag,
                    uint32_t* peer_flag, long long n_vec, int iters, uint32_t base, int leader,
                    int* status, unsigned long long* elapsed_ns) {
  __shared__ int sh_ok;
  unsigned long long t0 = 0;
  if (threadIdx.x == 0) {
    sh_ok = 1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  }
  __syncthreads();
  for (int i = 0; i < iters; ++i) {
    const uint32_t epoch = base + (uint32_t)i + 1;
    if (!leader) {
      // follower: wait for the ball first
      if (threadIdx.x == 0) sh_ok = flag_wait_ge<true>(my_flag, epoch, status) ? 1 : 0;
      __syncthreads();
      if (!sh_ok) return;
    }
    // send what is in my buffer to the peer (the follower sends back what it received)
    for (long long v = threadIdx.x; v < n_vec; v += blockDim.x) peer_buf[v] = my_buf[v];
    // the CTA barrier orders every thread's payload stores before thread 0's release store
    // (system scope, cumulative), so one release publishes the whole payload
    __syncthreads();
    if (threadIdx.x == 0) st_release_sys(peer_flag, epoch);
    if (leader) {
      if (threadIdx.x == 0) sh_ok = flag_wait_ge<true>(my_flag, epoch, status) ? 1 : 0;
      __syncthreads();
      if (!sh_ok) return;
    }
  }
  if (threadIdx.x == 0 && elapsed_ns) {
    unsigned long long t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    *elapsed_ns = t1 - t0;
  }
}

// my_buf / peer_buf: nbytes each (multiple of 16), in peer-mapped memory; my_flag / peer_flag:
// one u32 each on the respective GPU; `base`: flag value before this call (both ranks pass
// the same).  elapsed_ns (device memory, may be null) receives the leader's or follower's
// device time for all `iters` trips.
extern "C" int mb200_pingpong(void* my_buf, void* peer_buf, uint32_t* my_flag, uint32_t* peer_flag,
                              long long nbytes, int iters, uint32_t base, int leader, int* status,
                              unsigned long long* elapsed_ns, void* stream) {
  if (nbytes < 0 || (nbytes & 15) || iters <= 0) return 1001;
  pingpong_kernel<<<1, 256, 0, ST(stream)>>>(reinterpret_cast<uint4*>(my_buf),
                                              reinterpret_cast<uint4*>(peer_buf), my_flag,
                                              peer_flag, nbytes / 16, iters, base, leader, status,
                                              elapsed_ns);
  return (int)cudaGetLastError();
}

// ---- checked builds: this translation unit's table of allowed address ranges ----------
extern "C" int mb200_bounds_register_comm(const void* base, int64_t size) {
#ifdef MB200_BOUNDS_ACTIVE
  return bounds_table_add(reinterpret_cast<unsigned long long>(base), (unsigned long long)size);
#else
  (void)base; (void)size;
  return 0;
#endif
}
extern "C" int mb200_bounds_reset_comm(int* status) {
#ifdef MB200_BOUNDS_ACTIVE
  return bounds_table_reset(status);
#else
  (void)status;
  return 0;
#endif
}

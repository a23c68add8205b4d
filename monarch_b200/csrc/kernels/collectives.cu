// Mesh collectives for ordinary tensors (the distributed-tensor engine's reduce / gather /
// all-to-all / broadcast), written as plain kernels over a peer-mapped staging buffer.
//
// A communicator owns, on every rank, one staging buffer and one flag array that all
// ranks of the group have mapped (CUDA IPC handles exchanged over actor messages, or
// torch's symmetric memory).  A collective is two or three launches on the caller's stream:
//
//   coll_stage     copy the local tensor into this rank's staging half, then (last block out)
//                  publish the collective's epoch in slot 0 of every rank's flag array
//   coll_reduce    wait for all ranks' epoch, combine the same 16-byte vector of every rank's
//                  staging (fp32 accumulation for 16-bit floats) and write it to a local
//                  tensor (one-shot all-reduce, reduce-scatter, root reduce) or to every
//                  rank's result region (two-shot all-reduce; publishes slot 1 when done)
//   coll_gather    wait, then pull byte ranges of peers' staging into a local tensor
//                  (all-gather, all-to-all, broadcast, and the copy-out of the two-shot)
//
// When the staging buffer also has an NVSwitch multicast mapping, sums of f32/bf16/f16 use
// `multimem.ld_reduce` (the switch adds the ranks' copies; one load instead of `world`) and
// the two-shot broadcast half uses `multimem.st`.  Only multimem touches the multicast
// address; nothing here is a TMA or bulk load, multicast or otherwise.
//
// Staging is double-buffered by the caller (half = epoch & 1).  Every collective begins
// with "publish my epoch, wait for everyone's", and a rank publishes epoch e+1 only after
// its own work for e is finished (stream order), so nobody overwrites a half that a peer
// may still be reading.  All waits are bounded and report through the status word.
//
// The reference reaches the same operations through NCCL communicators
// (torch-sys-cuda/src/nccl.rs:464-835, monarch_tensor_worker/src/comm.rs).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#define MB200_BOUNDS_TU 1
#include "comm.cuh"

namespace mb200 {

enum : int { kF32 = 0, kBF16 = 1, kF16 = 2, kF64 = 3, kI32 = 4, kI64 = 5 };
enum : int { kSum = 0, kProd = 1, kMin = 2, kMax = 3, kBand = 4, kBor = 5, kBxor = 6 };

// ------------------------------------------------------------- 16-byte vector traits --
template <typename T>
struct VT;
template <>
struct VT<float> {
  using Acc = float;
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& u, Acc (&a)[N]) {
    a[0] = __uint_as_float(u.x); a[1] = __uint_as_float(u.y);
    a[2] = __uint_as_float(u.z); a[3] = __uint_as_float(u.w);
  }
  static __device__ __forceinline__ uint4 pack(const Acc (&a)[N]) {
    return make_uint4(__float_as_uint(a[0]), __float_as_uint(a[1]), __float_as_uint(a[2]),
                      __float_as_uint(a[3]));
  }
};
template <>
struct VT<__nv_bfloat16> {
  using Acc = float;
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& u, Acc (&a)[N]) {
    float2 x = unpack_bf16x2(u.x), y = unpack_bf16x2(u.y), z = unpack_bf16x2(u.z),
           w = unpack_bf16x2(u.w);
    a[0] = x.x; a[1] = x.y; a[2] = y.x; a[3] = y.y; a[4] = z.x; a[5] = z.y; a[6] = w.x; a[7] = w.y;
  }
  static __device__ __forceinline__ uint4 pack(const Acc (&a)[N]) {
    return make_uint4(pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]), pack_bf16x2(a[4], a[5]),
                      pack_bf16x2(a[6], a[7]));
  }
};
template <>
struct VT<__half> {
  using Acc = float;
  static constexpr int N = 8;
  static __device__ __forceinline__ float2 up(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2*>(&u));
  }
  static __device__ __forceinline__ uint32_t dn(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ void unpack(const uint4& u, Acc (&a)[N]) {
    float2 x = up(u.x), y = up(u.y), z = up(u.z), w = up(u.w);
    a[0] = x.x; a[1] = x.y; a[2] = y.x; a[3] = y.y; a[4] = z.x; a[5] = z.y; a[6] = w.x; a[7] = w.y;
  }
  static __device__ __forceinline__ uint4 pack(const Acc (&a)[N]) {
    return make_uint4(dn(a[0], a[1]), dn(a[2], a[3]), dn(a[4], a[5]), dn(a[6], a[7]));
  }
};
template <>
struct VT<double> {
  using Acc = double;
  static constexpr int N = 2;
  static __device__ __forceinline__ void unpack(const uint4& u, Acc (&a)[N]) {
    a[0] = __hiloint2double((int)u.y, (int)u.x);
    a[1] = __hiloint2double((int)u.w, (int)u.z);
  }
  static __device__ __forceinline__ uint4 pack(const Acc (&a)[N]) {
    return make_uint4((uint32_t)__double2loint(a[0]), (uint32_t)__double2hiint(a[0]),
                      (uint32_t)__double2loint(a[1]), (uint32_t)__double2hiint(a[1]));
  }
};
template <>
struct VT<int32_t> {
  using Acc = int32_t;
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& u, Acc (&a)[N]) {
    a[0] = (int32_t)u.x; a[1] = (int32_t)u.y; a[2] = (int32_t)u.z; a[3] = (int32_t)u.w;
  }
  static __device__ __forceinline__ uint4 pack(const Acc (&a)[N]) {
    return make_uint4((uint32_t)a[0], (uint32_t)a[1], (uint32_t)a[2], (uint32_t)a[3]);
  }
};
template <>
struct VT<int64_t> {
  using Acc = int64_t;
  static constexpr int N = 2;
  static __device__ __forceinline__ void unpack(const uint4& u, Acc (&a)[N]) {
    a[0] = (int64_t)(((uint64_t)u.y << 32) | u.x);
    a[1] = (int64_t)(((uint64_t)u.w << 32) | u.z);
  }
  static __device__ __forceinline__ uint4 pack(const Acc (&a)[N]) {
    return make_uint4((uint32_t)(uint64_t)a[0], (uint32_t)((uint64_t)a[0] >> 32),
                      (uint32_t)(uint64_t)a[1], (uint32_t)((uint64_t)a[1] >> 32));
  }
};

template <int OP, typename A>
__device__ __forceinline__ A combine(A x, A y) {
  if constexpr (OP == kSum) return x + y;
  if constexpr (OP == kProd) return x * y;
  if constexpr (OP == kMin) return y < x ? y : x;
  if constexpr (OP == kMax) return y > x ? y : x;
  if constexpr (std::is_integral<A>::value) {   // bitwise reductions: integer types only
    if constexpr (OP == kBand) return x & y;
    if constexpr (OP == kBor) return x | y;
    if constexpr (OP == kBxor) return x ^ y;
  }
  return x;
}

template <typename T>
struct McOk {
  static constexpr bool value = false;
};
template <>
struct McOk<float> {
  static constexpr bool value = true;
};
template <>
struct McOk<__nv_bfloat16> {
  static constexpr bool value = true;
};
template <>
struct McOk<__half> {
  static constexpr bool value = true;
};

// ---------------------------------------------------------------------------- stage --
// Local copy src -> dst (dst: this rank's staging), then the last block publishes `epoch`
// in `slot` on every rank.  nbytes may be 0 (a rank that only takes part in the handshake).
__global__ void __launch_bounds__(256)
    coll_stage_kernel(uint8_t* __restrict__ dst, const uint8_t* __restrict__ src, int64_t nbytes,
                      Peers flags, int rank, int world, int slot, uint32_t epoch,
                      unsigned int* counter) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t t0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0) {
    const int64_t nvec = nbytes >> 4;
    int64_t i = t0;
    for (; i + 3 * stride < nvec; i += 4 * stride) {
      uint4 a = reinterpret_cast<const uint4*>(src)[i];
      uint4 b = reinterpret_cast<const uint4*>(src)[i + stride];
      uint4 c = reinterpret_cast<const uint4*>(src)[i + 2 * stride];
      uint4 d = reinterpret_cast<const uint4*>(src)[i + 3 * stride];
      reinterpret_cast<uint4*>(dst)[i] = a;
      reinterpret_cast<uint4*>(dst)[i + stride] = b;
      reinterpret_cast<uint4*>(dst)[i + 2 * stride] = c;
      reinterpret_cast<uint4*>(dst)[i + 3 * stride] = d;
    }
    for (; i < nvec; i += stride)
      reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    for (int64_t b = (nvec << 4) + t0; b < nbytes; b += stride) dst[b] = src[b];
  } else {
    for (int64_t b = t0; b < nbytes; b += stride) dst[b] = src[b];
  }
  if (last_block_done(counter)) signal_all(flags, world, rank, slot, epoch, threadIdx.x);
}

// --------------------------------------------------------------------------- reduce --
struct ReduceArgs {
  Peers in;          // every rank's staged input (same layout on all ranks)
  Peers out_peers;   // every rank's result region (two-shot), or all null
  const void* mc_in; // multicast mapping of `in`, or null
  void* mc_out;      // multicast mapping of the result region, or null
  void* out_local;   // local destination, or null; vector `lo + i` lands at vector i
  int64_t lo, hi;    // range of 16-byte vectors this rank combines
  int64_t valid_bytes_local;  // bytes of out_local that may be written (the last vector may be partial)
  float scale;
  int apply_scale;
  Peers flags;
  int rank, world, wait_slot, signal_slot;  // signal_slot < 0: nothing to publish
  uint32_t epoch;
  unsigned int* counter;
  int* status;
  // one-launch form for small tensors: the kernel first copies stage_bytes from stage_src to
  // this rank's staging (stage_dst) and publishes `epoch` in wait_slot itself.  The blocks
  // then wait for that flag too, so the grid must be co-resident (the launcher caps it).
  const uint8_t* stage_src;
  uint8_t* stage_dst;
  int64_t stage_bytes;
  unsigned int* stage_counter;
};

template <typename T, int OP>
__global__ void __launch_bounds__(256) coll_reduce_kernel(const ReduceArgs a) {
  using V = VT<T>;
  using Acc = typename V::Acc;
  __shared__ int sh_ok;
  if (a.stage_src != nullptr) {
    const int64_t sstride = (int64_t)gridDim.x * blockDim.x;
    const int64_t t0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nvec = a.stage_bytes >> 4;       // both pointers are 16-byte aligned
    for (int64_t v = t0; v < nvec; v += sstride)
      reinterpret_cast<uint4*>(a.stage_dst)[v] = reinterpret_cast<const uint4*>(a.stage_src)[v];
    for (int64_t b = (nvec << 4) + t0; b < a.stage_bytes; b += sstride)
      a.stage_dst[b] = a.stage_src[b];
    if (last_block_done(a.stage_counter))
      signal_all(a.flags, a.world, a.rank, a.wait_slot, a.epoch, threadIdx.x);
  }
  if (!block_wait_all(a.flags.p[a.rank], a.world, a.wait_slot, a.epoch, a.status, &sh_ok)) {
    if (a.signal_slot >= 0) last_block_done(a.counter);
    return;
  }
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  constexpr bool kMc = McOk<T>::value && OP == kSum;
  const bool use_mc = kMc && a.mc_in != nullptr;
  int64_t i = a.lo + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if constexpr (kMc) {
    // the pure in-switch case (sum, no scale, full vectors): four reductions in flight per
    // thread, results to the local tensor and/or to every rank through one multicast store
    if (use_mc && !a.apply_scale && (a.mc_out || !a.out_peers.p[0])) {
      for (; i + 3 * stride < a.hi; i += 4 * stride) {
        if (a.out_local && ((i + 3 * stride - a.lo) << 4) + 16 > a.valid_bytes_local) break;
        uint4 r4[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          r4[j] = multimem_ld_sum<T>(reinterpret_cast<const uint4*>(a.mc_in) + i + j * stride);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int64_t ij = i + j * stride;
          if (a.out_local)
            *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(a.out_local) +
                                      ((ij - a.lo) << 4)) = r4[j];
          if (a.mc_out) multimem_st_v4(reinterpret_cast<uint4*>(a.mc_out) + ij, r4[j]);
        }
      }
    }
  }
  for (; i < a.hi; i += stride) {
    uint4 r;
    if (use_mc && !a.apply_scale) {
      if constexpr (kMc) r = multimem_ld_sum<T>(reinterpret_cast<const uint4*>(a.mc_in) + i);
    } else {
      Acc acc[V::N];
      if (use_mc) {
        if constexpr (kMc)
          V::unpack(multimem_ld_sum<T>(reinterpret_cast<const uint4*>(a.mc_in) + i), acc);
      } else {
        // all loads first (they are in flight together), then combine in rank order so that
        // every rank computes bit-identical results
        uint4 raw[kMaxRanks];
#pragma unroll
        for (int p = 0; p < kMaxRanks; ++p)
          if (p < a.world) raw[p] = ld_nc_v4(reinterpret_cast<const uint4*>(a.in.p[p]) + i);
        V::unpack(raw[0], acc);
#pragma unroll
        for (int p = 1; p < kMaxRanks; ++p) {
          if (p < a.world) {
            Acc tmp[V::N];
            V::unpack(raw[p], tmp);
#pragma unroll
            for (int j = 0; j < V::N; ++j) acc[j] = combine<OP, Acc>(acc[j], tmp[j]);
          }
        }
      }
      if (a.apply_scale) {
#pragma unroll
        for (int j = 0; j < V::N; ++j) acc[j] = (Acc)(acc[j] * (Acc)a.scale);
      }
      r = V::pack(acc);
    }
    if (a.out_local) {
      const int64_t off = (i - a.lo) << 4;
      if (off + 16 <= a.valid_bytes_local) {
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(a.out_local) + off) = r;
      } else {  // the last, partial vector: only the bytes that belong to the tensor
        const uint8_t* rb = reinterpret_cast<const uint8_t*>(&r);
        for (int64_t b = off; b < a.valid_bytes_local; ++b)
          reinterpret_cast<uint8_t*>(a.out_local)[b] = rb[b - off];
      }
    }
    if (a.mc_out) {
      multimem_st_v4(reinterpret_cast<uint4*>(a.mc_out) + i, r);
    } else if (a.out_peers.p[0]) {
#pragma unroll
      for (int k = 0; k < kMaxRanks; ++k)
        if (k < a.world) st_v4(reinterpret_cast<uint4*>(a.out_peers.p[(a.rank + k) % a.world]) + i, r);
    }
  }
  if (a.signal_slot >= 0 && last_block_done(a.counter))
    signal_all(a.flags, a.world, a.rank, a.signal_slot, a.epoch, threadIdx.x);
}

// --------------------------------------------------------------------------- gather --
struct GatherArgs {
  Peers src;                    // every rank's staging (base of the half in use)
  int64_t src_off[kMaxRanks];   // byte offset inside rank p's staging
  int64_t dst_off[kMaxRanks];   // byte offset inside `out`
  int64_t nbytes[kMaxRanks];    // 0: nothing from that rank
  uint8_t* out;
  void* my_flags;
  int rank, world, wait_slot;
  uint32_t epoch;
  int* status;
};

// grid.y = peer (staggered from this rank), grid.x strides over that peer's bytes.
__global__ void __launch_bounds__(256) coll_gather_kernel(const GatherArgs a) {
  __shared__ int sh_ok;
  if (!block_wait_all(a.my_flags, a.world, a.wait_slot, a.epoch, a.status, &sh_ok)) return;
  const int p = (a.rank + (int)blockIdx.y) % a.world;
  const int64_t n = a.nbytes[p];
  if (n <= 0) return;
  const uint8_t* src = reinterpret_cast<const uint8_t*>(a.src.p[p]) + a.src_off[p];
  uint8_t* dst = a.out + a.dst_off[p];
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t t0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0) {
    const int64_t nvec = n >> 4;
    int64_t i = t0;
    // four independent 16-byte loads in flight per thread: a pull over NVLink is bound by
    // outstanding loads
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
    for (int64_t b = (nvec << 4) + t0; b < n; b += stride)
      dst[b] = *reinterpret_cast<const volatile uint8_t*>(src + b);
  } else {
    for (int64_t b = t0; b < n; b += stride) dst[b] = *reinterpret_cast<const volatile uint8_t*>(src + b);
  }
}

static Peers peers_of(const void* const* ptrs, int world) {
  Peers p{};
  if (ptrs)
    for (int i = 0; i < world && i < kMaxRanks; ++i) p.p[i] = const_cast<void*>(ptrs[i]);
  return p;
}

static int grid_for(int64_t items, int per_block, int cap) {
  int64_t b = (items + per_block - 1) / per_block;
  if (b < 1) b = 1;
  return (int)(b < cap ? b : cap);
}

template <typename T>
static int launch_reduce_op(int op, int grid, cudaStream_t st, const ReduceArgs& a) {
  switch (op) {
    case kSum: coll_reduce_kernel<T, kSum><<<grid, 256, 0, st>>>(a); break;
    case kProd: coll_reduce_kernel<T, kProd><<<grid, 256, 0, st>>>(a); break;
    case kMin: coll_reduce_kernel<T, kMin><<<grid, 256, 0, st>>>(a); break;
    case kMax: coll_reduce_kernel<T, kMax><<<grid, 256, 0, st>>>(a); break;
    default:
      if constexpr (std::is_integral<T>::value) {
        if (op == kBand) { coll_reduce_kernel<T, kBand><<<grid, 256, 0, st>>>(a); break; }
        if (op == kBor) { coll_reduce_kernel<T, kBor><<<grid, 256, 0, st>>>(a); break; }
        if (op == kBxor) { coll_reduce_kernel<T, kBxor><<<grid, 256, 0, st>>>(a); break; }
      }
      return 1001;
  }
  return (int)cudaGetLastError();
}

}  // namespace mb200

using namespace mb200;
#define ST(s) reinterpret_cast<cudaStream_t>(s)

// The grids of these kernels are kept within what is co-resident on one GPU (blocks that
// wait on a flag must not keep the blocks that publish it from being scheduled).
extern "C" int mb200_coll_stage(void* stage_dst, const void* src, int64_t nbytes,
                                const void* const* flag_ptrs, int rank, int world, int slot,
                                uint32_t epoch, unsigned int* counter, int n_blocks, void* stream) {
  if (world > kMaxRanks || world < 1 || nbytes < 0) return 1001;
  const int grid = n_blocks > 0 ? n_blocks : grid_for(nbytes / 16 + 1, 256 * 8, 296);
  coll_stage_kernel<<<grid, 256, 0, ST(stream)>>>(reinterpret_cast<uint8_t*>(stage_dst),
                                                  reinterpret_cast<const uint8_t*>(src), nbytes,
                                                  peers_of(flag_ptrs, world), rank, world, slot,
                                                  epoch, counter);
  return (int)cudaGetLastError();
}

// Combine vectors [lo, hi) of all ranks' staging.  out_local (may be null) receives them at
// vector index i - lo, at most valid_bytes_local bytes; out_ptrs (may be null) are every
// rank's result region, written at vector index i (mc_out: their multicast mapping).
extern "C" int mb200_coll_reduce(const void* const* in_ptrs, const void* mc_in,
                                 const void* const* out_ptrs, void* mc_out, void* out_local,
                                 int64_t lo, int64_t hi, int64_t valid_bytes_local, int dtype, int op,
                                 float scale, int apply_scale, const void* const* flag_ptrs,
                                 int rank, int world, int wait_slot, int signal_slot,
                                 uint32_t epoch, unsigned int* counter, int n_blocks, int* status,
                                 void* stream, const void* stage_src, void* stage_dst,
                                 int64_t stage_bytes, unsigned int* stage_counter) {
  if (world > kMaxRanks || world < 1 || hi < lo) return 1001;
  if (stage_src != nullptr &&
      (((reinterpret_cast<uintptr_t>(stage_src) | reinterpret_cast<uintptr_t>(stage_dst)) & 15) != 0 ||
       stage_counter == nullptr || stage_bytes < 0))
    return 1001;
  ReduceArgs a{};
  a.stage_src = reinterpret_cast<const uint8_t*>(stage_src);
  a.stage_dst = reinterpret_cast<uint8_t*>(stage_dst);
  a.stage_bytes = stage_bytes;
  a.stage_counter = stage_counter;
  a.in = peers_of(in_ptrs, world);
  a.out_peers = peers_of(out_ptrs, world);
  a.mc_in = mc_in;
  a.mc_out = mc_out;
  a.out_local = out_local;
  a.lo = lo;
  a.hi = hi;
  a.valid_bytes_local = valid_bytes_local;
  a.scale = scale;
  a.apply_scale = apply_scale;
  a.flags = peers_of(flag_ptrs, world);
  a.rank = rank;
  a.world = world;
  a.wait_slot = wait_slot;
  a.signal_slot = signal_slot;
  a.epoch = epoch;
  a.counter = counter;
  a.status = status;
  int grid = n_blocks > 0 ? n_blocks : grid_for(hi - lo, 256 * 4, 296);
  if (stage_src != nullptr && grid > 148) grid = 148;   // its blocks wait on one another
  cudaStream_t st = ST(stream);
  switch (dtype) {
    case kF32: return launch_reduce_op<float>(op, grid, st, a);
    case kBF16: return launch_reduce_op<__nv_bfloat16>(op, grid, st, a);
    case kF16: return launch_reduce_op<__half>(op, grid, st, a);
    case kF64: return launch_reduce_op<double>(op, grid, st, a);
    case kI32: return launch_reduce_op<int32_t>(op, grid, st, a);
    case kI64: return launch_reduce_op<int64_t>(op, grid, st, a);
    default: return 1001;
  }
}

// Pull nbytes[p] bytes from rank p's staging (+ src_off[p]) to out + dst_off[p], for every p.
extern "C" int mb200_coll_gather(const void* const* src_ptrs, const int64_t* src_off,
                                 const int64_t* dst_off, const int64_t* nbytes, void* out,
                                 void* my_flags, int rank, int world, int wait_slot, uint32_t epoch,
                                 int n_blocks, int* status, void* stream) {
  if (world > kMaxRanks || world < 1) return 1001;
  GatherArgs a{};
  a.src = peers_of(src_ptrs, world);
  int64_t most = 0;
  for (int p = 0; p < world; ++p) {
    a.src_off[p] = src_off[p];
    a.dst_off[p] = dst_off[p];
    a.nbytes[p] = nbytes[p];
    if (nbytes[p] > most) most = nbytes[p];
  }
  a.out = reinterpret_cast<uint8_t*>(out);
  a.my_flags = my_flags;
  a.rank = rank;
  a.world = world;
  a.wait_slot = wait_slot;
  a.epoch = epoch;
  a.status = status;
  int gx = n_blocks > 0 ? n_blocks : grid_for(most / 16 + 1, 256 * 8, 296 / world > 0 ? 296 / world : 1);
  dim3 grid(gx, world);
  coll_gather_kernel<<<grid, 256, 0, ST(stream)>>>(a);
  return (int)cudaGetLastError();
}

// ---- checked builds: this translation unit's table of allowed address ranges ----------
extern "C" int mb200_bounds_register_coll(const void* base, int64_t size) {
#ifdef MB200_BOUNDS_ACTIVE
  return bounds_table_add(reinterpret_cast<unsigned long long>(base), (unsigned long long)size);
#else
  (void)base; (void)size;
  return 0;
#endif
}
extern "C" int mb200_bounds_reset_coll(int* status) {
#ifdef MB200_BOUNDS_ACTIVE
  return bounds_table_reset(status);
#else
  (void)status;
  return 0;
#endif
}

// Shared pieces of the NVLink kernels: the per-rank pointer table, epoch-flag signalling
// with bounded waits, and strong (system-scope) 16-byte loads for peer memory.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace mb200 {

constexpr int kMaxRanks = 8;
struct Peers {
  void* p[kMaxRanks];
};

__device__ __forceinline__ uint32_t* flag_ptr(void* base, int slot, int src_rank) {
  return reinterpret_cast<uint32_t*>(base) + (size_t)slot * kMaxRanks + src_rank;
}

// Publish `epoch` in slot `slot` of every rank's flag array (called by <= kMaxRanks
// threads of one block after the data it announces has been written).
__device__ __forceinline__ void signal_all(const Peers& flags, int world, int rank, int slot,
                                           uint32_t epoch, int tid) {
  if (tid < world) {
    __threadfence_system();
    st_release_sys(flag_ptr(flags.p[tid], slot, rank), epoch);
  }
}

// Wait until every rank has published >= epoch in `slot` of *my* flag array.
__device__ __forceinline__ bool wait_all(void* my_flags, int world, int slot, uint32_t epoch,
                                         int* status) {
  bool ok = true;
  for (int r = 0; r < world && ok; ++r)
    ok = flag_wait_ge<true>(flag_ptr(my_flags, slot, r), epoch, status);
  return ok;
}

// Block-wide: thread 0 waits, everyone learns the outcome.
__device__ __forceinline__ bool block_wait_all(void* my_flags, int world, int slot,
                                               uint32_t epoch, int* status, int* sh_ok) {
  if (threadIdx.x == 0) *sh_ok = wait_all(my_flags, world, slot, epoch, status) ? 1 : 0;
  __syncthreads();
  return *sh_ok != 0;
}

// "Last block out" notification: returns true in exactly one block (the one finishing
// last), after all other blocks' writes are visible.
__device__ __forceinline__ bool last_block_done(unsigned int* counter) {
  __shared__ bool is_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int prev = atomicAdd(counter, 1u);
    is_last = (prev == gridDim.x - 1);
    if (is_last) *counter = 0;  // ready for the next launch
  }
  __syncthreads();
  return is_last;
}

__device__ __forceinline__ void acc8(float (&a)[8], uint4 u) {
  float2 x = unpack_bf16x2(u.x), y = unpack_bf16x2(u.y), z = unpack_bf16x2(u.z),
         w = unpack_bf16x2(u.w);
  a[0] += x.x; a[1] += x.y; a[2] += y.x; a[3] += y.y;
  a[4] += z.x; a[5] += z.y; a[6] += w.x; a[7] += w.y;
}
// ------------------------------------------------------------- checked builds --
// With -DMB200_BOUNDS_CHECK (the library `_mb200_kernels_checked.so`) every access of the
// collective kernels to peer-mapped memory -- 16-byte loads, stores and multimem
// operations -- is first looked up in a table of registered address ranges.  An access
// outside every range is NOT performed: the kernel records kStatusBounds and the offending
// address in the status word (status[0], status[2..3]) and carries on with zeros, so a
// wrong offset or a stale peer pointer shows up as an error the host reads, not as a
// fault.  The table belongs to one translation unit; mb200_bounds_* (bounds.cu) fan out
// registrations to all of them.  A translation unit opts in by defining MB200_BOUNDS_TU
// before including this header (comm.cu and collectives.cu do: the collectives proper; the
// GEMM-fused kernels bound their accesses through their tensor maps and tile extents).
#if defined(MB200_BOUNDS_CHECK) && defined(MB200_BOUNDS_TU)
#define MB200_BOUNDS_ACTIVE 1
constexpr int kBoundsMax = 128;
struct BoundsTable {
  unsigned long long base[kBoundsMax];
  unsigned long long size[kBoundsMax];
  int n;
  int* status;
};
static __device__ BoundsTable g_bounds;

__device__ __forceinline__ bool bounds_ok(const void* p, unsigned long long bytes) {
  const unsigned long long a = reinterpret_cast<unsigned long long>(p);
  const int n = g_bounds.n;
  for (int i = 0; i < n; ++i)
    if (a >= g_bounds.base[i] && a + bytes <= g_bounds.base[i] + g_bounds.size[i]) return true;
  int* st = g_bounds.status;
  if (st && atomicCAS(st, kStatusOk, kStatusBounds) == kStatusOk) {
    st[2] = (int)(a & 0xffffffffull);
    st[3] = (int)(a >> 32);
  }
  return false;
}
#define MB200_IN_BOUNDS(p, bytes) bounds_ok((p), (bytes))

// Host side of the table of this translation unit.
static inline int bounds_table_add(unsigned long long base, unsigned long long size) {
  BoundsTable t;
  cudaError_t e = cudaMemcpyFromSymbol(&t, g_bounds, sizeof(t));
  if (e != cudaSuccess) return (int)e;
  if (t.n >= kBoundsMax) return 1001;
  t.base[t.n] = base;
  t.size[t.n] = size;
  ++t.n;
  return (int)cudaMemcpyToSymbol(g_bounds, &t, sizeof(t));
}
static inline int bounds_table_reset(int* status) {
  BoundsTable t{};
  t.status = status;
  return (int)cudaMemcpyToSymbol(g_bounds, &t, sizeof(t));
}
#else
#define MB200_IN_BOUNDS(p, bytes) true
#endif

__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (!MB200_IN_BOUNDS(p, 16)) return v;
  asm volatile("ld.global.relaxed.sys.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// 16-byte store to (possibly peer) memory.
__device__ __forceinline__ void st_v4(void* p, const uint4& v) {
  if (!MB200_IN_BOUNDS(p, 16)) return;
  *reinterpret_cast<uint4*>(p) = v;
}

// ------------------------------------------------------------------------ multimem --
// NVSwitch multicast ("NVLS") accesses.  `mc` is an address inside a multicast mapping that
// every rank of the group has bound its own buffer to.  A ld_reduce makes the switch add
// the ranks' copies (fp32 accumulation for the 16-bit types) and returns one 16-byte
// vector; a st writes the vector into every rank's copy.
template <typename T>
__device__ __forceinline__ uint4 multimem_ld_sum(const void* mc);
template <>
__device__ __forceinline__ uint4 multimem_ld_sum<float>(const void* mc) {
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (!MB200_IN_BOUNDS(mc, 16)) return v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
template <>
__device__ __forceinline__ uint4 multimem_ld_sum<__nv_bfloat16>(const void* mc) {
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (!MB200_IN_BOUNDS(mc, 16)) return v;
  asm volatile(
      "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(mc)
      : "memory");
  return v;
}
template <>
__device__ __forceinline__ uint4 multimem_ld_sum<__half>(const void* mc) {
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (!MB200_IN_BOUNDS(mc, 16)) return v;
  asm volatile(
      "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(mc)
      : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_v4(void* mc, const uint4& v) {
  if (!MB200_IN_BOUNDS(mc, 16)) return;
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

}  // namespace mb200

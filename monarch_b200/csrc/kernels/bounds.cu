// Registration of the address ranges that a checked build (-DMB200_BOUNDS_CHECK) lets the
// collective kernels touch.  Every translation unit with such kernels keeps its own device
// table (comm.cuh); the entry points here forward to all of them.  In a regular build the
// functions exist and report that checking is off.
#include <cuda_runtime.h>
#include <stdint.h>

extern "C" int mb200_bounds_register_comm(const void* base, int64_t size);
extern "C" int mb200_bounds_reset_comm(int* status);
extern "C" int mb200_bounds_register_coll(const void* base, int64_t size);
extern "C" int mb200_bounds_reset_coll(int* status);

// 1 when this library was built with the checks, else 0.
extern "C" int mb200_bounds_enabled() {
#ifdef MB200_BOUNDS_CHECK
  return 1;
#else
  return 0;
#endif
}

// Forget every range (on the current device) and make violations report to `status`.
extern "C" int mb200_bounds_reset(int* status) {
  int rc = mb200_bounds_reset_comm(status);
  if (!rc) rc = mb200_bounds_reset_coll(status);
  return rc;
}

// Allow accesses to [base, base + size) on the current device (a local buffer, a peer
// mapping, or a multicast mapping).
extern "C" int mb200_bounds_register(const void* base, int64_t size) {
  int rc = mb200_bounds_register_comm(base, size);
  if (!rc) rc = mb200_bounds_register_coll(base, size);
  return rc;
}

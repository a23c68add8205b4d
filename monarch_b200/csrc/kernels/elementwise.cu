// Memory-bound kernels of the transformer step: RMSNorm, RoPE, SwiGLU, cross-entropy,
// AdamW, embedding. All are 16-byte vectorised, one pass over HBM where possible.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "mb200.h"
#include "ptx.cuh"

namespace mb200 {

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z),
         d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Sum across the block; result valid in every thread. `red` holds >= 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// ------------------------------------------------------------------ RMSNorm --
__global__ void __launch_bounds__(256)
    rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                       __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int d, float eps) {
  __shared__ float red[33];
  const size_t row = blockIdx.x;
  const __nv_bfloat16* xr = x + row * d;
  float ss = 0.f;
  for (int c = threadIdx.x * 8; c < d; c += blockDim.x * 8) {
    float f[8];
    load8(xr + c, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  ss = block_sum(ss, red);
  const float rs = rsqrtf(ss / d + eps);
  if (threadIdx.x == 0 && rstd) rstd[row] = rs;
  __nv_bfloat16* yr = y + row * d;
  for (int c = threadIdx.x * 8; c < d; c += blockDim.x * 8) {
    float f[8], g[8];
    load8(xr + c, f);
    load8(w + c, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = f[i] * rs * g[i];
    store8(yr + c, f);
  }
}

constexpr int RMS_BWD_THREADS = 256;
constexpr int RMS_BWD_MAXCH = 4;  // d <= 256*8*4 = 8192

// One block walks rows blockIdx.x, blockIdx.x + gridDim.x, ...; a thread owns NCH chunks of
// 8 columns.  NCH is a template parameter so that the per-thread arrays are sized for the
// actual row length: with d = 4096 (NCH 2) the kernel needs about half the registers of the
// d = 8192 instance and two to three blocks are resident per SM -- rows in different phases
// (loads, block reduction, stores) overlap, which is what a kernel with a reduction in the
// middle of every row needs to stream at HBM speed.
template <int NCH>
__global__ void __launch_bounds__(RMS_BWD_THREADS, NCH <= 2 ? 3 : 1)
    rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                       const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                       const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                       float* __restrict__ dw_partial, int rows, int d) {
  __shared__ float red[33];
  float wv[NCH][8];
  float acc[NCH][8];
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch) {
    const int c = threadIdx.x * 8 + ch * RMS_BWD_THREADS * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[ch][i] = 0.f;
    if (c < d) load8(w + c, wv[ch]);
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* xr = x + (size_t)row * d;
    const __nv_bfloat16* gr = dy + (size_t)row * d;
    const float rs = rstd[row];
    float xh[NCH][8], g[NCH][8];
    float dot = 0.f;
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      const int c = threadIdx.x * 8 + ch * RMS_BWD_THREADS * 8;
      if (c < d) {
        load8(xr + c, xh[ch]);
        load8(gr + c, g[ch]);
      }
    }
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      const int c = threadIdx.x * 8 + ch * RMS_BWD_THREADS * 8;
      if (c < d) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xh[ch][i] *= rs;
          acc[ch][i] += g[ch][i] * xh[ch][i];
          g[ch][i] *= wv[ch][i];
          dot += g[ch][i] * xh[ch][i];
        }
      }
    }
    dot = block_sum(dot, red) / d;
    __nv_bfloat16* dxr = dx + (size_t)row * d;
#pragma unroll
    for (int ch = 0; ch < NCH; ++ch) {
      const int c = threadIdx.x * 8 + ch * RMS_BWD_THREADS * 8;
      if (c < d) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rs * (g[ch][i] - xh[ch][i] * dot);
        if (dres) {
          float r[8];
          load8(dres + (size_t)row * d + c, r);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += r[i];
        }
        store8(dxr + c, o);
      }
    }
  }
  float* out = dw_partial + (size_t)blockIdx.x * d;
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch) {
    const int c = threadIdx.x * 8 + ch * RMS_BWD_THREADS * 8;
    if (c < d) {
      *reinterpret_cast<float4*>(out + c) = make_float4(acc[ch][0], acc[ch][1], acc[ch][2], acc[ch][3]);
      *reinterpret_cast<float4*>(out + c + 4) =
          make_float4(acc[ch][4], acc[ch][5], acc[ch][6], acc[ch][7]);
    }
  }
}

// Column sums of the [nblocks, d] partials.  A block covers 32 columns: its 8 thread rows
// stride over the partial rows (each warp reads 128 contiguous bytes per row) and are
// combined through shared memory, so d / 32 blocks share the work instead of d / 256.
__global__ void __launch_bounds__(256)
    rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, int nblocks, int d,
                             __nv_bfloat16* __restrict__ dw, int accumulate) {
  __shared__ float sh[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (c < d)
    for (int b = ty; b < nblocks; b += 8) s += partial[(size_t)b * d + c];
  sh[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && c < d) {
#pragma unroll
    for (int k = 1; k < 8; ++k) s += sh[k][tx];
    if (accumulate) s += __bfloat162float(dw[c]);
    dw[c] = __float2bfloat16(s);
  }
}

// Launches the backward pair: nb row-striding blocks, then the column reduction.
static void launch_rmsnorm_bwd(int nb, const __nv_bfloat16* dy, const __nv_bfloat16* x,
                               const __nv_bfloat16* w, const float* rstd,
                               const __nv_bfloat16* dres, __nv_bfloat16* dx, float* dw_partial,
                               __nv_bfloat16* dw, int dw_accumulate, int rows, int d,
                               cudaStream_t st) {
  const int nch = (d + RMS_BWD_THREADS * 8 - 1) / (RMS_BWD_THREADS * 8);
  if (nch <= 1)
    rmsnorm_bwd_kernel<1><<<nb, RMS_BWD_THREADS, 0, st>>>(dy, x, w, rstd, dres, dx, dw_partial,
                                                          rows, d);
  else if (nch == 2)
    rmsnorm_bwd_kernel<2><<<nb, RMS_BWD_THREADS, 0, st>>>(dy, x, w, rstd, dres, dx, dw_partial,
                                                          rows, d);
  else
    rmsnorm_bwd_kernel<4><<<nb, RMS_BWD_THREADS, 0, st>>>(dy, x, w, rstd, dres, dx, dw_partial,
                                                          rows, d);
  rmsnorm_dw_reduce_kernel<<<(d + 31) / 32, 256, 0, st>>>(dw_partial, nb, d, dw, dw_accumulate);
}

// --------------------------------------------------------------------- RoPE --
__global__ void rope_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, long long total, int seq_len,
                            int n_rot_heads, int hd, int row_stride, int inverse) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int half = hd >> 1;
  const int per_head = half >> 3;  // threads per head (8 pairs each)
  const int j = (int)(idx % per_head);
  const long long hh = idx / per_head;
  const int h = (int)(hh % n_rot_heads);
  const long long row = hh / n_rot_heads;
  const int pos = (int)(row % seq_len);
  __nv_bfloat16* base = qkv + row * row_stride + (size_t)h * hd + j * 8;
  float a[8], b[8], c[8], s[8];
  load8(base, a);
  load8(base + half, b);
  const float* cp = cos_t + (size_t)pos * half + j * 8;
  const float* sp = sin_t + (size_t)pos * half + j * 8;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    c[i] = cp[i];
    s[i] = inverse ? -sp[i] : sp[i];
  }
  float o1[8], o2[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    o1[i] = a[i] * c[i] - b[i] * s[i];
    o2[i] = b[i] * c[i] + a[i] * s[i];
  }
  store8(base, o1);
  store8(base + half, o2);
}

// ------------------------------------------------------------------- SwiGLU --
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu,
                                  __nv_bfloat16* __restrict__ h, long long total, int F) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int per_row = F >> 3;
  const long long row = idx / per_row;
  const int c = (int)(idx % per_row) * 8;
  float g[8], u[8], o[8];
  load8(gu + row * 2 * F + c, g);
  load8(gu + row * 2 * F + F + c, u);
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = g[i] / (1.f + __expf(-g[i])) * u[i];
  store8(h + row * F + c, o);
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu,
                                  const __nv_bfloat16* __restrict__ dh,
                                  __nv_bfloat16* __restrict__ dgu, long long total, int F) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int per_row = F >> 3;
  const long long row = idx / per_row;
  const int c = (int)(idx % per_row) * 8;
  float g[8], u[8], d[8], dg[8], du[8];
  load8(gu + row * 2 * F + c, g);
  load8(gu + row * 2 * F + F + c, u);
  load8(dh + row * F + c, d);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float sg = 1.f / (1.f + __expf(-g[i]));
    const float silu = g[i] * sg;
    du[i] = d[i] * silu;
    dg[i] = d[i] * u[i] * sg * (1.f + g[i] * (1.f - sg));
  }
  store8(dgu + row * 2 * F + c, dg);
  store8(dgu + row * 2 * F + F + c, du);
}

// ------------------------------------------------------------ cross-entropy --
constexpr int CE_THREADS = 512;
__global__ void __launch_bounds__(CE_THREADS)
    cross_entropy_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                         float* __restrict__ loss_rows, int V, int ld, float grad_scale) {
  __shared__ float red_m[CE_THREADS / 32];
  __shared__ float red_s[CE_THREADS / 32];
  __shared__ float bc[2];
  const size_t row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  const int tgt = (int)targets[row];
  float m = -INFINITY, s = 0.f;
  const int vec_end = V & ~7;
  for (int c = threadIdx.x * 8; c < vec_end; c += CE_THREADS * 8) {
    float f[8];
    load8(lr + c, f);
    float cm = f[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) cm = fmaxf(cm, f[i]);
    const float nm = fmaxf(m, cm);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += __expf(f[i] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  for (int c = vec_end + threadIdx.x; c < V; c += CE_THREADS) {
    const float f = __bfloat162float(lr[c]);
    const float nm = fmaxf(m, f);
    s = s * __expf(m - nm) + __expf(f - nm);
    m = nm;
  }
  // combine (m, s) across the block
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float wm = warp_max(m);
  float ws = warp_sum(m == -INFINITY ? 0.f : s * __expf(m - wm));
  if (lane == 0) {
    red_m[warp] = wm;
    red_s[warp] = ws;
  }
  __syncthreads();
  if (warp == 0) {
    float mm = lane < CE_THREADS / 32 ? red_m[lane] : -INFINITY;
    float ss = lane < CE_THREADS / 32 ? red_s[lane] : 0.f;
    const float gm = warp_max(mm);
    ss = warp_sum(mm == -INFINITY ? 0.f : ss * __expf(mm - gm));
    if (lane == 0) {
      bc[0] = gm;
      bc[1] = ss;
    }
  }
  __syncthreads();
  const float gm = bc[0];
  const float inv = 1.f / bc[1];
  if (threadIdx.x == 0) {
    const float lt = __bfloat162float(lr[tgt]);
    loss_rows[row] = logf(bc[1]) + gm - lt;
  }
  __syncthreads();  // the target logit is read before anyone overwrites it
  for (int c = threadIdx.x * 8; c < vec_end; c += CE_THREADS * 8) {
    float f[8];
    load8(lr + c, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float p = __expf(f[i] - gm) * inv;
      if (c + i == tgt) p -= 1.f;
      f[i] = p * grad_scale;
    }
    store8(lr + c, f);
  }
  for (int c = vec_end + threadIdx.x; c < V; c += CE_THREADS) {
    float p = __expf(__bfloat162float(lr[c]) - gm) * inv;
    if (c == tgt) p -= 1.f;
    lr[c] = __float2bfloat16(p * grad_scale);
  }
}

// -------------------------------------------------------------------- AdamW --
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                             const void* __restrict__ g, __nv_bfloat16* __restrict__ pb, int64_t n,
                             int g_bf16, float lr, float beta1, float beta2, float eps, float wd,
                             float inv_bc1, float inv_sqrt_bc2, float grad_scale) {
  const int64_t i4 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i4 >= n) return;
  float pv[4], mv[4], vv[4], gv[4];
  const bool full = i4 + 4 <= n;
  if (full) {
    float4 a = *reinterpret_cast<const float4*>(p + i4);
    float4 b = *reinterpret_cast<const float4*>(m + i4);
    float4 c = *reinterpret_cast<const float4*>(v + i4);
    pv[0] = a.x; pv[1] = a.y; pv[2] = a.z; pv[3] = a.w;
    mv[0] = b.x; mv[1] = b.y; mv[2] = b.z; mv[3] = b.w;
    vv[0] = c.x; vv[1] = c.y; vv[2] = c.z; vv[3] = c.w;
    if (g_bf16) {
      uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(g) + i4);
      float2 x = unpack_bf16x2(u.x), y = unpack_bf16x2(u.y);
      gv[0] = x.x; gv[1] = x.y; gv[2] = y.x; gv[3] = y.y;
    } else {
      float4 d = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(g) + i4);
      gv[0] = d.x; gv[1] = d.y; gv[2] = d.z; gv[3] = d.w;
    }
  } else {
    for (int k = 0; k < 4; ++k) {
      const bool ok = i4 + k < n;
      pv[k] = ok ? p[i4 + k] : 0.f;
      mv[k] = ok ? m[i4 + k] : 0.f;
      vv[k] = ok ? v[i4 + k] : 0.f;
      gv[k] = !ok ? 0.f
                  : (g_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(g)[i4 + k])
                            : reinterpret_cast<const float*>(g)[i4 + k]);
    }
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float gg = gv[k] * grad_scale;
    pv[k] *= (1.f - lr * wd);
    mv[k] = beta1 * mv[k] + (1.f - beta1) * gg;
    vv[k] = beta2 * vv[k] + (1.f - beta2) * gg * gg;
    const float denom = sqrtf(vv[k]) * inv_sqrt_bc2 + eps;
    pv[k] -= lr * inv_bc1 * mv[k] / denom;
  }
  if (full) {
    *reinterpret_cast<float4*>(p + i4) = make_float4(pv[0], pv[1], pv[2], pv[3]);
    *reinterpret_cast<float4*>(m + i4) = make_float4(mv[0], mv[1], mv[2], mv[3]);
    *reinterpret_cast<float4*>(v + i4) = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (pb) {
      uint2 o;
      o.x = pack_bf16x2(pv[0], pv[1]);
      o.y = pack_bf16x2(pv[2], pv[3]);
      *reinterpret_cast<uint2*>(pb + i4) = o;
    }
  } else {
    for (int k = 0; k < 4 && i4 + k < n; ++k) {
      p[i4 + k] = pv[k];
      m[i4 + k] = mv[k];
      v[i4 + k] = vv[k];
      if (pb) pb[i4 + k] = __float2bfloat16(pv[k]);
    }
  }
}

// ---------------------------------------------------------------- embedding --
__global__ void embedding_fwd_kernel(const __nv_bfloat16* __restrict__ table,
                                     const int64_t* __restrict__ ids,
                                     __nv_bfloat16* __restrict__ out, long long total, int d) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int per_row = d >> 3;
  const long long row = idx / per_row;
  const int c = (int)(idx % per_row) * 8;
  const int64_t id = ids[row];
  *reinterpret_cast<uint4*>(out + row * d + c) =
      *reinterpret_cast<const uint4*>(table + id * d + c);
}
__global__ void embedding_bwd_kernel(const __nv_bfloat16* __restrict__ dout,
                                     const int64_t* __restrict__ ids,
                                     __nv_bfloat16* __restrict__ dtable, long long total, int d) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int per_row = d >> 1;
  const long long row = idx / per_row;
  const int c = (int)(idx % per_row) * 2;
  const int64_t id = ids[row];
  const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(dout + row * d + c);
  atomicAdd(reinterpret_cast<__nv_bfloat162*>(dtable + id * d + c), g);
}

__global__ void sumsq_kernel(const void* __restrict__ x, int64_t n, int is_bf16,
                             float* __restrict__ out) {
  __shared__ float red[33];
  float s = 0.f;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float f = is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(x)[i])
                            : reinterpret_cast<const float*>(x)[i];
    s += f * f;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

static inline unsigned blocks_for(long long total, int threads) {
  return (unsigned)((total + threads - 1) / threads);
}

}  // namespace mb200

using namespace mb200;
#define ST(s) reinterpret_cast<cudaStream_t>(s)
#define BF(p) reinterpret_cast<__nv_bfloat16*>(p)
#define CBF(p) reinterpret_cast<const __nv_bfloat16*>(p)

extern "C" int mb200_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows,
                                 int d, float eps, void* stream) {
  if (rows <= 0) return 0;
  if (d % 8) return 1001;
  rmsnorm_fwd_kernel<<<rows, 256, 0, ST(stream)>>>(CBF(x), CBF(w), BF(y), rstd, d, eps);
  return (int)cudaGetLastError();
}

extern "C" int mb200_rmsnorm_bwd_blocks(int rows) {
  const int cap = 148 * 3;   // one resident wave: three blocks per SM at d <= 4096
  return rows < cap ? rows : cap;
}

extern "C" int mb200_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                                 const void* dres, void* dx, float* dw_partial, void* dw,
                                 int dw_accumulate, int rows, int d, void* stream) {
  if (rows <= 0) return 0;
  if (d % 8 || d > RMS_BWD_THREADS * 8 * RMS_BWD_MAXCH) return 1001;
  const int nb = mb200_rmsnorm_bwd_blocks(rows);
  launch_rmsnorm_bwd(nb, CBF(dy), CBF(x), CBF(w), rstd, CBF(dres), BF(dx), dw_partial, BF(dw),
                     dw_accumulate, rows, d, ST(stream));
  return (int)cudaGetLastError();
}

extern "C" int mb200_rope_inplace(void* qkv, const float* cos_t, const float* sin_t, int rows,
                                  int seq_len, int n_rot_heads, int hd, int row_stride,
                                  int inverse, void* stream) {
  if (rows <= 0) return 0;
  if (hd % 16 || row_stride % 8) return 1001;
  const long long total = (long long)rows * n_rot_heads * (hd / 16);
  rope_kernel<<<blocks_for(total, 256), 256, 0, ST(stream)>>>(BF(qkv), cos_t, sin_t, total,
                                                              seq_len, n_rot_heads, hd, row_stride,
                                                              inverse);
  return (int)cudaGetLastError();
}

extern "C" int mb200_swiglu_fwd(const void* gu, void* h, int rows, int F, void* stream) {
  if (rows <= 0) return 0;
  if (F % 8) return 1001;
  const long long total = (long long)rows * (F / 8);
  swiglu_fwd_kernel<<<blocks_for(total, 256), 256, 0, ST(stream)>>>(CBF(gu), BF(h), total, F);
  return (int)cudaGetLastError();
}
extern "C" int mb200_swiglu_bwd(const void* gu, const void* dh, void* dgu, int rows, int F,
                                void* stream) {
  if (rows <= 0) return 0;
  if (F % 8) return 1001;
  const long long total = (long long)rows * (F / 8);
  swiglu_bwd_kernel<<<blocks_for(total, 256), 256, 0, ST(stream)>>>(CBF(gu), CBF(dh), BF(dgu),
                                                                    total, F);
  return (int)cudaGetLastError();
}

extern "C" int mb200_cross_entropy_fwd_bwd(void* logits, const int64_t* targets, float* loss_rows,
                                           int rows, int V, int ld, float grad_scale,
                                           void* stream) {
  if (rows <= 0) return 0;
  if (ld % 8) return 1001;
  cross_entropy_kernel<<<rows, CE_THREADS, 0, ST(stream)>>>(BF(logits), targets, loss_rows, V, ld,
                                                            grad_scale);
  return (int)cudaGetLastError();
}

extern "C" int mb200_adamw(float* p, float* m, float* v, const void* g, void* p_bf16, int64_t n,
                           int g_bf16, float lr, float beta1, float beta2, float eps, float wd,
                           int step, float grad_scale, void* stream) {
  if (n <= 0) return 0;
  const double bc1 = 1.0 - pow((double)beta1, (double)step);
  const double bc2 = 1.0 - pow((double)beta2, (double)step);
  const long long nthreads = (n + 3) / 4;
  adamw_kernel<<<blocks_for(nthreads, 256), 256, 0, ST(stream)>>>(
      p, m, v, g, BF(p_bf16), n, g_bf16, lr, beta1, beta2, eps, wd, (float)(1.0 / bc1),
      (float)(1.0 / sqrt(bc2)), grad_scale);
  return (int)cudaGetLastError();
}

extern "C" int mb200_embedding_fwd(const void* table, const int64_t* ids, void* out, int rows,
                                   int d, void* stream) {
  if (rows <= 0) return 0;
  if (d % 8) return 1001;
  const long long total = (long long)rows * (d / 8);
  embedding_fwd_kernel<<<blocks_for(total, 256), 256, 0, ST(stream)>>>(CBF(table), ids, BF(out),
                                                                       total, d);
  return (int)cudaGetLastError();
}
extern "C" int mb200_embedding_bwd(const void* dout, const int64_t* ids, void* dtable, int rows,
                                   int d, void* stream) {
  if (rows <= 0) return 0;
  if (d % 2) return 1001;
  const long long total = (long long)rows * (d / 2);
  embedding_bwd_kernel<<<blocks_for(total, 256), 256, 0, ST(stream)>>>(CBF(dout), ids, BF(dtable),
                                                                       total, d);
  return (int)cudaGetLastError();
}

extern "C" int mb200_sumsq(const void* x, int64_t n, int is_bf16, float* out, void* stream) {
  if (n <= 0) return 0;
  sumsq_kernel<<<592, 256, 0, ST(stream)>>>(x, n, is_bf16, out);
  return (int)cudaGetLastError();
}

// ------------------------------------------------- allocation-free RMSNorm backward ----
// See mb200_noalloc.h.  The partial weight-gradient sums live in this file-scope device
// array instead of a caller-provided buffer.  In host code `g_noalloc_scratch` is only a
// handle for the runtime, not a device address: the address the kernels receive comes
// from cudaGetSymbolAddress, resolved once per device.
#include <stdio.h>

#include <mutex>

#include "mb200_noalloc.h"

static __device__ __align__(256) float g_noalloc_scratch[MB200_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int kNoallocMaxDevices = 64;
std::mutex g_noalloc_mu;
float* g_noalloc_ptr[kNoallocMaxDevices] = {nullptr};

// Device address of the scratch on the current device (resolved on first use).
int noalloc_scratch(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kNoallocMaxDevices) return MB200_NOALLOC_ERR_SYMBOL;
  std::lock_guard<std::mutex> g(g_noalloc_mu);
  if (!g_noalloc_ptr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
    if (e != cudaSuccess || !p) {
      fprintf(stderr, "mb200_rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed on device %d: %s\n",
              dev, cudaGetErrorString(e));
      return e != cudaSuccess ? (int)e : MB200_NOALLOC_ERR_SYMBOL;
    }
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}
}  // namespace

extern "C" int mb200_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w,
                                         const float* rstd, const void* dres, void* dx, void* dw,
                                         int dw_accumulate, int rows, int d, void* stream) {
  if (rows < 0) {
    fprintf(stderr, "mb200_rmsnorm_bwd_noalloc: rows = %d is negative\n", rows);
    return MB200_NOALLOC_ERR_BAD_ROWS;
  }
  if (d <= 0 || d % 8 || d > MB200_NOALLOC_MAX_D) {
    fprintf(stderr,
            "mb200_rmsnorm_bwd_noalloc: d = %d is not supported (multiple of 8, at most %d: the "
            "built-in scratch holds %d floats)\n",
            d, MB200_NOALLOC_MAX_D, MB200_NOALLOC_SCRATCH_FLOATS);
    return MB200_NOALLOC_ERR_BAD_D;
  }
  if (rows == 0) return 0;
  float* scratch = nullptr;
  int rc = noalloc_scratch(&scratch);
  if (rc) return rc;
  // As many row-striding blocks as the scratch has room for ([blocks, d] floats).
  int nb = mb200_rmsnorm_bwd_blocks(rows);
  const int cap = MB200_NOALLOC_SCRATCH_FLOATS / d;
  if (nb > cap) nb = cap;
  launch_rmsnorm_bwd(nb, CBF(dy), CBF(x), CBF(w), rstd, CBF(dres), BF(dx), scratch, BF(dw),
                     dw_accumulate, rows, d, ST(stream));
  return (int)cudaGetLastError();
}

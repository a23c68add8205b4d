// C API of the sm_100a kernel library (loaded from Python with ctypes).
// Every function takes raw device pointers and a cudaStream_t (as void*), launches
// asynchronously and returns 0 or a cudaError_t / library error code (>= 1000).
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// C[M,N] = opA(A) opB(B) (+R) (+C).  a_mn=0: A is row-major [M,K]; a_mn=1: A is row-major
// [K,M].  b_mn=0: B is row-major [N,K] (C = A B^T); b_mn=1: B is row-major [K,N].
int mb200_gemm_bf16(const void* A, const void* B, void* C, const void* R, int M, int N, int K,
                    int lda, int ldb, int ldc, int ldr, int a_mn, int b_mn, int accumulate,
                    int* status, void* stream);

// Which GEMM kernel the library uses: 1 = single-CTA 128x256 tiles, 2 = CTA-pair 256x256
// tiles (default).  The fused collective+GEMM kernels follow the same setting.
int mb200_gemm_set_impl(int impl);
int mb200_gemm_get_impl(void);

// RMSNorm over the last dimension. x,y: [rows, d] bf16 (row stride = d); w: [d] bf16;
// rstd: [rows] fp32 (saved for backward).
int mb200_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int d,
                      float eps, void* stream);
// dx = d(loss)/dx (+ dres when given: the gradient arriving through the residual path);
// dw_partial: fp32 scratch [nblocks, d]; dw: [d] bf16. nblocks is returned by
// mb200_rmsnorm_bwd_blocks(rows).
int mb200_rmsnorm_bwd_blocks(int rows);
int mb200_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                      const void* dres, void* dx, float* dw_partial, void* dw, int dw_accumulate,
                      int rows, int d, void* stream);

// In-place rotary embedding (rotate-half convention) on the first n_rot_heads heads of
// each row of `qkv` ([rows, row_stride] bf16, head h at columns [h*hd, (h+1)*hd)).
// cos/sin: [seq_len, hd/2] fp32; position of row r is r % seq_len. inverse=1 applies
// the transpose rotation (used for the backward pass).
int mb200_rope_inplace(void* qkv, const float* cos_t, const float* sin_t, int rows, int seq_len,
                       int n_rot_heads, int hd, int row_stride, int inverse, void* stream);

// SwiGLU on a fused [rows, 2F] gate|up buffer: h = silu(gate) * up.
int mb200_swiglu_fwd(const void* gu, void* h, int rows, int F, void* stream);
int mb200_swiglu_bwd(const void* gu, const void* dh, void* dgu, int rows, int F, void* stream);

// Softmax cross-entropy with in-place gradient: logits [rows, V] bf16 are replaced by
// (softmax - onehot) * grad_scale; loss_rows[r] = -log softmax(logits[r])[target[r]].
int mb200_cross_entropy_fwd_bwd(void* logits, const int64_t* targets, float* loss_rows, int rows,
                                int V, int ld, float grad_scale, void* stream);

// Fused AdamW on flat buffers: fp32 master/m/v, bf16 (g_bf16=1) or fp32 gradient,
// writes the updated bf16 copy of the parameter. step >= 1.
int mb200_adamw(float* p, float* m, float* v, const void* g, void* p_bf16, int64_t n, int g_bf16,
                float lr, float beta1, float beta2, float eps, float wd, int step,
                float grad_scale, void* stream);

// Embedding gather and scatter-add (atomic) for the gradient.
int mb200_embedding_fwd(const void* table, const int64_t* ids, void* out, int rows, int d,
                        void* stream);
int mb200_embedding_bwd(const void* dout, const int64_t* ids, void* dtable, int rows, int d,
                        void* stream);

// Sum of squares of a bf16/fp32 buffer accumulated into *out (fp32, caller zeroes it).
int mb200_sumsq(const void* x, int64_t n, int is_bf16, float* out, void* stream);

// Causal grouped-query attention (flash style, tcgen05). q: [B,S,Hq,hd], k/v: [B,S,Hkv,hd]
// inside a fused qkv buffer with row stride `ld`; o: [B,S,Hq,hd] dense; lse: [B,Hq,S] fp32.
int mb200_pingpong(void* my_buf, void* peer_buf, uint32_t* my_flag, uint32_t* peer_flag,
                   long long nbytes, int iters, uint32_t base, int leader, int* status,
                   unsigned long long* elapsed_ns, void* stream);
int mb200_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S,
                   int Hq, int Hkv, int hd, int ld_qkv, int ld_o, float scale, int* status,
                   void* stream);
int mb200_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                   const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int S,
                   int Hq, int Hkv, int hd, int ld_qkv, int ld_o, int ld_dqkv, float scale,
                   int* status, void* stream);

#ifdef __cplusplus
}
#endif

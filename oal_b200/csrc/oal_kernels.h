// Internal launch interface between the C-ABI translation unit and the kernel files.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace oal {

// Arguments of the token-pair kernels (oal_pairs.cu).
struct PairArgs {
  int B, Hq, Hkv, N, G;
  int window;            // 0: whole causal prefix; >0: keys of the query's own chunk only (multiple of 64)
  int io_dt, out_dt;
  float scale, floor;
  const void *q, *k, *v;
  const int32_t *dim_perm, *group_start;
  const float *A, *Bc, *Cc;
  int32_t* status;
  // forward
  void* out;
  float *num, *den;
  int accumulate;        // num/den already hold the cross-chunk term
  // backward
  const float* g;        // [B,Hq,N,80] augmented upstream gradient
  void *dq, *dk, *dv;
  const float *dq_init, *dk_init, *dv_init;   // fp32 cross-chunk parts to add, or null
  float* coef_partial;   // [B][Hq][tiles][NCOEF] or null
};

cudaError_t pairs_forward(const PairArgs& a, cudaStream_t st);
cudaError_t pairs_backward_q(const PairArgs& a, cudaStream_t st);
cudaError_t pairs_backward_kv(const PairArgs& a, cudaStream_t st);
int pairs_tiles(int n);

cudaError_t norm_vjp(const void* grad_out, int out_dt, const float* grad_num, const float* grad_den,
                     const float* num, const float* den, float floor_v, float* g, size_t rows,
                     cudaStream_t st);

// extra: [Hq][NCOEF] slots already summed over the batch (cross-chunk term), or null
cudaError_t reduce_coefs(const float* p0, int tiles0, const float* extra, int B, int Hq, int G,
                         float* dA, float* dB, float* dC, cudaStream_t st);

// ---- tensor-core state kernels (oal_state.cu) ---------------------------------------
// rotary embedding fused with the layout move between [B, N, H, 64] and [B, H, N, 64] (bf16)
cudaError_t rope_to_heads(const void* src, void* dst, const float* cosv, const float* sinv, int B, int N, int H,
                          bool rotate, cudaStream_t st);
cudaError_t rope_to_flat(const void* src, void* dst, const float* cosv, const float* sinv, int B, int N, int H,
                         bool rotate, cudaStream_t st);

size_t state_rows();                       // feature rows of the running state (2432)
size_t state_image_bytes_per_chunk();      // bytes of one bf16 state image [19 slabs][10][128][8]
size_t state_slab_image_bytes();           // bytes of one slab image [10][128][8] bf16

cudaError_t build_coef_table(const int32_t* dim_perm, const int32_t* group_start, const float* A,
                             const float* Bc, const float* Cc, int Hq, int G, float scale, float* table,
                             cudaStream_t st);
cudaError_t state_update(const void* k, const void* v, float* ds, int units, int N, int NB, int32_t* status,
                         cudaStream_t st);
// image_lo: optional second image holding bf16(state - bf16(state))
cudaError_t state_scan(const float* ds, void* image, void* image_lo, const float* state_in, float* state_total,
                       int units, int NB, int reverse, cudaStream_t st);
cudaError_t cross_read(bool query, const void* x, const void* image, const float* coef_table, float* out64,
                       float* out1, int B, int H, int rep, int N, int NB, int32_t* status, cudaStream_t st);


// ---- tensor-core backward kernels (oal_state_bwd.cu) ----------------------------------
// carry_img / carry_lo: the saved state image and its remainder image (both or neither)
cudaError_t dstate_heads(const void* q, const void* gimg, const void* carry_img, const void* carry_lo, const float* coef_table,
                         float* dcarry, float* dcoef_partial, int B, int Hq, int Hkv, int N, int NB, float scale,
                         int32_t* status, cudaStream_t st);
cudaError_t feature_grad(bool query, const void* x, const void* gimg, const void* v, const void* image,
                         const float* coef_table, float* dx, int B, int H, int rep, int N, int NB, int32_t* status,
                         cudaStream_t st);
cudaError_t dcoef_reduce(const float* partial, int outer, int Hq, const int32_t* dim_perm,
                         const int32_t* group_start, float* dcoef, float* slots, cudaStream_t st);
cudaError_t norm_vjp_image(const void* grad_out, int out_dt, const float* grad_num, const float* grad_den,
                           const float* num, const float* den, float floor_v, float* g, void* gimg, int heads,
                           int N, int NB, int token_major_heads, cudaStream_t st);   // > 0: grad_out is [B, N, Hq, 64]


// ---- factored intra-chunk weight (oal_factor.cu) -----------------------------------------
// Per-head table of the factored quadratic form (c_r, l_r[d], back-transform, sign split).
size_t head_factor_bytes(int Hq);
// Packed lower-triangular factor rows [factor_rows (1 or Hq), (G+1)(G+2)/2] -> A, B, C, and the transpose map.
cudaError_t expand_factor(const float* factor, int factor_rows, int Hq, int G, float eps, float* A, float* B, float* C,
                          cudaStream_t st);
cudaError_t expand_factor_grad(const float* factor, int factor_rows, int Hq, int G, const float* dA, const float* dB,
                               const float* dC, float* dfactor, cudaStream_t st);
cudaError_t build_head_factors(const int32_t* dim_perm, const int32_t* group_start, const float* A, const float* Bc,
                               const float* Cc, int Hq, int G, float scale, void* table, cudaStream_t st);
// dA, dB, dC = back-transformed sum of the query-side partial sums [B][Hq][tiles][nu_stride] (rm terms,
// upper triangle) + extra ([Hq][NCOEF] slots of the cross-chunk term, or null).
cudaError_t intra_coef_finish(const float* partial, int tiles, int nu_stride, int rm, const void* table,
                              const float* extra, int B, int Hq, int G, float* dA, float* dB, float* dC,
                              cudaStream_t st);

// ---- tensor-core intra-chunk kernels (oal_intra.cu, oal_intra_bwd.cu): heads with at most 8 groups ----
int intra_coef_terms();          // terms per head this build handles (rows of the partial-sum triangle)
cudaError_t intra_forward(const void* q, const void* k, const void* v, const void* factors, void* out, float* num,
                          float* den, int32_t* status, int B, int Hq, int Hkv, int N, int NB, int out_dt,
                          float floor_v, bool out_token_major, cudaStream_t st);
cudaError_t intra_backward_q(const void* q, const void* k, const void* v, const void* gimg, const void* factors,
                             void* dq, const float* dq_init, float* coef_partial, int32_t* status, int B, int Hq,
                             int Hkv, int N, int NB, cudaStream_t st);
cudaError_t intra_backward_kv(const void* q, const void* k, const void* v, const void* gimg, const void* factors,
                              void* dk, void* dv, const float* dk_cross, const float* dv_cross, float* dk_part,
                              float* dv_part, int32_t* status, int B, int Hq, int Hkv, int N, int NB, cudaStream_t st);

}  // namespace oal

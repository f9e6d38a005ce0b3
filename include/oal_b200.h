/*
 * oal_b200 -- C ABI of the B200 (sm_100a) implementation of OAL's causal
 * grouped-quadratic linear attention, forward and backward.
 *
 * This is the drop-in boundary for one path of the reference project
 * (wuqianyue09/OAL): everything the reference computes between
 *   oal_attention/hd_block_gemm_autograd.py:85-204   (_HDParallelBlockGemmFunction)
 * and its dense-contraction seam
 *   oal_attention/hd_block_gemm_contractions.py:26-92 (_bmm_fp32 / _bmm_add_fp32)
 *   oal_attention/csrc/hd_cublas_compat.cpp:100-203   (bmm_fp32, the only native op)
 * is replaced by the entry points below.  Signatures use plain pointers and
 * sizes only; every pointer is a CUDA device pointer unless stated otherwise
 * and the library never allocates or frees device memory: the caller owns the
 * inputs, the outputs and one workspace blob whose size is returned by
 * oal_workspace_bytes().  All launches go to the stream that is passed in.
 *
 * Return value of every int function: 0 on success, a negative OAL_ERR_* code
 * on a contract violation (oal_last_error_string() describes it).  Numerical
 * conditions (non-finite result, non-positive denominator, a bounded wait that
 * ran out inside a kernel) are not return codes: kernels OR them into the
 * caller's device status word, which the host reads at the same point where
 * the reference synchronises (oal_attention/hd_block_gemm_runtime.py:392-408).
 */
#ifndef OAL_B200_H
#define OAL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OAL_HEAD_DIM 64      /* kernels are specialised for D = Dv = 64; the host zero-pads smaller heads */
#define OAL_MAX_GROUPS 16    /* dimension groups per query head handled by the kernels */
#define OAL_E_PAD 80         /* [v | 1] rows (65 values) padded to a multiple of 16 */

enum { OAL_DTYPE_F32 = 0, OAL_DTYPE_BF16 = 1, OAL_DTYPE_F16 = 2 };

/* precision modes of the reference (oal_attention/hd_block_gemm_plan.py:52) */
enum {
  OAL_PRECISION_FP32_IEEE = 0,      /* fp32 arithmetic throughout, exact causal pair sums            */
  OAL_PRECISION_BF16_TENSORCORE = 1 /* bf16 operands, fp32 accumulation, chunked state scan (tcgen05) */
};

enum {
  OAL_OK = 0,
  OAL_ERR_ARGUMENT = -1,   /* NULL pointer, bad size, unsupported geometry  -> ValueError */
  OAL_ERR_DTYPE = -2,      /* unsupported dtype / precision combination     -> TypeError  */
  OAL_ERR_WORKSPACE = -3,  /* workspace too small                            -> ValueError */
  OAL_ERR_CUDA = -4        /* a CUDA runtime call failed                     -> RuntimeError */
};

/* bits of the device status word */
enum {
  OAL_STATUS_NONFINITE = 1,      /* numerator or denominator not finite                    */
  OAL_STATUS_DENOMINATOR = 2,    /* denominator <= 0                                        */
  OAL_STATUS_WAIT_TIMEOUT = 4,   /* a bounded mbarrier wait inside a kernel gave up; bits 8..15
                                    then hold the id of the wait site                       */
  OAL_STATUS_BAD_LAYOUT = 8      /* reserved (no kernel raises it)                          */
};

/* gradient request mask, same order as the reference's requested_gradient_mask
 * (oal_attention/hd_block_gemm_adapters.py:27-43): q, k, v, A, B, C */
enum {
  OAL_GRAD_Q = 1, OAL_GRAD_K = 2, OAL_GRAD_V = 4, OAL_GRAD_COEF = 8,
  /* oal_forward / oal_backward: the workspace still holds what oal_forward_local_state /
   * oal_backward_local_state computed for this very call (same problem, same workspace, nothing
   * launched on it in between): skip that stage (the chunk-state increments, resp. the
   * normalisation VJP, dCarry and coefficient partial sums) */
  OAL_GRAD_REUSE_STATE_STAGE = 16
};

/* OalProblem.flags */
enum {
  /* `out` (oal_forward) and `grad_out` (oal_backward) are [B, N, Hq, 64] -- the layout the caller's output
   * projection reads, replacing its transpose + contiguous copy
   * (qwen_lora_experiment/attention/common.py:575-596) -- instead of [B, Hq, N, 64].  num and den keep the
   * head-first layout.  bf16_tensorcore with at most 8 groups per head only. */
  OAL_FLAG_OUT_TOKEN_MAJOR = 1
};

typedef struct OalProblem {
  int32_t batch;        /* B                                                            */
  int32_t q_heads;      /* Hq                                                           */
  int32_t kv_heads;     /* Hkv, Hq % Hkv == 0; query head h reads KV head h / (Hq/Hkv)  */
  int32_t seq_len;      /* N >= 1 (ragged tails are masked)                             */
  int32_t head_dim;     /* must be OAL_HEAD_DIM                                         */
  int32_t value_dim;    /* must be OAL_HEAD_DIM                                         */
  int32_t groups;       /* G: second extent of B [Hq,G] and C [Hq,G,G], 1..OAL_MAX_GROUPS */
  int32_t chunk;        /* tokens per chunk of the state scan: 128 (bf16_tensorcore)    */
  int32_t io_dtype;     /* dtype of q, k, v and of dq, dk, dv                           */
  int32_t out_dtype;    /* dtype of out and of the upstream gradient of out             */
  int32_t precision;    /* OAL_PRECISION_*                                              */
  int32_t grad_mask;    /* OAL_GRAD_* bits requested from oal_backward                  */
  float scale;          /* q is multiplied by this before anything else                 */
  float floor;          /* normalisation floor: out = num / max(den, floor)             */
  int32_t flags;        /* OAL_FLAG_* bits, 0 for the reference's layouts                   */
} OalProblem;

/* Bytes of workspace oal_forward (phase 0) / oal_backward (phase 1) need, and
 * bytes of the saved chunk-state buffer the forward hands to the backward
 * (phase 2; 0 in fp32_ieee mode).  Replaces the reference's buffer planner
 * (oal_attention/hd_block_gemm_buffers.py:108-368).  Returns < 0 on error. */
int64_t oal_workspace_bytes(const OalProblem* problem, int phase);

/*
 * Forward.  Replaces _hd_parallel_block_gemm_impl
 * (oal_attention/hd_block_gemm_runtime.py:617-805) including feature building,
 * block totals, the exclusive scan, the intra-chunk scores and the fused
 * normalisation (oal_attention/hd_block_gemm_normalization_ops.py:113).
 *
 *   q [B,Hq,N,64], k [B,Hkv,N,64], v [B,Hkv,N,64]   io_dtype, row-major contiguous
 *   dim_perm   int32 [Hq,64]   dims of each head sorted by group id
 *   group_start int32 [Hq,OAL_MAX_GROUPS+1]  offsets into dim_perm; group g of head h
 *              owns dim_perm[h, group_start[h,g] : group_start[h,g+1]]
 *   coef_a fp32 [Hq], coef_b fp32 [Hq,G], coef_c fp32 [Hq,G,G] (symmetric)
 *   out [B,Hq,N,64] out_dtype; num fp32 [B,Hq,N,64]; den fp32 [B,Hq,N]
 *   saved_state: oal_workspace_bytes(problem, 2) bytes kept for the backward
 *              (may be NULL when that size is 0)
 *   state_in:  sequence parallelism, may be NULL: the fp32 state
 *              [B*Hkv, OAL_STATE_ROWS, OAL_E_PAD] accumulated by the ranks that own earlier
 *              tokens (see oal_forward_local_state).
 */
int oal_forward(const OalProblem* problem, const void* q, const void* k, const void* v,
                const int32_t* dim_perm, const int32_t* group_start, const float* coef_a,
                const float* coef_b, const float* coef_c, void* out, float* num, float* den,
                void* saved_state, const float* state_in, void* workspace, size_t workspace_bytes,
                int32_t* status, void* stream);

/*
 * Backward.  Replaces _hd_parallel_block_gemm_autograd_backward_impl
 * (oal_attention/hd_block_gemm_autograd.py:207-347): normalisation VJP
 * (hd_block_gemm_backward.py:191-308), dCarry + reverse scan (:764-908), the
 * shared-wave VJP (:1455-1992) and the feature folds / coefficient partial
 * sums (hd_block_gemm_feature_backward.py:59-474).
 *
 *   grad_out out_dtype [B,Hq,N,64] or NULL; grad_num fp32 [B,Hq,N,64] or NULL;
 *   grad_den fp32 [B,Hq,N] or NULL
 *   dq, dk, dv io_dtype (each may be NULL if not requested in grad_mask)
 *   d_coef_a fp32 [Hq], d_coef_b fp32 [Hq,G], d_coef_c fp32 [Hq,G,G] (symmetric
 *   closed form sum dW s_g s_g'); NULL unless OAL_GRAD_COEF
 *   dstate_in: sequence parallelism, gradient of the state arriving from the
 *   ranks that own later tokens, or NULL.
 */
int oal_backward(const OalProblem* problem, const void* q, const void* k, const void* v,
                 const int32_t* dim_perm, const int32_t* group_start, const float* coef_a,
                 const float* coef_b, const float* coef_c, const float* num, const float* den,
                 const void* saved_state, const void* grad_out, const float* grad_num,
                 const float* grad_den, void* dq, void* dk, void* dv, float* d_coef_a,
                 float* d_coef_b, float* d_coef_c, const float* dstate_in, void* workspace,
                 size_t workspace_bytes, int32_t* status, void* stream);

/*
 * Sequence parallelism (new; the reference is single-GPU, there is nothing to be compatible with).
 * A rank that owns a contiguous token range first computes the sum of its own chunk-state
 * increments, the ranks exchange these (one all-gather of batch*kv_heads*OAL_STATE_ROWS*OAL_E_PAD
 * floats), and each rank passes the sum over the ranks before it as `state_in` to oal_forward.
 * Backward mirrors it with the state gradient: oal_backward_local_state, exchange, sum over the
 * ranks after it as `dstate_in` to oal_backward.  With OAL_GRAD_REUSE_STATE_STAGE in grad_mask the
 * second call of each pair (oal_forward, oal_backward) reuses what the first left in the same workspace
 * instead of computing it again.
 *   state_total / dstate_total: fp32 [batch*kv_heads, OAL_STATE_ROWS, OAL_E_PAD]
 *   workspace: oal_workspace_bytes(problem, 0) for the forward call, (problem, 1) for the backward.
 */
#define OAL_STATE_ROWS 2432
int oal_forward_local_state(const OalProblem* problem, const void* k, const void* v, float* state_total,
                            void* workspace, size_t workspace_bytes, int32_t* status, void* stream);
int oal_backward_local_state(const OalProblem* problem, const void* q, const int32_t* dim_perm,
                             const int32_t* group_start, const float* coef_a, const float* coef_b,
                             const float* coef_c, const float* num, const float* den, const void* saved_state,
                             const void* grad_out, const float* grad_num, const float* grad_den,
                             float* dstate_total, void* workspace, size_t workspace_bytes, int32_t* status,
                             void* stream);

/*
 * Forward for callers that cannot allocate (no counterpart in the reference, which allocates every
 * buffer with torch.empty).  Same computation and outputs as oal_forward in bf16_tensorcore mode, but
 * the scratch memory comes from a fixed array inside the library instead of a caller workspace, and
 * the call performs no cudaMalloc / cudaFree or other allocating call.  Meant for hosts whose device
 * memory is frozen after start-up (serving processes with a pre-carved pool, plugins run from
 * allocator-free callbacks).
 *   Limits: batch * kv_heads * ceil(seq_len / 128) <= 16 and q_heads <= 64; larger problems return
 *   OAL_ERR_WORKSPACE.  The array (about 13.1 MB) is resident on every GPU that loads the library.
 *   The first call on each device resolves the array's device address; make that call outside any
 *   stream capture, with the device current.
 *   All calls on a device share the array and it keeps the previous call's contents; every element
 *   that is read is rewritten first, so nothing needs clearing, but two calls that overlap on the GPU
 *   (different streams, or different host threads) race on it: serialise them.
 *   saved_state still belongs to the caller (oal_workspace_bytes(problem, 2) bytes).
 */
int oal_forward_static_scratch(const OalProblem* problem, const void* q, const void* k, const void* v,
                               const int32_t* dim_perm, const int32_t* group_start, const float* coef_a,
                               const float* coef_b, const float* coef_c, void* out, float* num, float* den,
                               void* saved_state, int32_t* status, void* stream);

/*
 * Layer prologue fused into one pass per tensor (replaces the reshape / transpose / rotary / contiguous
 * sequence of qwen_lora_experiment/attention/common.py:550-572).  bf16 only, head dimension 64.
 *   oal_rope_pack: q_flat [B, N, Hq*64], k_flat, v_flat [B, N, Hkv*64] (projection outputs) ->
 *     q, k rotated by position and v copied, all head-first [B, H, N, 64] contiguous, as oal_forward
 *     reads them.  cos, sin: fp32 [N, 64], rotate-half convention (32 frequencies repeated twice).
 *   oal_rope_unpack_grad: the transpose of that map, for the backward: gradients in head-first layout ->
 *     gradients of the projection outputs.
 * Any of the three tensors may be NULL (skipped).
 */
int oal_rope_pack(const void* q_flat, const void* k_flat, const void* v_flat, const float* cos, const float* sin,
                  void* q, void* k, void* v, int batch, int seq_len, int q_heads, int kv_heads, void* stream);
int oal_rope_unpack_grad(const void* dq, const void* dk, const void* dv, const float* cos, const float* sin,
                         void* dq_flat, void* dk_flat, void* dv_flat, int batch, int seq_len, int q_heads,
                         int kv_heads, void* stream);

/* Text of the last error returned on the calling thread (host pointer, never NULL). */
const char* oal_last_error_string(void);

/*
 * Self-test of the tensor-core building blocks (no counterpart in the reference, whose
 * only native op delegates to cuBLAS: oal_attention/csrc/hd_cublas_compat.cpp:177-200).
 * Runs one 128 x n x k bf16 GEMM with fp32 accumulation through tcgen05.mma:
 *   mode 0: a [128,k], b [n,k] (K contiguous)      d = a b^T
 *   mode 1: a [k,128], b [k,n] (M / N contiguous)  d = a^T b
 *   mode 2: as mode 0 with the A operand staged in tensor memory
 * n: multiple of 16 in 16..256, k: multiple of 16 in 16..128; a, b bf16, d fp32 [128,n].
 */
int oal_selftest_umma(int mode, int n, int k, const void* a, const void* b, float* d, int32_t* status,
                      void* stream);

/*
 * Self-test of the bounded-wait path every tensor-core kernel relies on (no counterpart in the reference,
 * which has no device-side waits).  One warp waits on a barrier that nothing arrives on, with a limit of
 * `limit_clocks` SM clocks (1 .. 1 000 000, i.e. at most about half a millisecond); the wait gives up and
 * the kernel ORs OAL_STATUS_WAIT_TIMEOUT | (0x7E << 8) into *status and returns normally, exactly as the
 * production kernels do after their 50 M-clock limit.  Nothing hangs or faults; the context stays usable.
 */
int oal_selftest_wait_timeout(int64_t limit_clocks, int32_t* status, void* stream);

/*
 * Launch accounting and opt-in per-kernel timing (thin counterpart of the reference's stage
 * profiler, oal_attention/hd_block_gemm_profiling.py:195-378).  oal_launch_count() is the number
 * of kernels this library has launched in the process so far.  After oal_profile_enable(1) every
 * launch is bracketed by a CUDA-event pair on its stream; oal_profile_report() waits for them and
 * writes a JSON object {"kernel": [launches, total_ms], ...} into the host buffer, then forgets
 * them.  oal_profile_enable(0) switches the events off again.
 */
int64_t oal_launch_count(void);
void oal_profile_enable(int enable);
int oal_profile_report(char* buffer, size_t capacity);

/*
 * Inside oal_forward / oal_backward a few kernels that the main chain does not wait for run on two
 * streams the library owns (created on first use, per device), forked from and joined back into the
 * caller's stream with events before the call returns: from outside every entry point is work on the one
 * stream that was passed in.  oal_set_overlap(0) keeps everything on the caller's stream (the per-kernel
 * times of oal_profile_report are only meaningful that way); the default is 1.  No counterpart in the
 * reference, which runs one stream.
 */
void oal_set_overlap(int enable);

/*
 * Packed factor -> coefficients: L = lower-triangular matrix whose rows, packed in the order of
 * torch.tril_indices, are `factor` [factor_rows, (G+1)(G+2)/2] with factor_rows 1 (shared) or q_heads;
 * M = L L^T, coef_a[h] = M00 + kernel_eps, coef_b[h, g] = 2 M[0, 1+g], coef_c[h, g, g'] = M[1+g, 1+g'].
 * Replaces _expand_factor_coefficients (oal_attention/grouped_quadratic.py:184-219) and, with
 * oal_expand_factor_grad (d_factor from d_coef_a/b/c; a shared factor row sums the heads in order), its
 * autograd graph.  fp32.
 */
int oal_expand_factor(const float* factor, int factor_rows, int q_heads, int groups, float kernel_eps, float* coef_a,
                      float* coef_b, float* coef_c, void* stream);
int oal_expand_factor_grad(const float* factor, int factor_rows, int q_heads, int groups, const float* d_coef_a,
                           const float* d_coef_b, const float* d_coef_c, float* d_factor, void* stream);

/*
 * Deferred status words.  The reference synchronises after every forward to read its checks
 * (oal_attention/hd_block_gemm_runtime.py:392-408); here a call leaves a status word on the device, and
 * oal_status_defer queues its copy to pinned host memory on a stream the library owns, ordered after
 * everything `stream` holds so far (the word must stay allocated until the ticket has been polled as
 * finished).  oal_status_poll returns 1 and the word once the copy has run, 0 while it has not (`block`
 * = 0), or waits for it (`block` = 1).  A ticket stays valid for the next 1023 oal_status_defer calls on
 * its device.
 */
int oal_status_defer(const int32_t* status, void* stream, int64_t* ticket);
int oal_status_poll(int64_t ticket, int block, int32_t* value);

/* Library / build identification: "oal_b200 <version> sm_100a". Host pointer. */
const char* oal_version_string(void);

#ifdef __cplusplus
}
#endif
#endif /* OAL_B200_H */

// Inter-chunk state kernels on the tensor cores (tcgen05 / TMEM).
//
// Chunked causal scan of the reference (oal_attention/hd_block_gemm_runtime.py:271-320
// block totals and exclusive cumsum, :552-560 cross contraction phi_q x carry) with 128-token
// chunks:
//   state_update : dS[u,c] = phi_k(chunk c)^T [v | 1]          (features are the MMA M dimension)
//   state_scan   : carry[u,c] = state_in + sum_{c'<c} dS[u,c'] (fp32), stored as the bf16
//                  operand image the MMAs read
//   cross_read   : Y[i,:] = phi_q(i) . carry[u,c(i)]           (tokens are the MMA M dimension)
// Feature tiles are generated in shared memory (oal_features.cuh) and never touch HBM.
// The fp32 accumulators live in tensor memory; state images are streamed with 1-D bulk
// async copies.  Every mbarrier wait is bounded (oal_umma.cuh).
#include "oal_features.cuh"
#include "oal_kernels.h"

namespace oal {
namespace {

using namespace umma;

// the 19 slabs are processed by four CTAs per (chunk, unit): slab groups 5, 5, 5, 4
constexpr int SU_GROUPS = 4;
__device__ __forceinline__ int group_first_slab(int g) { return 5 * g; }
__device__ __forceinline__ int group_slab_count(int g) { return g < 3 ? 5 : F_SLABS - 15; }

// ---------------------------------------------------------------------------
// per-head coefficient table in feature order (fp32 [Hq][F_ROWS]), query scale folded in:
// pair rows carry scale^2, linear rows scale (the query-side kernels read the unscaled q)
// ---------------------------------------------------------------------------
__global__ void coef_table_kernel(const int32_t* dim_perm, const int32_t* group_start, const float* A,
                                  const float* Bc, const float* Cc, int G, float scale, float* table) {
  __shared__ int gdim[HD];
  const int h = blockIdx.x;
  if (threadIdx.x < HD) {
    const int p = threadIdx.x;
    int g = 0;
    while (g < GMAX - 1 && p >= group_start[h * (GMAX + 1) + g + 1]) ++g;
    gdim[dim_perm[h * HD + p]] = g;
  }
  __syncthreads();
  for (int f = threadIdx.x; f < F_ROWS; f += blockDim.x) {
    float v = 0.f;
    const FeatureId id = feature_id(f);
    if (id.kind == 0 && id.live) {
      const int gr = min(gdim[id.r], G - 1), gc = min(gdim[id.c], G - 1);
      v = (id.r == id.c ? 1.f : 2.f) * Cc[((size_t)h * G + gr) * G + gc];
    } else if (id.kind == 1) {
      v = Bc[h * G + min(gdim[id.r], G - 1)];
    } else if (id.kind == 2) {
      v = A[h];
    }
    table[(size_t)h * F_ROWS + f] = v * feature_scale_factor(f, scale);
  }
}

// ---------------------------------------------------------------------------
// state_update: dS[u,c][slab rows] = phi_k^T U
//   grid (4 slab groups, chunks, units); 256 threads, thread = (token, half of the slab's chunks)
// ---------------------------------------------------------------------------
struct StateUpdateArgs {
  const __nv_bfloat16 *k, *v;   // [units, N, 64]
  float* ds;                    // [units, NB] chunks of F_ROWS x EP floats in state_inc_offset order
  int N, NB;
  int32_t* status;
};

__global__ void __launch_bounds__(GEN_THREADS, 2) state_update_kernel(const StateUpdateArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* Abuf = smem;                          // 2 x SLAB_A_BYTES
  unsigned char* Uimg = smem + 2 * SLAB_A_BYTES;       // [10][128 tokens][8 e]
  __shared__ uint64_t mma_done[2];
  __shared__ uint32_t tmem_base;
  __shared__ int dead;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = blockIdx.x, c = blockIdx.y, u = blockIdx.z;
  const int token = tid & 127, half = tid >> 7;
  if (warp == 0) tmem_alloc(&tmem_base, 256);
  if (tid == 0) {
    mbar_init(&mma_done[0], 1);
    mbar_init(&mma_done[1], 1);
    mbar_fence_init();
    dead = 0;
  }
  const int i = c * CT + token;
  const __nv_bfloat16* kbase = a.k + (size_t)u * a.N * HD;
  const __nv_bfloat16* vbase = a.v + (size_t)u * a.N * VD;
  uint32_t xp[HD / 2];
  load_row_packed(xp, kbase, i, a.N);
  for (int idx = tid; idx < (EP / 8) * CT; idx += GEN_THREADS) {
    const int ec = idx >> 7, t = idx & 127, j = c * CT + t;
    reinterpret_cast<uint4*>(Uimg)[idx] = u_image_chunk(vbase + (size_t)j * VD, ec, j < a.N);
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  Waiter w{&dead};
  const uint32_t tacc = tmem_base;
  const int s0 = group_first_slab(grp), ns = group_slab_count(grp);
  const uint32_t idesc = instr_desc_bf16(128, EP, 1, 1);
  const uint32_t u_addr = smem_u32(Uimg);
  float* ds_base = a.ds + ((size_t)u * a.NB + c) * F_ROWS * EP;

  auto epilogue = [&](int it) {
    w.wait(&mma_done[it & 1], (it >> 1) & 1);
    fence_after_sync();
    if (warp >= 8) return;          // warps 0-7 cover the 128 lanes x 80 columns
    const int row = (s0 + it) * 128 + 32 * (warp & 3) + lane;
    const int col0 = warp < 4 ? 0 : 48, ncol = warp < 4 ? 48 : 32;
    const uint32_t t = tacc + (uint32_t)((it & 1) * EP) + ((uint32_t)(32 * (warp & 3)) << 16) + col0;
    for (int cc = 0; cc < ncol; cc += 16) {
      float vv[16];
      tmem_ld16(t + cc, vv);
      tmem_ld_wait();
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4)
        *reinterpret_cast<float4*>(ds_base + state_inc_offset(row, col0 + cc + 4 * q4)) =
            make_float4(vv[4 * q4], vv[4 * q4 + 1], vv[4 * q4 + 2], vv[4 * q4 + 3]);
    }
    fence_before_sync();
  };

  for (int it = 0; it < ns; ++it) {
    const int buf = it & 1;
    // A[buf] and accumulator buf were released by epilogue(it-2), which every thread has passed
    keep_in_loop(xp);
    write_half_slab_raw(s0 + it, half, xp, reinterpret_cast<uint4*>(Abuf + buf * SLAB_A_BYTES) + token);
    fence_async_smem();
    __syncthreads();
    if (tid == 0) {
      fence_after_sync();
      const uint32_t a_addr = smem_u32(Abuf + buf * SLAB_A_BYTES);
#pragma unroll
      for (int ks = 0; ks < CT / 16; ++ks)
        mma_bf16_ss(tacc + buf * EP, smem_desc(a_addr + ks * 256, 128, CT * 16),
                    smem_desc(u_addr + ks * 256, 128, CT * 16), idesc, ks > 0);
      mma_commit(&mma_done[buf]);
    }
    if (it >= 1) epilogue(it - 1);
  }
  epilogue(ns - 1);
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 256);
  if (tid == 0 && dead) atomicOr(a.status, w.status_bits());
}

// ---------------------------------------------------------------------------
// state_scan: exclusive prefix over chunks (forward) or suffix (reverse), fp32 running sum,
// result stored as the bf16 MMA operand image  [u][c][slab][e/8][128 rows][8 e].
//   thread = (feature row f, e chunk): grid (F_ROWS*10/256, units)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) state_scan_kernel(const float* ds, __nv_bfloat16* image,
                                                         const float* state_in, float* state_total, int NB,
                                                         int reverse) {
  const int x = blockIdx.x * 256 + threadIdx.x;     // 0 .. F_ROWS*10
  const int u = blockIdx.y;
  if (x >= F_ROWS * (EP / 8)) return;
  const int ec = x / F_ROWS, f = x % F_ROWS;
  const int slab = f >> 7, fr = f & 127;
  float run[8];
  if (state_in) {
    const float4* p = reinterpret_cast<const float4*>(state_in + ((size_t)u * F_ROWS + f) * EP + 8 * ec);
    const float4 a0 = p[0], a1 = p[1];
    run[0] = a0.x; run[1] = a0.y; run[2] = a0.z; run[3] = a0.w;
    run[4] = a1.x; run[5] = a1.y; run[6] = a1.z; run[7] = a1.w;
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) run[j] = 0.f;
  }
  for (int n = 0; n < NB; ++n) {
    const int c = reverse ? NB - 1 - n : n;
    const float4* p =
        reinterpret_cast<const float4*>(ds + ((size_t)u * NB + c) * F_ROWS * EP + state_inc_offset(f, 8 * ec));
    const float4 a0 = p[0], a1 = p[1];
    if (image) {
      uint4 o = make_uint4(pack_bf16(run[0], run[1]), pack_bf16(run[2], run[3]), pack_bf16(run[4], run[5]),
                           pack_bf16(run[6], run[7]));
      reinterpret_cast<uint4*>(image)[((((size_t)u * NB + c) * F_SLABS + slab) * (EP / 8) + ec) * 128 + fr] = o;
    }
    run[0] += a0.x; run[1] += a0.y; run[2] += a0.z; run[3] += a0.w;
    run[4] += a1.x; run[5] += a1.y; run[6] += a1.z; run[7] += a1.w;
  }
  if (state_total) {
    float4* p = reinterpret_cast<float4*>(state_total + ((size_t)u * F_ROWS + f) * EP + 8 * ec);
    p[0] = make_float4(run[0], run[1], run[2], run[3]);
    p[1] = make_float4(run[4], run[5], run[6], run[7]);
  }
}

// ---------------------------------------------------------------------------
// cross_read: Y[i, 0:80] = phi(i) . state_image[u, c]   (sum over all 17 slabs)
//   QUERY : phi = phi_q of head h (coefficient table with the query scale folded in), x = q, output num/den
//   !QUERY: phi = phi_k, x = k, output columns 0..63 (the value part) to out64
// ---------------------------------------------------------------------------
struct CrossReadArgs {
  const __nv_bfloat16* x;        // q [B,Hq,N,64] or k [B,Hkv,N,64]
  const __nv_bfloat16* image;    // [units, NB, 17, 10, 128, 8]
  const float* coef_table;       // [Hq, F_ROWS] (QUERY)
  float* out64;                  // [B,H,N,64]
  float* out1;                   // [B,H,N] (QUERY: denominator)
  int N, NB, H, rep;             // rep = heads per state unit (Hq/Hkv for QUERY, 1 otherwise)
  int32_t* status;
};

constexpr int CR_STAGES = 2;      // two CTAs share an SM: the other CTA hides this one's copy latency

template <bool QUERY>
__global__ void __launch_bounds__(GEN_THREADS, 2) cross_read_kernel(const CrossReadArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* Abuf = smem;                                   // 2 x SLAB_A_BYTES
  unsigned char* Sbuf = smem + 2 * SLAB_A_BYTES;                // CR_STAGES x SLAB_S_BYTES
  // per-head coefficient table, read straight from global memory (warp-uniform, L1-resident)
  const float* coef = QUERY ? a.coef_table + (size_t)blockIdx.y * F_ROWS : nullptr;
  __shared__ uint64_t full[CR_STAGES];
  __shared__ uint64_t mma_done[2];
  __shared__ uint32_t tmem_base;
  __shared__ int dead;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int token = tid & 127, half = tid >> 7;
  const int unit = (b * a.H + h) / a.rep;
  if (warp == 0) tmem_alloc(&tmem_base, 128);
  if (tid == 0) {
    for (int s = 0; s < CR_STAGES; ++s) mbar_init(&full[s], 1);
    mbar_init(&mma_done[0], 1);
    mbar_init(&mma_done[1], 1);
    mbar_fence_init();
    dead = 0;
  }
  const int i = c * CT + token;
  uint32_t xp[HD / 2];
  load_row_packed(xp, a.x + (size_t)(b * a.H + h) * a.N * HD, i, a.N);
  f32x2 xq[QUERY ? HD / 2 : 1];
  if constexpr (QUERY) unpack_row(xp, xq);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  Waiter w{&dead};
  const uint32_t tacc = tmem_base;
  const unsigned char* img = reinterpret_cast<const unsigned char*>(a.image) +
                             ((size_t)unit * a.NB + c) * F_SLABS * SLAB_S_BYTES;
  if (tid == 0) {
    for (int s = 0; s < CR_STAGES; ++s) {
      mbar_arrive_expect_tx(&full[s], SLAB_S_BYTES);
      bulk_g2s(Sbuf + s * SLAB_S_BYTES, img + (size_t)s * SLAB_S_BYTES, SLAB_S_BYTES, &full[s]);
    }
  }
  const uint32_t idesc = instr_desc_bf16(128, EP, 0, 1);
  for (int s = 0; s < F_SLABS; ++s) {
    const int buf = s & 1;
    if (s >= 2) {
      w.wait(&mma_done[buf], ((s - 2) >> 1) & 1);      // slab s-2 finished: A[buf] and its state stage are free
      if (tid == 0 && s + CR_STAGES - 2 < F_SLABS) {
        const int nxt = s + CR_STAGES - 2, st = nxt % CR_STAGES;
        mbar_arrive_expect_tx(&full[st], SLAB_S_BYTES);
        bulk_g2s(Sbuf + st * SLAB_S_BYTES, img + (size_t)nxt * SLAB_S_BYTES, SLAB_S_BYTES, &full[st]);
      }
    }
    if constexpr (QUERY) {
      keep_in_loop(xq);
      write_half_slab_coef(s, half, xq, coef, reinterpret_cast<uint4*>(Abuf + buf * SLAB_A_BYTES) + token);
    } else {
      keep_in_loop(xp);
      write_half_slab_raw(s, half, xp, reinterpret_cast<uint4*>(Abuf + buf * SLAB_A_BYTES) + token);
    }
    fence_async_smem();
    __syncthreads();
    if (tid == 0) {
      w.wait(&full[s % CR_STAGES], (s / CR_STAGES) & 1);
      fence_after_sync();
      const uint32_t a_addr = smem_u32(Abuf + buf * SLAB_A_BYTES);
      const uint32_t s_addr = smem_u32(Sbuf + (s % CR_STAGES) * SLAB_S_BYTES);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)       // 16 features per step
        mma_bf16_ss(tacc, smem_desc(a_addr + ks * 2 * CT * 16, CT * 16, 128),
                    smem_desc(s_addr + ks * 256, 128, 128 * 16), idesc, (s > 0 || ks > 0));
      mma_commit(&mma_done[buf]);
    }
  }
  w.wait(&mma_done[1], ((F_SLABS - 2) >> 1) & 1);    // slab 15
  w.wait(&mma_done[0], ((F_SLABS - 1) >> 1) & 1);    // slab 16
  fence_after_sync();
  if (warp < 8) {
    const int row = c * CT + 32 * (warp & 3) + lane;
    const int col0 = warp < 4 ? 0 : 48, ncol = warp < 4 ? 48 : 32;
    const uint32_t t = tacc + ((uint32_t)(32 * (warp & 3)) << 16) + col0;
    const size_t orow = (size_t)(b * a.H + h) * a.N + row;
    for (int cc = 0; cc < ncol; cc += 16) {
      float vv[16];
      tmem_ld16(t + cc, vv);
      tmem_ld_wait();
      if (row < a.N && !dead) {
        const int col = col0 + cc;
        if (col < VD) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4)
            *reinterpret_cast<float4*>(a.out64 + orow * VD + col + 4 * q4) =
                make_float4(vv[4 * q4], vv[4 * q4 + 1], vv[4 * q4 + 2], vv[4 * q4 + 3]);
        } else if (QUERY) {
          a.out1[orow] = vv[0];
        }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 128);
  if (tid == 0 && dead) atomicOr(a.status, w.status_bits());
}

}  // namespace

// ---------------------------------------------------------------------------
// host-side launchers
// ---------------------------------------------------------------------------
cudaError_t build_coef_table(const int32_t* dim_perm, const int32_t* group_start, const float* A,
                             const float* Bc, const float* Cc, int Hq, int G, float scale, float* table,
                             cudaStream_t st) {
  coef_table_kernel<<<Hq, 256, 0, st>>>(dim_perm, group_start, A, Bc, Cc, G, scale, table);
  return cudaGetLastError();
}

cudaError_t state_update(const void* k, const void* v, float* ds, int units, int N, int NB, int32_t* status,
                         cudaStream_t st) {
  const int smem = 2 * SLAB_A_BYTES + SLAB_S_BYTES;
  cudaError_t e = cudaFuncSetAttribute(state_update_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  StateUpdateArgs a{static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), ds, N, NB, status};
  state_update_kernel<<<dim3(SU_GROUPS, NB, units), GEN_THREADS, smem, st>>>(a);
  return cudaGetLastError();
}

cudaError_t state_scan(const float* ds, void* image, const float* state_in, float* state_total, int units,
                       int NB, int reverse, cudaStream_t st) {
  state_scan_kernel<<<dim3((F_ROWS * (EP / 8) + 255) / 256, units), 256, 0, st>>>(
      ds, static_cast<__nv_bfloat16*>(image), state_in, state_total, NB, reverse);
  return cudaGetLastError();
}

cudaError_t cross_read(bool query, const void* x, const void* image, const float* coef_table, float* out64,
                       float* out1, int B, int H, int rep, int N, int NB, int32_t* status,
                       cudaStream_t st) {
  const int smem = 2 * SLAB_A_BYTES + CR_STAGES * SLAB_S_BYTES;
  CrossReadArgs a{static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(image), coef_table,
                  out64, out1, N, NB, H, rep, status};
  cudaError_t e;
  if (query) {
    e = cudaFuncSetAttribute(cross_read_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    cross_read_kernel<true><<<dim3(NB, H, B), GEN_THREADS, smem, st>>>(a);
  } else {
    e = cudaFuncSetAttribute(cross_read_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    cross_read_kernel<false><<<dim3(NB, H, B), GEN_THREADS, smem, st>>>(a);
  }
  return cudaGetLastError();
}

size_t state_rows() { return F_ROWS; }
size_t state_image_bytes_per_chunk() { return (size_t)F_SLABS * SLAB_S_BYTES; }
size_t state_slab_image_bytes() { return SLAB_S_BYTES; }

}  // namespace oal

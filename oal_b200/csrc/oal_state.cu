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
      const uint64_t da = smem_desc(smem_u32(Abuf + buf * SLAB_A_BYTES), 128, CT * 16);
      const uint64_t du = smem_desc(u_addr, 128, CT * 16);
#pragma unroll
      for (int ks = 0; ks < CT / 16; ++ks)
        mma_bf16_ss(tacc + buf * EP, desc_advance(da, ks * 256), desc_advance(du, ks * 256), idesc, ks > 0);
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
// image_lo (optional): a second image of the rounding remainders, bf16(state - bf16(state)); the
// coefficient-gradient dot products of the backward read state = image + image_lo.
__global__ void __launch_bounds__(256) state_scan_kernel(const float* ds, __nv_bfloat16* image,
                                                         __nv_bfloat16* image_lo, const float* state_in,
                                                         float* state_total, int NB, int reverse) {
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
      const size_t at = ((((size_t)u * NB + c) * F_SLABS + slab) * (EP / 8) + ec) * 128 + fr;
      reinterpret_cast<uint4*>(image)[at] = o;
      if (image_lo) {
        const uint32_t w[4] = {o.x, o.y, o.z, o.w};
        uint32_t l[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) l[k] = pack_bf16(run[2 * k] - bf16_lo(w[k]), run[2 * k + 1] - bf16_hi(w[k]));
        reinterpret_cast<uint4*>(image_lo)[at] = make_uint4(l[0], l[1], l[2], l[3]);
      }
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
// cross_read: Y[i, 0:80] = phi(i) . state_image[u, c]   (sum over all slabs)
//   QUERY : phi = phi_q of head h (coefficient table with the query scale folded in), x = q, output num/den
//   !QUERY: phi = phi_k, x = k, output columns 0..63 (the value part) to out64
// ---------------------------------------------------------------------------
struct CrossReadArgs {
  const __nv_bfloat16* x;        // q [B,Hq,N,64] or k [B,Hkv,N,64]
  const __nv_bfloat16* image;    // [units, NB, 17, 10, 128, 8]
  const float* coef_table;       // [Hq, F_ROWS] (QUERY)
  float* out64;                  // [B,H,N,64]
  float* out1;                   // [B,H,N] (QUERY: denominator)
  int N, NB, H, rep, B;          // rep = heads per state unit (Hq/Hkv for QUERY, 1 otherwise)
  int32_t* status;
};

// Persistent, warp-specialised kernel.  Work items are (batch, head, chunk) with the heads of one
// state unit adjacent, so CTAs running at the same time read the same state image from L2.  CTA k
// takes items k, k + gridDim.x, ...; the flat iteration `it` = (item, slab) drives four roles:
//   warps 0-7   generate feature slab `slab` of the item's 128 tokens into A[it % 3]
//   warp  13    lane 0 streams the state slab images into a 4-slot ring and the head's coefficient
//               table into one of two buffers (bulk copies)
//   warp  12    lane 0 issues the MMAs  acc[item & 1] += A . S  once both are full
//   warps 8-11  after the item's last slab: accumulator -> HBM, then release it
constexpr int CR_GEN_WARPS = 8, CR_EPI_WARPS = 4;
constexpr int CR_ISSUER = CR_GEN_WARPS + CR_EPI_WARPS, CR_LOADER = CR_ISSUER + 1;
constexpr int CR_THREADS = (CR_LOADER + 1) * 32;
constexpr int CR_ARING = 3, CR_SRING = 4;
static_assert(CR_GEN_WARPS * 32 == GEN_THREADS, "the slab generator is written for GEN_THREADS threads");

struct CrItem {
  int b, h, c;
};
// item index -> (batch, head, chunk): the `rep` heads of a state unit are adjacent, then chunks
__device__ __forceinline__ CrItem cr_item(int item, int H, int rep, int NB) {
  CrItem r;
  const int hh = item % rep, t = item / rep;
  r.c = t % NB;
  const int unit = t / NB, units_per_b = H / rep;
  r.b = unit / units_per_b;
  r.h = (unit % units_per_b) * rep + hh;
  return r;
}

template <bool QUERY>
__global__ void __launch_bounds__(CR_THREADS, 1) cross_read_kernel(const CrossReadArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* Abuf = smem;                                   // CR_ARING x SLAB_A_BYTES
  unsigned char* Sbuf = smem + CR_ARING * SLAB_A_BYTES;         // CR_SRING x SLAB_S_BYTES, then the head's coefficient table
  __shared__ uint64_t full_a[CR_ARING], a_free[CR_ARING], s_full[CR_SRING], s_free[CR_SRING], acc_full[2], acc_free[2];
  __shared__ uint64_t coef_full[2], coef_free[2];
  __shared__ uint32_t tmem_base;
  __shared__ int dead;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_items = a.B * a.H * a.NB;
  const int my_items = (int)blockIdx.x < n_items ? (n_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  if (warp == CR_ISSUER) tmem_alloc(&tmem_base, 256);
  if (tid == 0) {
    for (int s = 0; s < CR_ARING; ++s) {
      mbar_init(&full_a[s], CR_GEN_WARPS);
      mbar_init(&a_free[s], 1);
    }
    for (int s = 0; s < CR_SRING; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_free[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_free[s], CR_EPI_WARPS);
      mbar_init(&coef_full[s], 1);
      mbar_init(&coef_free[s], CR_GEN_WARPS);
    }
    mbar_fence_init();
    dead = 0;
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  Waiter w{&dead};

  if (warp < CR_GEN_WARPS) {
    // ---------------- generators: thread = (token, half of the slab's chunks) ----------------
    const int token = tid & 127, half = tid >> 7;
    int s3 = 0, use = 0;
    for (int k = 0; k < my_items; ++k) {
      const CrItem it = cr_item(blockIdx.x + k * gridDim.x, a.H, a.rep, a.NB);
      // this head's coefficient table, brought in by the loader warp (two buffers)
      const float* coef = reinterpret_cast<const float*>(Sbuf + CR_SRING * SLAB_S_BYTES) + (k & 1) * F_ROWS;
      if constexpr (QUERY) w.wait(&coef_full[k & 1], (k >> 1) & 1, 0x47);
      uint32_t xp[HD / 2];
      load_row_packed(xp, a.x + (size_t)(it.b * a.H + it.h) * a.N * HD, it.c * CT + token, a.N);
      f32x2 xq[QUERY ? HD / 2 : 1];
      if constexpr (QUERY) unpack_row(xp, xq);
      for (int s = 0; s < F_SLABS; ++s) {
        if (use > 0) w.wait(&a_free[s3], (use - 1) & 1, 0x41);      // the MMAs that read A[s3] have completed
        uint4* tile = reinterpret_cast<uint4*>(Abuf + s3 * SLAB_A_BYTES) + token;
        if constexpr (QUERY) {
          keep_in_loop(xq);
          write_half_slab_coef(s, half, xq, coef, tile);
        } else {
          keep_in_loop(xp);
          write_half_slab_raw(s, half, xp, tile);
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_a[s3]);
        if (++s3 == CR_ARING) { s3 = 0; ++use; }
      }
      if constexpr (QUERY) {
        __syncwarp();
        if (lane == 0) mbar_arrive(&coef_free[k & 1]);     // this warp no longer reads the table
      }
    }
  } else if (warp < CR_ISSUER) {
    // ---------------- accumulator -> HBM ----------------
    const uint32_t lane_off = (uint32_t)(32 * (warp & 3)) << 16;
    for (int k = 0; k < my_items; ++k) {
      const CrItem it = cr_item(blockIdx.x + k * gridDim.x, a.H, a.rep, a.NB);
      const int row = it.c * CT + 32 * (warp & 3) + lane;
      const size_t orow = (size_t)(it.b * a.H + it.h) * a.N + row;
      w.wait(&acc_full[k & 1], (k >> 1) & 1, 0x42);
      fence_after_sync();
      const uint32_t t = tmem_base + (k & 1) * EP + lane_off;
#pragma unroll
      for (int cc = 0; cc < EP; cc += 16) {
        if (cc < VD || QUERY) {
          float vv[16];
          tmem_ld16(t + cc, vv);
          tmem_ld_wait();
          if (row < a.N && !dead) {
            if (cc < VD) {
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4)
                *reinterpret_cast<float4*>(a.out64 + orow * VD + cc + 4 * q4) =
                    make_float4(vv[4 * q4], vv[4 * q4 + 1], vv[4 * q4 + 2], vv[4 * q4 + 3]);
            } else if (QUERY) {
              a.out1[orow] = vv[0];
            }
          }
        }
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_free[k & 1]);
    }
  } else if (warp == CR_ISSUER) {
    // ---------------- MMA issue ----------------
    if (lane == 0) {
      const uint32_t idesc = instr_desc_bf16(128, EP, 0, 1);
      // descriptors of slot 0 of both rings, advanced by adds: this thread is the serial path of every slab
      const uint64_t da0 = smem_desc(smem_u32(Abuf), CT * 16, 128), ds0 = smem_desc(smem_u32(Sbuf), 128, 128 * 16);
      int s3 = 0, use = 0, gs = 0, guse = 0;
      for (int k = 0; k < my_items; ++k) {
        const uint32_t tacc = tmem_base + (k & 1) * EP;
        if (k >= 2) w.wait(&acc_free[k & 1], ((k >> 1) - 1) & 1, 0x43);   // item k-2 has left this accumulator
        for (int s = 0; s < F_SLABS; ++s) {
          const uint64_t da = desc_advance(da0, s3 * SLAB_A_BYTES), dsl = desc_advance(ds0, gs * SLAB_S_BYTES);
          w.wait(&full_a[s3], use & 1, 0x44);
          w.wait(&s_full[gs], guse & 1, 0x45);
          fence_after_sync();
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)       // 16 features per step
            mma_bf16_ss(tacc, desc_advance(da, ks * 2 * CT * 16), desc_advance(dsl, ks * 256), idesc, (s > 0 || ks > 0));
          mma_commit(&a_free[s3]);
          mma_commit(&s_free[gs]);
          if (s == F_SLABS - 1) mma_commit(&acc_full[k & 1]);
          if (++s3 == CR_ARING) { s3 = 0; ++use; }
          if (++gs == CR_SRING) { gs = 0; ++guse; }
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- state image stream ----------------
    if (lane == 0) {
      int gs = 0, guse = 0;
      for (int k = 0; k < my_items; ++k) {
        const CrItem it = cr_item(blockIdx.x + k * gridDim.x, a.H, a.rep, a.NB);
        const int unit = (it.b * a.H + it.h) / a.rep;
        const unsigned char* img = reinterpret_cast<const unsigned char*>(a.image) +
                                   ((size_t)unit * a.NB + it.c) * F_SLABS * SLAB_S_BYTES;
        if constexpr (QUERY) {
          if (k >= 2) w.wait(&coef_free[k & 1], ((k >> 1) - 1) & 1, 0x48);   // item k-2 no longer reads this buffer
          mbar_arrive_expect_tx(&coef_full[k & 1], F_ROWS * (uint32_t)sizeof(float));
          bulk_g2s(Sbuf + CR_SRING * SLAB_S_BYTES + (k & 1) * F_ROWS * sizeof(float),
                   a.coef_table + (size_t)it.h * F_ROWS, F_ROWS * (uint32_t)sizeof(float), &coef_full[k & 1]);
        }
        for (int s = 0; s < F_SLABS; ++s) {
          if (guse > 0) w.wait(&s_free[gs], (guse - 1) & 1, 0x46);
          mbar_arrive_expect_tx(&s_full[gs], SLAB_S_BYTES);
          bulk_g2s(Sbuf + gs * SLAB_S_BYTES, img + (size_t)s * SLAB_S_BYTES, SLAB_S_BYTES, &s_full[gs]);
          if (++gs == CR_SRING) { gs = 0; ++guse; }
        }
      }
    }
    __syncwarp();
  }
  fence_before_sync();
  __syncthreads();
  if (warp == CR_ISSUER) tmem_dealloc(tmem_base, 256);
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

cudaError_t state_scan(const float* ds, void* image, void* image_lo, const float* state_in, float* state_total,
                       int units, int NB, int reverse, cudaStream_t st) {
  state_scan_kernel<<<dim3((F_ROWS * (EP / 8) + 255) / 256, units), 256, 0, st>>>(
      ds, static_cast<__nv_bfloat16*>(image), static_cast<__nv_bfloat16*>(image_lo), state_in, state_total, NB, reverse);
  return cudaGetLastError();
}

cudaError_t cross_read(bool query, const void* x, const void* image, const float* coef_table, float* out64,
                       float* out1, int B, int H, int rep, int N, int NB, int32_t* status,
                       cudaStream_t st) {
  const int smem = CR_ARING * SLAB_A_BYTES + CR_SRING * SLAB_S_BYTES + 2 * F_ROWS * (int)sizeof(float);
  CrossReadArgs a{static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(image), coef_table,
                  out64, out1, N, NB, H, rep, B, status};
  cudaError_t e;
  int dev = 0, sms = 0;
  if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
  if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
  const int items = B * H * NB, grid = items < sms ? items : sms;
  if (query) {
    e = cudaFuncSetAttribute(cross_read_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    cross_read_kernel<true><<<grid, CR_THREADS, smem, st>>>(a);
  } else {
    e = cudaFuncSetAttribute(cross_read_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    cross_read_kernel<false><<<grid, CR_THREADS, smem, st>>>(a);
  }
  return cudaGetLastError();
}

size_t state_rows() { return F_ROWS; }
size_t state_image_bytes_per_chunk() { return (size_t)F_SLABS * SLAB_S_BYTES; }
size_t state_slab_image_bytes() { return SLAB_S_BYTES; }

}  // namespace oal

// Backward of the inter-chunk state path on the tensor cores (tcgen05 / TMEM).
//
//   dstate_heads : Z_h[u,c] = phi_raw(q_h)^T G_h per query head (raw = coefficient-free features),
//                  dCarry[u,c] = sum_h diag(coef_h) Z_h accumulated in tensor memory, and the
//                  per-feature coefficient gradient  dcoef_h[f] += sum_e carry[u,c][f,e] Z_h[f,e]
//                  (reference: oal_attention/hd_block_gemm_backward.py:764-877 dCarry with GQA sum;
//                  coefficient partial sums oal_attention/hd_block_gemm_feature_backward.py:134-474)
//   feature_grad : dphi[i, f] = A_i . state[f, :]  with A = G (query side, state = carry) or
//                  A = [v | 1] (key side, state = reverse-scanned dCarry), folded on the fly through
//                  the feature map into dq / dk
//                  (reference: hd_block_gemm_backward_wave.py:335-342 and hd_block_gemm_backward.py:911-964
//                  contractions, hd_block_gemm_feature_backward.py:59-131,157-422 folds)
// The reverse scan and the key-side phi_k . dT contraction reuse state_scan / cross_read.
#include "oal_features.cuh"
#include "oal_kernels.h"

namespace oal {
namespace {

using namespace umma;

// nine slab groups (2,...,2,1): two 80-column accumulators plus one Z buffer fit in 256 columns, so two
// CTAs share an SM and fill each other's gaps
constexpr int HGROUPS = 9;
__device__ __forceinline__ int hgroup_first(int g) { return 2 * g; }
__device__ __forceinline__ int hgroup_count(int g) { return g < 8 ? 2 : 1; }

__device__ __forceinline__ void unpack_bf16x8(const uint4 t, float (&o)[8]) {
  const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[j]);
    o[2 * j] = __low2float(h);
    o[2 * j + 1] = __high2float(h);
  }
}

// ---------------------------------------------------------------------------
// dstate_heads
// ---------------------------------------------------------------------------
struct DStateArgs {
  const __nv_bfloat16* q;          // [B,Hq,N,64]
  const __nv_bfloat16* gimg;       // [B*Hq, NB, 10, 128, 8]
  const __nv_bfloat16* carry_img;  // [units, NB, 17, 10, 128, 8] or null (no coefficient gradients)
  const float* coef_table;         // [Hq, F_ROWS]
  float* dcarry;                   // [units, NB, F_ROWS, EP]
  float* dcoef_partial;            // [B, NB, Hq, F_ROWS] or null
  int N, NB, Hq, Hkv;
  float scale;
  int32_t* status;
};

__global__ void __launch_bounds__(GEN_THREADS, 2) dstate_heads_kernel(const DStateArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* Abuf = smem;                        // 2 x SLAB_A_BYTES
  unsigned char* Gbuf = smem + 2 * SLAB_A_BYTES;     // 2 x SLAB_S_BYTES  ([10][128 tokens][8 e])
  __shared__ uint64_t mma_done[2], gfull[2];
  __shared__ uint32_t tmem_base;
  __shared__ int dead;
  __shared__ float dsum[2][2][128];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = blockIdx.x, c = blockIdx.y, u = blockIdx.z;
  const int b = u / a.Hkv, kvh = u % a.Hkv, rep = a.Hq / a.Hkv;
  const int token = tid & 127, half = tid >> 7, wg = warp >> 2;
  if (warp == 0) tmem_alloc(&tmem_base, 256);
  if (tid == 0) {
    mbar_init(&mma_done[0], 1);
    mbar_init(&mma_done[1], 1);
    mbar_init(&gfull[0], 1);
    mbar_init(&gfull[1], 1);
    mbar_fence_init();
    dead = 0;
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  Waiter w{&dead};
  const int s0 = hgroup_first(grp), ns = hgroup_count(grp);
  const uint32_t tacc = tmem_base;                 // ns x 80 columns
  const uint32_t tz = tmem_base + 160;             // 80 columns
  const uint32_t lane_off = (uint32_t)(32 * (warp & 3)) << 16;
  const uint32_t idesc = instr_desc_bf16(128, EP, 1, 1);
  const int fr = 32 * (warp & 3) + lane;
  const int col0 = wg == 0 ? 0 : 48, ncol = wg == 0 ? 48 : 32;
  const size_t g_stride = (size_t)a.NB * SLAB_S_BYTES;   // bytes per (b,h) in gimg
  auto gimg_ptr = [&](int h) {
    return reinterpret_cast<const unsigned char*>(a.gimg) + (size_t)(b * a.Hq + h) * g_stride + (size_t)c * SLAB_S_BYTES;
  };
  if (tid == 0) {
    mbar_arrive_expect_tx(&gfull[0], SLAB_S_BYTES);
    bulk_g2s(Gbuf, gimg_ptr(kvh * rep), SLAB_S_BYTES, &gfull[0]);
  }
  const unsigned char* carry_base =
      a.carry_img ? reinterpret_cast<const unsigned char*>(a.carry_img) + ((size_t)u * a.NB + c) * F_SLABS * SLAB_S_BYTES
                  : nullptr;

  // epilogue of flattened iteration m = head_index * ns + slab_index
  auto epilogue = [&](int m) {
    const int hm = m / ns, im = m - hm * ns, h = kvh * rep + hm;
    w.wait(&mma_done[m & 1], (m >> 1) & 1);
    fence_after_sync();
    const int f = (s0 + im) * 128 + fr;
    if (warp < 8) {                 // warps 0-7 cover the 128 lanes x 80 columns
      const float cf = a.coef_table[(size_t)h * F_ROWS + f];
      float dot = 0.f;
      for (int cc = 0; cc < ncol; cc += 16) {
        float z[16];
        tmem_ld16(tz + lane_off + col0 + cc, z);
        float acc[16];
        if (hm > 0) tmem_ld16(tacc + im * EP + lane_off + col0 + cc, acc);
        tmem_ld_wait();
        if (carry_base) {
          const uint4* cp = reinterpret_cast<const uint4*>(carry_base + (size_t)(s0 + im) * SLAB_S_BYTES);
          const int ec = (col0 + cc) >> 3;
          float c0[8], c1[8];
          unpack_bf16x8(cp[ec * 128 + fr], c0);
          unpack_bf16x8(cp[(ec + 1) * 128 + fr], c1);
#pragma unroll
          for (int j = 0; j < 8; ++j) dot = fmaf(z[j], c0[j], fmaf(z[8 + j], c1[j], dot));
        }
        uint32_t o[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(hm > 0 ? fmaf(cf, z[j], acc[j]) : cf * z[j]);
        tmem_st16(tacc + im * EP + lane_off + col0 + cc, o);
      }
      tmem_st_wait();
      if (a.dcoef_partial) dsum[m & 1][wg][fr] = dot;
    }
    if (a.dcoef_partial) {
      __syncthreads();
      if (warp < 4)
        a.dcoef_partial[(((size_t)b * a.NB + c) * a.Hq + h) * F_ROWS + f] = dsum[m & 1][0][fr] + dsum[m & 1][1][fr];
    }
    fence_before_sync();
  };

  int n = 0;
  for (int hh = 0; hh < rep; ++hh) {
    const int h = kvh * rep + hh;
    float x[HD];
    load_row_bf16(x, a.q + (size_t)(b * a.Hq + h) * a.N * HD, c * CT + token, a.N, a.scale);
    for (int it = 0; it < ns; ++it, ++n) {
      const int buf = n & 1;
      write_half_slab<false>(s0 + it, half, x, nullptr, reinterpret_cast<uint4*>(Abuf + buf * SLAB_A_BYTES), token);
      // the single Z buffer must be drained before the next MMA is issued
      if (n >= 1) epilogue(n - 1);
      // every MMA of the previous head has completed: its G buffer can take the next head's image
      if (it == 0 && tid == 0 && hh + 1 < rep) {
        mbar_arrive_expect_tx(&gfull[(hh + 1) & 1], SLAB_S_BYTES);
        bulk_g2s(Gbuf + ((hh + 1) & 1) * SLAB_S_BYTES, gimg_ptr(h + 1), SLAB_S_BYTES, &gfull[(hh + 1) & 1]);
      }
      fence_async_smem();
      __syncthreads();
      if (tid == 0) {
        if (it == 0) w.wait(&gfull[hh & 1], (hh >> 1) & 1);
        fence_after_sync();
        const uint32_t a_addr = smem_u32(Abuf + buf * SLAB_A_BYTES);
        const uint32_t g_addr = smem_u32(Gbuf + (hh & 1) * SLAB_S_BYTES);
#pragma unroll
        for (int ks = 0; ks < CT / 16; ++ks)
          mma_bf16_ss(tz, smem_desc(a_addr + ks * 256, 128, CT * 16), smem_desc(g_addr + ks * 256, 128, CT * 16),
                      idesc, ks > 0);
        mma_commit(&mma_done[buf]);
      }
    }
  }
  epilogue(n - 1);
  fence_after_sync();
  // dCarry rows of this slab group: tensor memory -> HBM
  float* dbase = a.dcarry + ((size_t)u * a.NB + c) * F_ROWS * EP;
  for (int it = 0; it < ns && warp < 8; ++it) {
    float* dst = dbase + (size_t)((s0 + it) * 128 + fr) * EP + col0;
    for (int cc = 0; cc < ncol; cc += 16) {
      float vv[16];
      tmem_ld16(tacc + it * EP + lane_off + col0 + cc, vv);
      tmem_ld_wait();
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4)
        *reinterpret_cast<float4*>(dst + cc + 4 * q4) =
            make_float4(vv[4 * q4], vv[4 * q4 + 1], vv[4 * q4 + 2], vv[4 * q4 + 3]);
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 256);
  if (tid == 0 && dead) atomicOr(a.status, w.status_bits());
}

// ---------------------------------------------------------------------------
// fold of one 16-column load (two chunks of 8 features) of dphi into dx
// ---------------------------------------------------------------------------
template <int CH, bool QUERY, int OFF>
__device__ __forceinline__ void fold_chunk(const float (&v)[16], const float (&x)[HD], const float* coef,
                                           float (&dx)[HD]) {
  if constexpr (CH < F_CONST_CHUNK) {
    float t[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) t[j] = v[OFF + j];
    if constexpr (QUERY) {
      const float4 c0 = *reinterpret_cast<const float4*>(coef + 8 * CH);
      const float4 c1 = *reinterpret_cast<const float4*>(coef + 8 * CH + 4);
      t[0] *= c0.x; t[1] *= c0.y; t[2] *= c0.z; t[3] *= c0.w;
      t[4] *= c1.x; t[5] *= c1.y; t[6] *= c1.z; t[7] *= c1.w;
    }
    if constexpr (CH < F_PAIR_CHUNKS) {
      constexpr RC p0 = pair_rc(8 * CH + 0), p1 = pair_rc(8 * CH + 1), p2 = pair_rc(8 * CH + 2),
                   p3 = pair_rc(8 * CH + 3), p4 = pair_rc(8 * CH + 4), p5 = pair_rc(8 * CH + 5),
                   p6 = pair_rc(8 * CH + 6), p7 = pair_rc(8 * CH + 7);
#define OAL_FOLD(P, J)                         \
  dx[P.r] = fmaf(t[J], x[P.c], dx[P.r]);       \
  dx[P.c] = fmaf(t[J], x[P.r], dx[P.c]);
      OAL_FOLD(p0, 0) OAL_FOLD(p1, 1) OAL_FOLD(p2, 2) OAL_FOLD(p3, 3)
      OAL_FOLD(p4, 4) OAL_FOLD(p5, 5) OAL_FOLD(p6, 6) OAL_FOLD(p7, 7)
#undef OAL_FOLD
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) dx[8 * (CH - F_LIN_CHUNK0) + j] += t[j];
    }
  }
}

template <int S, int HALF, bool QUERY, int Q>
__device__ __forceinline__ void fold_quarter(uint32_t taddr, const float (&x)[HD], const float* coef,
                                             float (&dx)[HD]) {
  float v[16];
  tmem_ld16(taddr + HALF * 64 + 16 * Q, v);
  tmem_ld_wait();
  fold_chunk<S * 16 + HALF * 8 + 2 * Q, QUERY, 0>(v, x, coef, dx);
  fold_chunk<S * 16 + HALF * 8 + 2 * Q + 1, QUERY, 8>(v, x, coef, dx);
}

template <int S, int HALF, bool QUERY>
__device__ __forceinline__ void fold_half_slab_impl(uint32_t taddr, const float (&x)[HD], const float* coef,
                                                    float (&dx)[HD]) {
  fold_quarter<S, HALF, QUERY, 0>(taddr, x, coef, dx);
  fold_quarter<S, HALF, QUERY, 1>(taddr, x, coef, dx);
  fold_quarter<S, HALF, QUERY, 2>(taddr, x, coef, dx);
  fold_quarter<S, HALF, QUERY, 3>(taddr, x, coef, dx);
}

template <bool QUERY>
__device__ __forceinline__ void fold_half_slab(int s, int half, uint32_t taddr, const float (&x)[HD],
                                               const float* coef, float (&dx)[HD]) {
#define OAL_FOLD_CASE(S)                                                               \
  case S:                                                                              \
    if (half == 0) fold_half_slab_impl<S, 0, QUERY>(taddr, x, coef, dx);               \
    else fold_half_slab_impl<S, 1, QUERY>(taddr, x, coef, dx);                         \
    break;
  switch (s) {
    OAL_FOLD_CASE(0) OAL_FOLD_CASE(1) OAL_FOLD_CASE(2) OAL_FOLD_CASE(3) OAL_FOLD_CASE(4) OAL_FOLD_CASE(5)
    OAL_FOLD_CASE(6) OAL_FOLD_CASE(7) OAL_FOLD_CASE(8) OAL_FOLD_CASE(9) OAL_FOLD_CASE(10) OAL_FOLD_CASE(11)
    OAL_FOLD_CASE(12) OAL_FOLD_CASE(13) OAL_FOLD_CASE(14) OAL_FOLD_CASE(15) OAL_FOLD_CASE(16)
    default: break;
  }
#undef OAL_FOLD_CASE
}

// ---------------------------------------------------------------------------
// feature_grad
//   grid (chunks, heads, batch); 256 threads; thread = (token, half of the slab's features)
// ---------------------------------------------------------------------------
struct FeatGradArgs {
  const __nv_bfloat16* x;        // q [B,Hq,N,64] (QUERY) or k [B,Hkv,N,64]
  const __nv_bfloat16* gimg;     // QUERY: A-operand image of G  [B*Hq, NB, 10, 128, 8]
  const __nv_bfloat16* v;        // KEY: values, the A operand [v | 1] is built in shared memory
  const __nv_bfloat16* image;    // state image [units, NB, 17, 10, 128, 8]: carry (QUERY) / dT (KEY)
  const float* coef_table;       // QUERY
  float* dx;                     // [B,H,N,64] fp32
  int N, NB, H, rep;
  float mul, outmul;
  int32_t* status;
};

constexpr int FG_STAGES = 4;

template <bool QUERY>
__global__ void __launch_bounds__(256, 1) feature_grad_kernel(const FeatGradArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* Aimg = smem;                                        // SLAB_S_BYTES: [10][128 tokens][8 e]
  unsigned char* Sbuf = smem + SLAB_S_BYTES;                         // FG_STAGES x SLAB_S_BYTES
  float* coef = reinterpret_cast<float*>(Sbuf + FG_STAGES * SLAB_S_BYTES);   // F_ROWS
  float* red = coef + F_ROWS;                                        // [128][65]
  __shared__ uint64_t full[FG_STAGES], mma_done[2], afull;
  __shared__ uint32_t tmem_base;
  __shared__ int dead;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int wg = warp >> 2, token = 32 * (warp & 3) + lane;
  const int unit = (b * a.H + h) / a.rep;
  if (warp == 0) tmem_alloc(&tmem_base, 256);
  if (tid == 0) {
    for (int s = 0; s < FG_STAGES; ++s) mbar_init(&full[s], 1);
    mbar_init(&mma_done[0], 1);
    mbar_init(&mma_done[1], 1);
    mbar_init(&afull, 1);
    mbar_fence_init();
    dead = 0;
  }
  if (QUERY)
    for (int f = tid; f < F_ROWS; f += 256) coef[f] = a.coef_table[(size_t)h * F_ROWS + f];
  const int i = c * CT + token;
  const size_t head_off = (size_t)(b * a.H + h) * a.N;
  float x[HD], dx[HD];
  load_row_bf16(x, a.x + head_off * HD, i, a.N, a.mul);
#pragma unroll
  for (int d = 0; d < HD; ++d) dx[d] = 0.f;
  if (!QUERY) {
    for (int idx = tid; idx < (EP / 8) * CT; idx += 256) {
      const int ec = idx >> 7, t = idx & 127, j = c * CT + t;
      reinterpret_cast<uint4*>(Aimg)[idx] = u_image_chunk(a.v + (head_off + j) * VD, ec, j < a.N);
    }
    fence_async_smem();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  Waiter w{&dead};
  const unsigned char* img = reinterpret_cast<const unsigned char*>(a.image) +
                             ((size_t)unit * a.NB + c) * F_SLABS * SLAB_S_BYTES;
  if (tid == 0) {
    if (QUERY) {
      mbar_arrive_expect_tx(&afull, SLAB_S_BYTES);
      bulk_g2s(Aimg, reinterpret_cast<const unsigned char*>(a.gimg) + ((size_t)(b * a.H + h) * a.NB + c) * SLAB_S_BYTES,
               SLAB_S_BYTES, &afull);
    }
    for (int s = 0; s < FG_STAGES; ++s) {
      mbar_arrive_expect_tx(&full[s], SLAB_S_BYTES);
      bulk_g2s(Sbuf + s * SLAB_S_BYTES, img + (size_t)s * SLAB_S_BYTES, SLAB_S_BYTES, &full[s]);
    }
  }
  const uint32_t idesc = instr_desc_bf16(128, 128, 0, 0);
  const uint32_t lane_off = (uint32_t)(32 * (warp & 3)) << 16;
  const uint32_t a_addr = smem_u32(Aimg);

#define OAL_FOLD_SLAB(S_)                                                                   \
  do {                                                                                      \
    const int fs_ = (S_);                                                                   \
    w.wait(&mma_done[fs_ & 1], (fs_ >> 1) & 1);                                             \
    fence_after_sync();                                                                     \
    fold_half_slab<QUERY>(fs_, wg, tmem_base + (fs_ & 1) * 128 + lane_off, x, coef, dx);    \
    fence_before_sync();                                                                    \
  } while (0)

  for (int s = 0; s < F_SLABS; ++s) {
    __syncthreads();      // fold(s-2) is finished by every thread: accumulator s&1 may be overwritten
    if (tid == 0) {
      if (QUERY && s == 0) w.wait(&afull, 0);
      w.wait(&full[s % FG_STAGES], (s / FG_STAGES) & 1);
      fence_after_sync();
      const uint32_t s_addr = smem_u32(Sbuf + (s % FG_STAGES) * SLAB_S_BYTES);
#pragma unroll
      for (int ks = 0; ks < EP / 16; ++ks)
        mma_bf16_ss(tmem_base + (s & 1) * 128, smem_desc(a_addr + ks * 2 * CT * 16, CT * 16, 128),
                    smem_desc(s_addr + ks * 2 * 128 * 16, 128 * 16, 128), idesc, ks > 0);
      mma_commit(&mma_done[s & 1]);
    }
    if (s >= 1) {
      OAL_FOLD_SLAB(s - 1);
      // slab s-1 has been consumed by the tensor core: refill its stage
      if (tid == 0 && s + 3 < F_SLABS) {
        const int st = (s + 3) % FG_STAGES;
        mbar_arrive_expect_tx(&full[st], SLAB_S_BYTES);
        bulk_g2s(Sbuf + st * SLAB_S_BYTES, img + (size_t)(s + 3) * SLAB_S_BYTES, SLAB_S_BYTES, &full[st]);
      }
    }
  }
  OAL_FOLD_SLAB(F_SLABS - 1);
#undef OAL_FOLD_SLAB
  // combine the two halves of every token and write
  if (wg == 1) {
#pragma unroll
    for (int d = 0; d < HD; ++d) red[token * 65 + d] = dx[d];
  }
  __syncthreads();
  if (wg == 0 && i < a.N && !dead) {
    float* dst = a.dx + (head_off + i) * HD;
#pragma unroll
    for (int d4 = 0; d4 < HD; d4 += 4)
      *reinterpret_cast<float4*>(dst + d4) = make_float4(a.outmul * (dx[d4] + red[token * 65 + d4]),
                                                          a.outmul * (dx[d4 + 1] + red[token * 65 + d4 + 1]),
                                                          a.outmul * (dx[d4 + 2] + red[token * 65 + d4 + 2]),
                                                          a.outmul * (dx[d4 + 3] + red[token * 65 + d4 + 3]));
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 256);
  if (tid == 0 && dead) atomicOr(a.status, w.status_bits());
}

// ---------------------------------------------------------------------------
// coefficient gradients of the cross-chunk term: per-feature sums -> (A, B_g, C_gg') slots
// ---------------------------------------------------------------------------
__global__ void dcoef_sum_kernel(const float* partial, int outer /* B*NB */, int Hq, float* dcoef) {
  const int f = blockIdx.x * blockDim.x + threadIdx.x, h = blockIdx.y;
  if (f >= F_ROWS) return;
  float t = 0.f;
  for (int o = 0; o < outer; ++o) t += partial[((size_t)o * Hq + h) * F_ROWS + f];
  dcoef[(size_t)h * F_ROWS + f] = t;
}

__device__ __forceinline__ int tri_slot(int g, int g2) { return g * GMAX - (g * (g - 1)) / 2 + (g2 - g); }

__global__ void dcoef_slots_kernel(const float* dcoef, const int32_t* dim_perm, const int32_t* group_start,
                                   float* slots /* [Hq][NCOEF] */) {
  __shared__ int gdim[HD];
  __shared__ short fslot[F_ROWS];
  __shared__ float fval[F_ROWS];
  const int h = blockIdx.x;
  if (threadIdx.x < HD) {
    const int p = threadIdx.x;
    int g = 0;
    while (g < GMAX - 1 && p >= group_start[h * (GMAX + 1) + g + 1]) ++g;
    gdim[dim_perm[h * HD + p]] = g;
  }
  __syncthreads();
  for (int f = threadIdx.x; f < F_ROWS; f += blockDim.x) {
    int slot = -1;
    float wgt = 1.f;
    if (f < F_PAIR_CHUNKS * 8) {
      int r = (int)((sqrtf(8.f * f + 1.f) - 1.f) * 0.5f);
      while ((r + 1) * (r + 2) / 2 <= f) ++r;
      while (r * (r + 1) / 2 > f) --r;
      const int cdim = f - r * (r + 1) / 2;
      const int ga = min(gdim[r], gdim[cdim]), gb = max(gdim[r], gdim[cdim]);
      slot = 1 + GMAX + tri_slot(ga, gb);
      wgt = (ga == gb && r != cdim) ? 2.f : 1.f;
    } else if (f < F_CONST_CHUNK * 8) {
      slot = 1 + gdim[f - F_LIN_CHUNK0 * 8];
    } else if (f == F_CONST_CHUNK * 8) {
      slot = 0;
    }
    fslot[f] = (short)slot;
    fval[f] = slot >= 0 ? wgt * dcoef[(size_t)h * F_ROWS + f] : 0.f;
  }
  __syncthreads();
  for (int s = threadIdx.x; s < NCOEF; s += blockDim.x) {
    float t = 0.f;
    for (int f = 0; f < F_ROWS; ++f)
      if (fslot[f] == s) t += fval[f];
    slots[(size_t)h * NCOEF + s] = t;
  }
}

// normalisation VJP writing, besides the fp32 rows, the bf16 operand image of G
//   rows are enumerated over padded chunks so that tail tokens of the last chunk are zeroed
__global__ void __launch_bounds__(256) norm_vjp_image_kernel(const void* grad_out, int out_dt, const float* grad_num,
                                                             const float* grad_den, const float* num,
                                                             const float* den, float floor_v, float* g,
                                                             __nv_bfloat16* gimg, int N, int NB, int heads) {
  const size_t r = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const size_t per_head = (size_t)NB * CT;
  if (r >= per_head * heads) return;
  const size_t bh = r / per_head;
  const int t = (int)(r % per_head);
  const int cidx = t / CT, tl = t % CT;
  float gv[2] = {0.f, 0.f}, gd = 0.f;
  if (t < N) {
    const size_t row = bh * N + t;
    const float dn = den[row];
    const float dw = fmaxf(dn, floor_v);
    float dot = 0.f;
    if (grad_out) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const float go = load_elem(grad_out, row * VD + lane + 32 * c, out_dt);
        dot = fmaf(go, num[row * VD + lane + 32 * c], dot);
        gv[c] = go / dw;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      if (grad_num) gv[c] += grad_num[row * VD + lane + 32 * c];
      g[row * EP + lane + 32 * c] = gv[c];
    }
    if (grad_out) gd = (dn >= floor_v) ? -(dot / dw) / dw : 0.f;
    if (grad_den) gd += grad_den[row];
    if (lane < EP - VD) g[row * EP + VD + lane] = lane == 0 ? gd : 0.f;
  }
  // hi image = bf16(g); lo image = bf16(g - hi): dW = g . [v|1] is formed from both, because its two
  // large terms (dout.v / den and dout.num / den^2) nearly cancel
  __nv_bfloat16* img = gimg + (bh * NB + cidx) * (size_t)(SLAB_S_BYTES / 2);
  __nv_bfloat16* img_lo = img + (size_t)heads * NB * (SLAB_S_BYTES / 2);
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const int e = lane + 32 * c;
    const __nv_bfloat16 hi = __float2bfloat16_rn(gv[c]);
    img[((e >> 3) * CT + tl) * 8 + (e & 7)] = hi;
    img_lo[((e >> 3) * CT + tl) * 8 + (e & 7)] = __float2bfloat16_rn(gv[c] - __bfloat162float(hi));
  }
  if (lane < EP - VD) {
    const int e = VD + lane;
    const float val = lane == 0 ? gd : 0.f;
    const __nv_bfloat16 hi = __float2bfloat16_rn(val);
    img[((e >> 3) * CT + tl) * 8 + (e & 7)] = hi;
    img_lo[((e >> 3) * CT + tl) * 8 + (e & 7)] = __float2bfloat16_rn(val - __bfloat162float(hi));
  }
}

}  // namespace

cudaError_t dstate_heads(const void* q, const void* gimg, const void* carry_img, const float* coef_table,
                         float* dcarry, float* dcoef_partial, int B, int Hq, int Hkv, int N, int NB, float scale,
                         int32_t* status, cudaStream_t st) {
  const int smem = 2 * SLAB_A_BYTES + 2 * SLAB_S_BYTES;
  cudaError_t e = cudaFuncSetAttribute(dstate_heads_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  DStateArgs a{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(gimg),
               static_cast<const __nv_bfloat16*>(carry_img), coef_table, dcarry, dcoef_partial, N, NB, Hq, Hkv,
               scale, status};
  dstate_heads_kernel<<<dim3(HGROUPS, NB, B * Hkv), GEN_THREADS, smem, st>>>(a);
  return cudaGetLastError();
}

cudaError_t feature_grad(bool query, const void* x, const void* gimg, const void* v, const void* image,
                         const float* coef_table, float* dx, int B, int H, int rep, int N, int NB, float mul,
                         float outmul, int32_t* status, cudaStream_t st) {
  const int smem = SLAB_S_BYTES + FG_STAGES * SLAB_S_BYTES + F_ROWS * (int)sizeof(float) + 128 * 65 * (int)sizeof(float);
  FeatGradArgs a{static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(gimg),
                 static_cast<const __nv_bfloat16*>(v), static_cast<const __nv_bfloat16*>(image), coef_table, dx,
                 N, NB, H, rep, mul, outmul, status};
  cudaError_t e;
  if (query) {
    e = cudaFuncSetAttribute(feature_grad_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    feature_grad_kernel<true><<<dim3(NB, H, B), 256, smem, st>>>(a);
  } else {
    e = cudaFuncSetAttribute(feature_grad_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    feature_grad_kernel<false><<<dim3(NB, H, B), 256, smem, st>>>(a);
  }
  return cudaGetLastError();
}

cudaError_t dcoef_reduce(const float* partial, int outer, int Hq, const int32_t* dim_perm,
                         const int32_t* group_start, float* dcoef, float* slots, cudaStream_t st) {
  dcoef_sum_kernel<<<dim3((F_ROWS + 255) / 256, Hq), 256, 0, st>>>(partial, outer, Hq, dcoef);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  dcoef_slots_kernel<<<Hq, 256, 0, st>>>(dcoef, dim_perm, group_start, slots);
  return cudaGetLastError();
}

cudaError_t norm_vjp_image(const void* grad_out, int out_dt, const float* grad_num, const float* grad_den,
                           const float* num, const float* den, float floor_v, float* g, void* gimg, int heads,
                           int N, int NB, cudaStream_t st) {
  const size_t rows = (size_t)heads * NB * CT;
  norm_vjp_image_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(grad_out, out_dt, grad_num, grad_den, num, den,
                                                                   floor_v, g, static_cast<__nv_bfloat16*>(gimg), N,
                                                                   NB, heads);
  return cudaGetLastError();
}

}  // namespace oal

// Intra-chunk term of the chunked scan on the tensor cores (tcgen05 / TMEM), backward.
//
// Query side, per 16-key tile of a 128-token chunk (rows are queries):
//   U  = Q . stack(K)^T,  dW = G [v|1]^T (whole chunk, G as hi + lo bf16)      MMAs into tensor memory
//   P_r = 2 sgn_r dW u_r  (bf16 tile),  D[r][r'] += 2 dW u_r u_r'               registers
//     (here the stack is carried as bf16 value + bf16 remainder, two MMA chains: the coefficient
//      gradient is a sum of strongly cancelling terms -- sum_j dW_ij w_ij = 0 for every row -- and
//      needs u to more than 8 bits; sum dW and sum dW u_r are accumulated on their own for dA, dB)
//   dq += P . stack(K)                                                           MMA, K = 16 R
// Key / value side (rows are keys, 16 queries per tile): the same with q and k exchanged,
//   dk += P^T-tile . stack(Q),  dU += W^T G   with W = sum_r sgn_r u_r^2,
// per query head into fp32 partials that kv_head_reduce_kernel sums over the heads of a KV head in
// fixed order.  The stacked scaled tile (oal_intra.cuh) is rebuilt per tile in a three-slot ring by
// the warps themselves; lane 0 of one compute warp (the one whose rows the causal mask idles most) also issues
// every MMA, between that warp's own steps, driven by warp-granular mbarrier arrivals.  The cross-chunk parts computed by the state kernels arrive as fp32 buffers and are added
// before the final cast.  Reference stages replaced: oal_attention/hd_block_gemm_backward_wave.py:253-476
// (dS, local dphi_q / dphi_k / dU GEMMs) and the folds / coefficient partials of
// oal_attention/hd_block_gemm_feature_backward.py:59-474.
#include "oal_intra.cuh"
#include "oal_kernels.h"

namespace oal {
namespace {

using namespace umma;

struct IntraBwdArgs {
  const __nv_bfloat16 *q, *k, *v;
  const __nv_bfloat16* gimg;        // [2][B*Hq, NB, 10, 128, 8]: bf16(g) image, then the image of g - bf16(g)
  size_t gimg_lo_offset;            // bytes from the hi image to the lo image
  const HeadFactor* factors;
  void* dq;                         // io dtype (bf16), may be null
  const float* dq_init;             // fp32 cross part, or null
  float* dk_part;                   // fp32 [B,Hq,N,64]: this query head's intra-chunk share of dk
  float* dv_part;                   // fp32 [B,Hq,N,64]: this query head's intra-chunk share of dv
  float* coef_partial;              // [B][Hq][NB][NQ] or null: D upper triangle, sum t_r, sum 2 dW
  int32_t* status;
  int N, NB, Hq, Hkv;
};

constexpr int STAGE_OUT_FLOATS = CT * 65 + 3;   // one [128][65] fp32 output staging tile (padded to 16 bytes)

// the G images (hi, lo) of one (batch row, query head, chunk): two bulk copies on one barrier
__device__ __forceinline__ void fetch_g_images(const IntraBwdArgs& a, unsigned char* ghi, unsigned char* glo,
                                               uint64_t* bar, int b, int h, int c) {
  const size_t item = (size_t)(b * a.Hq + h) * a.NB + c;
  const unsigned char* gsrc = reinterpret_cast<const unsigned char*>(a.gimg) + item * SLAB_S_BYTES;
  mbar_arrive_expect_tx(bar, 2 * SLAB_S_BYTES);
  bulk_g2s(ghi, gsrc, SLAB_S_BYTES, bar);
  bulk_g2s(glo, gsrc + a.gimg_lo_offset, SLAB_S_BYTES, bar);
}

// ---------------------------------------------------------------------------
// query side
// ---------------------------------------------------------------------------
// shared memory: Qa | Kimg | 3 stacks | 2 remainder stacks | G hi, G lo, U (dead once dW is complete)
// tensor memory: U (16 R columns) | dW (128) | dq (64) | two P tiles (8 R columns each)
constexpr int BQ_SMEM = XA_BYTES + X_BYTES + 3 * ST_BYTES + 2 * STLO_BYTES + 3 * SLAB_S_BYTES;
constexpr int NQ = NU + RM + 1;                 // partial sums per CTA: D (upper triangle), sum t_r, sum 2 dW
static_assert(RM * KT + CT + HD + 2 * P_COLS <= 512, "tensor-memory columns of the query-side kernel");
static_assert(CT * 65 * 4 <= XA_BYTES + X_BYTES + 3 * ST_BYTES, "dq staging tile");


__global__ void __launch_bounds__(CTHREADS, 1) intra_bwd_q_kernel(const IntraBwdArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* Qa = smem;
  unsigned char* Kimg = Qa + XA_BYTES;
  unsigned char* St = Kimg + X_BYTES;                     // 3 x ST_BYTES
  unsigned char* Lo = St + 3 * ST_BYTES;                  // 2 x STLO_BYTES
  unsigned char* Gimg = Lo + 2 * STLO_BYTES;              // hi, lo
  unsigned char* Uimg = Gimg + 2 * SLAB_S_BYTES;
  __shared__ HeadFactorS hf;
  __shared__ uint64_t gfull, dw_done, u_done, u_free, p_ready[2], p_done[2], st_ready[3];
  __shared__ uint32_t tmem_base;
  __shared__ int dead;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (a.Hq / a.Hkv);
  const int half = (warp >> 2) & 1, row = 32 * (warp & 3) + lane;
  const bool issuer = warp == 0;
  if (warp == 0) tmem_alloc(&tmem_base, 512);
  if (tid == 0) {
    mbar_init(&gfull, 1);
    mbar_init(&dw_done, 1);
    mbar_init(&u_done, 1);
    mbar_init(&u_free, CWARPS);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&p_ready[s], CWARPS);
      mbar_init(&p_done[s], 1);
    }
    for (int s = 0; s < 3; ++s) mbar_init(&st_ready[s], CWARPS);
    mbar_fence_init();
    dead = 0;
  }
  __syncthreads();
  if (tid == 0) fetch_g_images(a, Gimg, Gimg + SLAB_S_BYTES, &gfull, b, h, c);
  const size_t qoff = (size_t)(b * a.Hq + h) * a.N, koff = (size_t)(b * a.Hkv + kvh) * a.N;
  load_head_factor(hf, a.factors, h, tid, CTHREADS);
  load_operand_image(Qa, a.q + qoff * HD, c * CT, a.N, true, tid, CTHREADS);
  load_operand_image(Kimg, a.k + koff * HD, c * CT, a.N, false, tid, CTHREADS);
  load_u_image(Uimg, a.v + koff * VD, c * CT, a.N, tid, CTHREADS);
  async_copies_wait();
  __syncthreads();
  const int tiles = min(CT / KT, (a.N - c * CT + KT - 1) / KT);
  const int rank = hf.rank, rpos = hf.rpos;
  for (int s = 0; s < 3; ++s) init_stack_constants(St + s * ST_BYTES, hf, tid, CTHREADS);
  if ((tid >> 7) < tiles)
    build_stack_piece(St + (tid >> 7) * ST_BYTES, Kimg, (tid >> 7) * KT, hf, tid & 127, Lo + (tid >> 7) * STLO_BYTES);
  fence_async_smem();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  Waiter w{&dead};
  const uint32_t tU = tmem_base, tW = tmem_base + RM * KT, tQ = tW + CT, tP = tQ + HD;
  const uint32_t lane_off = (uint32_t)(32 * (warp & 3)) << 16;
  f32x2 D2[NU], N2[RM], S2 = 0ull;
#pragma unroll
  for (int x = 0; x < NU; ++x) D2[x] = 0ull;
#pragma unroll
  for (int x = 0; x < RM; ++x) N2[x] = 0ull;

  const uint32_t q_addr = smem_u32(Qa), st_addr = smem_u32(St), lo_addr = smem_u32(Lo);
  if (issuer) {
    if (lane == 0) {
      w.wait(&gfull, 0, 0x20);
      fence_after_sync();
      issue_dw(tW, smem_u32(Gimg), true, smem_u32(Uimg), false);
      mma_commit(&dw_done);
      issue_stack_scores(tU, q_addr, st_addr, rank, lo_addr);
      mma_commit(&u_done);
    }
    __syncwarp();
  }
  w.wait(&dw_done, 0, 0x24);
  for (int kt = 0; kt < tiles; ++kt) {
    const int buf = kt & 1;
    const bool warp_active = 32 * (warp & 3) + 31 >= kt * KT;
    float u[RM][8], dw[8];
    w.wait(&u_done, kt & 1, 0x25);
    fence_after_sync();
    if (warp_active) {
#pragma unroll
      for (int r = 0; r < RM; ++r)
        if (r < rank) tmem_ld8(tU + lane_off + r * KT + 8 * half, u[r]);
      tmem_ld8(tW + lane_off + kt * KT + 8 * half, dw);
      tmem_ld_wait();
    }
    fence_before_sync();
    warp_arrive(&u_free, lane);
    if (issuer && kt + 1 < tiles) {
      if (lane == 0) {
        w.wait(&u_free, kt & 1, 0x21);                 // every warp holds U(kt)
        if (kt + 1 >= 2) w.wait(&st_ready[(kt + 1) % 3], ((kt - 1) / 3) & 1, 0x22);
        fence_after_sync();
        issue_stack_scores(tU, q_addr, st_addr + ((kt + 1) % 3) * ST_BYTES, rank, lo_addr + ((kt + 1) & 1) * STLO_BYTES);
        mma_commit(&u_done);
      }
      __syncwarp();
    }
    if (kt >= 2) w.wait(&p_done[buf], ((kt - 2) >> 1) & 1, 0x26);
    fence_after_sync();
    const uint32_t pt = tP + lane_off + buf * P_COLS;
    if (warp_active) {
      f32x2 dw2[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float d0 = dw[2 * j], d1 = dw[2 * j + 1];
        if (kt * KT + 8 * half + 2 * j > row) d0 = 0.f;
        if (kt * KT + 8 * half + 2 * j + 1 > row) d1 = 0.f;
        dw2[j] = f2_pack(2.f * d0, 2.f * d1);
        S2 = f2_add(S2, dw2[j]);
      }
      f32x2 u2[RM][4];
#pragma unroll
      for (int r = 0; r < RM; ++r)
#pragma unroll
        for (int j = 0; j < 4; ++j) u2[r][j] = f2_pack(u[r][2 * j], u[r][2 * j + 1]);
      int idx = 0;
#pragma unroll
      for (int r = 0; r < RM; ++r) {
        if (r < rank) {
          f32x2 t[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            t[j] = f2_mul(dw2[j], u2[r][j]);
            N2[r] = f2_add(N2[r], t[j]);
          }
          store_tile8(pt, r, half, t, r >= rpos);
#pragma unroll
          for (int r2 = r; r2 < RM; ++r2) {
            if (r2 < rank) {
#pragma unroll
              for (int j = 0; j < 4; ++j) D2[idx + r2 - r] = f2_fma(t[j], u2[r2][j], D2[idx + r2 - r]);
            }
          }
        }
        idx += RM - r;
      }
    } else {
      const f32x2 zero[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
      for (int r = 0; r < RM; ++r)
        if (r < rank) store_tile8(pt, r, half, zero, false);
    }
    tmem_st_wait();
    fence_before_sync();
    warp_arrive(&p_ready[buf], lane);
    // stack of tile kt + 2 into the slot whose last reader was the dq MMA of tile kt - 1
    if (kt + 2 < tiles) {
      if (kt >= 1) w.wait(&p_done[(kt - 1) & 1], ((kt - 1) >> 1) & 1, 0x27);
      // (the remainder tile of slot kt & 1 was last read by U(kt), complete since u_done(kt))
      if (half == (kt & 1))
        build_stack_piece(St + ((kt + 2) % 3) * ST_BYTES, Kimg, (kt + 2) * KT, hf, tid & 127, Lo + buf * STLO_BYTES);
      fence_async_smem();
      warp_arrive(&st_ready[(kt + 2) % 3], lane);
    }
    if (issuer) {
      if (lane == 0) {
        w.wait(&p_ready[buf], (kt >> 1) & 1, 0x23);     // P tile of tile kt is in shared memory
        fence_after_sync();
        issue_stack_grad(tQ, tP + buf * P_COLS, st_addr + (kt % 3) * ST_BYTES, rank, kt > 0);
        mma_commit(&p_done[buf]);
      }
      __syncwarp();
    }
  }
  if (tiles >= 2) w.wait(&p_done[(tiles - 2) & 1], ((tiles - 2) >> 1) & 1, 0x28);
  w.wait(&p_done[(tiles - 1) & 1], ((tiles - 1) >> 1) & 1, 0x29);
  fence_after_sync();
  // every MMA has completed: all shared-memory operands are free
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  float* stage_out = reinterpret_cast<float*>(smem);              // [128][65] fp32 over Qa / Kimg / stacks
  float* red = reinterpret_cast<float*>(smem + CT * 65 * 4 + 256);   // [NQ][CTHREADS] behind it
  static_assert(CT * 65 * 4 + 256 + NQ * CTHREADS * 4 <= BQ_SMEM, "staging tile and partial sums");
  {
    if (a.dq) {
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        float vv[16];
        tmem_ld16(tQ + lane_off + 32 * half + 16 * cc, vv);
        tmem_ld_wait();
#pragma unroll
        for (int x = 0; x < 16; ++x) stage_out[row * 65 + 32 * half + 16 * cc + x] = vv[x];
      }
    }
    if (a.coef_partial) {
#pragma unroll
      for (int x = 0; x < NQ; ++x) {
        float lo, hi;
        f2_unpack(x < NU ? D2[x < NU ? x : 0] : (x < NU + RM ? N2[x >= NU && x < NU + RM ? x - NU : 0] : S2), lo, hi);
        red[x * CTHREADS + tid] = lo + hi;
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (a.dq && !dead) {
    // coalesced write-out: 8 consecutive dims per thread, cross-chunk part added, one 16-byte store
    constexpr int PER = CT * 8 / CTHREADS;
    float4 i0[PER], i1[PER];
#pragma unroll
    for (int it = 0; it < PER; ++it) {
      const int x = tid + it * CTHREADS, r = x >> 3, seg = x & 7, i = c * CT + r;
      i0[it] = i1[it] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < a.N && a.dq_init) {
        const float* ip = a.dq_init + (qoff + i) * HD + seg * 8;
        i0[it] = *reinterpret_cast<const float4*>(ip);
        i1[it] = *reinterpret_cast<const float4*>(ip + 4);
      }
    }
#pragma unroll
    for (int it = 0; it < PER; ++it) {
      const int x = tid + it * CTHREADS, r = x >> 3, seg = x & 7, i = c * CT + r;
      if (i >= a.N) continue;
      const size_t o = (qoff + i) * HD + seg * 8;
      const float* sp = stage_out + r * 65 + seg * 8;
      const float val[8] = {sp[0] + i0[it].x, sp[1] + i0[it].y, sp[2] + i0[it].z, sp[3] + i0[it].w,
                            sp[4] + i1[it].x, sp[5] + i1[it].y, sp[6] + i1[it].z, sp[7] + i1[it].w};
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.dq) + o) =
          make_uint4(pack_bf16(val[0], val[1]), pack_bf16(val[2], val[3]), pack_bf16(val[4], val[5]), pack_bf16(val[6], val[7]));
    }
  }
  if (a.coef_partial) {
    // column sums of the per-thread partials: red[value][thread], one warp per value, fixed order
    float* dst = a.coef_partial + ((size_t)(b * a.Hq + h) * a.NB + c) * NQ;
    for (int v = warp; v < NQ; v += CWARPS) {
      float t = 0.f;
#pragma unroll
      for (int x = 0; x < CTHREADS / 32; ++x) t += red[v * CTHREADS + 32 * x + lane];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      if (lane == 0) dst[v] = t;
    }
  }
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
  if (tid == 0 && dead) atomicOr(a.status, w.status_bits());
}

// ---------------------------------------------------------------------------
// key / value side: one CTA per (chunk, query head, batch row); rows are keys
// ---------------------------------------------------------------------------
constexpr int KV_WARPS = 16, KV_THREADS = KV_WARPS * 32;   // 128 key rows x 4 quarters of a 16-query tile
// shared memory: Ka | Qimg | G hi | G lo | 3 stacks | 2 remainder stacks | U   (G lo and U are dead once dW
// is complete).  The stack is carried as value + remainder here too: its rounding acts like a perturbation
// of the query rows that is the same for every key, and with large cancelling dimensions that alone costs
// dk / dv more than the tolerance.
// tensor memory: U (16 R columns) | dW^T (128) | dk (64) | dU (80) | one P tile (8 R) | one W^T tile (8)
constexpr int BKV_SMEM = XA_BYTES + X_BYTES + SLAB_S_BYTES + 3 * ST_BYTES + 2 * STLO_BYTES + 2 * SLAB_S_BYTES;
static_assert(RM * KT + CT + HD + EP + P_COLS + KT / 2 <= 512, "tensor-memory columns of the key/value-side kernel");
static_assert(2 * STAGE_OUT_FLOATS * 4 <= XA_BYTES + X_BYTES + 2 * SLAB_S_BYTES + 3 * ST_BYTES, "staging tiles");

__global__ void __launch_bounds__(KV_THREADS, 1) intra_bwd_kv_kernel(const IntraBwdArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* Ka = smem;                               // augmented k image (rows are keys)
  unsigned char* Qimg = Ka + XA_BYTES;
  unsigned char* Ghi = Qimg + X_BYTES;
  unsigned char* Glo = Ghi + SLAB_S_BYTES;                // dead once dW is complete
  unsigned char* St = Glo + SLAB_S_BYTES;                 // 3 x ST_BYTES: stacked scaled query tiles
  unsigned char* Lo = St + 3 * ST_BYTES;                  // 2 x STLO_BYTES
  unsigned char* Uimg = Lo + 2 * STLO_BYTES;              // dead once dW is complete
  __shared__ HeadFactorS hf;
  __shared__ uint64_t gfull, dw_done, u_done, u_free, p_ready, p_done, st_ready[3];
  __shared__ uint32_t tmem_base;
  __shared__ int dead;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (a.Hq / a.Hkv);
  const int part = warp >> 2, row = 32 * (warp & 3) + lane;       // row = key index inside the chunk; part = 4 queries of a tile
  // Key rows 96..127 (warps 3, 7, 11, 15) are masked out of every tile but the last two, and every stack is
  // built before those: these four warps are the builders, so the warps of rows 0..31, which work in every
  // tile, never build.  Rows 64..95 are idle for the first four tiles: warp 2 issues the MMAs.
  const bool issuer = warp == 2, builder = (warp & 3) == 3;
  if (warp == 0) tmem_alloc(&tmem_base, 512);
  if (tid == 0) {
    mbar_init(&gfull, 1);
    mbar_init(&dw_done, 1);
    mbar_init(&u_done, 1);
    mbar_init(&u_free, KV_WARPS);
    mbar_init(&p_ready, KV_WARPS);
    mbar_init(&p_done, 1);
    for (int s = 0; s < 3; ++s) mbar_init(&st_ready[s], KV_WARPS);
    mbar_fence_init();
    dead = 0;
  }
  __syncthreads();
  if (tid == 0) fetch_g_images(a, Ghi, Glo, &gfull, b, h, c);
  const size_t qoff = (size_t)(b * a.Hq + h) * a.N, koff = (size_t)(b * a.Hkv + kvh) * a.N;
  load_head_factor(hf, a.factors, h, tid, KV_THREADS);
  load_operand_image(Ka, a.k + koff * HD, c * CT, a.N, true, tid, KV_THREADS);
  load_operand_image(Qimg, a.q + qoff * HD, c * CT, a.N, false, tid, KV_THREADS);
  load_u_image(Uimg, a.v + koff * VD, c * CT, a.N, tid, KV_THREADS);
  async_copies_wait();
  __syncthreads();
  const int tiles = min(CT / KT, (a.N - c * CT + KT - 1) / KT);
  const int rank = hf.rank, rpos = hf.rpos;
  for (int s = 0; s < 3; ++s) init_stack_constants(St + s * ST_BYTES, hf, tid, KV_THREADS);
  if (tid < 256 && (tid >> 7) < tiles)
    build_stack_piece(St + (tid >> 7) * ST_BYTES, Qimg, (tid >> 7) * KT, hf, tid & 127, Lo + (tid >> 7) * STLO_BYTES);
  fence_async_smem();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  Waiter w{&dead};
  const uint32_t tU = tmem_base, tW = tmem_base + RM * KT, tK = tW + CT, tV = tK + HD, tP = tV + EP, tWt = tP + P_COLS;
  const uint32_t lane_off = (uint32_t)(32 * (warp & 3)) << 16;

  const uint32_t k_addr = smem_u32(Ka), st_addr = smem_u32(St), g_addr = smem_u32(Ghi), lo_addr = smem_u32(Lo);
  const uint32_t idesc_du = instr_desc_bf16(128, EP, 0, 1);
  if (issuer) {
    if (lane == 0) {
      w.wait(&gfull, 0, 0x30);
      fence_after_sync();
      // dW^T[j, i] = [v|1]_j . g_i: rows from the U image, columns from the hi and lo images of G
      issue_dw(tW, smem_u32(Uimg), false, g_addr, true);
      mma_commit(&dw_done);
      issue_stack_scores(tU, k_addr, st_addr, rank, lo_addr);
      mma_commit(&u_done);
    }
    __syncwarp();
  }
  w.wait(&dw_done, 0, 0x34);
  for (int qt = 0; qt < tiles; ++qt) {
    // keys of this warp are all later than the tile's queries -> nothing survives the mask
    const bool warp_active = 32 * (warp & 3) <= qt * KT + KT - 1;
    float u[RM][4], dw[4];
    w.wait(&u_done, qt & 1, 0x35);
    fence_after_sync();
    if (warp_active) {
#pragma unroll
      for (int r = 0; r < RM; ++r)
        if (r < rank) tmem_ld4(tU + lane_off + r * KT + 4 * part, u[r]);
      tmem_ld4(tW + lane_off + qt * KT + 4 * part, dw);
      tmem_ld_wait();
    }
    fence_before_sync();
    warp_arrive(&u_free, lane);
    if (issuer && qt + 1 < tiles) {
      if (lane == 0) {
        w.wait(&u_free, qt & 1, 0x31);
        if (qt + 1 >= 2) w.wait(&st_ready[(qt + 1) % 3], ((qt - 1) / 3) & 1, 0x32);
        fence_after_sync();
        issue_stack_scores(tU, k_addr, st_addr + ((qt + 1) % 3) * ST_BYTES, rank, lo_addr + ((qt + 1) & 1) * STLO_BYTES);
        mma_commit(&u_done);
      }
      __syncwarp();
    }
    // one P tile and one W^T tile in tensor memory: the MMAs of the previous tile must have read them
    if (qt >= 1) w.wait(&p_done, (qt - 1) & 1, 0x36);
    fence_after_sync();
    const uint32_t pt = tP + lane_off + 2 * part;
    f32x2 wv[2] = {0ull, 0ull};
    if (warp_active) {
      f32x2 dw2[2], wp[2], wn[2];
      bool keep[4];
#pragma unroll
      for (int x = 0; x < 4; ++x) keep[x] = qt * KT + 4 * part + x >= row;      // query not earlier than the key
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        dw2[j] = f2_pack(keep[2 * j] ? 2.f * dw[2 * j] : 0.f, keep[2 * j + 1] ? 2.f * dw[2 * j + 1] : 0.f);
        wp[j] = wn[j] = 0ull;
      }
#pragma unroll
      for (int r = 0; r < RM; ++r) {
        if (r < rank) {
          const f32x2 ua = f2_pack(u[r][0], u[r][1]), ub = f2_pack(u[r][2], u[r][3]);
          const f32x2 ta = f2_mul(dw2[0], ua), tb = f2_mul(dw2[1], ub);
          if (r < rpos) { wp[0] = f2_fma(ua, ua, wp[0]); wp[1] = f2_fma(ub, ub, wp[1]); }
          else { wn[0] = f2_fma(ua, ua, wn[0]); wn[1] = f2_fma(ub, ub, wn[1]); }
          float a0, a1, b0, b1;
          f2_unpack(ta, a0, a1);
          f2_unpack(tb, b0, b1);
          uint32_t lo = pack_bf16(a0, a1), hi = pack_bf16(b0, b1);
          if (r >= rpos) { lo ^= 0x80008000u; hi ^= 0x80008000u; }
          tmem_st2(pt + r * (KT / 2), lo, hi);
        }
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        float p0, p1, n0, n1;
        f2_unpack(wp[j], p0, p1);
        f2_unpack(wn[j], n0, n1);
        wv[j] = f2_pack(keep[2 * j] ? p0 - n0 : 0.f, keep[2 * j + 1] ? p1 - n1 : 0.f);
      }
    } else {
#pragma unroll
      for (int r = 0; r < RM; ++r)
        if (r < rank) tmem_st2(pt + r * (KT / 2), 0u, 0u);
    }
    {
      float a0, a1, b0, b1;
      f2_unpack(wv[0], a0, a1);
      f2_unpack(wv[1], b0, b1);
      tmem_st2(tWt + lane_off + 2 * part, pack_bf16(a0, a1), pack_bf16(b0, b1));
    }
    tmem_st_wait();
    fence_before_sync();
    warp_arrive(&p_ready, lane);
    // stack of tile qt + 2 into the slot whose last reader was the dk MMA of tile qt - 1 (complete: see above)
    if (qt + 2 < tiles) {
      if (builder)
        build_stack_piece(St + ((qt + 2) % 3) * ST_BYTES, Qimg, (qt + 2) * KT, hf, 32 * part + lane, Lo + (qt & 1) * STLO_BYTES);
      fence_async_smem();
      warp_arrive(&st_ready[(qt + 2) % 3], lane);
    }
    if (issuer) {
      if (lane == 0) {
        w.wait(&p_ready, qt & 1, 0x33);
        fence_after_sync();
        issue_stack_grad(tK, tP, st_addr + (qt % 3) * ST_BYTES, rank, qt > 0);
        mma_bf16_ts(tV, tWt, smem_desc(g_addr + qt * KT * 16, 128, CT * 16), idesc_du, qt > 0);
        mma_commit(&p_done);
      }
      __syncwarp();
    }
  }
  w.wait(&p_done, (tiles - 1) & 1, 0x39);
  fence_after_sync();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  // tensor-memory loads are warp-collective: every thread of a compute warp executes them; rows
  // beyond N are dropped at the write-out
  float* stage_out = reinterpret_cast<float*>(smem);    // two [128][65] fp32 staging tiles: dk, then dv
  {
    float vv[16];
    tmem_ld16(tK + lane_off + 16 * part, vv);
    tmem_ld_wait();
#pragma unroll
    for (int x = 0; x < 16; ++x) stage_out[row * 65 + 16 * part + x] = vv[x];
    tmem_ld16(tV + lane_off + 16 * part, vv);
    tmem_ld_wait();
#pragma unroll
    for (int x = 0; x < 16; ++x) stage_out[STAGE_OUT_FLOATS + row * 65 + 16 * part + x] = vv[x];
  }
  fence_before_sync();
  __syncthreads();
  if (!dead) {
    for (int x = tid; x < 2 * CT * 16; x += KV_THREADS) {   // coalesced write-out, four dims per thread: dk, then dv
      const int which = x >= CT * 16, xx = x - which * CT * 16;
      const int r = xx >> 4, seg = xx & 15, j = c * CT + r;
      float* dst = which ? a.dv_part : a.dk_part;
      if (j >= a.N || dst == nullptr) continue;
      const float* sp = stage_out + which * STAGE_OUT_FLOATS + r * 65 + seg * 4;
      *reinterpret_cast<float4*>(dst + (qoff + j) * HD + seg * 4) = make_float4(sp[0], sp[1], sp[2], sp[3]);
    }
  }
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
  if (tid == 0 && dead) atomicOr(a.status, w.status_bits());
}

// dk / dv = cross-chunk part + sum over the query heads of the KV head of the per-head shares,
// fixed order, cast to bf16.  One thread per 4 consecutive dims of one key token.
__global__ void __launch_bounds__(256) kv_head_reduce_kernel(const float* part, const float* cross,
                                                            __nv_bfloat16* out, int B, int Hq, int Hkv, int N) {
  const size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x;       // over B*Hkv*N*16
  const size_t total = (size_t)B * Hkv * N * 16;
  if (idx >= total) return;
  const int d4 = (int)(idx & 15);
  const size_t tok = idx >> 4;                                     // (b*Hkv + kvh)*N + n
  const int n = (int)(tok % N);
  const size_t bk = tok / N;
  const int kvh = (int)(bk % Hkv), b = (int)(bk / Hkv), rep = Hq / Hkv;
  float4 acc = cross ? *reinterpret_cast<const float4*>(cross + tok * HD + 4 * d4) : make_float4(0.f, 0.f, 0.f, 0.f);
  for (int r = 0; r < rep; ++r) {
    const float4 t = *reinterpret_cast<const float4*>(part + (((size_t)b * Hq + kvh * rep + r) * N + n) * HD + 4 * d4);
    acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
  }
  *reinterpret_cast<uint2*>(out + tok * HD + 4 * d4) = make_uint2(pack_bf16(acc.x, acc.y), pack_bf16(acc.z, acc.w));
}

}  // namespace

int OAL_INTRA_NAME(intra_coef_terms)() { return RM; }

cudaError_t OAL_INTRA_NAME(intra_backward_q)(const void* q, const void* k, const void* v, const void* gimg,
                                             const void* factors, void* dq, const float* dq_init, float* coef_partial,
                                             int32_t* status, int B, int Hq, int Hkv, int N, int NB, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(intra_bwd_q_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BQ_SMEM);
  if (e != cudaSuccess) return e;
  IntraBwdArgs a{};
  a.q = static_cast<const __nv_bfloat16*>(q); a.k = static_cast<const __nv_bfloat16*>(k);
  a.v = static_cast<const __nv_bfloat16*>(v); a.gimg = static_cast<const __nv_bfloat16*>(gimg);
  a.factors = static_cast<const HeadFactor*>(factors);
  a.dq = dq; a.dq_init = dq_init; a.coef_partial = coef_partial; a.status = status;
  a.N = N; a.NB = NB; a.Hq = Hq; a.Hkv = Hkv;
  a.gimg_lo_offset = (size_t)B * Hq * NB * SLAB_S_BYTES;
  intra_bwd_q_kernel<<<dim3(NB, Hq, B), CTHREADS, BQ_SMEM, st>>>(a);
  return cudaGetLastError();
}

cudaError_t OAL_INTRA_NAME(intra_backward_kv)(const void* q, const void* k, const void* v, const void* gimg,
                                              const void* factors, void* dk, void* dv, const float* dk_cross,
                                              const float* dv_cross, float* dk_part, float* dv_part, int32_t* status,
                                              int B, int Hq, int Hkv, int N, int NB, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(intra_bwd_kv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BKV_SMEM);
  if (e != cudaSuccess) return e;
  IntraBwdArgs a{};
  a.q = static_cast<const __nv_bfloat16*>(q); a.k = static_cast<const __nv_bfloat16*>(k);
  a.v = static_cast<const __nv_bfloat16*>(v); a.gimg = static_cast<const __nv_bfloat16*>(gimg);
  a.factors = static_cast<const HeadFactor*>(factors);
  a.dk_part = dk ? dk_part : nullptr; a.dv_part = dv ? dv_part : nullptr; a.status = status;
  a.N = N; a.NB = NB; a.Hq = Hq; a.Hkv = Hkv;
  a.gimg_lo_offset = (size_t)B * Hq * NB * SLAB_S_BYTES;
  intra_bwd_kv_kernel<<<dim3(NB, Hq, B), KV_THREADS, BKV_SMEM, st>>>(a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const size_t total = (size_t)B * Hkv * N * 16;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dk) kv_head_reduce_kernel<<<blocks, 256, 0, st>>>(dk_part, dk_cross, static_cast<__nv_bfloat16*>(dk), B, Hq, Hkv, N);
  if (dv) kv_head_reduce_kernel<<<blocks, 256, 0, st>>>(dv_part, dv_cross, static_cast<__nv_bfloat16*>(dv), B, Hq, Hkv, N);
  return cudaGetLastError();
}

}  // namespace oal

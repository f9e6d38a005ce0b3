// Intra-chunk term of the chunked scan on the tensor cores (tcgen05 / TMEM), backward.
//
// Per 16-key (query side) or 16-query (key/value side) tile of a 128-token chunk:
//   S_g  = Q_g K_g^T,  dW = G [v|1]^T                          MMAs into tensor memory
//   ds_g = dW (B_g + 2 sum_g' C_gg' s_g'),  w = A + ...        registers, causal mask, bf16 tiles
//   dq~ += ds_g K_g          (query side)                      MMAs, accumulators in tensor memory
//   dk~ += ds_g^T Q_g, dU += W^T G   (key/value side, summed over the query heads of the KV head)
// plus the coefficient partial sums dA, dB_g, dC_gg' (query side, per-thread accumulators and a
// fixed-order block reduction).  Sixteen compute warps (128 rows x 4 column parts) never meet at a
// block-wide barrier inside the tile loop: a seventeenth warp issues all MMAs and is driven by
// warp-granular mbarrier arrivals (scores read, ds tiles written); tcgen05.commit signals back.  The cross-chunk parts computed by the state kernels arrive as
// fp32 buffers and are added before the final cast.  Reference stages replaced:
// oal_attention/hd_block_gemm_backward_wave.py:253-476 (dS, local dphi_q / dphi_k / dU GEMMs) and the
// folds / coefficient partials of oal_attention/hd_block_gemm_feature_backward.py:59-474.
#include "oal_intra.cuh"
#include "oal_kernels.h"

namespace oal {
namespace {

using namespace umma;

constexpr int IMG_BYTES = (DP_MAX / 8) * CT * 16;        // 45056
constexpr int TILE_BYTES = (KT / 8) * CT * 16;           // 4096: bf16 [2][128 rows][8]
constexpr int NTRI = IG * (IG + 1) / 2;
static_assert(STAGE_BYTES <= SLAB_S_BYTES && STAGE_BYTES <= 2 * IG * TILE_BYTES, "image staging areas");
constexpr int STAGE_OUT_FLOATS = CT * 65 + 3;   // one [128][65] fp32 output staging tile (padded to 16 bytes)
static_assert(2 * STAGE_OUT_FLOATS * 4 <= 2 * IMG_BYTES + 3 * SLAB_S_BYTES, "output staging tiles must fit in the images");
constexpr int NVAL = 1 + IG + NTRI;      // coefficient-gradient partial sums per thread: A, B_g, C_gg' (g <= g')
constexpr int BT = 512;                 // compute threads per CTA: 128 rows x 4 column parts
constexpr int BT_ALL = BT + 32;         // plus one warp whose lane 0 issues every MMA
constexpr int CWARPS = BT / 32;         // compute warps: arrival count of the warp-level barriers
constexpr int CW = KT / (BT / CT);      // columns of a tile handled by one thread (4)

// One arrival per warp on an mbarrier after every lane has finished what precedes (shared-memory
// stores made visible to the async proxy, or tensor-memory loads).
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}

// 8 bytes (4 bf16) of a [2][128 rows][8] tile image: columns 4*part .. 4*part+3 of `row`
__device__ __forceinline__ void store_tile4(unsigned char* tile, int part, int row, const float (&t)[4]) {
  *reinterpret_cast<uint2*>(tile + ((part >> 1) * CT + row) * 16 + (part & 1) * 8) =
      make_uint2(pack_bf16(t[0], t[1]), pack_bf16(t[2], t[3]));
}

__device__ __forceinline__ int tri8(int g, int g2) { return g * GMAX - (g * (g - 1)) / 2 + (g2 - g); }

struct IntraBwdArgs {
  const __nv_bfloat16 *q, *k, *v;
  const __nv_bfloat16* gimg;        // [2][B*Hq, NB, 10, 128, 8]: bf16(g) image, then the image of g - bf16(g)
  size_t gimg_lo_offset;            // bytes from the hi image to the lo image
  const int32_t *dim_perm, *group_start;
  const float *A, *Bc, *Cc;
  void *dq, *dk, *dv;               // io dtype outputs (bf16), may be null
  const float* dq_init;             // fp32 cross part (already scaled), or null
  float* dk_part;                   // fp32 [B,Hq,N,64]: this query head's intra-chunk share of dk
  float* dv_part;                   // fp32 [B,Hq,N,64]: this query head's intra-chunk share of dv
  float* coef_partial;              // [B][Hq][NB][NCOEF] or null
  int32_t* status;
  int N, NB, Hq, Hkv, G;
  float scale;
  // padded q / k operand images and [v | 1] images made by pad_images, and the bytes of one q / k slot
  const unsigned char *qimg, *kimg, *uimg;
  int img_stride;
};

// All operand images of one CTA arrive by bulk copy on one barrier: G (hi, lo), q, k, [v | 1].
// A head whose padded layout does not fit the image slots is refused (status word) and copies nothing.
__device__ __forceinline__ bool fetch_images(const IntraBwdArgs& a, const PaddedGroups& pg, unsigned char* Qimg,
                                             unsigned char* Kimg, unsigned char* Uimg, unsigned char* Gimg,
                                             uint64_t* bar, int b, int h, int kvh, int c) {
  const uint32_t bytes = (uint32_t)pg.k16_start[IG] * 4096u;
  if (bytes > (uint32_t)a.img_stride) {
    atomicOr(a.status, OAL_STATUS_BAD_LAYOUT);
    return false;
  }
  const size_t item = (size_t)(b * a.Hq + h) * a.NB + c;
  const unsigned char* gsrc = reinterpret_cast<const unsigned char*>(a.gimg) + item * SLAB_S_BYTES;
  mbar_arrive_expect_tx(bar, 3 * SLAB_S_BYTES + 2 * bytes);
  bulk_g2s(Gimg, gsrc, SLAB_S_BYTES, bar);
  bulk_g2s(Gimg + SLAB_S_BYTES, gsrc + a.gimg_lo_offset, SLAB_S_BYTES, bar);
  bulk_g2s(Qimg, a.qimg + item * (size_t)a.img_stride, bytes, bar);
  bulk_g2s(Kimg, a.kimg + item * (size_t)a.img_stride, bytes, bar);
  bulk_g2s(Uimg, a.uimg + ((size_t)(b * a.Hkv + kvh) * a.NB + c) * SLAB_S_BYTES, SLAB_S_BYTES, bar);
  return true;
}

// scores -> (ds_g tiles, w) for 8 columns of one row.  ss = scale * s.
struct PairOut {
  float w[8];
};

// ---------------------------------------------------------------------------
// query side
// ---------------------------------------------------------------------------
constexpr int BQ_SMEM = 2 * IMG_BYTES + 3 * SLAB_S_BYTES + 2 * IG * TILE_BYTES;

__global__ void __launch_bounds__(BT_ALL, 1) intra_bwd_q_kernel(const IntraBwdArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* Qimg = smem;
  unsigned char* Kimg = Qimg + IMG_BYTES;
  unsigned char* Uimg = Kimg + IMG_BYTES;
  unsigned char* Gimg = Uimg + SLAB_S_BYTES;               // hi image, lo image
  unsigned char* DS = Gimg + 2 * SLAB_S_BYTES;            // [2][IG][TILE_BYTES]
  __shared__ PaddedGroups pg;
  __shared__ uint64_t s_done[2], s_free[2], ds_ready[2], ds_done[2], gfull;
  __shared__ uint32_t tmem_base;
  __shared__ int dead;
  __shared__ bool bad;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (a.Hq / a.Hkv);
  const int part = (warp >> 2) & 3, row = 32 * (warp & 3) + lane;
  const bool issuer = warp == CWARPS;
  if (warp == 0) tmem_alloc(&tmem_base, 512);
  if (tid == 0) {
    mbar_init(&s_done[0], 1);
    mbar_init(&s_done[1], 1);
    mbar_init(&s_free[0], CWARPS);
    mbar_init(&s_free[1], CWARPS);
    mbar_init(&ds_ready[0], CWARPS);
    mbar_init(&ds_ready[1], CWARPS);
    mbar_init(&ds_done[0], 1);
    mbar_init(&ds_done[1], 1);
    mbar_init(&gfull, 1);
    mbar_fence_init();
    dead = 0;
  }
  load_padded_groups(pg, a.dim_perm, a.group_start, a.A, a.Bc, a.Cc, a.G, h, 1.f, 2.f, 2.f, tid, BT_ALL);
  const size_t qoff = (size_t)(b * a.Hq + h) * a.N, koff = (size_t)(b * a.Hkv + kvh) * a.N;
  if (tid == 0) bad = !fetch_images(a, pg, Qimg, Kimg, Uimg, Gimg, &gfull, b, h, kvh, c);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  if (bad) {                        // refused layout: nothing was fetched, nothing is computed
    if (warp == 0) tmem_dealloc(tmem_base, 512);
    return;
  }
  Waiter w{&dead};
  // two score buffers (S_g tiles + dW tile each): the MMAs of tile kt+2 start as soon as every warp has
  // read tile kt, so a warp never waits for scores after its combine
  constexpr uint32_t SBUF = IG * KT + KT;
  static_assert(2 * SBUF + DP_MAX <= 512, "tensor-memory columns");
  const uint32_t tS = tmem_base, tW = tmem_base + IG * KT, tQ = tmem_base + 2 * SBUF;
  const uint32_t lane_off = (uint32_t)(32 * (warp & 3)) << 16;
  const int tiles = min(CT / KT, (a.N - c * CT + KT - 1) / KT);
  // every MMA has completed when the tile loop is left, so the q / k images are free by then:
  // they hold the [128][65] fp32 staging tile of the coalesced dq write-out
  static_assert(2 * IMG_BYTES >= CT * 65 * 4, "staging tile must fit in the two operand images");
  float* stage_out = reinterpret_cast<float*>(smem);
  float cA = 0.f, cB[IG], cC[NTRI];
#pragma unroll
  for (int g = 0; g < IG; ++g) cB[g] = 0.f;
#pragma unroll
  for (int x = 0; x < NTRI; ++x) cC[x] = 0.f;

  if (issuer) {
    if (lane == 0) {
      const uint32_t q_addr = smem_u32(Qimg), k_addr = smem_u32(Kimg), u_addr = smem_u32(Uimg), g_addr = smem_u32(Gimg);
      const uint32_t idesc16 = instr_desc_bf16(128, KT, 0, 0);
      const uint32_t idesc_dq = instr_desc_bf16(128, 16, 0, 1);
      auto issue_scores = [&](int kt) {
        const uint32_t off = (kt & 1) * SBUF;
        issue_group_scores(tS + off, q_addr, k_addr, kt * KT, pg);
#pragma unroll
        for (int ks = 0; ks < 2 * (EP / 16); ++ks) {       // G = hi + lo: the K extent is walked twice
          const int gp = ks / (EP / 16), kk = ks % (EP / 16);
          mma_bf16_ss(tW + off, smem_desc(g_addr + gp * SLAB_S_BYTES + kk * 4096, CT * 16, 128),
                      smem_desc(u_addr + kk * 4096 + kt * KT * 16, CT * 16, 128), idesc16, ks > 0);
        }
        mma_commit(&s_done[kt & 1]);
      };
      w.wait(&gfull, 0, 0x20);
      fence_after_sync();
      issue_scores(0);
      if (tiles > 1) issue_scores(1);
      for (int kt = 0; kt < tiles; ++kt) {
        const int buf = kt & 1;
        if (kt + 2 < tiles) {
          w.wait(&s_free[buf], (kt >> 1) & 1, 0x25);   // every compute warp holds the scores of tile kt
          fence_after_sync();
          issue_scores(kt + 2);
        }
        w.wait(&ds_ready[buf], (kt >> 1) & 1, 0x26);  // ds tiles of tile kt are in shared memory
        fence_after_sync();
        const uint32_t ds_addr = smem_u32(DS + buf * IG * TILE_BYTES);
#pragma unroll 1
        for (int g = 0; g < IG; ++g)
          for (int k16 = pg.k16_start[g]; k16 < pg.k16_start[g + 1]; ++k16)
            mma_bf16_ss(tQ + k16 * 16, smem_desc(ds_addr + g * TILE_BYTES, CT * 16, 128),
                        smem_desc(k_addr + k16 * 4096 + kt * KT * 16, 128, CT * 16), idesc_dq, kt > 0);
        mma_commit(&ds_done[buf]);
      }
    }
    __syncwarp();
  } else {
    for (int kt = 0; kt < tiles; ++kt) {
      const int buf = kt & 1;
      float s[IG][CW], dw[CW];
      w.wait(&s_done[buf], (kt >> 1) & 1, 0x21);
      fence_after_sync();
      const uint32_t soff = buf * SBUF;
#pragma unroll
      for (int g = 0; g < IG; ++g) {
        if (pg.k16_start[g + 1] > pg.k16_start[g]) tmem_ld4(tS + soff + lane_off + g * KT + CW * part, s[g]);
        else {
#pragma unroll
          for (int x = 0; x < CW; ++x) s[g][x] = 0.f;
        }
      }
      tmem_ld4(tW + soff + lane_off + CW * part, dw);
      tmem_ld_wait();
      fence_before_sync();
      warp_arrive(&s_free[buf], lane);
      const bool warp_active = 32 * (warp & 3) + 31 >= kt * KT;
      if (kt >= 2) w.wait(&ds_done[buf], ((kt - 2) >> 1) & 1, 0x22);
      unsigned char* dsb = DS + buf * IG * TILE_BYTES;
      if (warp_active) {
#pragma unroll
        for (int x = 0; x < CW; ++x) {
          if (kt * KT + CW * part + x > row) dw[x] = 0.f;
          cA += dw[x];
        }
        // packed pairs of columns: (0,1) and (2,3)
        f32x2 s2[IG][2];
        const f32x2 sc2 = f2_bcast(a.scale);
        const f32x2 dw2[2] = {f2_pack(dw[0], dw[1]), f2_pack(dw[2], dw[3])};
#pragma unroll
        for (int g = 0; g < IG; ++g) {
          s2[g][0] = f2_mul(f2_pack(s[g][0], s[g][1]), sc2);
          s2[g][1] = f2_mul(f2_pack(s[g][2], s[g][3]), sc2);
          f2_unpack(s2[g][0], s[g][0], s[g][1]);
          f2_unpack(s2[g][1], s[g][2], s[g][3]);
        }
#pragma unroll
        for (int g = 0; g < IG; ++g) {
          f32x2 t0 = pg.B2[g], t1 = t0;
#pragma unroll
          for (int g2 = 0; g2 < IG; ++g2) {
            const f32x2 c2 = pg.C2[g * IG + g2];
            t0 = f2_fma(c2, s2[g2][0], t0);
            t1 = f2_fma(c2, s2[g2][1], t1);
          }
          t0 = f2_mul(t0, dw2[0]);
          t1 = f2_mul(t1, dw2[1]);
          float t[CW];
          f2_unpack(t0, t[0], t[1]);
          f2_unpack(t1, t[2], t[3]);
          store_tile4(dsb + g * TILE_BYTES, part, row, t);
        }
        int idx = 0;
#pragma unroll
        for (int g = 0; g < IG; ++g) {
          float ws[CW];
#pragma unroll
          for (int x = 0; x < CW; ++x) {
            ws[x] = dw[x] * s[g][x];
            cB[g] += ws[x];
          }
#pragma unroll
          for (int g2 = g; g2 < IG; ++g2) {
#pragma unroll
            for (int x = 0; x < CW; ++x) cC[idx] = fmaf(ws[x], s[g2][x], cC[idx]);
            ++idx;
          }
        }
      } else {
        const float zero[CW] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int g = 0; g < IG; ++g) store_tile4(dsb + g * TILE_BYTES, part, row, zero);
      }
      fence_async_smem();
      warp_arrive(&ds_ready[buf], lane);
    }
    if (tiles >= 2) w.wait(&ds_done[(tiles - 2) & 1], ((tiles - 2) >> 1) & 1, 0x23);
    w.wait(&ds_done[(tiles - 1) & 1], ((tiles - 1) >> 1) & 1, 0x24);
    fence_after_sync();
    // dq~ (padded, group-sorted columns) -> row-major staging tile in shared memory (original dim order)
    if (a.dq) {
      const int nslab = pg.k16_start[IG];
      for (int k16 = part; k16 < nslab; k16 += BT / CT) {
        float vv[16];
        tmem_ld16(tQ + lane_off + k16 * 16, vv);
        tmem_ld_wait();
#pragma unroll
        for (int x = 0; x < 16; ++x) {
          const int src = pg.src[k16 * 16 + x];
          if (src >= 0) stage_out[row * 65 + src] = a.scale * vv[x];
        }
      }
    }
  }
  if (a.coef_partial) {
    // U, G and the ds tiles are idle once the last MMA has completed: park the partial sums there
    static_assert(NVAL * BT * 4 <= 3 * SLAB_S_BYTES + 2 * IG * TILE_BYTES, "partial sums must fit");
    float* red = reinterpret_cast<float*>(Uimg);
    if (!issuer) {
      red[tid] = cA;
#pragma unroll
      for (int g = 0; g < IG; ++g) red[(1 + g) * BT + tid] = cB[g];
#pragma unroll
      for (int x = 0; x < NTRI; ++x) red[(1 + IG + x) * BT + tid] = cC[x];
    }
    float* dst = a.coef_partial + ((size_t)(b * a.Hq + h) * a.NB + c) * NCOEF;
    for (int x = tid; x < NCOEF; x += BT_ALL) dst[x] = 0.f;      // slots of groups this build does not have
  }
  fence_before_sync();
  __syncthreads();
  if (a.dq && !dead) {
    // coalesced write-out: 8 consecutive dims per thread, cross-chunk part added, one 16-byte store
    for (int x = tid; x < CT * 8; x += BT_ALL) {
      const int r = x >> 3, seg = x & 7, i = c * CT + r;
      if (i >= a.N) continue;
      const size_t o = (qoff + i) * HD + seg * 8;
      float val[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) val[j] = stage_out[r * 65 + seg * 8 + j];
      if (a.dq_init) {
        const float4 i0 = *reinterpret_cast<const float4*>(a.dq_init + o), i1 = *reinterpret_cast<const float4*>(a.dq_init + o + 4);
        val[0] += i0.x; val[1] += i0.y; val[2] += i0.z; val[3] += i0.w;
        val[4] += i1.x; val[5] += i1.y; val[6] += i1.z; val[7] += i1.w;
      }
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.dq) + o) =
          make_uint4(pack_bf16(val[0], val[1]), pack_bf16(val[2], val[3]), pack_bf16(val[4], val[5]), pack_bf16(val[6], val[7]));
    }
  }
  if (a.coef_partial) {
    // column sums of the per-thread partials: red[value][thread], one warp per value
    const float* red = reinterpret_cast<const float*>(Uimg);
    float* dst = a.coef_partial + ((size_t)(b * a.Hq + h) * a.NB + c) * NCOEF;
    for (int v = warp; v < NVAL; v += BT_ALL / 32) {
      float t = 0.f;
#pragma unroll
      for (int x = 0; x < BT / 32; ++x) t += red[v * BT + 32 * x + lane];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      if (lane == 0) {
        int slot = v;                                  // 0: A, 1..IG: B_g
        if (v > IG) {                                  // C_gg', g <= g', in the order of the accumulators
          int g = 0, rest = v - 1 - IG;
          while (rest >= IG - g) {
            rest -= IG - g;
            ++g;
          }
          slot = 1 + GMAX + tri8(g, g + rest);
        }
        dst[slot] = t;
      }
    }
  }
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
  if (tid == 0 && dead) atomicOr(a.status, w.status_bits());
}

// ---------------------------------------------------------------------------
// key / value side: one CTA per (chunk, query head, batch row); the per-head shares of dk and dv are
// summed over the query heads of a KV head afterwards, in fixed order, by kv_head_reduce_kernel
// ---------------------------------------------------------------------------
constexpr int BKV_SMEM = 2 * IMG_BYTES + 3 * SLAB_S_BYTES + 2 * IG * TILE_BYTES + 2 * TILE_BYTES;

__global__ void __launch_bounds__(BT_ALL, 1) intra_bwd_kv_kernel(const IntraBwdArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* Kimg = smem;
  unsigned char* Qimg = Kimg + IMG_BYTES;
  unsigned char* Uimg = Qimg + IMG_BYTES;
  unsigned char* Gimg = Uimg + SLAB_S_BYTES;               // hi image, lo image
  unsigned char* DS = Gimg + 2 * SLAB_S_BYTES;             // [2][IG][TILE_BYTES]
  unsigned char* WT = DS + 2 * IG * TILE_BYTES;            // [2][TILE_BYTES]
  __shared__ PaddedGroups pg;
  __shared__ uint64_t s_done, s_free, ds_ready[2], ds_done[2], gfull;
  __shared__ uint32_t tmem_base;
  __shared__ int dead;
  __shared__ bool bad;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (a.Hq / a.Hkv);
  const int part = (warp >> 2) & 3, row = 32 * (warp & 3) + lane;     // row = key index inside the chunk
  const bool issuer = warp == CWARPS;
  if (warp == 0) tmem_alloc(&tmem_base, 512);
  if (tid == 0) {
    mbar_init(&s_done, 1);
    mbar_init(&s_free, CWARPS);
    mbar_init(&ds_ready[0], CWARPS);
    mbar_init(&ds_ready[1], CWARPS);
    mbar_init(&ds_done[0], 1);
    mbar_init(&ds_done[1], 1);
    mbar_init(&gfull, 1);
    mbar_fence_init();
    dead = 0;
  }
  load_padded_groups(pg, a.dim_perm, a.group_start, a.A, a.Bc, a.Cc, a.G, h, 1.f, 1.f, 1.f, tid, BT_ALL);
  const size_t koff = (size_t)(b * a.Hkv + kvh) * a.N, qoff = (size_t)(b * a.Hq + h) * a.N;
  if (tid == 0) bad = !fetch_images(a, pg, Qimg, Kimg, Uimg, Gimg, &gfull, b, h, kvh, c);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  if (bad) {                        // refused layout: nothing was fetched, nothing is computed
    if (warp == 0) tmem_dealloc(tmem_base, 512);
    return;
  }
  Waiter w{&dead};
  const uint32_t tS = tmem_base, tW = tmem_base + IG * KT, tK = tmem_base + IG * KT + KT, tU = tK + DP_MAX;
  const uint32_t lane_off = (uint32_t)(32 * (warp & 3)) << 16;
  const int tiles = min(CT / KT, (a.N - c * CT + KT - 1) / KT);

  if (issuer) {
    if (lane == 0) {
      const uint32_t q_addr = smem_u32(Qimg), k_addr = smem_u32(Kimg), u_addr = smem_u32(Uimg), g_addr = smem_u32(Gimg);
      const uint32_t idesc16 = instr_desc_bf16(128, KT, 0, 0);
      const uint32_t idesc_dk = instr_desc_bf16(128, 16, 0, 1);
      const uint32_t idesc_du = instr_desc_bf16(128, EP, 0, 1);
      auto issue_scores = [&](int qt) {
        issue_group_scores(tS, k_addr, q_addr, qt * KT, pg);         // S^T: key rows x 16 queries
#pragma unroll
        for (int ks = 0; ks < 2 * (EP / 16); ++ks) {     // G = hi + lo
          const int gp = ks / (EP / 16), kk = ks % (EP / 16);
          mma_bf16_ss(tW, smem_desc(u_addr + kk * 4096, CT * 16, 128),
                      smem_desc(g_addr + gp * SLAB_S_BYTES + kk * 4096 + qt * KT * 16, CT * 16, 128), idesc16, ks > 0);
        }
        mma_commit(&s_done);
      };
      w.wait(&gfull, 0, 0x30);
      fence_after_sync();
      issue_scores(0);
      for (int qt = 0; qt < tiles; ++qt) {
        const int buf = qt & 1;
        if (qt + 1 < tiles) {
          w.wait(&s_free, qt & 1, 0x35);
          fence_after_sync();
          issue_scores(qt + 1);
        }
        w.wait(&ds_ready[buf], (qt >> 1) & 1, 0x36);
        fence_after_sync();
        const uint32_t ds_addr = smem_u32(DS + buf * IG * TILE_BYTES);
#pragma unroll 1
        for (int g = 0; g < IG; ++g)
          for (int k16 = pg.k16_start[g]; k16 < pg.k16_start[g + 1]; ++k16)
            mma_bf16_ss(tK + k16 * 16, smem_desc(ds_addr + g * TILE_BYTES, CT * 16, 128),
                        smem_desc(q_addr + k16 * 4096 + qt * KT * 16, 128, CT * 16), idesc_dk, qt > 0);
        mma_bf16_ss(tU, smem_desc(smem_u32(WT + buf * TILE_BYTES), CT * 16, 128),
                    smem_desc(g_addr + qt * KT * 16, 128, CT * 16), idesc_du, qt > 0);
        mma_commit(&ds_done[buf]);
      }
    }
    __syncwarp();
  } else {
    for (int qt = 0; qt < tiles; ++qt) {
      const int buf = qt & 1;
      float s[IG][CW], dw[CW];
      w.wait(&s_done, qt & 1, 0x31);
      fence_after_sync();
#pragma unroll
      for (int g = 0; g < IG; ++g) {
        if (pg.k16_start[g + 1] > pg.k16_start[g]) tmem_ld4(tS + lane_off + g * KT + CW * part, s[g]);
        else {
#pragma unroll
          for (int x = 0; x < CW; ++x) s[g][x] = 0.f;
        }
      }
      tmem_ld4(tW + lane_off + CW * part, dw);
      tmem_ld_wait();
      fence_before_sync();
      warp_arrive(&s_free, lane);
      // keys of this warp are all later than the tile's queries -> nothing survives the mask
      const bool warp_active = 32 * (warp & 3) <= qt * KT + KT - 1;
      if (qt >= 2) w.wait(&ds_done[buf], ((qt - 2) >> 1) & 1, 0x32);
      unsigned char* dsb = DS + buf * IG * TILE_BYTES;
      float wv[CW];
      if (warp_active) {
#pragma unroll
        for (int x = 0; x < CW; ++x) {
          wv[x] = pg.A;
          if (qt * KT + CW * part + x < row) dw[x] = 0.f;          // query earlier than the key
        }
        // packed pairs of columns: (0,1) and (2,3)
        f32x2 s2[IG][2];
        const f32x2 sc2 = f2_bcast(a.scale), two2 = f2_bcast(2.f);
        const f32x2 dw2[2] = {f2_pack(dw[0], dw[1]), f2_pack(dw[2], dw[3])};
        f32x2 w0 = f2_bcast(pg.A), w1 = w0;
#pragma unroll
        for (int g = 0; g < IG; ++g) {
          s2[g][0] = f2_mul(f2_pack(s[g][0], s[g][1]), sc2);
          s2[g][1] = f2_mul(f2_pack(s[g][2], s[g][3]), sc2);
        }
#pragma unroll
        for (int g = 0; g < IG; ++g) {
          f32x2 t0 = f2_bcast(0.f), t1 = t0;
#pragma unroll
          for (int g2 = 0; g2 < IG; ++g2) {
            const f32x2 c2 = pg.C2[g * IG + g2];
            t0 = f2_fma(c2, s2[g2][0], t0);
            t1 = f2_fma(c2, s2[g2][1], t1);
          }
          const f32x2 bg = pg.B2[g];
          // w += s_g (B_g + t);  ds_g = dw (B_g + 2 t)
          w0 = f2_fma(s2[g][0], f2_fma(t0, f2_bcast(1.f), bg), w0);
          w1 = f2_fma(s2[g][1], f2_fma(t1, f2_bcast(1.f), bg), w1);
          t0 = f2_mul(dw2[0], f2_fma(two2, t0, bg));
          t1 = f2_mul(dw2[1], f2_fma(two2, t1, bg));
          float t[CW];
          f2_unpack(t0, t[0], t[1]);
          f2_unpack(t1, t[2], t[3]);
          store_tile4(dsb + g * TILE_BYTES, part, row, t);
        }
        f2_unpack(w0, wv[0], wv[1]);
        f2_unpack(w1, wv[2], wv[3]);
#pragma unroll
        for (int x = 0; x < CW; ++x)
          if (qt * KT + CW * part + x < row) wv[x] = 0.f;
      } else {
#pragma unroll
        for (int x = 0; x < CW; ++x) wv[x] = 0.f;
#pragma unroll
        for (int g = 0; g < IG; ++g) store_tile4(dsb + g * TILE_BYTES, part, row, wv);
      }
      store_tile4(WT + buf * TILE_BYTES, part, row, wv);
      fence_async_smem();
      warp_arrive(&ds_ready[buf], lane);
    }
    if (tiles >= 2) w.wait(&ds_done[(tiles - 2) & 1], ((tiles - 2) >> 1) & 1, 0x33);
    w.wait(&ds_done[(tiles - 1) & 1], ((tiles - 1) >> 1) & 1, 0x34);
    fence_after_sync();
    // tensor-memory loads are warp-collective: every thread executes them; rows beyond N are dropped at
    // the write-out
    const int nslab = pg.k16_start[IG];
    float* stage_out = reinterpret_cast<float*>(smem);    // the k / q images are free: [128][65] fp32 staging tile
    for (int k16 = part; k16 < nslab; k16 += BT / CT) {
      float vv[16];
      tmem_ld16(tK + lane_off + k16 * 16, vv);
      tmem_ld_wait();
#pragma unroll
      for (int x = 0; x < 16; ++x) {
        const int src = pg.src[k16 * 16 + x];
        if (src >= 0) stage_out[row * 65 + src] = a.scale * vv[x];   // Q image holds unscaled q
      }
    }
    {
      const int col0 = 16 * part;
      float vv[16];
      tmem_ld16(tU + lane_off + col0, vv);
      tmem_ld_wait();
      // second staging tile, behind the first: the q / k / U / G images are all idle by now
#pragma unroll
      for (int x = 0; x < 16; ++x) stage_out[STAGE_OUT_FLOATS + row * 65 + col0 + x] = vv[x];
    }
  }
  fence_before_sync();
  __syncthreads();
  if (!dead) {
    const float* stage_out = reinterpret_cast<const float*>(smem);
    for (int x = tid; x < 2 * CT * 16; x += BT_ALL) {   // coalesced write-out, four dims per thread: dk, then dv
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

cudaError_t OAL_INTRA_NAME(intra_backward_q)(const void* q, const void* k, const void* v, const void* gimg, const int32_t* dim_perm,
                             const int32_t* group_start, const float* A, const float* Bc, const float* Cc, void* dq,
                             const float* dq_init, float* coef_partial, int32_t* status, int B, int Hq, int Hkv,
                             int N, int NB, int G, float scale, const void* qimg, const void* kimg,
                             const void* uimg, int img_stride, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(intra_bwd_q_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BQ_SMEM);
  if (e != cudaSuccess) return e;
  IntraBwdArgs a{};
  a.q = static_cast<const __nv_bfloat16*>(q); a.k = static_cast<const __nv_bfloat16*>(k);
  a.v = static_cast<const __nv_bfloat16*>(v); a.gimg = static_cast<const __nv_bfloat16*>(gimg);
  a.dim_perm = dim_perm; a.group_start = group_start; a.A = A; a.Bc = Bc; a.Cc = Cc;
  a.dq = dq; a.dq_init = dq_init; a.coef_partial = coef_partial; a.status = status;
  a.N = N; a.NB = NB; a.Hq = Hq; a.Hkv = Hkv; a.G = G; a.scale = scale;
  a.gimg_lo_offset = (size_t)B * Hq * NB * SLAB_S_BYTES;
  a.qimg = static_cast<const unsigned char*>(qimg); a.kimg = static_cast<const unsigned char*>(kimg);
  a.uimg = static_cast<const unsigned char*>(uimg); a.img_stride = img_stride;
  intra_bwd_q_kernel<<<dim3(NB, Hq, B), BT_ALL, BQ_SMEM, st>>>(a);
  return cudaGetLastError();
}

cudaError_t OAL_INTRA_NAME(intra_backward_kv)(const void* q, const void* k, const void* v, const void* gimg, const int32_t* dim_perm,
                              const int32_t* group_start, const float* A, const float* Bc, const float* Cc, void* dk,
                              void* dv, const float* dk_cross, const float* dv_cross, float* dk_part, float* dv_part,
                              int32_t* status, int B, int Hq, int Hkv, int N, int NB, int G, float scale,
                              const void* qimg, const void* kimg, const void* uimg, int img_stride, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(intra_bwd_kv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, BKV_SMEM);
  if (e != cudaSuccess) return e;
  IntraBwdArgs a{};
  a.q = static_cast<const __nv_bfloat16*>(q); a.k = static_cast<const __nv_bfloat16*>(k);
  a.v = static_cast<const __nv_bfloat16*>(v); a.gimg = static_cast<const __nv_bfloat16*>(gimg);
  a.dim_perm = dim_perm; a.group_start = group_start; a.A = A; a.Bc = Bc; a.Cc = Cc;
  a.dk_part = dk ? dk_part : nullptr; a.dv_part = dv ? dv_part : nullptr; a.status = status;
  a.N = N; a.NB = NB; a.Hq = Hq; a.Hkv = Hkv; a.G = G; a.scale = scale;
  a.gimg_lo_offset = (size_t)B * Hq * NB * SLAB_S_BYTES;
  a.qimg = static_cast<const unsigned char*>(qimg); a.kimg = static_cast<const unsigned char*>(kimg);
  a.uimg = static_cast<const unsigned char*>(uimg); a.img_stride = img_stride;
  intra_bwd_kv_kernel<<<dim3(NB, Hq, B), BT_ALL, BKV_SMEM, st>>>(a);
  e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const size_t total = (size_t)B * Hkv * N * 16;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dk) kv_head_reduce_kernel<<<blocks, 256, 0, st>>>(dk_part, dk_cross, static_cast<__nv_bfloat16*>(dk), B, Hq, Hkv, N);
  if (dv) kv_head_reduce_kernel<<<blocks, 256, 0, st>>>(dv_part, dv_cross, static_cast<__nv_bfloat16*>(dv), B, Hq, Hkv, N);
  return cudaGetLastError();
}

}  // namespace oal

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
  const __nv_bfloat16* carry_img;  // [units, NB, 19, 10, 128, 8] or null (no coefficient gradients)
  const __nv_bfloat16* carry_lo;   // same layout: bf16(state - bf16(state)); the dot products below see hi + lo,
                                   // because they are sums of strongly cancelling terms
  const float* coef_table;         // [Hq, F_ROWS]
  float* dcarry;                   // [units, NB] chunks of F_ROWS x EP floats in state_inc_offset order
  float* dcoef_partial;            // [B, NB, 2 column halves, Hq, F_ROWS] or null
  int N, NB, Hq, Hkv, units;
  float scale;
  int32_t* status;
};

// Persistent, warp-specialised kernel.  Work items are (batch x KV head, chunk, feature slab); CTA k
// takes items k, k + gridDim.x, ... and walks the query heads of the KV head for each, so the flat
// iteration `it` = (item, head) drives four pipelined roles:
//   warps 0-3   thread = token: generate the coefficient-free, unscaled feature slab of (item, head)
//               from the packed bf16 q row into A[it % 3]
//   warp  13    lane 0 streams the head's G image into a 4-slot ring (bulk copies)
//   warp  12    lane 0 issues the MMAs  Z[it % 3] = A^T G  once A and G are full and Z[it % 3] is drained
//   warps 4-11  drain Z, thread = (feature row, half of the 80 columns): dot with the carry row for
//               the coefficient gradient, acc += coef_h * Z in registers; after the last head
//               acc -> dCarry
// A slot and Z buffer share the index it % 3, so the MMA-completion barrier of that index tells the
// generators "A is free" and the drain warps "Z is ready".
constexpr int DS_GEN_WARPS = 4, DS_EPI_WARPS = 8;
constexpr int DS_ISSUER = DS_GEN_WARPS + DS_EPI_WARPS, DS_LOADER = DS_ISSUER + 1;
constexpr int DS_THREADS = (DS_LOADER + 1) * 32;
constexpr int DS_RING = 3;      // A slots in shared memory = Z buffers in tensor memory
constexpr int DS_GRING = 4;     // G image slots
constexpr int DS_COLS = EP / 2; // columns per drain thread
static_assert(DS_GEN_WARPS * 32 == CT, "one generator thread per token");
static_assert(DS_GEN_WARPS % 4 == 0, "drain warp w must sit on tensor-memory lane quadrant w % 4");

// (item, head) cursor of one role; the divisions happen only when the item changes
struct DsCursor {
  int u, c, slab, hh, item;
  int b, h0;          // batch row and first query head of the item's KV head
  __device__ __forceinline__ void set_item(int it_item, int NB, int Hkv, int rep) {
    item = it_item;
    slab = item % F_SLABS;
    const int r = item / F_SLABS;
    c = r % NB;
    u = r / NB;
    b = u / Hkv;
    h0 = (u - b * Hkv) * rep;
  }
  __device__ __forceinline__ void start(int NB, int Hkv, int rep) {
    hh = 0;
    set_item(blockIdx.x, NB, Hkv, rep);
  }
  __device__ __forceinline__ void next(int rep, int NB, int Hkv) {
    if (++hh == rep) {
      hh = 0;
      set_item(item + gridDim.x, NB, Hkv, rep);
    }
  }
};

__global__ void __launch_bounds__(DS_THREADS, 1) dstate_heads_kernel(const DStateArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* Abuf = smem;                              // DS_RING x SLAB_A_BYTES
  unsigned char* Gbuf = smem + DS_RING * SLAB_A_BYTES;     // DS_GRING x SLAB_S_BYTES  ([10][128 tokens][8 e])
  __shared__ uint64_t full_a[DS_RING], mma_done[DS_RING], z_free[DS_RING], g_full[DS_GRING], g_free[DS_GRING];
  __shared__ uint32_t tmem_base;
  __shared__ int dead;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rep = a.Hq / a.Hkv;
  const int n_items = F_SLABS * a.NB * a.units;
  const int my_items = (int)blockIdx.x < n_items ? (n_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  const int T = my_items * rep;
  if (warp == DS_ISSUER) tmem_alloc(&tmem_base, 256);
  if (tid == 0) {
    for (int s = 0; s < DS_RING; ++s) {
      mbar_init(&full_a[s], DS_GEN_WARPS);
      mbar_init(&mma_done[s], 1);
      mbar_init(&z_free[s], DS_EPI_WARPS);
    }
    for (int s = 0; s < DS_GRING; ++s) {
      mbar_init(&g_full[s], 1);
      mbar_init(&g_free[s], 1);
    }
    mbar_fence_init();
    dead = 0;
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  Waiter w{&dead};

  if (warp < DS_GEN_WARPS) {
    // ---------------- generators ----------------
    const int token = tid;
    uint4 nx[8];                               // packed q row of the next (item, head)
    auto fetch = [&](const DsCursor& d) {
      const int h = d.h0 + d.hh, i = d.c * CT + token;
      if (i < a.N) {
        const uint4* p = reinterpret_cast<const uint4*>(a.q + ((size_t)(d.b * a.Hq + h) * a.N + i) * HD);
#pragma unroll
        for (int j = 0; j < 8; ++j) nx[j] = p[j];
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) nx[j] = make_uint4(0u, 0u, 0u, 0u);
      }
    };
    DsCursor cur;
    cur.start(a.NB, a.Hkv, rep);
    if (T > 0) fetch(cur);
    int s = 0, use = 0;                       // ring slot of `it` and how often it has been used before
    for (int it = 0; it < T; ++it) {
      const int slab = cur.slab;
      uint32_t xp[HD / 2];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        xp[4 * j] = nx[j].x;
        xp[4 * j + 1] = nx[j].y;
        xp[4 * j + 2] = nx[j].z;
        xp[4 * j + 3] = nx[j].w;
      }
      cur.next(rep, a.NB, a.Hkv);
      if (it + 1 < T) fetch(cur);             // in flight while this slab is generated
      if (use > 0) w.wait(&mma_done[s], (use - 1) & 1, 0x31);   // the MMA that read A[s] has completed
      write_slab_raw(slab, xp, reinterpret_cast<uint4*>(Abuf + s * SLAB_A_BYTES) + token);
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&full_a[s]);
      if (++s == DS_RING) { s = 0; ++use; }
    }
  } else if (warp < DS_ISSUER) {
    // ---------------- drain warps ----------------
    const int fr = 32 * (warp & 3) + lane, ch = (warp - DS_GEN_WARPS) >> 2, col0 = ch * DS_COLS;
    const uint32_t lane_off = (uint32_t)(32 * (warp & 3)) << 16;
    // packed fp32 pairs: the drain is bound by issue slots, and a packed multiply-add is one slot for two columns
    f32x2 acc[DS_COLS / 2];        // this thread's part of the dCarry row, summed over the heads of the item
    f32x2 carry[DS_COLS / 2];      // this thread's part of the carry row (value + remainder), fp32, once per item
#pragma unroll
    for (int j = 0; j < DS_COLS / 2; ++j) carry[j] = 0ull;
    DsCursor d, dn;
    d.start(a.NB, a.Hkv, rep);
    dn = d;
    int s = 0, use = 0;
    float cf_next = T > 0 ? a.coef_table[(size_t)d.h0 * F_ROWS + d.slab * 128 + fr] : 0.f;
    for (int it = 0; it < T; ++it) {
      const int b = d.b, h = d.h0 + d.hh, f = d.slab * 128 + fr;
      const float fs = feature_scale_factor(f, a.scale);   // d(table entry) / d(coefficient)
      const float cf = cf_next;
      dn.next(rep, a.NB, a.Hkv);
      if (it + 1 < T)       // coefficient of the next (item, head): in flight during this drain
        cf_next = a.coef_table[(size_t)(dn.h0 + dn.hh) * F_ROWS + dn.slab * 128 + fr];
      if (d.hh == 0 && a.carry_img) {
        const uint4* cp = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(a.carry_img) +
                                                         (((size_t)d.u * a.NB + d.c) * F_SLABS + d.slab) * SLAB_S_BYTES);
        const uint4* cl = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(a.carry_lo) +
                                                         (((size_t)d.u * a.NB + d.c) * F_SLABS + d.slab) * SLAB_S_BYTES);
        uint4 cpk[DS_COLS / 8], cpl[DS_COLS / 8];
#pragma unroll
        for (int e = 0; e < DS_COLS / 8; ++e) {
          cpk[e] = cp[(col0 / 8 + e) * 128 + fr];
          cpl[e] = cl[(col0 / 8 + e) * 128 + fr];
        }
#pragma unroll
        for (int e = 0; e < DS_COLS / 8; ++e) {
          float c0[8], c1[8];
          unpack_bf16x8(cpk[e], c0);
          unpack_bf16x8(cpl[e], c1);
#pragma unroll
          for (int j = 0; j < 4; ++j) carry[4 * e + j] = f2_pack(c0[2 * j] + c1[2 * j], c0[2 * j + 1] + c1[2 * j + 1]);
        }
      }
      w.wait(&mma_done[s], use & 1, 0x32);
      fence_after_sync();
      const uint32_t tz = tmem_base + EP * s + col0;
      if (d.hh == 0) {
#pragma unroll
        for (int j = 0; j < DS_COLS / 2; ++j) acc[j] = 0ull;
      }
      f32x2 dot[2] = {0ull, 0ull};
      const f32x2 cf2 = f2_bcast(cf);
      // two register stages: the loads of the next 8 columns are in flight while these are combined
      float z[2][8];
      tmem_ld8(tz + lane_off, z[0]);
#pragma unroll
      for (int r = 0; r < DS_COLS / 8; ++r) {
        tmem_ld_wait();
        if (r + 1 < DS_COLS / 8) tmem_ld8(tz + lane_off + 8 * (r + 1), z[(r + 1) & 1]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const f32x2 z2 = f2_pack(z[r & 1][2 * j], z[r & 1][2 * j + 1]);
          dot[j & 1] = f2_fma(z2, carry[4 * r + j], dot[j & 1]);
          acc[4 * r + j] = f2_fma(cf2, z2, acc[4 * r + j]);
        }
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&z_free[s]);      // every lane has its Z values in registers
      float d0, d1, d2, d3;
      f2_unpack(dot[0], d0, d1);
      f2_unpack(dot[1], d2, d3);
      const float dot_sum = (d0 + d2) + (d1 + d3);
      if (a.dcoef_partial)      // one partial per column half, summed by the reduction over (batch, chunk, half)
        a.dcoef_partial[((((size_t)b * a.NB + d.c) * 2 + ch) * a.Hq + h) * F_ROWS + f] =
            fs * dot_sum;
      if (d.hh == rep - 1) {
        // dCarry rows of this slab -> HBM; the next group of 8 columns of a row lies one 128-row block further
        float* dst = a.dcarry + ((size_t)d.u * a.NB + d.c) * F_ROWS * EP + state_inc_offset(f, col0);
#pragma unroll
        for (int r = 0; r < DS_COLS / 8; ++r) {
          float o[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) f2_unpack(acc[4 * r + j], o[2 * j], o[2 * j + 1]);
          *reinterpret_cast<float4*>(dst + r * 1024) = make_float4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<float4*>(dst + r * 1024 + 4) = make_float4(o[4], o[5], o[6], o[7]);
        }
      }
      d = dn;
      if (++s == DS_RING) { s = 0; ++use; }
    }
  } else if (warp == DS_ISSUER) {
    // ---------------- MMA issue ----------------
    if (lane == 0) {
      const uint32_t idesc = instr_desc_bf16(128, EP, 1, 1);
      // descriptors of slot 0 of both rings, advanced by adds: this thread is the serial path of every slab
      const uint64_t da0 = smem_desc(smem_u32(Abuf), 128, CT * 16), dg0 = smem_desc(smem_u32(Gbuf), 128, CT * 16);
      int s = 0, use = 0, gs = 0, guse = 0;
      for (int it = 0; it < T; ++it) {
        const uint64_t da = desc_advance(da0, s * SLAB_A_BYTES), dg = desc_advance(dg0, gs * SLAB_S_BYTES);
        const uint32_t tz = tmem_base + EP * s;
        w.wait(&full_a[s], use & 1, 0x33);
        w.wait(&g_full[gs], guse & 1, 0x34);
        if (use > 0) w.wait(&z_free[s], (use - 1) & 1, 0x35);
        fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < CT / 16; ++ks)
          mma_bf16_ss(tz, desc_advance(da, ks * 256), desc_advance(dg, ks * 256), idesc, ks > 0);
        mma_commit(&mma_done[s]);
        mma_commit(&g_free[gs]);               // the loader may refill this G slot when these MMAs are done
        if (++s == DS_RING) { s = 0; ++use; }
        if (++gs == DS_GRING) { gs = 0; ++guse; }
      }
    }
    __syncwarp();
  } else {
    // ---------------- G image stream ----------------
    if (lane == 0) {
      DsCursor d;
      d.start(a.NB, a.Hkv, rep);
      int gs = 0, guse = 0;
      for (int it = 0; it < T; ++it) {
        const int h = d.h0 + d.hh;
        const unsigned char* src =
            reinterpret_cast<const unsigned char*>(a.gimg) + ((size_t)(d.b * a.Hq + h) * a.NB + d.c) * SLAB_S_BYTES;
        if (guse > 0) w.wait(&g_free[gs], (guse - 1) & 1, 0x36);
        mbar_arrive_expect_tx(&g_full[gs], SLAB_S_BYTES);
        bulk_g2s(Gbuf + gs * SLAB_S_BYTES, src, SLAB_S_BYTES, &g_full[gs]);
        d.next(rep, a.NB, a.Hkv);
        if (++gs == DS_GRING) { gs = 0; ++guse; }
      }
    }
    __syncwarp();
  }
  fence_before_sync();
  __syncthreads();
  if (warp == DS_ISSUER) tmem_dealloc(tmem_base, 256);
  if (tid == 0 && dead) atomicOr(a.status, w.status_bits());
}

// ---------------------------------------------------------------------------
// fold of dphi (tensor memory, thread = token, columns = the 128 features of a slab) through the
// feature map into dx.  x and dx are fp32 rows held as packed pairs (element 2k, 2k+1 in pair k);
// every index is a compile-time constant.  Per pair chunk (cb, r), with t_j = dphi_j (* coef_j):
//   dx[r]        += sum_j t_j x[8 cb + j]        dx[8 cb + j] += t_j x[r]
// ---------------------------------------------------------------------------
template <int Q, bool QUERY, int OFF>
__device__ __forceinline__ void fold_chunk(const float (&v)[16], const f32x2 (&xq)[HD / 2], const float* coef,
                                           f32x2 (&dxq)[HD / 2]) {
  if constexpr (Q < F_CONST_CHUNK) {
    f32x2 t[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) t[k] = f2_pack(v[OFF + 2 * k], v[OFF + 2 * k + 1]);
    if constexpr (QUERY) {
      const ulonglong2 ca = *reinterpret_cast<const ulonglong2*>(coef + 8 * Q);
      const ulonglong2 cb2 = *reinterpret_cast<const ulonglong2*>(coef + 8 * Q + 4);
      t[0] = f2_mul(t[0], ca.x);
      t[1] = f2_mul(t[1], ca.y);
      t[2] = f2_mul(t[2], cb2.x);
      t[3] = f2_mul(t[3], cb2.y);
    }
    if constexpr (Q < F_PAIR_CHUNKS) {
      constexpr PairCursor pc = pair_pos(Q);
      constexpr int nv = pc.valid();
      float xlo, xhi;
      f2_unpack(xq[pc.r / 2], xlo, xhi);
      const f32x2 xr2 = f2_bcast((pc.r & 1) ? xhi : xlo);
      f32x2 sr2 = 0ull;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (2 * k < nv) {                       // pairs entirely above the diagonal do not exist
          if (2 * k + 1 >= nv) {                // the pair straddles the diagonal: drop its upper element
            float lo, hi;
            f2_unpack(t[k], lo, hi);
            t[k] = f2_pack(lo, 0.f);
          }
          sr2 = f2_fma(t[k], xq[4 * pc.cb + k], sr2);
          dxq[4 * pc.cb + k] = f2_fma(t[k], xr2, dxq[4 * pc.cb + k]);
        }
      }
      float slo, shi, dlo, dhi;
      f2_unpack(sr2, slo, shi);
      f2_unpack(dxq[pc.r / 2], dlo, dhi);
      if (pc.r & 1) dhi += slo + shi;
      else dlo += slo + shi;
      dxq[pc.r / 2] = f2_pack(dlo, dhi);
    } else {
      const f32x2 one2 = f2_bcast(1.f);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        dxq[4 * (Q - F_LIN_CHUNK0) + k] = f2_fma(t[k], one2, dxq[4 * (Q - F_LIN_CHUNK0) + k]);
    }
  }
}

// Eight chunks = four 16-column loads; the next load is in flight while the previous one is folded.
template <int S, int HALF, bool QUERY>
__device__ __forceinline__ void fold_half_slab_impl(uint32_t taddr, const f32x2 (&xq)[HD / 2], const float* coef,
                                                    f32x2 (&dxq)[HD / 2]) {
  constexpr int Q0 = S * 16 + HALF * 8;
  float va[16], vb[16];
  tmem_ld16(taddr + HALF * 64, va);
  tmem_ld_wait();
  tmem_ld16(taddr + HALF * 64 + 16, vb);
  fold_chunk<Q0 + 0, QUERY, 0>(va, xq, coef, dxq);
  fold_chunk<Q0 + 1, QUERY, 8>(va, xq, coef, dxq);
  tmem_ld_wait();
  tmem_ld16(taddr + HALF * 64 + 32, va);
  fold_chunk<Q0 + 2, QUERY, 0>(vb, xq, coef, dxq);
  fold_chunk<Q0 + 3, QUERY, 8>(vb, xq, coef, dxq);
  tmem_ld_wait();
  tmem_ld16(taddr + HALF * 64 + 48, vb);
  fold_chunk<Q0 + 4, QUERY, 0>(va, xq, coef, dxq);
  fold_chunk<Q0 + 5, QUERY, 8>(va, xq, coef, dxq);
  tmem_ld_wait();
  fold_chunk<Q0 + 6, QUERY, 0>(vb, xq, coef, dxq);
  fold_chunk<Q0 + 7, QUERY, 8>(vb, xq, coef, dxq);
}

template <bool QUERY>
__device__ __forceinline__ void fold_half_slab(int s, int half, uint32_t taddr, const f32x2 (&xq)[HD / 2],
                                               const float* coef, f32x2 (&dxq)[HD / 2]) {
#define OAL_CASE(S)                                                                    \
  case S:                                                                              \
    if (half == 0) fold_half_slab_impl<S, 0, QUERY>(taddr, xq, coef, dxq);             \
    else fold_half_slab_impl<S, 1, QUERY>(taddr, xq, coef, dxq);                       \
    break;
  OAL_SLAB_SWITCH(s, OAL_CASE)
#undef OAL_CASE
}

// ---------------------------------------------------------------------------
// feature_grad: persistent, warp-specialised.  Work items are (batch, head, chunk) with the heads of
// one state unit adjacent; CTA k takes items k, k + gridDim.x, ...  Roles:
//   warps 0-7  fold: thread = (token, half of the slab's 128 features); drains dphi of slab `s` from
//              tensor memory (three buffers) into its packed dx row; halves are combined per item
//   warp  8    lane 0 issues  dphi[s] = A . S[s]^T  (M = tokens, N = 128 features, K = 80)
//   warp  9    lane 0 streams the state slab images (4-slot ring) and, per item, the A operand
//              image (QUERY: the image of G) and the head's coefficient table (two buffers each)
// KEY: the A operand [v | 1] is built in shared memory by the fold warps.
// ---------------------------------------------------------------------------
struct FeatGradArgs {
  const __nv_bfloat16* x;        // q [B,Hq,N,64] (QUERY) or k [B,Hkv,N,64]
  const __nv_bfloat16* gimg;     // QUERY: A-operand image of G  [B*Hq, NB, 10, 128, 8]
  const __nv_bfloat16* v;        // KEY: values, the A operand [v | 1] is built in shared memory
  const __nv_bfloat16* image;    // state image [units, NB, 19, 10, 128, 8]: carry (QUERY) / dT (KEY)
  const float* coef_table;       // QUERY
  float* dx;                     // [B,H,N,64] fp32
  int N, NB, H, rep, B;
  int32_t* status;
};

constexpr int FG_FOLD_WARPS = 8, FG_ISSUER = FG_FOLD_WARPS, FG_LOADER = FG_ISSUER + 1;
constexpr int FG_THREADS = (FG_LOADER + 1) * 32;
constexpr int FG_SRING = 4, FG_DRING = 3;

struct FgItem {
  int b, h, c;
};
__device__ __forceinline__ FgItem fg_item(int item, int H, int rep, int NB) {
  FgItem r;
  const int hh = item % rep, t = item / rep;
  r.c = t % NB;
  const int unit = t / NB, units_per_b = H / rep;
  r.b = unit / units_per_b;
  r.h = (unit % units_per_b) * rep + hh;
  return r;
}

template <bool QUERY>
__global__ void __launch_bounds__(FG_THREADS, 1) feature_grad_kernel(const FeatGradArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* Sbuf = smem;                                        // FG_SRING x SLAB_S_BYTES
  unsigned char* Aimg = Sbuf + FG_SRING * SLAB_S_BYTES;              // 2 x SLAB_S_BYTES: [10][128 tokens][8 e]
  float* coef_s = reinterpret_cast<float*>(Aimg + 2 * SLAB_S_BYTES); // 2 x F_ROWS
  float* red = coef_s + 2 * F_ROWS;                                  // [128][65]
  __shared__ uint64_t s_full[FG_SRING], s_free[FG_SRING], a_full[2], a_free[2], coef_full[2], coef_free[2];
  __shared__ uint64_t d_full[FG_DRING], d_free[FG_DRING];
  __shared__ uint32_t tmem_base;
  __shared__ int dead;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_items = a.B * a.H * a.NB;
  const int my_items = (int)blockIdx.x < n_items ? (n_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  if (warp == FG_ISSUER) tmem_alloc(&tmem_base, 512);
  if (tid == 0) {
    for (int s = 0; s < FG_SRING; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_free[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&a_full[s], QUERY ? 1 : FG_FOLD_WARPS);
      mbar_init(&a_free[s], 1);
      mbar_init(&coef_full[s], 1);
      mbar_init(&coef_free[s], FG_FOLD_WARPS);
    }
    for (int s = 0; s < FG_DRING; ++s) {
      mbar_init(&d_full[s], 1);
      mbar_init(&d_free[s], FG_FOLD_WARPS);
    }
    mbar_fence_init();
    dead = 0;
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  Waiter w{&dead};

  if (warp < FG_FOLD_WARPS) {
    // ---------------- fold warps ----------------
    const int wg = warp >> 2, token = 32 * (warp & 3) + lane;
    const uint32_t lane_off = (uint32_t)(32 * (warp & 3)) << 16;
    int ds = 0, duse = 0;
    for (int k = 0; k < my_items; ++k) {
      const FgItem it = fg_item(blockIdx.x + k * gridDim.x, a.H, a.rep, a.NB);
      const int i = it.c * CT + token;
      const size_t head_off = (size_t)(it.b * a.H + it.h) * a.N;
      f32x2 xq[HD / 2], dxq[HD / 2];
      {
        uint32_t xp[HD / 2];
        load_row_packed(xp, a.x + head_off * HD, i, a.N);
        unpack_row(xp, xq);
      }
#pragma unroll
      for (int d = 0; d < HD / 2; ++d) dxq[d] = 0ull;
      if (!QUERY) {
        // A operand [v | 1] of this item, once the MMAs of item k-2 have left the buffer
        if (k >= 2) w.wait(&a_free[k & 1], ((k >> 1) - 1) & 1, 0x51);
        uint4* dst = reinterpret_cast<uint4*>(Aimg + (k & 1) * SLAB_S_BYTES);
        for (int idx = tid; idx < (EP / 8) * CT; idx += FG_FOLD_WARPS * 32) {
          const int ec = idx >> 7, t = idx & 127, j = it.c * CT + t;
          dst[idx] = u_image_chunk(a.v + (head_off + j) * VD, ec, j < a.N);
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&a_full[k & 1]);
      }
      const float* coef = coef_s + (k & 1) * F_ROWS;
      if (QUERY) w.wait(&coef_full[k & 1], (k >> 1) & 1, 0x52);
      for (int s = 0; s < F_SLABS; ++s) {
        w.wait(&d_full[ds], duse & 1, 0x53);
        fence_after_sync();
        fold_half_slab<QUERY>(s, wg, tmem_base + ds * 128 + lane_off, xq, coef, dxq);
        fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&d_free[ds]);
        if (++ds == FG_DRING) { ds = 0; ++duse; }
      }
      if (QUERY) {
        __syncwarp();
        if (lane == 0) mbar_arrive(&coef_free[k & 1]);
      }
      // combine the two halves of every token and write
      float dx[HD];
#pragma unroll
      for (int d = 0; d < HD / 2; ++d) f2_unpack(dxq[d], dx[2 * d], dx[2 * d + 1]);
      if (wg == 1) {
#pragma unroll
        for (int d = 0; d < HD; ++d) red[token * 65 + d] = dx[d];
      }
      asm volatile("bar.sync 1, %0;" ::"n"(FG_FOLD_WARPS * 32) : "memory");
      if (wg == 0 && i < a.N && !dead) {
        float* dst = a.dx + (head_off + i) * HD;
#pragma unroll
        for (int d4 = 0; d4 < HD; d4 += 4)
          *reinterpret_cast<float4*>(dst + d4) =
              make_float4(dx[d4] + red[token * 65 + d4], dx[d4 + 1] + red[token * 65 + d4 + 1],
                          dx[d4 + 2] + red[token * 65 + d4 + 2], dx[d4 + 3] + red[token * 65 + d4 + 3]);
      }
      asm volatile("bar.sync 1, %0;" ::"n"(FG_FOLD_WARPS * 32) : "memory");
    }
  } else if (warp == FG_ISSUER) {
    // ---------------- MMA issue ----------------
    if (lane == 0) {
      const uint32_t idesc = instr_desc_bf16(128, 128, 0, 0);
      const uint64_t da0 = smem_desc(smem_u32(Aimg), CT * 16, 128), ds0 = smem_desc(smem_u32(Sbuf), 128 * 16, 128);
      int gs = 0, guse = 0, ds = 0, duse = 0;
      for (int k = 0; k < my_items; ++k) {
        const uint64_t da = desc_advance(da0, (k & 1) * SLAB_S_BYTES);
        w.wait(&a_full[k & 1], (k >> 1) & 1, 0x54);
        for (int s = 0; s < F_SLABS; ++s) {
          const uint64_t dsl = desc_advance(ds0, gs * SLAB_S_BYTES);
          w.wait(&s_full[gs], guse & 1, 0x55);
          if (duse > 0) w.wait(&d_free[ds], (duse - 1) & 1, 0x56);
          fence_after_sync();
#pragma unroll
          for (int ks = 0; ks < EP / 16; ++ks)
            mma_bf16_ss(tmem_base + ds * 128, desc_advance(da, ks * 2 * CT * 16), desc_advance(dsl, ks * 2 * 128 * 16), idesc,
                        ks > 0);
          mma_commit(&d_full[ds]);
          mma_commit(&s_free[gs]);
          if (s == F_SLABS - 1) mma_commit(&a_free[k & 1]);
          if (++gs == FG_SRING) { gs = 0; ++guse; }
          if (++ds == FG_DRING) { ds = 0; ++duse; }
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- image / table stream ----------------
    if (lane == 0) {
      int gs = 0, guse = 0;
      for (int k = 0; k < my_items; ++k) {
        const FgItem it = fg_item(blockIdx.x + k * gridDim.x, a.H, a.rep, a.NB);
        const int unit = (it.b * a.H + it.h) / a.rep;
        const unsigned char* img = reinterpret_cast<const unsigned char*>(a.image) +
                                   ((size_t)unit * a.NB + it.c) * F_SLABS * SLAB_S_BYTES;
        if (QUERY) {
          if (k >= 2) {
            w.wait(&a_free[k & 1], ((k >> 1) - 1) & 1, 0x57);
            w.wait(&coef_free[k & 1], ((k >> 1) - 1) & 1, 0x58);
          }
          mbar_arrive_expect_tx(&a_full[k & 1], SLAB_S_BYTES);
          bulk_g2s(Aimg + (k & 1) * SLAB_S_BYTES,
                   reinterpret_cast<const unsigned char*>(a.gimg) + ((size_t)(it.b * a.H + it.h) * a.NB + it.c) * SLAB_S_BYTES,
                   SLAB_S_BYTES, &a_full[k & 1]);
          mbar_arrive_expect_tx(&coef_full[k & 1], F_ROWS * (uint32_t)sizeof(float));
          bulk_g2s(coef_s + (k & 1) * F_ROWS, a.coef_table + (size_t)it.h * F_ROWS, F_ROWS * (uint32_t)sizeof(float),
                   &coef_full[k & 1]);
        }
        for (int s = 0; s < F_SLABS; ++s) {
          if (guse > 0) w.wait(&s_free[gs], (guse - 1) & 1, 0x59);
          mbar_arrive_expect_tx(&s_full[gs], SLAB_S_BYTES);
          bulk_g2s(Sbuf + gs * SLAB_S_BYTES, img + (size_t)s * SLAB_S_BYTES, SLAB_S_BYTES, &s_full[gs]);
          if (++gs == FG_SRING) { gs = 0; ++guse; }
        }
      }
    }
    __syncwarp();
  }
  fence_before_sync();
  __syncthreads();
  if (warp == FG_ISSUER) tmem_dealloc(tmem_base, 512);
  if (tid == 0 && dead) atomicOr(a.status, w.status_bits());
}

// ---------------------------------------------------------------------------
// coefficient gradients of the cross-chunk term: per-feature sums -> (A, B_g, C_gg') slots
// ---------------------------------------------------------------------------
// block = 32 feature rows x 8 segments of the outer index; the segments are added in fixed order
__global__ void __launch_bounds__(256) dcoef_sum_kernel(const float* partial, int outer /* B*NB*2 */, int Hq,
                                                        float* dcoef) {
  __shared__ float seg_sum[8][32];
  const int lane = threadIdx.x & 31, seg = threadIdx.x >> 5;
  const int f = blockIdx.x * 32 + lane, h = blockIdx.y;
  const int per = (outer + 7) / 8, o0 = seg * per, o1 = min(outer, o0 + per);
  float t = 0.f;
#pragma unroll 4
  for (int o = o0; o < o1; ++o) t += partial[((size_t)o * Hq + h) * F_ROWS + f];
  seg_sum[seg][lane] = t;
  __syncthreads();
  if (seg == 0) {
    float r = 0.f;
#pragma unroll
    for (int x = 0; x < 8; ++x) r += seg_sum[x][lane];
    dcoef[(size_t)h * F_ROWS + f] = r;
  }
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
    const FeatureId id = feature_id(f);
    if (id.kind == 0 && id.live) {
      const int ga = min(gdim[id.r], gdim[id.c]), gb = max(gdim[id.r], gdim[id.c]);
      slot = 1 + GMAX + tri_slot(ga, gb);
      wgt = (ga == gb && id.r != id.c) ? 2.f : 1.f;
    } else if (id.kind == 1) {
      slot = 1 + gdim[id.r];
    } else if (id.kind == 2) {
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

// normalisation VJP writing the bf16 operand images of G (hi, lo) and, when `g` is given, its fp32 rows
//   CTA = 32 consecutive tokens of one (head, chunk); warp = 8 consecutive columns, lane = token, so a
//   warp stores 512 contiguous bytes of an image chunk.  Rows are enumerated over padded chunks so
//   that tail tokens of the last chunk are zeroed.
__global__ void __launch_bounds__(256) norm_vjp_image_kernel(const void* grad_out, int out_dt, const float* grad_num,
                                                             const float* grad_den, const float* num,
                                                             const float* den, float floor_v, float* g,
                                                             __nv_bfloat16* gimg, int N, int NB, int heads,
                                                             int tm_heads) {
  __shared__ float part[8][32];
  const int ec = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t per_head = (size_t)NB * CT;
  const size_t r = (size_t)blockIdx.x * 32 + lane;          // grid covers heads * per_head rows exactly
  const size_t bh = r / per_head;
  const int t = (int)(r % per_head);
  const int cidx = t / CT, tl = t % CT;
  const bool live = t < N;
  const size_t row = bh * N + t;
  // row of the upstream gradient of out: head-first [B, Hq, N, 64], or token-major [B, N, Hq, 64] (tm_heads = Hq)
  const size_t grow = tm_heads > 0 ? ((bh / tm_heads) * N + t) * tm_heads + bh % tm_heads : row;
  float gv[8], dot = 0.f, dn = 1.f, dw = 1.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) gv[j] = 0.f;
  if (live) {
    dn = den[row];
    dw = fmaxf(dn, floor_v);
    if (grad_out) {
      float go[8];
      if (out_dt == OAL_DTYPE_BF16) {
        const uint4 w = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(grad_out) + grow * VD + 8 * ec);
        unpack_bf16x8(w, go);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) go[j] = load_elem(grad_out, grow * VD + 8 * ec + j, out_dt);
      }
      const float4 n0 = *reinterpret_cast<const float4*>(num + row * VD + 8 * ec);
      const float4 n1 = *reinterpret_cast<const float4*>(num + row * VD + 8 * ec + 4);
      const float nn[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        dot = fmaf(go[j], nn[j], dot);
        gv[j] = go[j] / dw;
      }
    }
    if (grad_num) {
      const float4 a0 = *reinterpret_cast<const float4*>(grad_num + row * VD + 8 * ec);
      const float4 a1 = *reinterpret_cast<const float4*>(grad_num + row * VD + 8 * ec + 4);
      gv[0] += a0.x; gv[1] += a0.y; gv[2] += a0.z; gv[3] += a0.w;
      gv[4] += a1.x; gv[5] += a1.y; gv[6] += a1.z; gv[7] += a1.w;
    }
  }
  part[ec][lane] = dot;
  // hi image = bf16(g); lo image = bf16(g - hi): dW = g . [v|1] is formed from both, because its two
  // large terms (dout.v / den and dout.num / den^2) nearly cancel
  uint4* img = reinterpret_cast<uint4*>(gimg + (bh * NB + cidx) * (size_t)(SLAB_S_BYTES / 2));
  uint4* img_lo = reinterpret_cast<uint4*>(gimg + ((size_t)heads * NB + bh * NB + cidx) * (size_t)(SLAB_S_BYTES / 2));
  {
    uint32_t hi[4], lo[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const __nv_bfloat16 h0 = __float2bfloat16_rn(gv[2 * k]), h1 = __float2bfloat16_rn(gv[2 * k + 1]);
      hi[k] = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
      lo[k] = pack_bf16(gv[2 * k] - __bfloat162float(h0), gv[2 * k + 1] - __bfloat162float(h1));
    }
    img[ec * CT + tl] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    img_lo[ec * CT + tl] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
  }
  if (g && live) {
    *reinterpret_cast<float4*>(g + row * EP + 8 * ec) = make_float4(gv[0], gv[1], gv[2], gv[3]);
    *reinterpret_cast<float4*>(g + row * EP + 8 * ec + 4) = make_float4(gv[4], gv[5], gv[6], gv[7]);
  }
  __syncthreads();
  if (ec < 2) {            // columns 64..79: [d den, 0 x 15]
    float gd = 0.f;
    if (ec == 0 && live) {
      float d = 0.f;
#pragma unroll
      for (int x = 0; x < 8; ++x) d += part[x][lane];
      if (grad_out) gd = (dn >= floor_v) ? -(d / dw) / dw : 0.f;
      if (grad_den) gd += grad_den[row];
    }
    const __nv_bfloat16 h0 = __float2bfloat16_rn(gd);
    img[(VD / 8 + ec) * CT + tl] = make_uint4((uint32_t)__bfloat16_as_ushort(h0), 0u, 0u, 0u);
    img_lo[(VD / 8 + ec) * CT + tl] = make_uint4(pack_bf16(gd - __bfloat162float(h0), 0.f), 0u, 0u, 0u);
    if (g && live) {
      *reinterpret_cast<float4*>(g + row * EP + VD + 8 * ec) = make_float4(gd, 0.f, 0.f, 0.f);
      *reinterpret_cast<float4*>(g + row * EP + VD + 8 * ec + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
}

}  // namespace

cudaError_t dstate_heads(const void* q, const void* gimg, const void* carry_img, const void* carry_lo, const float* coef_table,
                         float* dcarry, float* dcoef_partial, int B, int Hq, int Hkv, int N, int NB, float scale,
                         int32_t* status, cudaStream_t st) {
  const int smem = DS_RING * SLAB_A_BYTES + DS_GRING * SLAB_S_BYTES;
  cudaError_t e = cudaFuncSetAttribute(dstate_heads_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  int dev = 0, sms = 0;
  if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
  if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
  const int items = F_SLABS * NB * B * Hkv;
  DStateArgs a{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(gimg),
               static_cast<const __nv_bfloat16*>(carry_img), static_cast<const __nv_bfloat16*>(carry_lo), coef_table,
               dcarry, dcoef_partial, N, NB, Hq, Hkv,
               B * Hkv, scale, status};
  dstate_heads_kernel<<<items < sms ? items : sms, DS_THREADS, smem, st>>>(a);
  return cudaGetLastError();
}

cudaError_t feature_grad(bool query, const void* x, const void* gimg, const void* v, const void* image,
                         const float* coef_table, float* dx, int B, int H, int rep, int N, int NB, int32_t* status,
                         cudaStream_t st) {
  const int smem = FG_SRING * SLAB_S_BYTES + 2 * SLAB_S_BYTES + 2 * F_ROWS * (int)sizeof(float) +
                   128 * 65 * (int)sizeof(float);
  FeatGradArgs a{static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(gimg),
                 static_cast<const __nv_bfloat16*>(v), static_cast<const __nv_bfloat16*>(image), coef_table, dx,
                 N, NB, H, rep, B, status};
  cudaError_t e;
  int dev = 0, sms = 0;
  if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
  if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
  const int items = B * H * NB, grid = items < sms ? items : sms;
  if (query) {
    e = cudaFuncSetAttribute(feature_grad_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    feature_grad_kernel<true><<<grid, FG_THREADS, smem, st>>>(a);
  } else {
    e = cudaFuncSetAttribute(feature_grad_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    feature_grad_kernel<false><<<grid, FG_THREADS, smem, st>>>(a);
  }
  return cudaGetLastError();
}

cudaError_t dcoef_reduce(const float* partial, int outer, int Hq, const int32_t* dim_perm,
                         const int32_t* group_start, float* dcoef, float* slots, cudaStream_t st) {
  dcoef_sum_kernel<<<dim3(F_ROWS / 32, Hq), 256, 0, st>>>(partial, outer, Hq, dcoef);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  dcoef_slots_kernel<<<Hq, 256, 0, st>>>(dcoef, dim_perm, group_start, slots);
  return cudaGetLastError();
}

cudaError_t norm_vjp_image(const void* grad_out, int out_dt, const float* grad_num, const float* grad_den,
                           const float* num, const float* den, float floor_v, float* g, void* gimg, int heads,
                           int N, int NB, int token_major_heads, cudaStream_t st) {
  const size_t rows = (size_t)heads * NB * CT;      // a multiple of 32
  norm_vjp_image_kernel<<<(unsigned)(rows / 32), 256, 0, st>>>(grad_out, out_dt, grad_num, grad_den, num, den,
                                                                   floor_v, g, static_cast<__nv_bfloat16*>(gimg), N,
                                                                   NB, heads, token_major_heads);
  return cudaGetLastError();
}

}  // namespace oal

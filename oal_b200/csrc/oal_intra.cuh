// Shared pieces of the tensor-core intra-chunk kernels.
//
// Per token pair (i, j) of one query head the kernel weight is a quadratic form in
// v = [1, s_1 .. s_G], s_g = sum_{d in g} (scale q_i[d]) k_j[d]:
//     w = v^T M v,   M = [[A, B/2], [B/2, C]]          (oal_attention/grouped_reference.py:61-99)
// With the eigen-decomposition M = V diag(sigma) V^T (head_factor_kernel, one per call) and
// lambda_r = sqrt|sigma_r| the weight is a signed sum of squares
//     w = sum_r sgn_r u_r^2,   u_r(i,j) = c_r + sum_d q_i[d] (l_r[d] k_j[d]),
//     c_r = lambda_r V[0][r],  l_r[d] = scale lambda_r V[1 + g(d)][r],
// so every u_r is one plain 64-long dot product of the query row with a per-dimension scaled copy
// of the key row.  The kernels stack the R = G + 1 scaled copies of a 16-key tile as the N rows of
// one MMA (N = 16 R, K = 64 + one step that adds c_r), read u from tensor memory and spend R
// multiply-adds per pair instead of the G^2 of the direct form; the backward reuses the same stack
// for dq / dk and accumulates the coefficient gradient as D[r][r'] = sum dW u_r u_r', which
// intra_coef_finish maps back to (dA, dB, dC).  Dimension groups need no sorting or padding.
#pragma once

#include "oal_features.cuh"

namespace oal {

#ifndef OAL_RM
#define OAL_RM 9                     // terms handled by this build: heads with at most OAL_RM - 1 groups
#endif
#ifndef OAL_INTRA_NAME
#define OAL_INTRA_NAME(name) name
#endif

constexpr int KT = 16;                               // keys (query side) or queries (key side) per tile
constexpr int RM = OAL_RM;
constexpr int NU = RM * (RM + 1) / 2;                // D[r][r'], r <= r'
constexpr int RMAX_ALL = OAL_MAX_GROUPS + 1;         // 17: extent of the per-head factor table
constexpr int NU_ALL = RMAX_ALL * (RMAX_ALL + 1) / 2;
constexpr int XA_CHUNKS = 10;                        // augmented operand image: 64 dims + 16 (constant step)
constexpr int XA_BYTES = XA_CHUNKS * CT * 16;        // 20480
constexpr int X_BYTES = 8 * CT * 16;                 // 16384: plain 128 x 64 operand image
constexpr int ST_BYTES = XA_CHUNKS * RM * KT * 16;   // stacked scaled tile [10 chunks][16 R rows][8]
constexpr int STLO_BYTES = 8 * RM * KT * 16;         // its rounding remainders [8 chunks][16 R rows][8]
constexpr int P_COLS = RM * KT / 2;                  // tensor-memory columns of a bf16 tile [128 rows][16 R]
constexpr int CWARPS = 8;                            // warps of a CTA: 128 rows x 2 halves of a tile
constexpr int CTHREADS = CWARPS * 32;                // lane 0 of warp 0 also issues every MMA (rows 0..31 are
                                                     // masked out of most tiles, so that warp has the time)

// Per-head factor table in global memory (written by head_factor_kernel).
struct HeadFactor {
  float c[RMAX_ALL];                 // c_r
  float l[RMAX_ALL][HD];             // l_r[d], original dimension order
  float t[RMAX_ALL][RMAX_ALL];       // t[a][r] = V[a][r] / lambda_r  (v = t u)
  int rank;                          // R = G + 1
  int rpos;                          // terms r < rpos enter with +, the others with -
  int pad[2];
};

// The part of it a kernel keeps in shared memory.
struct HeadFactorS {
  float l[RM][HD];
  float c[RM];
  int rank, rpos;
};

__device__ __forceinline__ void load_head_factor(HeadFactorS& s, const HeadFactor* table, int h, int tid, int nthreads) {
  const HeadFactor& f = table[h];
  for (int x = tid; x < RM * HD; x += nthreads) s.l[x / HD][x % HD] = f.l[x / HD][x % HD];
  for (int x = tid; x < RM; x += nthreads) s.c[x] = f.c[x];
  if (tid == 0) {
    s.rank = min(f.rank, RM);
    s.rpos = min(f.rpos, RM);
  }
}

// 16-byte asynchronous copy global -> shared (zero fill when `valid` is false); completion with
// async_copies_wait().  All copies of a thread are in flight together, so a tile costs one memory
// latency instead of one per 16 bytes.
__device__ __forceinline__ void async_copy16(void* dst_smem, const void* src, bool valid) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(umma::smem_u32(dst_smem)), "l"(src),
               "r"(valid ? 16 : 0)
               : "memory");
}
__device__ __forceinline__ void async_copies_wait() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// Rows [row0, row0 + 128) of a bf16 [.., N, 64] tensor -> operand image [chunks][128 rows][8]
// (rows beyond N are zero), by asynchronous copies: call async_copies_wait() and a block barrier
// before reading.  With `augment` the image has two more chunks: (1, 1, 0 ...) for the rows that
// exist and zeros, which is the K step that adds c_r (as c_hi + c_lo) to every u_r.
__device__ __forceinline__ void load_operand_image(unsigned char* img, const __nv_bfloat16* base, int row0, int N,
                                                   bool augment, int tid, int nthreads) {
  for (int x = tid; x < 8 * CT; x += nthreads) {
    const int c8 = x >> 7, r = x & 127, i = row0 + r;
    async_copy16(img + (size_t)x * 16, base + (size_t)min(i, N - 1) * HD + c8 * 8, i < N);
  }
  if (augment) {
    for (int x = tid; x < 2 * CT; x += nthreads) {
      const int r = x & 127, i = row0 + r;
      reinterpret_cast<uint4*>(img)[8 * CT + x] = make_uint4((x < CT && i < N) ? 0x3F803F80u : 0u, 0u, 0u, 0u);   // bf16 (1, 1)
    }
  }
}

// [v | 1 | 0] image of the chunk's tokens (asynchronous copies for the value part).
__device__ __forceinline__ void load_u_image(unsigned char* img, const __nv_bfloat16* vbase, int row0, int N, int tid,
                                             int nthreads) {
  for (int x = tid; x < (VD / 8) * CT; x += nthreads) {
    const int ec = x >> 7, t = x & 127, j = row0 + t;
    async_copy16(img + (size_t)x * 16, vbase + (size_t)min(j, N - 1) * VD + ec * 8, j < N);
  }
  for (int x = tid; x < (EP / 8 - VD / 8) * CT; x += nthreads) {
    const int t = x & 127, j = row0 + t;
    reinterpret_cast<uint4*>(img)[(VD / 8) * CT + x] = make_uint4((x < CT && j < N) ? 0x00003F80u : 0u, 0u, 0u, 0u);
  }
}

// Constant chunks of a stacked tile: row (r, j) of chunk 8 holds (bf16(c_r), bf16(c_r - bf16(c_r)), 0 ...),
// chunk 9 is zero.  Written once per buffer; the scaled chunks 0..7 are rebuilt for every tile.
__device__ __forceinline__ void init_stack_constants(unsigned char* st, const HeadFactorS& hf, int tid, int nthreads) {
  const int nr = hf.rank * KT;
  for (int x = tid; x < 2 * nr; x += nthreads) {
    const int which = x >= nr, n = x - which * nr;
    uint4 t = make_uint4(0u, 0u, 0u, 0u);
    if (!which) {
      const float c = hf.c[n / KT];
      const __nv_bfloat16 hi = __float2bfloat16_rn(c);
      const __nv_bfloat16 lo = __float2bfloat16_rn(c - __bfloat162float(hi));
      t.x = (uint32_t)__bfloat16_as_ushort(hi) | ((uint32_t)__bfloat16_as_ushort(lo) << 16);
    }
    reinterpret_cast<uint4*>(st)[(8 + which) * nr + n] = t;
  }
}

// Scaled chunks of the stacked tile of rows [row0, row0 + 16) of the plain image `x`:
//   st[c8][r * 16 + j][0..7] = bf16(l_r[8 c8 + e] * x[row0 + j][8 c8 + e]),  one rounding.
// `bt` in 0..127 is the builder thread: (j, c8) = (bt & 15, bt >> 4), so the loads from the image and
// the stores of one r are contiguous across 16 lanes.  With `st_lo` the remainders of the rounding
// (product - bf16(product), itself rounded to bf16) go to a second tile of the same row order: a
// consumer that adds both MMA chains sees the scaled keys to about 16 bits.
__device__ __forceinline__ void build_stack_piece(unsigned char* st, const unsigned char* x, int row0,
                                                  const HeadFactorS& hf, int bt, unsigned char* st_lo = nullptr) {
  const int j = bt & 15, c8 = bt >> 4;
  const int nr = hf.rank * KT;
  const uint4 raw = reinterpret_cast<const uint4*>(x)[c8 * CT + row0 + j];
  const f32x2 xv[4] = {f2_pack(bf16_lo(raw.x), bf16_hi(raw.x)), f2_pack(bf16_lo(raw.y), bf16_hi(raw.y)),
                       f2_pack(bf16_lo(raw.z), bf16_hi(raw.z)), f2_pack(bf16_lo(raw.w), bf16_hi(raw.w))};
  uint4* dst = reinterpret_cast<uint4*>(st) + c8 * nr + j;
#pragma unroll
  for (int r = 0; r < RM; ++r) {
    if (r < hf.rank) {
      const ulonglong2 la = *reinterpret_cast<const ulonglong2*>(&hf.l[r][8 * c8]);
      const ulonglong2 lb = *reinterpret_cast<const ulonglong2*>(&hf.l[r][8 * c8 + 4]);
      const f32x2 p[4] = {f2_mul(xv[0], la.x), f2_mul(xv[1], la.y), f2_mul(xv[2], lb.x), f2_mul(xv[3], lb.y)};
      const uint4 hi = pack_pairs_bf16(p);
      dst[r * KT] = hi;
      if (st_lo) {
        const uint32_t hw[4] = {hi.x, hi.y, hi.z, hi.w};
        uint32_t lw[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float a, b;
          f2_unpack(p[k], a, b);
          lw[k] = umma::pack_bf16(a - bf16_lo(hw[k]), b - bf16_hi(hw[k]));
        }
        reinterpret_cast<uint4*>(st_lo)[c8 * nr + r * KT + j] = make_uint4(lw[0], lw[1], lw[2], lw[3]);
      }
    }
  }
}

// 32 lanes x 32-bit, 4 consecutive columns per thread.
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, float (&v)[4]) {
  uint32_t r[4];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(taddr)
               : "memory");
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = __uint_as_float(r[i]);
}

// One arrival per warp on an mbarrier after every lane has finished what precedes (shared-memory
// stores made visible to the async proxy, or tensor-memory loads).
__device__ __forceinline__ void warp_arrive(uint64_t* bar, int lane) {
  __syncwarp();
  if (lane == 0) umma::mbar_arrive(bar);
}

// U[128, 16 R] = X (128 rows, augmented image) . stack^T : five K steps (64 dims + the constant step),
// plus four over the remainder tile when `lo_addr` is given.  Descriptors are built once and advanced
// by adds: the issuing thread is on the critical path of every tile.
__device__ __forceinline__ void issue_stack_scores(uint32_t tmem_u, uint32_t xa_addr, uint32_t st_addr, int rank,
                                                   uint32_t lo_addr = 0) {
  const uint32_t nr = (uint32_t)rank * KT;
  const uint32_t idesc = umma::instr_desc_bf16(128, (int)nr, 0, 0);
  const uint64_t da = umma::smem_desc(xa_addr, CT * 16, 128), db = umma::smem_desc(st_addr, nr * 16, 128);
#pragma unroll
  for (int ks = 0; ks < XA_CHUNKS / 2; ++ks)
    umma::mma_bf16_ss(tmem_u, umma::desc_advance(da, ks * 2 * CT * 16), umma::desc_advance(db, ks * 2 * nr * 16), idesc,
                      ks > 0);
  if (lo_addr) {
    const uint64_t dl = umma::smem_desc(lo_addr, nr * 16, 128);
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
      umma::mma_bf16_ss(tmem_u, umma::desc_advance(da, ks * 2 * CT * 16), umma::desc_advance(dl, ks * 2 * nr * 16), idesc, 1);
  }
}

// acc[128, 64] (+)= P (128 rows, K = 16 R, in tensor memory: row = lane, bf16 pairs, 8 columns per
// term) . stack (rows are K, the 64 dims are N).
__device__ __forceinline__ void issue_stack_grad(uint32_t tmem_acc, uint32_t tmem_p, uint32_t st_addr, int rank,
                                                 bool accumulate) {
  const uint32_t nr = (uint32_t)rank * KT;
  const uint32_t idesc = umma::instr_desc_bf16(128, HD, 0, 1);
  const uint64_t db = umma::smem_desc(st_addr, 128, nr * 16);
#pragma unroll
  for (int r = 0; r < RM; ++r)
    if (r < rank)
      umma::mma_bf16_ts(tmem_acc, tmem_p + r * (KT / 2), umma::desc_advance(db, r * 256), idesc, accumulate || r > 0);
}

// Columns 8*half .. 8*half+7 of block r of this thread's row of a tile in tensor memory (bf16 pairs).
__device__ __forceinline__ void store_tile8(uint32_t tmem_tile_lane, int r, int half, const f32x2 (&t)[4], bool negate) {
  uint4 o = pack_pairs_bf16(t);
  if (negate) { o.x ^= 0x80008000u; o.y ^= 0x80008000u; o.z ^= 0x80008000u; o.w ^= 0x80008000u; }
  umma::tmem_st4(tmem_tile_lane + r * (KT / 2) + 4 * half, o.x, o.y, o.z, o.w);
}

// dW[128, 128] = rows . cols^T over the 80-long augmented value axis, ten K steps: `rows` and `cols` are
// [10][128][8] images; the one flagged hi_lo is followed by its remainder image and walked twice.
__device__ __forceinline__ void issue_dw(uint32_t tmem_dw, uint32_t rows_addr, bool rows_hi_lo, uint32_t cols_addr,
                                         bool cols_hi_lo) {
  const uint32_t idesc = umma::instr_desc_bf16(128, CT, 0, 0);
  const uint64_t da = umma::smem_desc(rows_addr, CT * 16, 128), db = umma::smem_desc(cols_addr, CT * 16, 128);
#pragma unroll
  for (int ks = 0; ks < 2 * (EP / 16); ++ks) {
    const int gp = ks / (EP / 16), kk = ks % (EP / 16);
    umma::mma_bf16_ss(tmem_dw, umma::desc_advance(da, (rows_hi_lo ? gp * SLAB_S_BYTES : 0) + kk * 2 * CT * 16),
                      umma::desc_advance(db, (cols_hi_lo ? gp * SLAB_S_BYTES : 0) + kk * 2 * CT * 16), idesc, ks > 0);
  }
}

}  // namespace oal

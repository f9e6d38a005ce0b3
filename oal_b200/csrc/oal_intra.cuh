// Shared pieces of the tensor-core intra-chunk kernels: per-head padded group layout, operand
// images of q / k with every group padded to a multiple of 16 dimensions, and the per-pair
// combine  w = A + sum_g s_g (B_g + sum_g' C_gg' s_g').
#pragma once

#include "oal_features.cuh"

namespace oal {

// The intra-chunk kernels are compiled twice: for up to 8 groups per head (default) and, with
// OAL_IG = 4, for up to 4 groups (the per-pair combine is quadratic in the compiled group bound).
#ifndef OAL_IG
#define OAL_IG 8
#endif
#ifndef OAL_INTRA_NAME
#define OAL_INTRA_NAME(name) name
#endif
constexpr int KT = 16;                       // keys (or queries) per tile of the intra-chunk kernels
constexpr int IG = OAL_IG;                   // groups handled by this build of the kernels
constexpr int DP_MAX = 64 + (IG - 1) * 16;   // padded dims: every group rounded up to 16 (176 for 8 groups)

// Padded, group-sorted dimension layout of one head.
struct PaddedGroups {
  int k16_start[IG + 1];     // first 16-dim slab of group g; k16_start[IG] = number of slabs
  short src[DP_MAX];         // original dimension of padded position p, or -1 for zero padding
  float A;
  // coefficients as (c, c) pairs, so one 64-bit shared-memory load feeds a packed FMA:
  // B times `bscale`; C[g][g] times `cdiag`, C[g][g'] times `coff`
  f32x2 B2[IG], C2[IG * IG];
};

// Layout part: first slab of every group and the source dimension of every padded position.
// Contains two block-wide barriers.
__device__ __forceinline__ void load_group_layout(PaddedGroups& pg, const int32_t* dim_perm, const int32_t* group_start,
                                                  int h, int tid, int nthreads) {
  if (tid == 0) {
    int acc = 0;
    for (int g = 0; g < IG; ++g) {
      pg.k16_start[g] = acc;
      const int n = group_start[h * (GMAX + 1) + g + 1] - group_start[h * (GMAX + 1) + g];
      acc += (n + 15) >> 4;
    }
    pg.k16_start[IG] = acc;
  }
  __syncthreads();
  for (int p = tid; p < DP_MAX; p += nthreads) {
    int g = 0;
    while (g < IG - 1 && p >= 16 * pg.k16_start[g + 1]) ++g;
    const int t = p - 16 * pg.k16_start[g];
    const int s0 = group_start[h * (GMAX + 1) + g], n = group_start[h * (GMAX + 1) + g + 1] - s0;
    pg.src[p] = (p < 16 * pg.k16_start[IG] && t < n) ? (short)dim_perm[h * HD + s0 + t] : (short)-1;
  }
  __syncthreads();
}

__device__ __forceinline__ void load_padded_groups(PaddedGroups& pg, const int32_t* dim_perm,
                                                   const int32_t* group_start, const float* A, const float* Bc,
                                                   const float* Cc, int G, int h, float bscale, float cdiag,
                                                   float coff, int tid, int nthreads) {
  if (tid == 0) pg.A = A[h];
  for (int x = tid; x < IG; x += nthreads) {
    const float v = x < G ? bscale * Bc[h * G + x] : 0.f;
    pg.B2[x] = ((f32x2)__float_as_uint(v) << 32) | __float_as_uint(v);
  }
  for (int x = tid; x < IG * IG; x += nthreads) {
    const int g = x / IG, g2 = x % IG;
    const float v = (g < G && g2 < G) ? (g == g2 ? cdiag : coff) * Cc[((size_t)h * G + g) * G + g2] : 0.f;
    pg.C2[x] = ((f32x2)__float_as_uint(v) << 32) | __float_as_uint(v);
  }
  load_group_layout(pg, dim_perm, group_start, h, tid, nthreads);
}

constexpr int STAGE_WORDS = CT * 33;      // raw 128 x 64 bf16 tile, row pitch 33 words (conflict-free column walks)
constexpr int STAGE_BYTES = STAGE_WORDS * 4;

// Rows [row0, row0+128) of a bf16 [.., N, 64] tensor -> operand image [slabs*2][128 rows][8] with the
// padded group layout (rows beyond N are zero).  The tile is first copied row-major into `stage`
// with coalesced 16-byte loads, then gathered column by column from shared memory.
// Contains two block-wide barriers; `stage` is free again when it returns.
__device__ __forceinline__ void build_padded_image(unsigned char* img, uint32_t* stage, const __nv_bfloat16* base,
                                                   int row0, int N, const PaddedGroups& pg, int tid, int nthreads) {
  for (int x = tid; x < CT * 8; x += nthreads) {
    const int r = x >> 3, seg = x & 7, i = row0 + r;
    uint4 t = make_uint4(0u, 0u, 0u, 0u);
    if (i < N) t = *reinterpret_cast<const uint4*>(base + (size_t)i * HD + seg * 8);
    uint32_t* d = stage + r * 33 + seg * 4;
    d[0] = t.x; d[1] = t.y; d[2] = t.z; d[3] = t.w;
  }
  __syncthreads();
  const int chunks = 2 * pg.k16_start[IG];
  const unsigned short* raw = reinterpret_cast<const unsigned short*>(stage);
  for (int x = tid; x < chunks * CT; x += nthreads) {
    const int c8 = x >> 7, r = x & 127;
    unsigned short e[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int s = pg.src[c8 * 8 + j];
      e[j] = s >= 0 ? raw[r * 66 + s] : (unsigned short)0;
    }
    reinterpret_cast<uint4*>(img)[x] = make_uint4(e[0] | ((uint32_t)e[1] << 16), e[2] | ((uint32_t)e[3] << 16),
                                                  e[4] | ((uint32_t)e[5] << 16), e[6] | ((uint32_t)e[7] << 16));
  }
  __syncthreads();
}

// Both images of a CTA at once: the q and k tiles travel to their staging areas in one round of
// global loads, one barrier, one gather pass, one barrier.
__device__ __forceinline__ void build_padded_images(unsigned char* img_a, unsigned char* img_b, uint32_t* stage_a,
                                                    uint32_t* stage_b, const __nv_bfloat16* base_a,
                                                    const __nv_bfloat16* base_b, int row0, int N,
                                                    const PaddedGroups& pg, int tid, int nthreads) {
  for (int x = tid; x < 2 * CT * 8; x += nthreads) {
    const int which = x >= CT * 8, xx = x - which * CT * 8;
    const int r = xx >> 3, seg = xx & 7, i = row0 + r;
    uint4 t = make_uint4(0u, 0u, 0u, 0u);
    if (i < N) t = *reinterpret_cast<const uint4*>((which ? base_b : base_a) + (size_t)i * HD + seg * 8);
    uint32_t* d = (which ? stage_b : stage_a) + r * 33 + seg * 4;
    d[0] = t.x; d[1] = t.y; d[2] = t.z; d[3] = t.w;
  }
  __syncthreads();
  const int per_img = 2 * pg.k16_start[IG] * CT;
  for (int x = tid; x < 2 * per_img; x += nthreads) {
    const int which = x >= per_img, xx = x - which * per_img;
    const int c8 = xx >> 7, r = xx & 127;
    const unsigned short* raw = reinterpret_cast<const unsigned short*>(which ? stage_b : stage_a);
    unsigned short e[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int sd = pg.src[c8 * 8 + j];
      e[j] = sd >= 0 ? raw[r * 66 + sd] : (unsigned short)0;
    }
    reinterpret_cast<uint4*>(which ? img_b : img_a)[xx] =
        make_uint4(e[0] | ((uint32_t)e[1] << 16), e[2] | ((uint32_t)e[3] << 16), e[4] | ((uint32_t)e[5] << 16),
                   e[6] | ((uint32_t)e[7] << 16));
  }
  __syncthreads();
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

// Issue the per-group score MMAs  S_g[128 x KT] = X_g (128 rows) . Y_g (KT rows)^T  for one tile.
//   x_addr: image whose 128 rows are the MMA M dimension; y_addr: image, rows [yrow0, yrow0+KT) are N
__device__ __forceinline__ void issue_group_scores(uint32_t tmem_s, uint32_t x_addr, uint32_t y_addr, int yrow0,
                                                   const PaddedGroups& pg) {
  const uint32_t idesc = umma::instr_desc_bf16(128, KT, 0, 0);
#pragma unroll 1
  for (int g = 0; g < IG; ++g) {
    const int k0 = pg.k16_start[g], k1 = pg.k16_start[g + 1];
    for (int k16 = k0; k16 < k1; ++k16)
      umma::mma_bf16_ss(tmem_s + g * KT, umma::smem_desc(x_addr + k16 * 4096, CT * 16, 128),
                        umma::smem_desc(y_addr + k16 * 4096 + yrow0 * 16, CT * 16, 128), idesc, k16 > k0);
  }
}

}  // namespace oal

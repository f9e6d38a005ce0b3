// Quadratic feature map of the chunked scan, laid out for the tensor cores.
//
// The reference materialises phi_k = [1, k_d, k_r k_c (r >= c)] and
// phi_q = [A, B_{g(d)} q_d, m C_{g(r)g(c)} q_r q_c] as [tokens, 2145] matrices in HBM
// (oal_attention/hd_block_gemm_feature_forward.py:225-253, :373-385; pair order
// oal_attention/hd_block_gemm_cache.py:105-121).  Here a feature tile only ever exists
// in shared memory: each thread owns one token, keeps its 64-element row in registers
// and emits 16-byte chunks of 8 consecutive features as bf16.  The feature order is
// internal (the running state is never exposed), chosen so that every index below is a
// compile-time constant:
//   chunks   0..259  pair features p = 8*chunk + j, p = r(r+1)/2 + c  (r >= c)
//   chunks 260..267  linear features d = 8*(chunk-260) + j
//   chunk  268       [constant, 0 x 7]
//   chunks 269..271  zero padding
// 16 chunks (128 features) form a slab: 17 slabs, 2176 feature rows.
#pragma once

#include <utility>

#include "oal_common.cuh"
#include "oal_umma.cuh"

namespace oal {

constexpr int F_PAIR_CHUNKS = 260;
constexpr int F_LIN_CHUNK0 = 260;
constexpr int F_CONST_CHUNK = 268;
constexpr int F_CHUNKS = 272;
constexpr int F_SLABS = 17;
constexpr int F_ROWS = F_SLABS * 128;          // 2176
constexpr int CT = 128;                        // tokens per chunk of the scan
constexpr int SLAB_A_BYTES = 128 * CT * 2;     // feature slab tile  [16 chunks][128 tokens][8] bf16
constexpr int SLAB_S_BYTES = (EP / 8) * 128 * 16;   // state slab image [10][128 features][8 e] bf16

// Per-chunk fp32 state increments (and state-gradient increments) are stored like the bf16 state
// image, [slab][e / 8][128 rows][8 e], so that a warp whose lanes are consecutive feature rows writes
// and reads contiguous kilobytes.  Float index of (feature row f, column e) inside one chunk:
__host__ __device__ constexpr size_t state_inc_offset(int f, int e) {
  return ((size_t)((f >> 7) * (EP / 8) + (e >> 3)) * 128 + (f & 127)) * 8 + (e & 7);
}

struct RC {
  int r, c;
};
__host__ __device__ constexpr RC pair_rc(int p) {
  int r = 0;
  while ((r + 1) * (r + 2) / 2 <= p) ++r;
  return RC{r, p - r * (r + 1) / 2};
}

// One chunk of 8 features of the token whose row is x[64].  QUERY multiplies by the
// per-head coefficient table (same feature order, fp32, in shared memory).
template <int CH, bool QUERY>
__device__ __forceinline__ uint4 feature_chunk(const float (&x)[HD], const float* coef) {
  float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if constexpr (CH < F_PAIR_CHUNKS) {
    constexpr RC p0 = pair_rc(8 * CH + 0), p1 = pair_rc(8 * CH + 1), p2 = pair_rc(8 * CH + 2),
                 p3 = pair_rc(8 * CH + 3), p4 = pair_rc(8 * CH + 4), p5 = pair_rc(8 * CH + 5),
                 p6 = pair_rc(8 * CH + 6), p7 = pair_rc(8 * CH + 7);
    f[0] = x[p0.r] * x[p0.c]; f[1] = x[p1.r] * x[p1.c]; f[2] = x[p2.r] * x[p2.c]; f[3] = x[p3.r] * x[p3.c];
    f[4] = x[p4.r] * x[p4.c]; f[5] = x[p5.r] * x[p5.c]; f[6] = x[p6.r] * x[p6.c]; f[7] = x[p7.r] * x[p7.c];
  } else if constexpr (CH < F_CONST_CHUNK) {
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = x[8 * (CH - F_LIN_CHUNK0) + j];
  } else if constexpr (CH == F_CONST_CHUNK) {
    f[0] = 1.f;
#pragma unroll
    for (int j = 1; j < 8; ++j) f[j] = 0.f;
  } else {
    return make_uint4(0u, 0u, 0u, 0u);
  }
  if constexpr (QUERY) {
    const float4 c0 = *reinterpret_cast<const float4*>(coef + 8 * CH);
    const float4 c1 = *reinterpret_cast<const float4*>(coef + 8 * CH + 4);
    f[0] *= c0.x; f[1] *= c0.y; f[2] *= c0.z; f[3] *= c0.w;
    f[4] *= c1.x; f[5] *= c1.y; f[6] *= c1.z; f[7] *= c1.w;
  }
  return make_uint4(umma::pack_bf16(f[0], f[1]), umma::pack_bf16(f[2], f[3]), umma::pack_bf16(f[4], f[5]),
                    umma::pack_bf16(f[6], f[7]));
}

// ---- coefficient-free features straight from the packed bf16 row ------------------------------
// xp[k] holds (x[2k], x[2k+1]).  The product of two bf16 values rounded once to bf16 is what the
// fp32 multiply followed by a conversion gives, so the packed multiply yields the same bits at two
// features per instruction and needs no unpacked copy of the row.
template <int A, int B>
__device__ __forceinline__ uint32_t pick2(const uint32_t (&xp)[HD / 2]) {   // (x[A], x[B])
  if constexpr ((A & 1) == 0 && B == A + 1) {
    return xp[A / 2];
  } else {
    constexpr uint32_t lo = (A & 1) * 2, hi = 4 + (B & 1) * 2;
    return __byte_perm(xp[A / 2], xp[B / 2], lo | ((lo + 1) << 4) | (hi << 8) | ((hi + 1) << 12));
  }
}
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

template <int CH>
__device__ __forceinline__ uint4 feature_chunk_bf16(const uint32_t (&xp)[HD / 2]) {
  if constexpr (CH < F_PAIR_CHUNKS) {
    constexpr RC p0 = pair_rc(8 * CH + 0), p1 = pair_rc(8 * CH + 1), p2 = pair_rc(8 * CH + 2),
                 p3 = pair_rc(8 * CH + 3), p4 = pair_rc(8 * CH + 4), p5 = pair_rc(8 * CH + 5),
                 p6 = pair_rc(8 * CH + 6), p7 = pair_rc(8 * CH + 7);
    return make_uint4(mul_bf16x2(pick2<p0.r, p1.r>(xp), pick2<p0.c, p1.c>(xp)),
                      mul_bf16x2(pick2<p2.r, p3.r>(xp), pick2<p2.c, p3.c>(xp)),
                      mul_bf16x2(pick2<p4.r, p5.r>(xp), pick2<p4.c, p5.c>(xp)),
                      mul_bf16x2(pick2<p6.r, p7.r>(xp), pick2<p6.c, p7.c>(xp)));
  } else if constexpr (CH < F_CONST_CHUNK) {
    constexpr int k = 4 * (CH - F_LIN_CHUNK0);
    return make_uint4(xp[k], xp[k + 1], xp[k + 2], xp[k + 3]);
  } else if constexpr (CH == F_CONST_CHUNK) {
    return make_uint4(0x00003F80u, 0u, 0u, 0u);   // bf16(1.0) in element 0
  } else {
    return make_uint4(0u, 0u, 0u, 0u);
  }
}

template <int S, int... J>
__device__ __forceinline__ void slab_bf16_impl(const uint32_t (&xp)[HD / 2], uint4* tile, int token,
                                               std::integer_sequence<int, J...>) {
  ((tile[J * CT + token] = feature_chunk_bf16<S * 16 + J>(xp)), ...);
}

// All 16 chunks of slab s of one token (coefficient-free, unscaled) into the slab tile.
__device__ __forceinline__ void write_slab_bf16(int s, const uint32_t (&xp)[HD / 2], uint4* tile, int token) {
#define OAL_SLAB_CASE(S)                                                               \
  case S:                                                                              \
    slab_bf16_impl<S>(xp, tile, token, std::make_integer_sequence<int, 16>{});          \
    break;
  switch (s) {
    OAL_SLAB_CASE(0) OAL_SLAB_CASE(1) OAL_SLAB_CASE(2) OAL_SLAB_CASE(3) OAL_SLAB_CASE(4) OAL_SLAB_CASE(5)
    OAL_SLAB_CASE(6) OAL_SLAB_CASE(7) OAL_SLAB_CASE(8) OAL_SLAB_CASE(9) OAL_SLAB_CASE(10) OAL_SLAB_CASE(11)
    OAL_SLAB_CASE(12) OAL_SLAB_CASE(13) OAL_SLAB_CASE(14) OAL_SLAB_CASE(15) OAL_SLAB_CASE(16)
    default: break;
  }
#undef OAL_SLAB_CASE
}

// Power of the query scale a coefficient-free, unscaled feature row lacks: pair features scale^2,
// linear features scale, the constant feature 1.
__device__ __forceinline__ float feature_scale_factor(int f, float scale) {
  return f < 8 * F_PAIR_CHUNKS ? scale * scale : (f < 8 * F_CONST_CHUNK ? scale : 1.f);
}

// Threads per CTA of the kernels that generate feature slabs: 128 tokens x GEN_PARTS threads per
// token, each thread writing 16 / GEN_PARTS chunks of a slab.
constexpr int GEN_THREADS = 256;
constexpr int GEN_PARTS = GEN_THREADS / CT;
constexpr int GEN_CHUNKS = 16 / GEN_PARTS;

template <int S, int PART, bool QUERY, int... J>
__device__ __forceinline__ void part_slab_impl(const float (&x)[HD], const float* coef, uint4* tile, int token,
                                               std::integer_sequence<int, J...>) {
  ((tile[(PART * GEN_CHUNKS + J) * CT + token] = feature_chunk<S * 16 + PART * GEN_CHUNKS + J, QUERY>(x, coef)), ...);
}

template <int S, bool QUERY>
__device__ __forceinline__ void part_slab_select(int part, const float (&x)[HD], const float* coef, uint4* tile,
                                                 int token) {
  using Seq = std::make_integer_sequence<int, GEN_CHUNKS>;
  if constexpr (GEN_PARTS == 2) {
    if (part == 0) part_slab_impl<S, 0, QUERY>(x, coef, tile, token, Seq{});
    else part_slab_impl<S, 1, QUERY>(x, coef, tile, token, Seq{});
  } else {
    switch (part) {
      case 0: part_slab_impl<S, 0, QUERY>(x, coef, tile, token, Seq{}); break;
      case 1: part_slab_impl<S, 1, QUERY>(x, coef, tile, token, Seq{}); break;
      case 2: part_slab_impl<S, 2 % GEN_PARTS, QUERY>(x, coef, tile, token, Seq{}); break;
      default: part_slab_impl<S, 3 % GEN_PARTS, QUERY>(x, coef, tile, token, Seq{}); break;
    }
  }
}

// Write this thread's chunks of slab s of its token into the slab tile ([16 chunks][128 tokens] x
// 16 bytes).  s and part are runtime values; the bodies are static.
template <bool QUERY>
__device__ __forceinline__ void write_half_slab(int s, int part, const float (&x)[HD], const float* coef,
                                                uint4* tile, int token) {
#define OAL_SLAB_CASE(S)                                      \
  case S:                                                     \
    part_slab_select<S, QUERY>(part, x, coef, tile, token);   \
    break;
  switch (s) {
    OAL_SLAB_CASE(0) OAL_SLAB_CASE(1) OAL_SLAB_CASE(2) OAL_SLAB_CASE(3) OAL_SLAB_CASE(4) OAL_SLAB_CASE(5)
    OAL_SLAB_CASE(6) OAL_SLAB_CASE(7) OAL_SLAB_CASE(8) OAL_SLAB_CASE(9) OAL_SLAB_CASE(10) OAL_SLAB_CASE(11)
    OAL_SLAB_CASE(12) OAL_SLAB_CASE(13) OAL_SLAB_CASE(14) OAL_SLAB_CASE(15) OAL_SLAB_CASE(16)
    default: break;
  }
#undef OAL_SLAB_CASE
}

// Row `i` (or zeros when i >= N) of a bf16 [.., N, 64] tensor into registers, times mul.
__device__ __forceinline__ void load_row_bf16(float (&x)[HD], const __nv_bfloat16* base, int i, int N, float mul) {
  if (i < N) {
    const uint4* p = reinterpret_cast<const uint4*>(base + (size_t)i * HD);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint4 t = p[c];
      const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[j]);
        x[8 * c + 2 * j] = mul * __low2float(h);
        x[8 * c + 2 * j + 1] = mul * __high2float(h);
      }
    }
  } else {
#pragma unroll
    for (int d = 0; d < HD; ++d) x[d] = 0.f;
  }
}

// Bounded mbarrier waits for one CTA: the first wait that expires raises a shared flag and every
// later wait returns at once, so a kernel always terminates; the flag ends up in the status word.
struct Waiter {
  int* dead;          // shared flag: a wait expired somewhere in this CTA (holds the site id, >= 1)
  __device__ __forceinline__ void wait(uint64_t* bar, uint32_t parity, int site = 1) {
    if (*reinterpret_cast<volatile int*>(dead)) return;
    if (!umma::mbar_wait(bar, parity)) *reinterpret_cast<volatile int*>(dead) = site;
  }
  // status bits to OR into the caller's word: the timeout flag plus the site id in bits 8..15
  __device__ __forceinline__ int status_bits() const {
    const int d = *reinterpret_cast<volatile int*>(dead);
    return d ? (OAL_STATUS_WAIT_TIMEOUT | ((d & 0xFF) << 8)) : 0;
  }
};


// 16-byte image chunk (8 consecutive e of one token) of U = [v | 1 | 0]
__device__ __forceinline__ uint4 u_image_chunk(const __nv_bfloat16* vrow, int ec, bool valid) {
  if (!valid) return make_uint4(0u, 0u, 0u, 0u);
  if (ec < VD / 8) return *reinterpret_cast<const uint4*>(vrow + 8 * ec);
  if (ec == VD / 8) return make_uint4(0x00003F80u, 0u, 0u, 0u);   // bf16(1.0) in element 0
  return make_uint4(0u, 0u, 0u, 0u);
}


}  // namespace oal

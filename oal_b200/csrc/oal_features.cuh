// Quadratic feature map of the chunked scan, laid out for the tensor cores.
//
// The reference materialises phi_k = [1, k_d, k_r k_c (r >= c)] and
// phi_q = [A, B_{g(d)} q_d, m C_{g(r)g(c)} q_r q_c] as [tokens, 2145] matrices in HBM
// (oal_attention/hd_block_gemm_feature_forward.py:225-253, :373-385; pair order
// oal_attention/hd_block_gemm_cache.py:105-121).  Here a feature tile only ever exists in
// shared memory, as 16-byte chunks of 8 features in bf16.  The feature order is internal (the
// running state is never exposed) and chosen so that a chunk multiplies one row element with eight
// adjacent column elements, which the packed bf16 / fp32 multiplies do two at a time:
//   pair chunk (cb, r), r = 8 cb .. 63:  features x[r] * x[8 cb + j], j = 0..7, zero where
//       8 cb + j > r.  Chunks are ordered by cb, then r: while cb stays the same the eight
//       column values stay in registers and only x[r] changes.
//       chunk index = 64 cb - 4 cb (cb - 1) + (r - 8 cb); 288 pair chunks
//   chunks 288..295  linear features d = 8 (chunk - 288) + j
//   chunk  296       [constant, 0 x 7]
//   chunks 297..303  zero padding
// 16 chunks (128 features) form a slab: 19 slabs, 2432 feature rows.
// Each thread owns one token and keeps its row in registers; every index in the generated code is a
// compile-time constant.  Pairs (x[8 cb + 2k], x[8 cb + 2k + 1]) are adjacent in the packed row, so a
// chunk is one broadcast of x[r] and four packed multiplies.
#pragma once

#include <utility>

#include "oal_common.cuh"
#include "oal_umma.cuh"

namespace oal {

constexpr int F_PAIR_CHUNKS = 288;
constexpr int F_LIN_CHUNK0 = 288;
constexpr int F_CONST_CHUNK = 296;
constexpr int F_CHUNKS = 304;
constexpr int F_SLABS = 19;
constexpr int F_ROWS = F_SLABS * 128;          // 2432
constexpr int CT = 128;                        // tokens per chunk of the scan
constexpr int SLAB_A_BYTES = 128 * CT * 2;     // feature slab tile  [16 chunks][128 tokens][8] bf16
constexpr int SLAB_S_BYTES = (EP / 8) * 128 * 16;   // state slab image [10][128 features][8 e] bf16

// Per-chunk fp32 state increments (and state-gradient increments) are stored like the bf16 state
// image, [slab][e / 8][128 rows][8 e], so that a warp whose lanes are consecutive feature rows writes
// and reads contiguous kilobytes.  Float index of (feature row f, column e) inside one chunk:
__host__ __device__ constexpr size_t state_inc_offset(int f, int e) {
  return ((size_t)((f >> 7) * (EP / 8) + (e >> 3)) * 128 + (f & 127)) * 8 + (e & 7);
}

// Position in the pair-chunk order.
struct PairCursor {
  int r, cb;
  __host__ __device__ constexpr void seek(int q) {      // q < F_PAIR_CHUNKS
    cb = 0;
    int base = 0;
    while (q >= base + HD - 8 * cb) {
      base += HD - 8 * cb;
      ++cb;
    }
    r = 8 * cb + (q - base);
  }
  // number of features of the chunk that exist (c <= r); 8 or more means all
  __host__ __device__ constexpr int valid() const { return r - 8 * cb + 1; }
};
__host__ __device__ constexpr PairCursor pair_pos(int q) {
  PairCursor pc{0, 0};
  pc.seek(q);
  return pc;
}

// What feature row f is: kind 0 pair (r, c; `live` false for the zero entries above the diagonal),
// 1 linear (r = dimension), 2 constant, 3 padding.
struct FeatureId {
  int kind, r, c;
  bool live;
};
__host__ __device__ inline FeatureId feature_id(int f) {
  const int q = f >> 3, j = f & 7;
  FeatureId id{3, 0, 0, false};
  if (q < F_PAIR_CHUNKS) {
    const PairCursor pc = pair_pos(q);
    id.kind = 0;
    id.r = pc.r;
    id.c = 8 * pc.cb + j;
    id.live = id.c <= id.r;
  } else if (q < F_CONST_CHUNK) {
    id.kind = 1;
    id.r = 8 * (q - F_LIN_CHUNK0) + j;
    id.live = true;
  } else if (q == F_CONST_CHUNK && j == 0) {
    id.kind = 2;
    id.live = true;
  }
  return id;
}

// Power of the query scale folded into the per-head coefficient table: the query-side kernels work
// on the unscaled q, so pair coefficients carry scale^2 and linear ones scale.
__host__ __device__ inline float feature_scale_factor(int f, float scale) {
  return f < 8 * F_PAIR_CHUNKS ? scale * scale : (f < 8 * F_CONST_CHUNK ? scale : 1.f);
}

__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// ---- coefficient-free chunk from the packed bf16 row  xp[k] = (x[2k], x[2k+1]) -------------------
// The product of two bf16 values rounded once to bf16 is what an fp32 multiply followed by a
// conversion gives, so the packed multiply yields those bits at two features per instruction.
template <int Q>
__device__ __forceinline__ uint4 raw_chunk(const uint32_t (&xp)[HD / 2]) {
  if constexpr (Q < F_PAIR_CHUNKS) {
    constexpr PairCursor pc = pair_pos(Q);
    constexpr int nv = pc.valid();
    const uint32_t w = xp[pc.r / 2];
    const uint32_t xr2 = __byte_perm(w, w, (pc.r & 1) ? 0x3232u : 0x1010u);
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t mask = (2 * k < nv ? 0x0000FFFFu : 0u) | (2 * k + 1 < nv ? 0xFFFF0000u : 0u);
      o[k] = mask == 0u ? 0u : (mul_bf16x2(xr2, xp[4 * pc.cb + k]) & mask);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
  } else if constexpr (Q < F_CONST_CHUNK) {
    constexpr int k = 4 * (Q - F_LIN_CHUNK0);
    return make_uint4(xp[k], xp[k + 1], xp[k + 2], xp[k + 3]);
  } else if constexpr (Q == F_CONST_CHUNK) {
    return make_uint4(0x00003F80u, 0u, 0u, 0u);   // bf16(1.0) in element 0
  } else {
    return make_uint4(0u, 0u, 0u, 0u);
  }
}

// ---- chunk times the per-head coefficient table (query side of the forward) -----------------------
//   xq   : fp32 row as packed pairs, xq[k] = (x[2k], x[2k+1]), unscaled
//   coef : table of the head in feature order, query scale folded in, zero above the diagonal and in
//          the padding; every lane reads the same address, so global memory through L1 is fine
__device__ __forceinline__ uint4 pack_pairs_bf16(const f32x2 (&f)[4]) {
  uint32_t o[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float lo, hi;
    f2_unpack(f[k], lo, hi);
    o[k] = umma::pack_bf16(lo, hi);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

template <int Q>
__device__ __forceinline__ uint4 coef_chunk(const f32x2 (&xq)[HD / 2], const float* coef) {
  if constexpr (Q <= F_CONST_CHUNK) {
    const ulonglong2 ca = *reinterpret_cast<const ulonglong2*>(coef + 8 * Q);
    const ulonglong2 cb2 = *reinterpret_cast<const ulonglong2*>(coef + 8 * Q + 4);
    const f32x2 cf[4] = {ca.x, ca.y, cb2.x, cb2.y};
    f32x2 f[4];
    if constexpr (Q < F_PAIR_CHUNKS) {
      constexpr PairCursor pc = pair_pos(Q);
      float lo, hi;
      f2_unpack(xq[pc.r / 2], lo, hi);
      const f32x2 xr2 = f2_bcast((pc.r & 1) ? hi : lo);
#pragma unroll
      for (int k = 0; k < 4; ++k) f[k] = f2_mul(f2_mul(xr2, xq[4 * pc.cb + k]), cf[k]);
    } else if constexpr (Q < F_CONST_CHUNK) {
#pragma unroll
      for (int k = 0; k < 4; ++k) f[k] = f2_mul(xq[4 * (Q - F_LIN_CHUNK0) + k], cf[k]);
    } else {
      f[0] = cf[0];          // (A, 0): the table is zero in the padding
      f[1] = f[2] = f[3] = 0ull;
    }
    return pack_pairs_bf16(f);
  } else {
    return make_uint4(0u, 0u, 0u, 0u);
  }
}

// Threads per CTA of the kernels whose threads split a slab as (token, half of the 16 chunks).
constexpr int GEN_THREADS = 256;

// Chunks [J0, J0 + NJ) of slab S of one token into the slab tile ([16 chunks][128 tokens] x 16 bytes);
// `tile` points at the token's column.
template <int S, int J0, int... J>
__device__ __forceinline__ void raw_chunks_impl(const uint32_t (&xp)[HD / 2], uint4* tile,
                                                std::integer_sequence<int, J...>) {
  ((tile[(J0 + J) * CT] = raw_chunk<S * 16 + J0 + J>(xp)), ...);
}
template <int S, int J0, int... J>
__device__ __forceinline__ void coef_chunks_impl(const f32x2 (&xq)[HD / 2], const float* coef, uint4* tile,
                                                 std::integer_sequence<int, J...>) {
  ((tile[(J0 + J) * CT] = coef_chunk<S * 16 + J0 + J>(xq, coef)), ...);
}

#define OAL_SLAB_SWITCH(s, CASE)                                                                      \
  switch (s) {                                                                                        \
    CASE(0) CASE(1) CASE(2) CASE(3) CASE(4) CASE(5) CASE(6) CASE(7) CASE(8) CASE(9) CASE(10) CASE(11) \
    CASE(12) CASE(13) CASE(14) CASE(15) CASE(16) CASE(17) CASE(18)                                    \
    default: break;                                                                                   \
  }
static_assert(F_SLABS == 19, "OAL_SLAB_SWITCH enumerates the slabs");

// All 16 chunks of slab s (s is a run-time value; the bodies are static).
__device__ __forceinline__ void write_slab_raw(int s, const uint32_t (&xp)[HD / 2], uint4* tile) {
#define OAL_CASE(S) case S: raw_chunks_impl<S, 0>(xp, tile, std::make_integer_sequence<int, 16>{}); break;
  OAL_SLAB_SWITCH(s, OAL_CASE)
#undef OAL_CASE
}
// Half of the chunks of slab s: half 0 = chunks 0..7, half 1 = chunks 8..15.
template <int J0>
__device__ __forceinline__ void write_half_slab_raw_impl(int s, const uint32_t (&xp)[HD / 2], uint4* tile) {
#define OAL_CASE(S) case S: raw_chunks_impl<S, J0>(xp, tile, std::make_integer_sequence<int, 8>{}); break;
  OAL_SLAB_SWITCH(s, OAL_CASE)
#undef OAL_CASE
}
__device__ __forceinline__ void write_half_slab_raw(int s, int half, const uint32_t (&xp)[HD / 2], uint4* tile) {
  if (half == 0) write_half_slab_raw_impl<0>(s, xp, tile);
  else write_half_slab_raw_impl<8>(s, xp, tile);
}
__device__ __forceinline__ void write_half_slab_coef(int s, int half, const f32x2 (&xq)[HD / 2], const float* coef,
                                                     uint4* tile) {
#define OAL_CASE(S)                                                                                 \
  case S:                                                                                           \
    if (half == 0) coef_chunks_impl<S, 0>(xq, coef, tile, std::make_integer_sequence<int, 8>{});    \
    else coef_chunks_impl<S, 8>(xq, coef, tile, std::make_integer_sequence<int, 8>{});              \
    break;
  OAL_SLAB_SWITCH(s, OAL_CASE)
#undef OAL_CASE
}

// The row stays the same while a kernel walks the slabs, and every feature is a pure function of it:
// without this barrier the compiler hoists the features of all slabs out of the slab loop and spills
// them.  Costs no instruction.
__device__ __forceinline__ void keep_in_loop(uint32_t (&xp)[HD / 2]) {
#pragma unroll
  for (int w = 0; w < HD / 2; ++w) asm volatile("" : "+r"(xp[w]));
}
__device__ __forceinline__ void keep_in_loop(f32x2 (&xq)[HD / 2]) {
#pragma unroll
  for (int w = 0; w < HD / 2; ++w) asm volatile("" : "+l"(xq[w]));
}

// Row `i` (or zeros when i >= N) of a bf16 [.., N, 64] tensor as packed words / as fp32 pairs.
__device__ __forceinline__ void load_row_packed(uint32_t (&xp)[HD / 2], const __nv_bfloat16* base, int i, int N) {
  if (i < N) {
    const uint4* p = reinterpret_cast<const uint4*>(base + (size_t)i * HD);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint4 t = p[c];
      xp[4 * c] = t.x;
      xp[4 * c + 1] = t.y;
      xp[4 * c + 2] = t.z;
      xp[4 * c + 3] = t.w;
    }
  } else {
#pragma unroll
    for (int w = 0; w < HD / 2; ++w) xp[w] = 0u;
  }
}
__device__ __forceinline__ void unpack_row(const uint32_t (&xp)[HD / 2], f32x2 (&xq)[HD / 2]) {
#pragma unroll
  for (int w = 0; w < HD / 2; ++w) xq[w] = f2_pack(bf16_lo(xp[w]), bf16_hi(xp[w]));
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
    if (umma::mbar_test(bar, parity)) return;           // already complete: the common case costs one probe
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

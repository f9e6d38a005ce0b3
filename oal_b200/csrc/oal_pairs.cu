// Token-pair kernels (fp32 CUDA-core arithmetic).
//
// They evaluate the kernel weight of a (query i, key j) pair directly from the
// per-group dot products
//     s_g(i,j) = sum_{d in g} (scale q_i[d]) k_j[d]
//     w(i,j)   = A + sum_g B_g s_g + sum_{g,g'} C_gg' s_g s_g'
// and accumulate  num_i, den_i = sum_{j<=i} w(i,j) [v_j, 1]  together with the
// first-order gradients.  `window` selects the key range of a query:
//   window == 0 : the whole causal prefix -> the exact fp32 mode of the operator
//                 (reference semantics: oal_attention/grouped_reference.py:102-178,
//                 dense statement tests/operators/test_grouped_quadratic.py:31-84);
//   window  > 0 : only keys in the query's own chunk of `window` tokens -> the
//                 intra-chunk term of the chunked scan, added onto the cross-chunk
//                 term that the state kernels left in num/den (reference:
//                 oal_attention/hd_block_gemm_runtime.py:530-597 local score, tril,
//                 score x U; backward oal_attention/hd_block_gemm_backward_wave.py:253-476).
// Dimensions of a head are visited in group-sorted order (dim_perm), so a group is
// a contiguous range and s_g needs no gather.
#include "oal_common.cuh"
#include "oal_kernels.h"

namespace oal {

namespace {

constexpr int TP = 64;       // pair tile edge
constexpr int P65 = 65;      // row pitch that keeps column walks conflict-free

__device__ __forceinline__ int tri_index(int g, int g2) {   // g <= g2 < GMAX
  return g * GMAX - (g * (g - 1)) / 2 + (g2 - g);
}

template <int GCAP>
struct Coefs {
  float A;
  float B[GCAP];
  float C[GCAP * GCAP];
};

template <int GCAP>
__device__ __forceinline__ void load_coefs(Coefs<GCAP>& c, const PairArgs& a, int h, int tid) {
  if (tid == 0) c.A = a.A[h];
  for (int x = tid; x < GCAP; x += blockDim.x) c.B[x] = x < a.G ? a.Bc[h * a.G + x] : 0.f;
  for (int x = tid; x < GCAP * GCAP; x += blockDim.x) {
    int g = x / GCAP, g2 = x % GCAP;
    c.C[x] = (g < a.G && g2 < a.G) ? a.Cc[(h * a.G + g) * a.G + g2] : 0.f;
  }
}

// rows [row0, row0+64) of a [.., N, 64] tensor -> smem [64][65], columns permuted, scaled
__device__ __forceinline__ void load_tile_perm(float* dst, const void* src, size_t base, int row0,
                                               int N, int dt, float mul, const int* perm, int tid) {
  for (int x = tid; x < TP * HD; x += 256) {
    int r = x >> 6, p = x & 63, i = row0 + r;
    float v = 0.f;
    if (i < N) v = mul * load_elem(src, base + (size_t)i * HD + perm[p], dt);
    dst[r * P65 + p] = v;
  }
}

// ---------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------
template <int GCAP>
__global__ void __launch_bounds__(256) fwd_pairs_kernel(const PairArgs a) {
  extern __shared__ __align__(16) float sm[];
  float* Qs = sm;                 // [64][65]  scaled, permuted
  float* Ks = Qs + TP * P65;      // [64][65]  permuted
  float* Us = Ks + TP * P65;      // [64][80]  [v | 1 | 0]
  float* WT = Us + TP * EP;       // [64 j][64 i]
  __shared__ HeadGroups hg;
  __shared__ Coefs<GCAP> co;
  const int tid = threadIdx.x, it = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (a.Hq / a.Hkv);
  const int N = a.N, i0 = it * TP;
  load_head_groups(hg, a.dim_perm, a.group_start, h, tid, 256);
  load_coefs<GCAP>(co, a, h, tid);
  __syncthreads();
  const size_t qbase = (size_t)(b * a.Hq + h) * N * HD;
  const size_t kbase = (size_t)(b * a.Hkv + kvh) * N * HD;
  load_tile_perm(Qs, a.q, qbase, i0, N, a.io_dt, a.scale, hg.perm, tid);

  const int ty = tid >> 4, tx = tid & 15;
  float acc[4][5];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 5; ++c) acc[r][c] = 0.f;

  const int jt_begin = a.window ? ((i0 / a.window) * a.window) / TP : 0;
  const int il = tid & 63, jb = tid >> 6;
  for (int jt = jt_begin; jt <= it; ++jt) {
    const int j0 = jt * TP;
    load_tile_perm(Ks, a.k, kbase, j0, N, a.io_dt, 1.f, hg.perm, tid);
    for (int x = tid; x < TP * EP; x += 256) {
      int r = x / EP, e = x % EP, j = j0 + r;
      float v = 0.f;
      if (j < N) v = e < VD ? load_elem(a.v, kbase + (size_t)j * VD + e, a.io_dt) : (e == VD ? 1.f : 0.f);
      Us[x] = v;
    }
    __syncthreads();
    // pair phase: thread = (query row il, key slots jb + 4m)
#pragma unroll 1
    for (int pz = 0; pz < 2; ++pz) {
      float s[8][GCAP];
#pragma unroll
      for (int m = 0; m < 8; ++m)
#pragma unroll
        for (int g = 0; g < GCAP; ++g) s[m][g] = 0.f;
#pragma unroll
      for (int g = 0; g < GCAP; ++g) {
        const int d1 = hg.start[g + 1];
        for (int d = hg.start[g]; d < d1; ++d) {
          const float qv = Qs[il * P65 + d];
#pragma unroll
          for (int m = 0; m < 8; ++m) s[m][g] = fmaf(qv, Ks[(jb + 4 * (pz * 8 + m)) * P65 + d], s[m][g]);
        }
      }
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        const int jl = jb + 4 * (pz * 8 + m);
        float w = co.A;
#pragma unroll
        for (int g = 0; g < GCAP; ++g) {
          float t = co.B[g];
#pragma unroll
          for (int g2 = 0; g2 < GCAP; ++g2) t = fmaf(co.C[g * GCAP + g2], s[m][g2], t);
          w = fmaf(s[m][g], t, w);
        }
        const int gi = i0 + il, gj = j0 + jl;
        WT[jl * TP + il] = (gj <= gi && gi < N) ? w : 0.f;
      }
    }
    __syncthreads();
    // Y[i][e] += sum_j W[i][j] U[j][e]
#pragma unroll 4
    for (int j = 0; j < TP; ++j) {
      const float4 av = *reinterpret_cast<const float4*>(&WT[j * TP + 4 * ty]);
      const float ar[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
      for (int c = 0; c < 5; ++c) {
        const float bv = Us[j * EP + 5 * tx + c];
#pragma unroll
        for (int r = 0; r < 4; ++r) acc[r][c] = fmaf(ar[r], bv, acc[r][c]);
      }
    }
    __syncthreads();
  }
  // epilogue: stage Y in shared memory, add the cross-chunk part, normalise
  float* Ys = Us;
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 5; ++c) Ys[(4 * ty + r) * EP + 5 * tx + c] = acc[r][c];
  __syncthreads();
  int flags = 0;
  for (int x = tid; x < TP * 16; x += 256) {
    const int r = x >> 4, c4 = (x & 15) * 4, i = i0 + r;
    if (i >= N) continue;
    const size_t row = (size_t)(b * a.Hq + h) * N + i;
    float den = Ys[r * EP + VD];
    if (a.accumulate) den += a.den[row];
    float nv[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) nv[c] = Ys[r * EP + c4 + c];
    if (a.accumulate) {
      const float4 o = *reinterpret_cast<const float4*>(a.num + row * VD + c4);
      nv[0] += o.x; nv[1] += o.y; nv[2] += o.z; nv[3] += o.w;
    }
    *reinterpret_cast<float4*>(a.num + row * VD + c4) = make_float4(nv[0], nv[1], nv[2], nv[3]);
    const float dn = fmaxf(den, a.floor);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      if (!finite_f(nv[c])) flags |= OAL_STATUS_NONFINITE;
      store_elem(a.out, row * VD + c4 + c, a.out_dt, nv[c] / dn);
    }
    if (c4 == 0) {
      if (!finite_f(den)) flags |= OAL_STATUS_NONFINITE;
      else if (!(den > 0.f)) flags |= OAL_STATUS_DENOMINATOR;
    }
  }
  __syncthreads();           // every thread has read its old den before any is overwritten
  for (int r = tid; r < TP; r += 256) {
    const int i = i0 + r;
    if (i >= N) continue;
    const size_t row = (size_t)(b * a.Hq + h) * N + i;
    float den = Ys[r * EP + VD];
    if (a.accumulate) den += a.den[row];
    a.den[row] = den;
  }
  if (flags) atomicOr(a.status, flags);
}

// ---------------------------------------------------------------------------
// backward, query side: dq and the coefficient partial sums
// ---------------------------------------------------------------------------
template <int GCAP>
struct BwdCfg {
  static constexpr int SUB = GCAP > 8 ? 16 : 32;   // keys (queries) per sub-tile
  static constexpr int MB = SUB / 4;               // pairs per thread per sub-tile
};

template <int GCAP>
__device__ __forceinline__ void block_reduce_coefs(float cA, const float (&cB)[GCAP],
                                                   const float (&cC)[GCAP * (GCAP + 1) / 2],
                                                   float* red /* [8][NCOEF] smem */, float* dst,
                                                   int tid) {
  const int warp = tid >> 5, lane = tid & 31;
  auto wsum = [](float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
  };
  for (int x = lane; x < NCOEF; x += 32) red[warp * NCOEF + x] = 0.f;
  __syncwarp();
  float v = wsum(cA);
  if (lane == 0) red[warp * NCOEF + 0] = v;
#pragma unroll
  for (int g = 0; g < GCAP; ++g) {
    v = wsum(cB[g]);
    if (lane == 0) red[warp * NCOEF + 1 + g] = v;
  }
  int idx = 0;
#pragma unroll
  for (int g = 0; g < GCAP; ++g)
#pragma unroll
    for (int g2 = g; g2 < GCAP; ++g2) {
      v = wsum(cC[idx]);
      if (lane == 0) red[warp * NCOEF + 1 + GMAX + tri_index(g, g2)] = v;
      ++idx;
    }
  __syncthreads();
  for (int x = tid; x < NCOEF; x += 256) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w * NCOEF + x];
    dst[x] = t;
  }
}

template <int GCAP>
__global__ void __launch_bounds__(256) bwd_q_pairs_kernel(const PairArgs a) {
  constexpr int SUB = BwdCfg<GCAP>::SUB, MB = BwdCfg<GCAP>::MB;
  extern __shared__ __align__(16) float sm[];
  float* Qs = sm;                     // [64][65]
  float* Ks = Qs + TP * P65;          // [64][65]
  float* gT = Ks + TP * P65;          // [65 e][64 i]
  float* UT = gT + E1 * TP;           // [65 e][64 j]
  float* dWs = UT + E1 * TP;          // [64 i][65]
  float* DS = dWs + TP * P65;         // [GCAP][SUB j][64 i]   (also reduction scratch at the end)
  __shared__ HeadGroups hg;
  __shared__ Coefs<GCAP> co;
  const int tid = threadIdx.x, it = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (a.Hq / a.Hkv);
  const int N = a.N, i0 = it * TP;
  load_head_groups(hg, a.dim_perm, a.group_start, h, tid, 256);
  load_coefs<GCAP>(co, a, h, tid);
  __syncthreads();
  const size_t qbase = (size_t)(b * a.Hq + h) * N * HD;
  const size_t kbase = (size_t)(b * a.Hkv + kvh) * N * HD;
  const size_t gbase = (size_t)(b * a.Hq + h) * N * EP;
  load_tile_perm(Qs, a.q, qbase, i0, N, a.io_dt, a.scale, hg.perm, tid);
  for (int x = tid; x < E1 * TP; x += 256) {
    int r = x / E1, e = x % E1, i = i0 + r;
    gT[e * TP + r] = i < N ? a.g[gbase + (size_t)i * EP + e] : 0.f;
  }
  const int ty = tid >> 4, tx = tid & 15;
  int gcol[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) gcol[c] = hg.group_of[4 * tx + c];
  float acc[4][4];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[r][c] = 0.f;
  float cA = 0.f, cB[GCAP], cC[GCAP * (GCAP + 1) / 2];
#pragma unroll
  for (int g = 0; g < GCAP; ++g) cB[g] = 0.f;
#pragma unroll
  for (int x = 0; x < GCAP * (GCAP + 1) / 2; ++x) cC[x] = 0.f;

  const int jt_begin = a.window ? ((i0 / a.window) * a.window) / TP : 0;
  const int il = tid & 63, jb = tid >> 6;
  for (int jt = jt_begin; jt <= it; ++jt) {
    const int j0 = jt * TP;
    load_tile_perm(Ks, a.k, kbase, j0, N, a.io_dt, 1.f, hg.perm, tid);
    for (int x = tid; x < E1 * TP; x += 256) {
      int r = x / E1, e = x % E1, j = j0 + r;
      float v = 0.f;
      if (j < N) v = e < VD ? load_elem(a.v, kbase + (size_t)j * VD + e, a.io_dt) : 1.f;
      UT[e * TP + r] = v;
    }
    __syncthreads();
    {  // dW[i][j] = g_i . u_j
      float d[4][4];
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) d[r][c] = 0.f;
#pragma unroll 5
      for (int e = 0; e < E1; ++e) {
        const float4 av = *reinterpret_cast<const float4*>(&gT[e * TP + 4 * ty]);
        const float4 bv = *reinterpret_cast<const float4*>(&UT[e * TP + 4 * tx]);
        const float ar[4] = {av.x, av.y, av.z, av.w}, br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
          for (int c = 0; c < 4; ++c) d[r][c] = fmaf(ar[r], br[c], d[r][c]);
      }
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) dWs[(4 * ty + r) * P65 + 4 * tx + c] = d[r][c];
    }
    __syncthreads();
#pragma unroll 1
    for (int js = 0; js < TP / SUB; ++js) {
      {
        float s[MB][GCAP];
#pragma unroll
        for (int m = 0; m < MB; ++m)
#pragma unroll
          for (int g = 0; g < GCAP; ++g) s[m][g] = 0.f;
#pragma unroll
        for (int g = 0; g < GCAP; ++g) {
          const int d1 = hg.start[g + 1];
          for (int d = hg.start[g]; d < d1; ++d) {
            const float qv = Qs[il * P65 + d];
#pragma unroll
            for (int m = 0; m < MB; ++m)
              s[m][g] = fmaf(qv, Ks[(js * SUB + jb + 4 * m) * P65 + d], s[m][g]);
          }
        }
#pragma unroll
        for (int m = 0; m < MB; ++m) {
          const int jl = js * SUB + jb + 4 * m;
          const int gi = i0 + il, gj = j0 + jl;
          const float dw = (gj <= gi && gi < N) ? dWs[il * P65 + jl] : 0.f;
          cA += dw;
          int idx = 0;
#pragma unroll
          for (int g = 0; g < GCAP; ++g) {
            float t = co.B[g];
#pragma unroll
            for (int g2 = 0; g2 < GCAP; ++g2) t = fmaf(2.f * co.C[g * GCAP + g2], s[m][g2], t);
            DS[(g * SUB + jb + 4 * m) * TP + il] = dw * t;
            const float ws = dw * s[m][g];
            cB[g] += ws;
#pragma unroll
            for (int g2 = g; g2 < GCAP; ++g2) {
              cC[idx] = fmaf(ws, s[m][g2], cC[idx]);
              ++idx;
            }
          }
        }
      }
      __syncthreads();
      // dq~[i][p] += sum_j ds_{g(p)}(i,j) k[j][p]
#pragma unroll 2
      for (int jj = 0; jj < SUB; ++jj) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float4 av = *reinterpret_cast<const float4*>(&DS[(gcol[c] * SUB + jj) * TP + 4 * ty]);
          const float bv = Ks[(js * SUB + jj) * P65 + 4 * tx + c];
          acc[0][c] = fmaf(av.x, bv, acc[0][c]);
          acc[1][c] = fmaf(av.y, bv, acc[1][c]);
          acc[2][c] = fmaf(av.z, bv, acc[2][c]);
          acc[3][c] = fmaf(av.w, bv, acc[3][c]);
        }
      }
      __syncthreads();
    }
  }
  if (a.dq) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int i = i0 + 4 * ty + r;
      if (i >= N) continue;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const size_t o = qbase + (size_t)i * HD + hg.perm[4 * tx + c];
        float v = a.scale * acc[r][c];
        if (a.dq_init) v += a.dq_init[o];
        store_elem(a.dq, o, a.io_dt, v);
      }
    }
  }
  if (a.coef_partial) {
    float* dst = a.coef_partial + ((size_t)(b * a.Hq + h) * gridDim.x + it) * NCOEF;
    block_reduce_coefs<GCAP>(cA, cB, cC, DS, dst, tid);
  }
}

// ---------------------------------------------------------------------------
// backward, key/value side: dk and dv (sums over the query heads of the KV head)
// ---------------------------------------------------------------------------
template <int GCAP>
__global__ void __launch_bounds__(256) bwd_kv_pairs_kernel(const PairArgs a) {
  constexpr int SUB = BwdCfg<GCAP>::SUB, MB = BwdCfg<GCAP>::MB;
  extern __shared__ __align__(16) float sm[];
  float* Ks = sm;                     // [64 j][65] permuted for the current head
  float* Qs = Ks + TP * P65;          // [64 i][65]
  float* dWs = Qs + TP * P65;         // [64 i][65]
  float* UT = dWs + TP * P65;         // [65 e][64 j]
  float* gT = UT + E1 * TP;           // [65 e][64 i]
  float* gs = gT + E1 * TP;           // [64 i][80]
  float* Ws = gs + TP * EP;           // [SUB i][64 j]
  float* DS = Ws + SUB * TP;          // [GCAP][SUB i][64 j]
  float* dkacc = DS + GCAP * SUB * TP;  // [64 j][64 d]  original dimension order
  __shared__ HeadGroups hg;
  __shared__ Coefs<GCAP> co;
  const int tid = threadIdx.x, jt = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int rep = a.Hq / a.Hkv;
  const int N = a.N, j0 = jt * TP;
  const size_t kbase = (size_t)(b * a.Hkv + kvh) * N * HD;
  const int ty = tid >> 4, tx = tid & 15;
  for (int x = tid; x < E1 * TP; x += 256) {
    int r = x / E1, e = x % E1, j = j0 + r;
    float v = 0.f;
    if (j < N) v = e < VD ? load_elem(a.v, kbase + (size_t)j * VD + e, a.io_dt) : 1.f;
    UT[e * TP + r] = v;
  }
  float adu[4][5];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 5; ++c) adu[r][c] = 0.f;
  const int last_tile = (N - 1) / TP;
  const int it_end = a.window ? min(last_tile, ((j0 / a.window + 1) * a.window) / TP - 1) : last_tile;
  const int jl = tid & 63, ib = tid >> 6;

  for (int hh = 0; hh < rep; ++hh) {
    const int h = kvh * rep + hh;
    __syncthreads();
    load_head_groups(hg, a.dim_perm, a.group_start, h, tid, 256);
    load_coefs<GCAP>(co, a, h, tid);
    __syncthreads();
    load_tile_perm(Ks, a.k, kbase, j0, N, a.io_dt, 1.f, hg.perm, tid);
    int gcol[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) gcol[c] = hg.group_of[4 * tx + c];
    float adk[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) adk[r][c] = 0.f;
    const size_t qbase = (size_t)(b * a.Hq + h) * N * HD;
    const size_t gbase = (size_t)(b * a.Hq + h) * N * EP;
    for (int it = jt; it <= it_end; ++it) {
      const int i0 = it * TP;
      load_tile_perm(Qs, a.q, qbase, i0, N, a.io_dt, a.scale, hg.perm, tid);
      for (int x = tid; x < TP * EP; x += 256) {
        int r = x / EP, e = x % EP, i = i0 + r;
        const float v = i < N ? a.g[gbase + (size_t)i * EP + e] : 0.f;
        gs[x] = v;
        if (e < E1) gT[e * TP + r] = v;
      }
      __syncthreads();
      {
        float d[4][4];
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
          for (int c = 0; c < 4; ++c) d[r][c] = 0.f;
#pragma unroll 5
        for (int e = 0; e < E1; ++e) {
          const float4 av = *reinterpret_cast<const float4*>(&gT[e * TP + 4 * ty]);
          const float4 bv = *reinterpret_cast<const float4*>(&UT[e * TP + 4 * tx]);
          const float ar[4] = {av.x, av.y, av.z, av.w}, br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
          for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c) d[r][c] = fmaf(ar[r], br[c], d[r][c]);
        }
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
          for (int c = 0; c < 4; ++c) dWs[(4 * ty + r) * P65 + 4 * tx + c] = d[r][c];
      }
      __syncthreads();
#pragma unroll 1
      for (int is = 0; is < TP / SUB; ++is) {
        {
          float s[MB][GCAP];
#pragma unroll
          for (int m = 0; m < MB; ++m)
#pragma unroll
            for (int g = 0; g < GCAP; ++g) s[m][g] = 0.f;
#pragma unroll
          for (int g = 0; g < GCAP; ++g) {
            const int d1 = hg.start[g + 1];
            for (int d = hg.start[g]; d < d1; ++d) {
              const float kv = Ks[jl * P65 + d];
#pragma unroll
              for (int m = 0; m < MB; ++m)
                s[m][g] = fmaf(Qs[(is * SUB + ib + 4 * m) * P65 + d], kv, s[m][g]);
            }
          }
#pragma unroll
          for (int m = 0; m < MB; ++m) {
            const int ii = ib + 4 * m, ilq = is * SUB + ii;
            const int gi = i0 + ilq, gj = j0 + jl;
            const bool valid = gj <= gi && gi < N;
            const float dw = valid ? dWs[ilq * P65 + jl] : 0.f;
            float w = co.A;
#pragma unroll
            for (int g = 0; g < GCAP; ++g) {
              float t = 0.f;
#pragma unroll
              for (int g2 = 0; g2 < GCAP; ++g2) t = fmaf(co.C[g * GCAP + g2], s[m][g2], t);
              w = fmaf(s[m][g], co.B[g] + t, w);
              DS[(g * SUB + ii) * TP + jl] = dw * (co.B[g] + 2.f * t);
            }
            Ws[ii * TP + jl] = valid ? w : 0.f;
          }
        }
        __syncthreads();
#pragma unroll 2
        for (int ii = 0; ii < SUB; ++ii) {
          const int ilq = is * SUB + ii;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const float4 av = *reinterpret_cast<const float4*>(&DS[(gcol[c] * SUB + ii) * TP + 4 * ty]);
            const float bv = Qs[ilq * P65 + 4 * tx + c];
            adk[0][c] = fmaf(av.x, bv, adk[0][c]);
            adk[1][c] = fmaf(av.y, bv, adk[1][c]);
            adk[2][c] = fmaf(av.z, bv, adk[2][c]);
            adk[3][c] = fmaf(av.w, bv, adk[3][c]);
          }
          const float4 wv = *reinterpret_cast<const float4*>(&Ws[ii * TP + 4 * ty]);
          const float wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
          for (int c = 0; c < 5; ++c) {
            const float bv = gs[ilq * EP + 5 * tx + c];
#pragma unroll
            for (int r = 0; r < 4; ++r) adu[r][c] = fmaf(wr[r], bv, adu[r][c]);
          }
        }
        __syncthreads();
      }
    }
    // fold this head's dk (permuted columns) into the shared accumulator
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float* dst = &dkacc[(4 * ty + r) * HD + hg.perm[4 * tx + c]];
        *dst = hh == 0 ? adk[r][c] : *dst + adk[r][c];
      }
  }
  __syncthreads();
  if (a.dk) {
    for (int x = tid; x < TP * HD; x += 256) {
      const int r = x >> 6, j = j0 + r;
      if (j >= N) continue;
      const size_t o = kbase + (size_t)j * HD + (x & 63);
      float v = dkacc[x];
      if (a.dk_init) v += a.dk_init[o];
      store_elem(a.dk, o, a.io_dt, v);
    }
  }
  if (a.dv) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int j = j0 + 4 * ty + r;
      if (j >= N) continue;
#pragma unroll
      for (int c = 0; c < 5; ++c) {
        const int e = 5 * tx + c;
        if (e >= VD) continue;
        const size_t o = kbase + (size_t)j * VD + e;
        float v = adu[r][c];
        if (a.dv_init) v += a.dv_init[o];
        store_elem(a.dv, o, a.io_dt, v);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// normalisation VJP: g_i = [dnum_i, dden_i]
//   den' = max(den, floor); dnum = dout/den' + grad_num;
//   dden = -(dout . num)/den'^2 [den >= floor] + grad_den
// (oal_attention/hd_block_gemm_backward.py:272-307)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) norm_vjp_kernel(const void* grad_out, int out_dt,
                                                       const float* grad_num, const float* grad_den,
                                                       const float* num, const float* den,
                                                       float floor_v, float* g, size_t rows) {
  const size_t row = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float dn = den[row];
  const float dw = fmaxf(dn, floor_v);
  float gv[2] = {0.f, 0.f}, dot = 0.f;
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
  if (lane < EP - VD) {
    float v = 0.f;
    if (lane == 0) {
      if (grad_out) v = (dn >= floor_v) ? -(dot / dw) / dw : 0.f;
      if (grad_den) v += grad_den[row];
    }
    g[row * EP + VD + lane] = v;
  }
}

// Fixed-order reduction of the per-tile coefficient partial sums.
//   partial [B][Hq][tiles][NCOEF]; extra [Hq][NCOEF] (already summed over the batch) or null
__global__ void reduce_coefs_kernel(const float* p0, int tiles0, const float* extra, int B, int Hq, int G,
                                    float* dA, float* dB, float* dC) {
  const int h = blockIdx.x;
  for (int x = threadIdx.x; x < 1 + G + G * G; x += blockDim.x) {
    int slot;
    if (x == 0) slot = 0;
    else if (x <= G) slot = x;            // 1 + g
    else {
      int g = (x - 1 - G) / G, g2 = (x - 1 - G) % G;
      slot = 1 + GMAX + (g <= g2 ? tri_index(g, g2) : tri_index(g2, g));
    }
    float t = extra ? extra[(size_t)h * NCOEF + slot] : 0.f;
    for (int b = 0; b < B; ++b)
      for (int i = 0; i < tiles0; ++i) t += p0[((size_t)(b * Hq + h) * tiles0 + i) * NCOEF + slot];
    if (x == 0) dA[h] = t;
    else if (x <= G) dB[h * G + x - 1] = t;
    else dC[(size_t)h * G * G + (x - 1 - G)] = t;
  }
}

template <int GCAP>
size_t fwd_smem() { return sizeof(float) * (2 * TP * P65 + TP * EP + TP * TP); }
template <int GCAP>
size_t bwd_q_smem() {
  return sizeof(float) * (3 * TP * P65 + 2 * E1 * TP + GCAP * BwdCfg<GCAP>::SUB * TP);
}
template <int GCAP>
size_t bwd_kv_smem() {
  return sizeof(float) * (3 * TP * P65 + 2 * E1 * TP + TP * EP + BwdCfg<GCAP>::SUB * TP +
                          GCAP * BwdCfg<GCAP>::SUB * TP + TP * HD);
}

template <int GCAP>
cudaError_t launch_pairs(const PairArgs& a, int which, cudaStream_t st) {
  const int tiles = (a.N + TP - 1) / TP;
  cudaError_t e;
  if (which == 0) {
    e = cudaFuncSetAttribute(fwd_pairs_kernel<GCAP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)fwd_smem<GCAP>());
    if (e != cudaSuccess) return e;
    fwd_pairs_kernel<GCAP><<<dim3(tiles, a.Hq, a.B), 256, fwd_smem<GCAP>(), st>>>(a);
  } else if (which == 1) {
    e = cudaFuncSetAttribute(bwd_q_pairs_kernel<GCAP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)bwd_q_smem<GCAP>());
    if (e != cudaSuccess) return e;
    bwd_q_pairs_kernel<GCAP><<<dim3(tiles, a.Hq, a.B), 256, bwd_q_smem<GCAP>(), st>>>(a);
  } else {
    e = cudaFuncSetAttribute(bwd_kv_pairs_kernel<GCAP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)bwd_kv_smem<GCAP>());
    if (e != cudaSuccess) return e;
    bwd_kv_pairs_kernel<GCAP><<<dim3(tiles, a.Hkv, a.B), 256, bwd_kv_smem<GCAP>(), st>>>(a);
  }
  return cudaGetLastError();
}

cudaError_t dispatch_pairs(const PairArgs& a, int which, cudaStream_t st) {
  if (a.G <= 4) return launch_pairs<4>(a, which, st);
  if (a.G <= 8) return launch_pairs<8>(a, which, st);
  return launch_pairs<16>(a, which, st);
}

}  // namespace

cudaError_t pairs_forward(const PairArgs& a, cudaStream_t st) { return dispatch_pairs(a, 0, st); }
cudaError_t pairs_backward_q(const PairArgs& a, cudaStream_t st) { return dispatch_pairs(a, 1, st); }
cudaError_t pairs_backward_kv(const PairArgs& a, cudaStream_t st) { return dispatch_pairs(a, 2, st); }
int pairs_tiles(int n) { return (n + TP - 1) / TP; }

cudaError_t norm_vjp(const void* grad_out, int out_dt, const float* grad_num, const float* grad_den,
                     const float* num, const float* den, float floor_v, float* g, size_t rows,
                     cudaStream_t st) {
  norm_vjp_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(grad_out, out_dt, grad_num, grad_den, num,
                                                             den, floor_v, g, rows);
  return cudaGetLastError();
}

cudaError_t reduce_coefs(const float* p0, int tiles0, const float* extra, int B, int Hq, int G,
                         float* dA, float* dB, float* dC, cudaStream_t st) {
  reduce_coefs_kernel<<<Hq, 128, 0, st>>>(p0, tiles0, extra, B, Hq, G, dA, dB, dC);
  return cudaGetLastError();
}

}  // namespace oal

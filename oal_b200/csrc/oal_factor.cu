// Per-head factorisation of the kernel's quadratic form, and the way back for its gradient.
//
// head_factor_kernel: M = [[A, B/2], [B/2, C]] (symmetric, (G+1) x (G+1), any signature) is
// diagonalised by cyclic Jacobi rotations (fp32; the eigenvalues are re-evaluated as Rayleigh quotients
// of the untouched matrix), one warp per query head, the rotations of a round (disjoint index pairs of
// a round-robin tournament) applied together.  The result is stored as the
// table the intra-chunk kernels read (oal_intra.cuh): c_r, l_r[d], the back-transform t and the count
// of positive terms.  Replaces nothing in the reference, which evaluates the direct form
// (oal_attention/grouped_reference.py:61-99); the values of w are the same.
//
// intra_coef_finish_kernel: sums the per-(batch row, chunk) partial sums of the query-side backward in
// fixed order -- D'[r][r'] = 2 sum dW u_r u_r', n'[r] = 2 sum dW u_r, s' = 2 sum dW -- and maps them to
// dM = sum dW v v^T with v = t u:  dM[a][b] = 1/2 (t D' t^T)[a][b] for a, b >= 1, dM[0][b] = 1/2 (t n')[b]
// and dM[0][0] = s' / 2 (v_0 = 1 is exact, so its row never goes through the rotation); adds the
// cross-chunk coefficient gradient of the state kernels and writes dA, dB, dC
// (oal_attention/hd_block_gemm_feature_backward.py:59-131 coefficient partials).
#include "oal_intra.cuh"
#include "oal_kernels.h"

namespace oal {
namespace {

constexpr int JN = RMAX_ALL;          // 17
constexpr int JP = JN + 1;            // row pitch
constexpr int JH = (JN + 1) / 2;      // index pairs per round (9)

// One warp per head.  Lane = (pair index i = lane & 15, row parity lane >> 4): the two lanes of a pair
// compute the same rotation from the untouched matrix and then update every other row (column) of
// the two columns (rows) of their pair, so no index arithmetic needs a division.
__global__ void __launch_bounds__(32) head_factor_kernel(const int32_t* dim_perm, const int32_t* group_start,
                                                         const float* A, const float* Bc, const float* Cc, int G,
                                                         float scale, HeadFactor* table) {
  __shared__ float M[JN][JP], V[JN][JP], M0[JN][JP];
  __shared__ int gdim[HD];
  __shared__ int order[JN];
  __shared__ float lam[JN], sig[JN];
  __shared__ int gstart[GMAX + 1];
  __shared__ float coefC[GMAX * GMAX], coefB[GMAX];
  const int h = blockIdx.x, lane = threadIdx.x;
  const int n = G + 1;
  // one coalesced pass over the head's tables (the loops below would otherwise chain global latencies)
  if (lane <= GMAX) gstart[lane] = group_start[h * (GMAX + 1) + lane];
  if (lane < G) coefB[lane] = Bc[h * G + lane];
  for (int x = lane; x < G * G; x += 32) coefC[x] = Cc[(size_t)h * G * G + x];
  const float coefA = A[h];
  const int perm0 = dim_perm[h * HD + lane], perm1 = dim_perm[h * HD + lane + 32];
  __syncwarp();
  for (int half_i = 0; half_i < 2; ++half_i) {
    const int p = lane + 32 * half_i;
    int g = 0;
    while (g < GMAX - 1 && p >= gstart[g + 1]) ++g;
    gdim[half_i ? perm1 : perm0] = min(g, G - 1);
  }
  if (lane < n) {
    const int a = lane;
    for (int b = 0; b < n; ++b) {
      float v;
      if (a == 0 && b == 0) v = coefA;
      else if (a == 0) v = 0.5f * coefB[b - 1];
      else if (b == 0) v = 0.5f * coefB[a - 1];
      else v = 0.5f * (coefC[(a - 1) * G + b - 1] + coefC[(b - 1) * G + a - 1]);
      M[a][b] = v;
      M0[a][b] = v;
      V[a][b] = a == b ? 1.f : 0.f;
    }
  }
  __syncwarp();
  const int m = (n & 1) ? n + 1 : n;          // players of the tournament; index n (if any) is a bye
  const int half = m / 2;
  const int pi = lane & 15, lg = lane >> 4;
  for (int sweep = 0; sweep < 12; ++sweep) {
    float off = 0.f, all = 0.f;
    if (lane < n)
      for (int b = 0; b < n; ++b) {
        const float v = M[lane][b];
        all = fmaf(v, v, all);
        if (b != lane) off = fmaf(v, v, off);
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      off += __shfl_xor_sync(0xffffffffu, off, o);
      all += __shfl_xor_sync(0xffffffffu, all, o);
    }
    if (off <= 1e-11f * all) break;     // off-diagonal norm below 3e-6 of the whole: the Rayleigh quotients finish the job
    for (int t = 0; t < m - 1; ++t) {
      int p = 0, q = -1;
      float c = 1.f, s = 0.f;
      if (pi < half) {
        if (pi == 0) { p = m - 1; q = t; }
        else { p = t + pi; if (p >= m - 1) p -= m - 1; q = t - pi; if (q < 0) q += m - 1; }
        if (p > q) { const int x = p; p = q; q = x; }
        if (q < n) {
          const float apq = M[p][q];
          if (fabsf(apq) > 1e-30f) {
            const float tau = (M[q][q] - M[p][p]) / (2.f * apq);
            const float tt = (tau >= 0.f ? 1.f : -1.f) / (fabsf(tau) + sqrtf(1.f + tau * tau));
            c = rsqrtf(1.f + tt * tt);
            s = tt * c;
          }
        } else {
          q = -1;
        }
      }
      __syncwarp();
      // all loads of a phase are issued before its first store (the compiler cannot reorder them itself:
      // same array), so a phase costs one shared-memory latency instead of one per row
      if (q >= 0) {
        float xm[JH], ym[JH], xv[JH], yv[JH];
#pragma unroll
        for (int it = 0; it < JH; ++it) {           // columns p, q of M and V, rows l = lg, lg + 2, ...
          const int l = min(lg + 2 * it, n - 1);
          xm[it] = M[l][p]; ym[it] = M[l][q];
          xv[it] = V[l][p]; yv[it] = V[l][q];
        }
#pragma unroll
        for (int it = 0; it < JH; ++it) {
          const int l = lg + 2 * it;
          if (l < n) {
            M[l][p] = c * xm[it] - s * ym[it]; M[l][q] = s * xm[it] + c * ym[it];
            V[l][p] = c * xv[it] - s * yv[it]; V[l][q] = s * xv[it] + c * yv[it];
          }
        }
      }
      __syncwarp();
      if (q >= 0) {
        float xm[JH], ym[JH];
#pragma unroll
        for (int it = 0; it < JH; ++it) {           // rows p, q of M
          const int l = min(lg + 2 * it, n - 1);
          xm[it] = M[p][l]; ym[it] = M[q][l];
        }
#pragma unroll
        for (int it = 0; it < JH; ++it) {
          const int l = lg + 2 * it;
          if (l < n) { M[p][l] = c * xm[it] - s * ym[it]; M[q][l] = s * xm[it] + c * ym[it]; }
        }
      }
      __syncwarp();
    }
  }
  // eigenvalues as Rayleigh quotients of the untouched matrix (second-order accurate in the
  // remaining rotation error)
  if (lane < n) {
    float acc = 0.f;
    for (int a = 0; a < n; ++a) {
      float row = 0.f;
      for (int b = 0; b < n; ++b) row = fmaf(M0[a][b], V[b][lane], row);
      acc = fmaf(V[a][lane], row, acc);
    }
    sig[lane] = acc;
  }
  __syncwarp();
  // order: positive eigenvalues first; lambda_r = sqrt(max(|sigma_r|, tiny relative floor))
  if (lane == 0) {
    float smax = 0.f;
    for (int r = 0; r < n; ++r) smax = fmaxf(smax, fabsf(sig[r]));
    const float floor_v = fmaxf(1e-12f * smax, 1e-30f);
    int k = 0;
    for (int r = 0; r < n; ++r) if (sig[r] >= 0.f) order[k++] = r;
    const int rpos = k;
    for (int r = 0; r < n; ++r) if (sig[r] < 0.f) order[k++] = r;
    for (int r = 0; r < n; ++r) lam[r] = sqrtf(fmaxf(fabsf(sig[order[r]]), floor_v));
    table[h].rank = n;
    table[h].rpos = rpos;
    table[h].pad[0] = table[h].pad[1] = 0;
  }
  __syncwarp();
  HeadFactor& out = table[h];
  if (lane < RMAX_ALL) out.c[lane] = lane < n ? lam[lane] * V[0][order[lane]] : 0.f;
  for (int r = 0; r < RMAX_ALL; ++r) {
    const bool live = r < n;
    const float sl = live ? scale * lam[r] : 0.f;
    const int col = live ? order[r] : 0;
    out.l[r][lane] = live ? sl * V[1 + gdim[lane]][col] : 0.f;
    out.l[r][lane + 32] = live ? sl * V[1 + gdim[lane + 32]][col] : 0.f;
    if (lane < RMAX_ALL) out.t[lane][r] = (live && lane < n) ? V[lane][col] / lam[r] : 0.f;
  }
}

__device__ __forceinline__ int tri_all(int g, int g2) { return g * GMAX - (g * (g - 1)) / 2 + (g2 - g); }

// partial: [B][Hq][tiles][nu_stride]: entries r <= r' in row-major upper-triangle order of an rm x rm
// matrix, then the rm sums n'[r], then s'.
__global__ void __launch_bounds__(128) intra_coef_finish_kernel(const float* partial, int tiles, int nu_stride, int rm,
                                                                const HeadFactor* table, const float* extra, int B,
                                                                int Hq, int G, float* dA, float* dB, float* dC) {
  __shared__ float D[RMAX_ALL][RMAX_ALL];
  __shared__ float T[RMAX_ALL][RMAX_ALL];
  __shared__ float X[RMAX_ALL][RMAX_ALL];       // t D'
  __shared__ float N1[RMAX_ALL + 1];            // n'[r], then s'
  const int h = blockIdx.x, tid = threadIdx.x;
  const int n = G + 1;
  for (int x = tid; x < RMAX_ALL * RMAX_ALL; x += 128) {
    D[x / RMAX_ALL][x % RMAX_ALL] = 0.f;
    T[x / RMAX_ALL][x % RMAX_ALL] = table[h].t[x / RMAX_ALL][x % RMAX_ALL];
  }
  __syncthreads();
  const int nu = rm * (rm + 1) / 2;
  for (int x = tid; x < nu; x += 128) {
    int r = 0, rest = x;
    while (rest >= rm - r) { rest -= rm - r; ++r; }
    const int r2 = r + rest;
    float t = 0.f;
    if (partial)
      for (int b = 0; b < B; ++b)
        for (int i = 0; i < tiles; ++i) t += partial[((size_t)(b * Hq + h) * tiles + i) * nu_stride + x];
    if (r < RMAX_ALL && r2 < RMAX_ALL) { D[r][r2] = t; D[r2][r] = t; }
  }
  for (int x = tid; x < RMAX_ALL + 1; x += 128) {
    float t = 0.f;
    const int src = x < RMAX_ALL ? nu + x : nu + rm;
    if (partial && (x < rm || x == RMAX_ALL))
      for (int b = 0; b < B; ++b)
        for (int i = 0; i < tiles; ++i) t += partial[((size_t)(b * Hq + h) * tiles + i) * nu_stride + src];
    N1[x] = t;
  }
  __syncthreads();
  for (int x = tid; x < n * n; x += 128) {
    const int a = x / n, r2 = x % n;
    float t = 0.f;
    for (int r = 0; r < n; ++r) t += T[a][r] * D[r][r2];
    X[a][r2] = t;
  }
  __syncthreads();
  for (int x = tid; x < n * n; x += 128) {
    const int a = x / n, b = x % n;
    float t = 0.f;
    if (a == 0 && b == 0) t = N1[RMAX_ALL];
    else if (a == 0 || b == 0) { for (int r = 0; r < n; ++r) t += T[a + b][r] * N1[r]; }
    else { for (int r2 = 0; r2 < n; ++r2) t += X[a][r2] * T[b][r2]; }
    t *= 0.5f;
    if (a == 0 && b == 0) dA[h] = t + (extra ? extra[(size_t)h * NCOEF] : 0.f);
    else if (a == 0) dB[h * G + b - 1] = t + (extra ? extra[(size_t)h * NCOEF + b] : 0.f);
    else if (b > 0) {
      const int g = a - 1, g2 = b - 1;
      const int slot = 1 + GMAX + (g <= g2 ? tri_all(g, g2) : tri_all(g2, g));
      dC[((size_t)h * G + g) * G + g2] = t + (extra ? extra[(size_t)h * NCOEF + slot] : 0.f);
    }
  }
}


// ---------------------------------------------------------------------------
// Packed factor -> coefficients and back.  L is the lower-triangular matrix whose packed rows
// (row-major over (row, col <= row), the order of torch.tril_indices) are `factor`; M = L L^T;
// A = M00 + eps, B = 2 M[0, 1:], C = M[1:, 1:].  One block per query head, thread = (i, j).
// Replaces the tensor-op sequence of oal_attention/grouped_quadratic.py (_expand_factor_coefficients there)
// and its autograd graph: two launches per step instead of about forty.
// ---------------------------------------------------------------------------
constexpr int XS = GMAX + 1;     // largest side of L

__device__ __forceinline__ float packed_l(const float* f, int r, int c) { return c <= r ? f[r * (r + 1) / 2 + c] : 0.f; }

__global__ void __launch_bounds__(XS * XS) expand_factor_kernel(const float* factor, int factor_rows, int G, float eps,
                                                                float* A, float* B, float* C) {
  const int h = blockIdx.x, side = G + 1;
  const float* f = factor + (size_t)(factor_rows == 1 ? 0 : h) * (side * (side + 1) / 2);
  const int i = threadIdx.x / side, j = threadIdx.x % side;
  if (i >= side) return;
  float m = 0.f;
  for (int k = 0; k <= min(i, j); ++k) m = fmaf(packed_l(f, i, k), packed_l(f, j, k), m);
  if (i == 0 && j == 0) A[h] = m + eps;
  else if (i == 0) B[(size_t)h * G + j - 1] = 2.f * m;
  else if (j > 0) C[((size_t)h * G + i - 1) * G + j - 1] = m;
}

// dL = (S + S^T) L on the lower triangle, S[0][0] = dA, S[0][j] = 2 dB[j-1], S[i][j] = dC[i-1][j-1] (i, j >= 1),
// S[i][0] = 0.  With one shared factor row (factor_rows == 1) a single block walks the heads in order.
__global__ void __launch_bounds__(XS * XS) expand_factor_grad_kernel(const float* factor, int factor_rows, int Hq, int G,
                                                                     const float* dA, const float* dB, const float* dC,
                                                                     float* dfactor) {
  const int side = G + 1, P = side * (side + 1) / 2;
  const int i = threadIdx.x / side, k = threadIdx.x % side;
  const bool mine = i < side && k <= i;
  const int h0 = factor_rows == 1 ? 0 : blockIdx.x, h1 = factor_rows == 1 ? Hq : h0 + 1;
  const float* f = factor + (size_t)(factor_rows == 1 ? 0 : h0) * P;
  float acc = 0.f;
  for (int h = h0; h < h1 && mine; ++h) {
    auto S = [&](int r, int c) -> float {
      if (r == 0) return c == 0 ? dA[h] : 2.f * dB[(size_t)h * G + c - 1];
      return c == 0 ? 0.f : dC[((size_t)h * G + r - 1) * G + c - 1];
    };
    for (int j = k; j < side; ++j) acc = fmaf(S(i, j) + S(j, i), packed_l(f, j, k), acc);
  }
  if (mine) dfactor[(size_t)(factor_rows == 1 ? 0 : h0) * P + i * (i + 1) / 2 + k] = acc;
}

}  // namespace

size_t head_factor_bytes(int Hq) { return (size_t)Hq * sizeof(HeadFactor); }

cudaError_t build_head_factors(const int32_t* dim_perm, const int32_t* group_start, const float* A, const float* Bc,
                               const float* Cc, int Hq, int G, float scale, void* table, cudaStream_t st) {
  head_factor_kernel<<<Hq, 32, 0, st>>>(dim_perm, group_start, A, Bc, Cc, G, scale, static_cast<HeadFactor*>(table));
  return cudaGetLastError();
}

cudaError_t intra_coef_finish(const float* partial, int tiles, int nu_stride, int rm, const void* table,
                              const float* extra, int B, int Hq, int G, float* dA, float* dB, float* dC,
                              cudaStream_t st) {
  intra_coef_finish_kernel<<<Hq, 128, 0, st>>>(partial, tiles, nu_stride, rm, static_cast<const HeadFactor*>(table),
                                               extra, B, Hq, G, dA, dB, dC);
  return cudaGetLastError();
}


cudaError_t expand_factor(const float* factor, int factor_rows, int Hq, int G, float eps, float* A, float* B, float* C,
                          cudaStream_t st) {
  expand_factor_kernel<<<Hq, (GMAX + 1) * (GMAX + 1), 0, st>>>(factor, factor_rows, G, eps, A, B, C);
  return cudaGetLastError();
}

cudaError_t expand_factor_grad(const float* factor, int factor_rows, int Hq, int G, const float* dA, const float* dB,
                               const float* dC, float* dfactor, cudaStream_t st) {
  expand_factor_grad_kernel<<<factor_rows == 1 ? 1 : Hq, (GMAX + 1) * (GMAX + 1), 0, st>>>(factor, factor_rows, Hq, G, dA,
                                                                                           dB, dC, dfactor);
  return cudaGetLastError();
}

}  // namespace oal

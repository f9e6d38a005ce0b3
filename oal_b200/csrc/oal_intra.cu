// Intra-chunk term of the chunked scan on the tensor cores (tcgen05 / TMEM), forward.
//
// For one (batch row, query head, 128-token chunk), 16 keys at a time:
//   U  = Q . stack^T         one MMA chain, N = 16 R columns: u_r(i, j) for the R terms of the factored
//                            weight (oal_intra.cuh); the stack is rebuilt per tile in shared memory
//   W  = sum_r sgn_r u_r^2   R multiply-adds per pair in registers, causal mask, bf16
//   Y += W [v | 1]           second MMA, accumulator shared by all key tiles
// then adds the cross-chunk part left in num / den by cross_read, normalises and writes out / num /
// den and the status flags.  Eight warps (128 rows x 2 halves of a tile); lane 0 of warp 0 also issues
// the MMAs between its own steps; hand-offs are warp-granular mbarrier arrivals; two CTAs share an SM.  Replaces, per chunk, the
// reference's F-wide local score GEMM, tril, bf16 cast, score x U GEMM, merge and normalise stages
// (oal_attention/hd_block_gemm_runtime.py:530-597, hd_block_gemm_normalization_ops.py:113).
#include "oal_intra.cuh"
#include "oal_kernels.h"

namespace oal {
namespace {

using namespace umma;

struct IntraFwdArgs {
  const __nv_bfloat16 *q, *k, *v;
  const HeadFactor* factors;
  void* out;
  float *num, *den;
  int32_t* status;
  int N, Hq, Hkv, out_dt;
  float floor;
  int out_token_major;      // out is [B, N, Hq, 64] instead of [B, Hq, N, 64]
};

constexpr int FWD_SMEM = XA_BYTES + X_BYTES + SLAB_S_BYTES + 2 * ST_BYTES;
static_assert(CT * 65 * 4 <= XA_BYTES + X_BYTES + SLAB_S_BYTES, "output staging tile must fit in the operand images");
// tensor memory: U (16 R columns) | Y (80) | two weight tiles (8 columns each: 16 keys as bf16 pairs)
constexpr uint32_t FWD_TMEM_U = 0, FWD_TMEM_Y = RM * KT, FWD_TMEM_W = RM * KT + EP;
static_assert(RM * KT + EP + 2 * (KT / 2) <= 256, "tensor-memory columns of the forward kernel");

__global__ void __launch_bounds__(CTHREADS, 2) intra_fwd_kernel(const IntraFwdArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* Qa = smem;                         // augmented q image
  unsigned char* Kimg = Qa + XA_BYTES;
  unsigned char* Uimg = Kimg + X_BYTES;
  unsigned char* St = Uimg + SLAB_S_BYTES;          // two stacked key tiles
  __shared__ HeadFactorS hf;
  __shared__ uint64_t u_done, u_free, w_ready[2], w_done[2], st_ready[2];
  __shared__ uint32_t tmem_base;
  __shared__ int dead;
  __shared__ float den_s[CT];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (a.Hq / a.Hkv);
  const int half = (warp >> 2) & 1, row = 32 * (warp & 3) + lane;
  const bool issuer = warp == 0;
  if (warp == 0) tmem_alloc(&tmem_base, 256);
  if (tid == 0) {
    mbar_init(&u_done, 1);
    mbar_init(&u_free, CWARPS);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&w_ready[s], CWARPS);
      mbar_init(&w_done[s], 1);
      mbar_init(&st_ready[s], CWARPS / 2);
    }
    mbar_fence_init();
    dead = 0;
  }
  const size_t qoff = (size_t)(b * a.Hq + h) * a.N, koff = (size_t)(b * a.Hkv + kvh) * a.N;
  load_head_factor(hf, a.factors, h, tid, CTHREADS);
  load_operand_image(Qa, a.q + qoff * HD, c * CT, a.N, true, tid, CTHREADS);
  load_operand_image(Kimg, a.k + koff * HD, c * CT, a.N, false, tid, CTHREADS);
  load_u_image(Uimg, a.v + koff * VD, c * CT, a.N, tid, CTHREADS);
  async_copies_wait();
  __syncthreads();
  const int tiles = min(CT / KT, (a.N - c * CT + KT - 1) / KT);
  const int rank = hf.rank, rpos = hf.rpos;
  init_stack_constants(St, hf, tid, CTHREADS);
  init_stack_constants(St + ST_BYTES, hf, tid, CTHREADS);
  if (tid < CTHREADS && (tid >> 7) < tiles) build_stack_piece(St + (tid >> 7) * ST_BYTES, Kimg, (tid >> 7) * KT, hf, tid & 127);
  fence_async_smem();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  Waiter w{&dead};
  const uint32_t tU = tmem_base + FWD_TMEM_U, tY = tmem_base + FWD_TMEM_Y, tWt = tmem_base + FWD_TMEM_W;
  const uint32_t lane_off = (uint32_t)(32 * (warp & 3)) << 16;

  const uint32_t q_addr = smem_u32(Qa), u_addr = smem_u32(Uimg), st_addr = smem_u32(St);
  const uint32_t idesc_y = instr_desc_bf16(128, EP, 0, 1);
  if (issuer) {
    if (lane == 0) {
      issue_stack_scores(tU, q_addr, st_addr, rank);
      mma_commit(&u_done);
    }
    __syncwarp();
  }
  for (int kt = 0; kt < tiles; ++kt) {
    const int buf = kt & 1;
    const bool warp_active = 32 * (warp & 3) + 31 >= kt * KT;       // else every pair of the warp is masked
    f32x2 wp[4], wn[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) wp[j] = wn[j] = 0ull;
    w.wait(&u_done, kt & 1, 0x14);
    fence_after_sync();
    // two batches of terms: the loads of the second overlap the arithmetic of the first.  A positive
    // semi-definite form (every term enters with +, the usual case) takes the loop without sign tests.
    constexpr int R0 = (RM + 1) / 2;
    float u0[R0][8], u1[RM - R0][8];
    if (warp_active) {
#pragma unroll
      for (int r = 0; r < R0; ++r)
        if (r < rank) tmem_ld8(tU + lane_off + r * KT + 8 * half, u0[r]);
      tmem_ld_wait();
#pragma unroll
      for (int r = R0; r < RM; ++r)
        if (r < rank) tmem_ld8(tU + lane_off + r * KT + 8 * half, u1[r - R0]);
      if (rpos == rank) {
#pragma unroll
        for (int r = 0; r < R0; ++r)
          if (r < rank) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const f32x2 u2 = f2_pack(u0[r][2 * j], u0[r][2 * j + 1]);
              wp[j] = f2_fma(u2, u2, wp[j]);
            }
          }
      } else {
#pragma unroll
        for (int r = 0; r < R0; ++r)
          if (r < rank) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const f32x2 u2 = f2_pack(u0[r][2 * j], u0[r][2 * j + 1]);
              if (r < rpos) wp[j] = f2_fma(u2, u2, wp[j]);
              else wn[j] = f2_fma(u2, u2, wn[j]);
            }
          }
      }
      tmem_ld_wait();
    }
    fence_before_sync();
    warp_arrive(&u_free, lane);
    if (issuer && kt + 1 < tiles) {
      if (lane == 0) {
        w.wait(&u_free, kt & 1, 0x11);                                   // every warp holds U(kt)
        if (kt + 1 >= 2) w.wait(&st_ready[(kt + 1) & 1], ((kt - 1) >> 1) & 1, 0x12);
        fence_after_sync();
        issue_stack_scores(tU, q_addr, st_addr + ((kt + 1) & 1) * ST_BYTES, rank);
        mma_commit(&u_done);
      }
      __syncwarp();
    }
    if (warp_active) {
      if (rpos == rank) {
#pragma unroll
        for (int r = R0; r < RM; ++r)
          if (r < rank) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const f32x2 u2 = f2_pack(u1[r - R0][2 * j], u1[r - R0][2 * j + 1]);
              wp[j] = f2_fma(u2, u2, wp[j]);
            }
          }
      } else {
#pragma unroll
        for (int r = R0; r < RM; ++r)
          if (r < rank) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const f32x2 u2 = f2_pack(u1[r - R0][2 * j], u1[r - R0][2 * j + 1]);
              if (r < rpos) wp[j] = f2_fma(u2, u2, wp[j]);
              else wn[j] = f2_fma(u2, u2, wn[j]);
            }
          }
      }
    }
    float wv[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float p0, p1, n0, n1;
      f2_unpack(wp[j], p0, p1);
      f2_unpack(wn[j], n0, n1);
      wv[2 * j] = p0 - n0;
      wv[2 * j + 1] = p1 - n1;
    }
#pragma unroll
    for (int x = 0; x < 8; ++x)
      if (!warp_active || kt * KT + 8 * half + x > row) wv[x] = 0.f;
    if (kt >= 2) w.wait(&w_done[buf], ((kt - 2) >> 1) & 1, 0x15);     // the MMA that read W[buf] two tiles ago
    fence_after_sync();
    // the weight tile is the A operand of the second MMA, read from tensor memory: row = lane, bf16 pairs
    tmem_st4(tWt + lane_off + buf * (KT / 2) + 4 * half, pack_bf16(wv[0], wv[1]), pack_bf16(wv[2], wv[3]),
             pack_bf16(wv[4], wv[5]), pack_bf16(wv[6], wv[7]));
    tmem_st_wait();
    fence_before_sync();
    warp_arrive(&w_ready[buf], lane);
    // stack of tile kt + 2 into the buffer U(kt) has finished reading; the two halves take turns
    if (kt + 2 < tiles && half == (kt & 1)) {
      build_stack_piece(St + buf * ST_BYTES, Kimg, (kt + 2) * KT, hf, tid & 127);
      fence_async_smem();
      warp_arrive(&st_ready[buf], lane);
    }
    if (issuer) {
      if (lane == 0) {
        w.wait(&w_ready[buf], (kt >> 1) & 1, 0x13);
        fence_after_sync();
        mma_bf16_ts(tY, tWt + buf * (KT / 2), smem_desc(u_addr + kt * KT * 16, 128, CT * 16), idesc_y, kt > 0);
        mma_commit(&w_done[buf]);
      }
      __syncwarp();
    }
  }
  if (tiles >= 2) w.wait(&w_done[(tiles - 2) & 1], ((tiles - 2) >> 1) & 1, 0x16);
  if (tiles >= 1) w.wait(&w_done[(tiles - 1) & 1], ((tiles - 1) >> 1) & 1, 0x17);
  fence_after_sync();
  // every MMA has completed (or the CTA is dead): the operand images are free
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  // epilogue: add the cross-chunk part, normalise, status.  The intra-chunk numerators go through a
  // row-major staging tile in shared memory so that the global reads and writes below are full 16-
  // and 32-byte vectors, contiguous across the lanes of a warp.
  float* stage_out = reinterpret_cast<float*>(smem);        // [128][65] fp32
  int flags = 0;
  {
    const int i = c * CT + row;
    const size_t orow = qoff + i;
    const int col0 = half == 0 ? 0 : 48, ncol = half == 0 ? 48 : 32;
#pragma unroll
    for (int cc = 0; cc < 48; cc += 16) {
      if (cc < ncol) {
        float vv[16];
        tmem_ld16(tY + lane_off + col0 + cc, vv);
        tmem_ld_wait();
        if (col0 + cc < VD) {
#pragma unroll
          for (int x = 0; x < 16; ++x) stage_out[row * 65 + col0 + cc + x] = vv[x];
        } else {
          float den = vv[0];                    // column 64
          if (i < a.N && !dead) {
            den += a.den[orow];
            a.den[orow] = den;
            if (!finite_f(den)) flags |= OAL_STATUS_NONFINITE;
            else if (!(den > 0.f)) flags |= OAL_STATUS_DENOMINATOR;
          }
          den_s[row] = den;
        }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (!dead) {
    // 128 rows x 8 segments of 8 columns = 4 per thread; the reads of the cross-chunk numerators are
    // all issued before the first use
    constexpr int PER = CT * 8 / CTHREADS;
    float4 o0[PER], o1[PER];
#pragma unroll
    for (int it = 0; it < PER; ++it) {
      const int x = tid + it * CTHREADS, r = x >> 3, seg = x & 7, ii = c * CT + r;
      if (ii < a.N) {
        const float* np = a.num + (qoff + ii) * VD + seg * 8;
        o0[it] = *reinterpret_cast<const float4*>(np);
        o1[it] = *reinterpret_cast<const float4*>(np + 4);
      }
    }
#pragma unroll
    for (int it = 0; it < PER; ++it) {
      const int x = tid + it * CTHREADS, r = x >> 3, seg = x & 7, ii = c * CT + r;
      if (ii >= a.N) continue;
      const float inv = 1.f / fmaxf(den_s[r], a.floor);
      const size_t oo = (qoff + ii) * VD + seg * 8;
      const size_t ot = a.out_token_major ? (((size_t)b * a.N + ii) * a.Hq + h) * VD + seg * 8 : oo;
      float* np = a.num + oo;
      const float* sp = stage_out + r * 65 + seg * 8;
      const float n[8] = {sp[0] + o0[it].x, sp[1] + o0[it].y, sp[2] + o0[it].z, sp[3] + o0[it].w,
                          sp[4] + o1[it].x, sp[5] + o1[it].y, sp[6] + o1[it].z, sp[7] + o1[it].w};
      *reinterpret_cast<float4*>(np) = make_float4(n[0], n[1], n[2], n[3]);
      *reinterpret_cast<float4*>(np + 4) = make_float4(n[4], n[5], n[6], n[7]);
      bool fin = true;
#pragma unroll
      for (int j = 0; j < 8; ++j) fin = fin && finite_f(n[j]);
      if (!fin) flags |= OAL_STATUS_NONFINITE;
      if (a.out_dt == OAL_DTYPE_BF16) {
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.out) + ot) =
            make_uint4(pack_bf16(n[0] * inv, n[1] * inv), pack_bf16(n[2] * inv, n[3] * inv),
                       pack_bf16(n[4] * inv, n[5] * inv), pack_bf16(n[6] * inv, n[7] * inv));
      } else if (a.out_dt == OAL_DTYPE_F32) {
        float* op = reinterpret_cast<float*>(a.out) + ot;
        *reinterpret_cast<float4*>(op) = make_float4(n[0] * inv, n[1] * inv, n[2] * inv, n[3] * inv);
        *reinterpret_cast<float4*>(op + 4) = make_float4(n[4] * inv, n[5] * inv, n[6] * inv, n[7] * inv);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) store_elem(a.out, ot + j, a.out_dt, n[j] * inv);
      }
    }
  }
  if (flags) atomicOr(a.status, flags);
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 256);
  if (tid == 0 && dead) atomicOr(a.status, w.status_bits());
}

}  // namespace

cudaError_t OAL_INTRA_NAME(intra_forward)(const void* q, const void* k, const void* v, const void* factors, void* out,
                                          float* num, float* den, int32_t* status, int B, int Hq, int Hkv, int N, int NB,
                                          int out_dt, float floor_v, bool out_token_major, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(intra_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM);
  if (e != cudaSuccess) return e;
  IntraFwdArgs a{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k),
                 static_cast<const __nv_bfloat16*>(v), static_cast<const HeadFactor*>(factors), out, num, den, status,
                 N, Hq, Hkv, out_dt, floor_v, out_token_major ? 1 : 0};
  intra_fwd_kernel<<<dim3(NB, Hq, B), CTHREADS, FWD_SMEM, st>>>(a);
  return cudaGetLastError();
}

}  // namespace oal

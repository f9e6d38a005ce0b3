// Intra-chunk term of the chunked scan on the tensor cores (tcgen05 / TMEM), forward.
//
// For one (batch, query head, 128-token chunk) the kernel forms, 16 keys at a time,
//   S_g = Q_g K_g^T              one small MMA chain per dimension group (groups padded to 16 dims)
//   W   = A + sum_g s_g (B_g + sum_g' C_gg' s_g')   in registers, causal mask, bf16
//   Y  += W [v | 1]              second MMA, accumulator shared by all key tiles
// then adds the cross-chunk part left in num/den by cross_read, normalises and writes out / num /
// den and the status flags.  It replaces, per chunk, the reference's F-wide local score GEMM,
// tril, bf16 cast, score x U GEMM, merge and normalise stages
// (oal_attention/hd_block_gemm_runtime.py:530-597, hd_block_gemm_normalization_ops.py:113).
#include "oal_intra.cuh"
#include "oal_kernels.h"

namespace oal {
namespace {

using namespace umma;

struct IntraFwdArgs {
  const __nv_bfloat16 *q, *k, *v;
  const int32_t *dim_perm, *group_start;
  const float *A, *Bc, *Cc;
  void* out;
  float *num, *den;
  int32_t* status;
  int N, Hq, Hkv, G, out_dt;
  int slabs;            // upper bound on the padded 16-dim slabs of any head (image size)
  float scale, floor;
  // operand images made by pad_images (null: build them here from q, k, v)
  const unsigned char *qimg, *kimg, *uimg;
};

// ---------------------------------------------------------------------------
// pad_images: the padded q / k operand images of every (batch, query head, chunk) and the [v | 1]
// image of every (batch, KV head, chunk), written once to HBM so that the intra-chunk kernels fetch
// them with bulk copies instead of gathering them again in each of the three kernels.
//   qimg, kimg: [B*Hq*NB][slabs * 4096 bytes]   uimg: [B*Hkv*NB][SLAB_S_BYTES]
// ---------------------------------------------------------------------------
struct PadArgs {
  const __nv_bfloat16 *q, *k, *v;
  const int32_t *dim_perm, *group_start;
  unsigned char *qimg, *kimg, *uimg;
  int32_t* status;
  int N, NB, Hq, Hkv, slabs;
};

__global__ void __launch_bounds__(256) pad_images_kernel(const PadArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  uint32_t* stage_a = reinterpret_cast<uint32_t*>(smem);      // raw q tile, row pitch 33 words
  uint32_t* stage_b = stage_a + STAGE_WORDS;                  // raw k tile
  __shared__ PaddedGroups pg;
  const int tid = threadIdx.x;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int rep = a.Hq / a.Hkv, kvh = h / rep;
  const size_t qoff = (size_t)(b * a.Hq + h) * a.N, koff = (size_t)(b * a.Hkv + kvh) * a.N;
  // the raw tiles are on their way while the layout is worked out
  for (int x = tid; x < 2 * CT * 8; x += 256) {
    const int which = x >= CT * 8, xx = x - which * CT * 8;
    const int r = xx >> 3, seg = xx & 7, i = c * CT + r;
    uint4 t = make_uint4(0u, 0u, 0u, 0u);
    if (i < a.N) t = *reinterpret_cast<const uint4*>((which ? a.k + koff * HD : a.q + qoff * HD) + (size_t)i * HD + seg * 8);
    uint32_t* d = (which ? stage_b : stage_a) + r * 33 + seg * 4;
    d[0] = t.x; d[1] = t.y; d[2] = t.z; d[3] = t.w;
  }
  load_group_layout(pg, a.dim_perm, a.group_start, h, tid, 256);     // its barriers also cover the staging stores
  const int nslab = pg.k16_start[IG];
  if (nslab > a.slabs) {            // the consumer kernels refuse this head too
    if (tid == 0) atomicOr(a.status, OAL_STATUS_BAD_LAYOUT);
    return;
  }
  const size_t item = (size_t)(b * a.Hq + h) * a.NB + c;
  const size_t img_bytes = (size_t)a.slabs * 4096;
  const int per_img = 2 * nslab * CT;
  for (int x = tid; x < 2 * per_img; x += 256) {       // gather straight into the images in HBM, 16 bytes per thread
    const int which = x >= per_img, xx = x - which * per_img;
    const int c8 = xx >> 7, r = xx & 127;
    const unsigned short* raw = reinterpret_cast<const unsigned short*>(which ? stage_b : stage_a);
    unsigned short e[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int sd = pg.src[c8 * 8 + j];
      e[j] = sd >= 0 ? raw[r * 66 + sd] : (unsigned short)0;
    }
    reinterpret_cast<uint4*>((which ? a.kimg : a.qimg) + item * img_bytes)[xx] =
        make_uint4(e[0] | ((uint32_t)e[1] << 16), e[2] | ((uint32_t)e[3] << 16), e[4] | ((uint32_t)e[5] << 16),
                   e[6] | ((uint32_t)e[7] << 16));
  }
  if (h % rep == 0) {
    uint4* du = reinterpret_cast<uint4*>(a.uimg + ((size_t)(b * a.Hkv + kvh) * a.NB + c) * SLAB_S_BYTES);
    for (int idx = tid; idx < (EP / 8) * CT; idx += 256) {
      const int ec = idx >> 7, t = idx & 127, j = c * CT + t;
      du[idx] = u_image_chunk(a.v + (koff + j) * VD, ec, j < a.N);
    }
  }
}

constexpr int W_BYTES = (KT / 8) * CT * 16;              // 4096: one bf16 weight tile [2][128 rows][8 keys]
__host__ __device__ constexpr int fwd_smem_bytes(int slabs) {
  return 2 * slabs * 4096 + SLAB_S_BYTES + 2 * W_BYTES + STAGE_BYTES;
}

__global__ void __launch_bounds__(256, 2) intra_fwd_kernel(const IntraFwdArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int img_bytes = a.slabs * 4096;                  // padded q / k operand image [slabs*2][128][8]
  unsigned char* Qimg = smem;
  unsigned char* Kimg = Qimg + img_bytes;
  unsigned char* Uimg = Kimg + img_bytes;
  unsigned char* Wbuf = Uimg + SLAB_S_BYTES;
  uint32_t* stage = reinterpret_cast<uint32_t*>(Wbuf + 2 * W_BYTES);
  __shared__ PaddedGroups pg;
  __shared__ uint64_t s_done, w_done[2], imgfull;
  __shared__ uint32_t tmem_base;
  __shared__ int dead;
  __shared__ float den_s[CT];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (a.Hq / a.Hkv);
  const int half = warp >> 2, row = 32 * (warp & 3) + lane;
  if (warp == 0) tmem_alloc(&tmem_base, 256);
  if (tid == 0) {
    mbar_init(&s_done, 1);
    mbar_init(&w_done[0], 1);
    mbar_init(&w_done[1], 1);
    mbar_init(&imgfull, 1);
    mbar_fence_init();
    dead = 0;
  }
  load_padded_groups(pg, a.dim_perm, a.group_start, a.A, a.Bc, a.Cc, a.G, h, a.scale, a.scale * a.scale, 2.f * a.scale * a.scale, tid, 256);
  const size_t qoff = (size_t)(b * a.Hq + h) * a.N, koff = (size_t)(b * a.Hkv + kvh) * a.N;
  // a head with more padded slabs than the caller announced would not fit the images: refuse it
  const bool bad = pg.k16_start[IG] > a.slabs;
  const bool prebuilt = a.qimg != nullptr;
  if (prebuilt) {
    // the images were made by pad_images: three bulk copies, awaited by the thread that issues the MMAs
    if (tid == 0 && !bad) {
      const uint32_t bytes = (uint32_t)pg.k16_start[IG] * 4096u;
      const size_t item = (size_t)(b * a.Hq + h) * gridDim.x + c;
      mbar_arrive_expect_tx(&imgfull, 2 * bytes + SLAB_S_BYTES);
      bulk_g2s(Qimg, a.qimg + item * (size_t)img_bytes, bytes, &imgfull);
      bulk_g2s(Kimg, a.kimg + item * (size_t)img_bytes, bytes, &imgfull);
      bulk_g2s(Uimg, a.uimg + ((size_t)(b * a.Hkv + kvh) * gridDim.x + c) * SLAB_S_BYTES, SLAB_S_BYTES, &imgfull);
    }
  } else {
    if (!bad) {
      // second staging area: the U image, which is built right after
      build_padded_images(Qimg, Kimg, stage, reinterpret_cast<uint32_t*>(Uimg), a.q + qoff * HD, a.k + koff * HD, c * CT,
                          a.N, pg, tid, 256);
    }
    for (int idx = tid; idx < (EP / 8) * CT; idx += 256) {
      const int ec = idx >> 7, t = idx & 127, j = c * CT + t;
      reinterpret_cast<uint4*>(Uimg)[idx] = u_image_chunk(a.v + (koff + j) * VD, ec, j < a.N);
    }
  }
  if (bad && tid == 0) atomicOr(a.status, OAL_STATUS_BAD_LAYOUT);
  fence_async_smem();
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  Waiter w{&dead};
  const uint32_t tS = tmem_base, tY = tmem_base + IG * KT;
  const uint32_t lane_off = (uint32_t)(32 * (warp & 3)) << 16;
  const uint32_t q_addr = smem_u32(Qimg), k_addr = smem_u32(Kimg), u_addr = smem_u32(Uimg);
  const uint32_t idesc_y = instr_desc_bf16(128, EP, 0, 1);
  const int tiles = bad ? 0 : min(CT / KT, (a.N - c * CT + KT - 1) / KT);
  if (tid == 0 && !bad) {
    if (prebuilt) {
      w.wait(&imgfull, 0, 0x15);
      fence_after_sync();
    }
    issue_group_scores(tS, q_addr, k_addr, 0, pg);
    mma_commit(&s_done);
  }
  for (int kt = 0; kt < tiles; ++kt) {
    const int buf = kt & 1;
    float s[IG][8];
    w.wait(&s_done, kt & 1, 0x11);
    fence_after_sync();
#pragma unroll
    for (int g = 0; g < IG; ++g) {
      if (pg.k16_start[g + 1] > pg.k16_start[g]) tmem_ld8(tS + lane_off + g * KT + 8 * half, s[g]);
      else {
#pragma unroll
        for (int x = 0; x < 8; ++x) s[g][x] = 0.f;
      }
    }
    tmem_ld_wait();
    fence_before_sync();
    __syncthreads();                       // every thread holds its scores: S may be overwritten
    if (tid == 0 && kt + 1 < tiles) {
      fence_after_sync();
      issue_group_scores(tS, q_addr, k_addr, (kt + 1) * KT, pg);
      mma_commit(&s_done);
    }
    // combine (rows whose whole warp lies above the tile's keys are masked out entirely)
    float wv[8];
    const bool warp_active = 32 * (warp & 3) + 31 >= kt * KT;
    if (warp_active) {
      // packed pairs of columns (2j, 2j+1)
      f32x2 s2[IG][4], w2[4];
#pragma unroll
      for (int g = 0; g < IG; ++g)
#pragma unroll
        for (int j = 0; j < 4; ++j) s2[g][j] = f2_pack(s[g][2 * j], s[g][2 * j + 1]);
#pragma unroll
      for (int j = 0; j < 4; ++j) w2[j] = f2_bcast(pg.A);
#pragma unroll
      for (int g = 0; g < IG; ++g) {
        f32x2 t[4];
        const f32x2 bg = pg.B2[g], cgg = pg.C2[g * IG + g];
#pragma unroll
        for (int j = 0; j < 4; ++j) t[j] = f2_fma(cgg, s2[g][j], bg);
#pragma unroll
        for (int g2 = 0; g2 < g; ++g2) {
          const f32x2 c2 = pg.C2[g * IG + g2];
#pragma unroll
          for (int j = 0; j < 4; ++j) t[j] = f2_fma(c2, s2[g2][j], t[j]);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) w2[j] = f2_fma(s2[g][j], t[j], w2[j]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) f2_unpack(w2[j], wv[2 * j], wv[2 * j + 1]);
#pragma unroll
      for (int x = 0; x < 8; ++x)
        if (kt * KT + 8 * half + x > row) wv[x] = 0.f;
    } else {
#pragma unroll
      for (int x = 0; x < 8; ++x) wv[x] = 0.f;
    }
    if (kt >= 2) w.wait(&w_done[buf], ((kt - 2) >> 1) & 1, 0x12);     // the MMA that read W[buf] two tiles ago
    reinterpret_cast<uint4*>(Wbuf + buf * W_BYTES)[half * CT + row] =
        make_uint4(pack_bf16(wv[0], wv[1]), pack_bf16(wv[2], wv[3]), pack_bf16(wv[4], wv[5]), pack_bf16(wv[6], wv[7]));
    fence_async_smem();
    __syncthreads();
    if (tid == 0) {
      fence_after_sync();
      mma_bf16_ss(tY, smem_desc(smem_u32(Wbuf + buf * W_BYTES), CT * 16, 128),
                  smem_desc(u_addr + kt * KT * 16, 128, CT * 16), idesc_y, kt > 0);
      mma_commit(&w_done[buf]);
    }
  }
  // all weight MMAs done
  if (tiles >= 2) w.wait(&w_done[(tiles - 2) & 1], ((tiles - 2) >> 1) & 1, 0x13);
  if (tiles >= 1) w.wait(&w_done[(tiles - 1) & 1], ((tiles - 1) >> 1) & 1, 0x14);
  fence_after_sync();
  // epilogue: add the cross-chunk part, normalise, status.  The intra-chunk numerators go through a
  // row-major staging tile in shared memory (the q / k / U images are idle now) so that the global
  // reads and writes below are full 16- and 32-byte vectors, contiguous across the lanes of a warp.
  const int i = c * CT + row;
  const size_t orow = qoff + i;
  const int col0 = half == 0 ? 0 : 48, ncol = half == 0 ? 48 : 32;
  float* stage_out = reinterpret_cast<float*>(smem);        // [128][65] fp32, fits in Qimg + Kimg + Uimg
  int flags = 0;
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
        if (i < a.N && !bad) {
          den += a.den[orow];
          a.den[orow] = den;
          if (!finite_f(den)) flags |= OAL_STATUS_NONFINITE;
          else if (!(den > 0.f)) flags |= OAL_STATUS_DENOMINATOR;
        }
        den_s[row] = den;
      }
    }
  }
  __syncthreads();
  if (!dead && !bad) {
    for (int x = tid; x < CT * 8; x += 256) {
      const int r = x >> 3, seg = x & 7, ii = c * CT + r;
      if (ii >= a.N) continue;
      const float dn = fmaxf(den_s[r], a.floor);
      const size_t oo = (qoff + ii) * VD + seg * 8;
      float* np = a.num + oo;
      const float4 o0 = *reinterpret_cast<const float4*>(np), o1 = *reinterpret_cast<const float4*>(np + 4);
      const float* sp = stage_out + r * 65 + seg * 8;
      const float n[8] = {sp[0] + o0.x, sp[1] + o0.y, sp[2] + o0.z, sp[3] + o0.w,
                          sp[4] + o1.x, sp[5] + o1.y, sp[6] + o1.z, sp[7] + o1.w};
      *reinterpret_cast<float4*>(np) = make_float4(n[0], n[1], n[2], n[3]);
      *reinterpret_cast<float4*>(np + 4) = make_float4(n[4], n[5], n[6], n[7]);
      bool fin = true;
#pragma unroll
      for (int j = 0; j < 8; ++j) fin = fin && finite_f(n[j]);
      if (!fin) flags |= OAL_STATUS_NONFINITE;
      if (a.out_dt == OAL_DTYPE_BF16) {
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.out) + oo) =
            make_uint4(pack_bf16(n[0] / dn, n[1] / dn), pack_bf16(n[2] / dn, n[3] / dn),
                       pack_bf16(n[4] / dn, n[5] / dn), pack_bf16(n[6] / dn, n[7] / dn));
      } else if (a.out_dt == OAL_DTYPE_F32) {
        float* op = reinterpret_cast<float*>(a.out) + oo;
        *reinterpret_cast<float4*>(op) = make_float4(n[0] / dn, n[1] / dn, n[2] / dn, n[3] / dn);
        *reinterpret_cast<float4*>(op + 4) = make_float4(n[4] / dn, n[5] / dn, n[6] / dn, n[7] / dn);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) store_elem(a.out, oo + j, a.out_dt, n[j] / dn);
      }
    }
  }
  if (flags) atomicOr(a.status, flags);
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 256);
  if (tid == 0 && dead) atomicOr(a.status, w.status_bits());
}

}  // namespace

cudaError_t OAL_INTRA_NAME(intra_forward)(const void* q, const void* k, const void* v, const int32_t* dim_perm,
                          const int32_t* group_start, const float* A, const float* Bc, const float* Cc, void* out,
                          float* num, float* den, int32_t* status, int B, int Hq, int Hkv, int N, int NB, int G,
                          int out_dt, int slabs, float scale, float floor_v, const void* qimg, const void* kimg,
                          const void* uimg, cudaStream_t st) {
  if (slabs < 1 || slabs > DP_MAX / 16) slabs = DP_MAX / 16;
  const int smem = fwd_smem_bytes(slabs);
  cudaError_t e = cudaFuncSetAttribute(intra_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       fwd_smem_bytes(DP_MAX / 16));
  if (e != cudaSuccess) return e;
  IntraFwdArgs a{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k),
                 static_cast<const __nv_bfloat16*>(v), dim_perm, group_start, A, Bc, Cc, out, num, den, status,
                 N, Hq, Hkv, G, out_dt, slabs, scale, floor_v, static_cast<const unsigned char*>(qimg),
                 static_cast<const unsigned char*>(kimg), static_cast<const unsigned char*>(uimg)};
  intra_fwd_kernel<<<dim3(NB, Hq, B), 256, smem, st>>>(a);
  return cudaGetLastError();
}

// Bytes of one q (or k) image slot for a given slab bound, and the pad_images launcher.
size_t OAL_INTRA_NAME(pad_image_bytes)(int slabs) {
  if (slabs < 1 || slabs > DP_MAX / 16) slabs = DP_MAX / 16;
  return (size_t)slabs * 4096;
}

cudaError_t OAL_INTRA_NAME(pad_images)(const void* q, const void* k, const void* v, const int32_t* dim_perm,
                                       const int32_t* group_start, void* qimg, void* kimg, void* uimg,
                                       int32_t* status, int B, int Hq, int Hkv, int N, int NB, int slabs,
                                       cudaStream_t st) {
  if (slabs < 1 || slabs > DP_MAX / 16) slabs = DP_MAX / 16;
  const int smem = 2 * STAGE_BYTES;
  cudaError_t e = cudaSuccess;
  PadArgs a{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k),
            static_cast<const __nv_bfloat16*>(v), dim_perm, group_start, static_cast<unsigned char*>(qimg),
            static_cast<unsigned char*>(kimg), static_cast<unsigned char*>(uimg), status, N, NB, Hq, Hkv, slabs};
  pad_images_kernel<<<dim3(NB, Hq, B), 256, smem, st>>>(a);
  return cudaGetLastError();
}

}  // namespace oal

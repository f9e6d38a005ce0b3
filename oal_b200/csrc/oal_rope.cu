// Prologue of the operator inside a transformer layer: rotary embedding of q and k fused with the
// move from the projection layout [B, N, H * 64] to the head-first layout [B, H, N, 64] the operator
// reads, and its backward (inverse rotation fused with the move back).  The reference does this with
// separate element-wise passes (qwen_lora_experiment/attention/common.py:550-572: reshape, transpose,
// apply_rotary_pos_emb, three .contiguous() copies).  Rotate-half convention: dimension d pairs with
// d + 32; cos / sin are fp32 [N, 64] with the 32 frequencies repeated twice.
// One thread handles 8 dimensions of the lower half and their 8 partners: two 16-byte loads, two
// 16-byte stores; a token's head row is 128 contiguous bytes on both sides.
#include "oal_common.cuh"
#include "oal_kernels.h"
#include "oal_umma.cuh"

namespace oal {
namespace {

__device__ __forceinline__ void unpack8(const uint4 t, float (&o)[8]) {
  const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    o[2 * j] = __uint_as_float(w[j] << 16);
    o[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
  }
}
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  return make_uint4(umma::pack_bf16(v[0], v[1]), umma::pack_bf16(v[2], v[3]), umma::pack_bf16(v[4], v[5]),
                    umma::pack_bf16(v[6], v[7]));
}

// TO_HEADS: flat [B, N, H, 64] -> heads [B, H, N, 64], rotation by +angle (ROTATE) or plain copy.
// !TO_HEADS: heads -> flat, rotation by -angle (the transpose of the forward map).
template <bool TO_HEADS, bool ROTATE>
__global__ void __launch_bounds__(256) rope_move_kernel(const __nv_bfloat16* src, __nv_bfloat16* dst,
                                                        const float* cosv, const float* sinv, int B, int N, int H) {
  const size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x;     // over B * N * H * 4
  const size_t total = (size_t)B * N * H * 4;
  if (idx >= total) return;
  const int j = (int)(idx & 3);
  const size_t t = idx >> 2;                                       // (b, n, h) in flat order
  const int h = (int)(t % H);
  const size_t bn = t / H;
  const int n = (int)(bn % N), b = (int)(bn / N);
  const size_t flat = ((size_t)(b * N + n) * H + h) * HD;
  const size_t heads = ((size_t)(b * H + h) * N + n) * HD;
  const __nv_bfloat16* s = src + (TO_HEADS ? flat : heads);
  __nv_bfloat16* d = dst + (TO_HEADS ? heads : flat);
  const uint4 lo = *reinterpret_cast<const uint4*>(s + 8 * j);
  const uint4 hi = *reinterpret_cast<const uint4*>(s + 32 + 8 * j);
  if (!ROTATE) {
    *reinterpret_cast<uint4*>(d + 8 * j) = lo;
    *reinterpret_cast<uint4*>(d + 32 + 8 * j) = hi;
    return;
  }
  float xl[8], xh[8], ol[8], oh[8];
  unpack8(lo, xl);
  unpack8(hi, xh);
  const float4 c0 = *reinterpret_cast<const float4*>(cosv + (size_t)n * HD + 8 * j);
  const float4 c1 = *reinterpret_cast<const float4*>(cosv + (size_t)n * HD + 8 * j + 4);
  const float4 s0 = *reinterpret_cast<const float4*>(sinv + (size_t)n * HD + 8 * j);
  const float4 s1 = *reinterpret_cast<const float4*>(sinv + (size_t)n * HD + 8 * j + 4);
  const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float sg = TO_HEADS ? sn[e] : -sn[e];
    ol[e] = xl[e] * cs[e] - xh[e] * sg;
    oh[e] = xh[e] * cs[e] + xl[e] * sg;
  }
  *reinterpret_cast<uint4*>(d + 8 * j) = pack8(ol);
  *reinterpret_cast<uint4*>(d + 32 + 8 * j) = pack8(oh);
}

template <bool TO_HEADS, bool ROTATE>
cudaError_t launch(const void* src, void* dst, const float* cosv, const float* sinv, int B, int N, int H,
                   cudaStream_t st) {
  const size_t total = (size_t)B * N * H * 4;
  if (total == 0) return cudaSuccess;
  rope_move_kernel<TO_HEADS, ROTATE><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(src), static_cast<__nv_bfloat16*>(dst), cosv, sinv, B, N, H);
  return cudaGetLastError();
}

}  // namespace

cudaError_t rope_to_heads(const void* src, void* dst, const float* cosv, const float* sinv, int B, int N, int H,
                          bool rotate, cudaStream_t st) {
  return rotate ? launch<true, true>(src, dst, cosv, sinv, B, N, H, st)
                : launch<true, false>(src, dst, cosv, sinv, B, N, H, st);
}
cudaError_t rope_to_flat(const void* src, void* dst, const float* cosv, const float* sinv, int B, int N, int H,
                         bool rotate, cudaStream_t st) {
  return rotate ? launch<false, true>(src, dst, cosv, sinv, B, N, H, st)
                : launch<false, false>(src, dst, cosv, sinv, B, N, H, st);
}

}  // namespace oal

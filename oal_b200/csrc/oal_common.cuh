// Shared device helpers for the oal_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/oal_b200.h"

namespace oal {

constexpr int HD = OAL_HEAD_DIM;      // head dimension of q/k (padded by the host)
constexpr int VD = OAL_HEAD_DIM;      // value dimension
constexpr int E1 = VD + 1;            // [v | 1]
constexpr int EP = OAL_E_PAD;         // E1 padded to a multiple of 16
constexpr int GMAX = OAL_MAX_GROUPS;
constexpr int NCOEF = 1 + GMAX + GMAX * (GMAX + 1) / 2;   // A, B[g], C[g<=g'] partial-sum slots

// ---- dtype-generic element access (io tensors are fp32, bf16 or fp16) -------
__device__ __forceinline__ float load_elem(const void* p, size_t i, int dt) {
  if (dt == OAL_DTYPE_F32) return reinterpret_cast<const float*>(p)[i];
  if (dt == OAL_DTYPE_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}

__device__ __forceinline__ void store_elem(void* p, size_t i, int dt, float v) {
  if (dt == OAL_DTYPE_F32) reinterpret_cast<float*>(p)[i] = v;
  else if (dt == OAL_DTYPE_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
}

// Four consecutive elements starting at a multiple of four.
__device__ __forceinline__ void load4(const void* p, size_t i, int dt, float (&o)[4]) {
  if (dt == OAL_DTYPE_F32) {
    float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
    o[0] = t.x; o[1] = t.y; o[2] = t.z; o[3] = t.w;
  } else if (dt == OAL_DTYPE_BF16) {
    uint2 t = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p) + i);
    __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&t.x);
    __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&t.y);
    o[0] = __low2float(a); o[1] = __high2float(a); o[2] = __low2float(b); o[3] = __high2float(b);
  } else {
    uint2 t = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(p) + i);
    __half2 a = *reinterpret_cast<__half2*>(&t.x);
    __half2 b = *reinterpret_cast<__half2*>(&t.y);
    o[0] = __low2float(a); o[1] = __high2float(a); o[2] = __low2float(b); o[3] = __high2float(b);
  }
}

__device__ __forceinline__ bool finite_f(float x) { return fabsf(x) <= 3.402823466e38f; }

// Per-head description of the dimension groups, staged in shared memory.
struct HeadGroups {
  int perm[HD];            // permuted position p holds original dimension perm[p]
  int start[GMAX + 1];     // group g owns permuted positions [start[g], start[g+1])
  int group_of[HD];        // group id of permuted position p
};

__device__ __forceinline__ void load_head_groups(HeadGroups& hg, const int32_t* dim_perm,
                                                 const int32_t* group_start, int h, int tid,
                                                 int nthreads) {
  for (int x = tid; x < HD; x += nthreads) hg.perm[x] = dim_perm[h * HD + x];
  for (int x = tid; x <= GMAX; x += nthreads) hg.start[x] = group_start[h * (GMAX + 1) + x];
  __syncthreads();
  for (int x = tid; x < HD; x += nthreads) {
    int g = 0;
    while (g < GMAX - 1 && x >= hg.start[g + 1]) ++g;
    hg.group_of[x] = g;
  }
}

}  // namespace oal

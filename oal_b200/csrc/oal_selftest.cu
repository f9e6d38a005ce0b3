// Self-test of the tensor-core building blocks: one 128 x N x K bf16 GEMM through
// tcgen05.mma with each operand arrangement the attention kernels rely on.
// It exists so that a wrong descriptor encoding shows up as a failed unit test with
// a small, readable error instead of as a parity failure of the whole operator.
#include "oal_common.cuh"
#include "oal_umma.cuh"

namespace oal {
namespace {

using namespace umma;

// mode 0: A [128][K] and B [N][K] row-major (K contiguous)     -> both operands K-major in smem
// mode 1: A [K][128] and B [K][N] row-major (M / N contiguous) -> both operands MN-major in smem
// mode 2: A [128][K] written to TMEM as packed bf16 pairs, B [N][K] K-major in smem
// D [128][N] fp32 = A * B^T (modes 0, 2) or A^T * B (mode 1).
__global__ void __launch_bounds__(128) umma_selftest_kernel(const __nv_bfloat16* A, const __nv_bfloat16* B,
                                                            float* D, int N, int K, int mode, int* status) {
  extern __shared__ __align__(128) unsigned char smem[];
  __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(smem);
  __nv_bfloat16* Bs = As + 128 * K;
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (mode == 1) {
    for (int x = tid; x < 128 * K; x += 128) {
      int k = x / 128, m = x % 128;
      As[((m >> 3) * K + k) * 8 + (m & 7)] = A[x];
    }
    for (int x = tid; x < N * K; x += 128) {
      int k = x / N, n = x % N;
      Bs[((n >> 3) * K + k) * 8 + (n & 7)] = B[x];
    }
  } else {
    for (int x = tid; x < 128 * K; x += 128) {
      int m = x / K, k = x % K;
      As[((k >> 3) * 128 + m) * 8 + (k & 7)] = A[x];
    }
    for (int x = tid; x < N * K; x += 128) {
      int n = x / K, k = x % K;
      Bs[((k >> 3) * N + n) * 8 + (k & 7)] = B[x];
    }
  }
  fence_async_smem();
  if (warp == 0) tmem_alloc(&tmem_base, 512);
  if (tid == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tacc = tmem_base;            // columns [0, N)
  const uint32_t ta = tmem_base + 256;        // columns [256, 256 + K/2) for mode 2
  if (mode == 2) {
    // each thread owns one row (lane of TMEM) and writes its K/2 packed columns
    const int m = warp * 32 + lane;
    for (int c0 = 0; c0 < K / 2; c0 += 16) {
      uint32_t r[16];
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const int k = 2 * (c0 + c);
        r[c] = pack_bf16(__bfloat162float(A[m * K + k]), __bfloat162float(A[m * K + k + 1]));
      }
      tmem_st16(ta + ((uint32_t)(warp * 32) << 16) + c0, r);
    }
    tmem_st_wait();
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
  }
  if (tid == 0) {
    const uint32_t idesc = instr_desc_bf16(128, N, mode == 1, mode == 1);
    const uint32_t a0 = smem_u32(As), b0 = smem_u32(Bs);
    for (int ks = 0; ks < K / 16; ++ks) {
      uint64_t ad, bd;
      if (mode == 1) {
        ad = smem_desc(a0 + ks * 256, 128, K * 16);
        bd = smem_desc(b0 + ks * 256, 128, K * 16);
      } else {
        ad = smem_desc(a0 + ks * 2 * 128 * 16, 128 * 16, 128);
        bd = smem_desc(b0 + ks * 2 * N * 16, N * 16, 128);
      }
      if (mode == 2) mma_bf16_ts(tacc, ta + ks * 8, bd, idesc, ks > 0);
      else mma_bf16_ss(tacc, ad, bd, idesc, ks > 0);
    }
    mma_commit(&bar);
  }
  const bool ok = mbar_wait(&bar, 0);
  fence_after_sync();
  if (ok) {
    const int m = warp * 32 + lane;
    for (int c0 = 0; c0 < N; c0 += 16) {
      float v[16];
      tmem_ld16(tacc + ((uint32_t)(warp * 32) << 16) + c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int c = 0; c < 16; ++c) D[m * N + c0 + c] = v[c];
    }
  } else if (tid == 0) {
    atomicOr(status, OAL_STATUS_WAIT_TIMEOUT);
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, 512);
}

// One warp waits on an mbarrier that nothing ever arrives on, with a short limit: the wait gives up,
// the kernel records the status word exactly as the production kernels do (timeout flag + site id)
// and returns normally.  Nothing hangs, traps or faults; the context stays usable.
constexpr int SELFTEST_WAIT_SITE = 0x7E;
__global__ void __launch_bounds__(32) wait_timeout_selftest_kernel(long long limit_clocks, int* status) {
  __shared__ uint64_t bar;
  __shared__ int dead;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
    dead = 0;
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    if (!mbar_wait(&bar, 0, limit_clocks)) dead = SELFTEST_WAIT_SITE;
    if (dead) atomicOr(status, OAL_STATUS_WAIT_TIMEOUT | ((dead & 0xFF) << 8));
  }
}

}  // namespace
}  // namespace oal

extern "C" int oal_selftest_wait_timeout(int64_t limit_clocks, int32_t* status, void* stream) {
  if (!status || limit_clocks < 1 || limit_clocks > 1000000) return OAL_ERR_ARGUMENT;
  oal::wait_timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>((long long)limit_clocks, status);
  return cudaGetLastError() == cudaSuccess ? OAL_OK : OAL_ERR_CUDA;
}

extern "C" int oal_selftest_umma(int mode, int n, int k, const void* a, const void* b, float* d,
                                 int32_t* status, void* stream) {
  if (mode < 0 || mode > 2 || n < 16 || n > 256 || n % 16 || k < 16 || k > 128 || k % 16 || !a || !b || !d || !status)
    return OAL_ERR_ARGUMENT;
  const size_t smem = (size_t)(128 + n) * k * sizeof(__nv_bfloat16);
  cudaError_t e = cudaFuncSetAttribute(oal::umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem);
  if (e != cudaSuccess) return OAL_ERR_CUDA;
  oal::umma_selftest_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), d, n, k, mode, status);
  return cudaGetLastError() == cudaSuccess ? OAL_OK : OAL_ERR_CUDA;
}

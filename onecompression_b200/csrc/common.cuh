// Shared helpers for the sm_100a kernels of the GPTQ / QEP path.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

// Status codes returned by every extern "C" entry point.
#define OC_OK 0
#define OC_ERR_INVALID_ARG (-1)
#define OC_ERR_CUDA (-2)
#define OC_ERR_UNSUPPORTED (-3)
#define OC_ERR_WORKSPACE (-4)
#define OC_ERR_TOO_LARGE (-5)

#define OC_CHECK_LAUNCH()                                   \
  do {                                                      \
    oc_count_launches(1);                                   \
    cudaError_t e__ = cudaGetLastError();                   \
    if (e__ != cudaSuccess) {                               \
      oc_set_last_error(cudaGetErrorString(e__));           \
      return OC_ERR_CUDA;                                   \
    }                                                       \
  } while (0)

#define OC_CUDA(call)                                       \
  do {                                                      \
    cudaError_t e__ = (call);                               \
    if (e__ != cudaSuccess) {                               \
      oc_set_last_error(cudaGetErrorString(e__));           \
      return OC_ERR_CUDA;                                   \
    }                                                       \
  } while (0)

#define OC_REQUIRE(cond, msg)                               \
  do {                                                      \
    if (!(cond)) {                                          \
      oc_set_last_error(msg);                               \
      return OC_ERR_INVALID_ARG;                            \
    }                                                       \
  } while (0)

void oc_set_last_error(const char* msg);
void oc_count_launches(int n);

// 16-bit element types of weights and activations (the `dtype` arguments of the C ABI)
enum : int { OC_DTYPE_F16 = 0, OC_DTYPE_BF16 = 1 };

__device__ __forceinline__ float oc_ld16(const void* p, long long i, int bf16) {
  return bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i])
              : __half2float(static_cast<const __half*>(p)[i]);
}
__device__ __forceinline__ void oc_st16(void* p, long long i, float v, int bf16) {
  if (bf16) static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else static_cast<__half*>(p)[i] = __float2half_rn(v);
}

static inline int oc_div_up(long long a, long long b) { return (int)((a + b - 1) / b); }

// Function attributes (the opt-in to more than 48 KB of dynamic shared memory) and device
// properties belong to a device, and one process may drive several: keep "done" flags and cached
// values per device.  OC_MAX_DEVICES bounds the tables; OC_CURRENT_DEVICE(dev) fetches the index.
#define OC_MAX_DEVICES 64
#define OC_CURRENT_DEVICE(dev)                                            \
  int dev = 0;                                                            \
  OC_CUDA(cudaGetDevice(&dev));                                           \
  OC_REQUIRE(dev >= 0 && dev < OC_MAX_DEVICES, "device index out of range")

// Raises the dynamic shared memory limit of `kernel` to `bytes` once per device.
#define OC_OPT_IN_SMEM(kernel, bytes)                                                             \
  do {                                                                                            \
    static bool done__[OC_MAX_DEVICES] = {};                                                      \
    OC_CURRENT_DEVICE(dev__);                                                                     \
    if (!done__[dev__]) {                                                                         \
      OC_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));  \
      done__[dev__] = true;                                                                       \
    }                                                                                             \
  } while (0)

// ---- engines of oc_moment_accum (its `engine` argument) ---------------------
enum : int {
  OC_MOMENT_AUTO = 0,    // tensor cores when the shapes allow, else FMA
  OC_MOMENT_SIMT = 1,    // fp32 FMA kernel
  OC_MOMENT_SINGLE = 2,  // tcgen05, one CTA per 128 x 256 tile
  OC_MOMENT_PAIR = 3,    // tcgen05 cta_group::2, one CTA pair per 256 x 256 tile
};
#ifndef OC_MOMENT_AUTO_USES_PAIRS
#define OC_MOMENT_AUTO_USES_PAIRS 0
#endif

// ---- fp32 GEMM engine (gemm.cu) -------------------------------------------
// C[M,N] = beta*C + alpha * opA(A) * opB(B), all fp32, exact FMA arithmetic.
//   transA = 0: A is [M,K] row-major (lda);  1: A is [K,M] row-major.
//   transB = 0: B is [K,N] row-major (ldb);  1: B is [N,K] row-major.
// Flags restrict work to the structurally non-zero part of triangular
// operands; coordinates are relative to the sub-matrices passed in.
enum : int {
  OC_GEMM_SKIP_UPPER_TILES = 1,  // do not compute tiles entirely above the diagonal of C
  OC_GEMM_KLO_FROM_N = 2,        // op(B)[k,n] == 0 for k < n   (k range starts at tile's first n)
  OC_GEMM_KHI_FROM_M = 4,        // op(A)[m,k] == 0 for k > m   (k range ends at tile's last m)
  OC_GEMM_KHI_FROM_N = 8,        // op(B)[k,n] == 0 for k > n   (k range ends at tile's last n)
  OC_GEMM_KLO_FROM_M = 16,       // op(A)[m,k] == 0 for k < m   (k range starts at tile's first m)
};

struct OcGemm {
  const float* A; long long lda; long long strideA;
  const float* B; long long ldb; long long strideB;
  float* C; long long ldc; long long strideC;
  int M, N, K;
  float alpha, beta;
  int transA, transB, flags, batch;
};

int oc_gemm_f32_launch(const OcGemm& g, cudaStream_t stream);

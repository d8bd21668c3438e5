// Fused RMSNorm for the block passes of the QEP driver:
//   y = weight * fp16( float(x) * rsqrt( mean(float(x)^2) + eps ) )
// i.e. the formula of the Llama / Mistral / Qwen RMSNorm modules that the block passes
// otherwise run as seven elementwise kernels through fp32 temporaries (upcast, square, mean,
// rsqrt, scale, downcast, weight multiply).  One CTA per row; HBM bound (2 bytes in, 2 out per
// element).  Rounding points are the module's: fp32 up to the downcast, fp16 weight product.
#include "common.cuh"

namespace {

__global__ void __launch_bounds__(256) rmsnorm_f16_kernel(const __half* __restrict__ x, long long ldx,
                                                          const __half* __restrict__ w, float eps, int d,
                                                          __half* __restrict__ y, long long ldy) {
  const long long row = blockIdx.x;
  const __half* xr = x + row * ldx;
  __half* yr = y + row * ldy;
  __shared__ float red[8];
  float ss = 0.f;
  const bool vec = (d % 8 == 0) && (ldx % 8 == 0) && (ldy % 8 == 0) &&
                   ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) |
                     reinterpret_cast<uintptr_t>(w)) & 15) == 0;
  if (vec) {
    for (int i = threadIdx.x * 8; i < d; i += 256 * 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
      const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) { const float2 f = __half22float2(h[k]); ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss); }
    }
  } else {
    for (int i = threadIdx.x; i < d; i += 256) { const float f = __half2float(xr[i]); ss = fmaf(f, f, ss); }
  }
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) tot += red[k];
  const float r = rsqrtf(tot / (float)d + eps);
  if (vec) {
    for (int i = threadIdx.x * 8; i < d; i += 256 * 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(xr + i);
      const uint4 g = *reinterpret_cast<const uint4*>(w + i);
      const __half2* h = reinterpret_cast<const __half2*>(&v);
      const __half2* gw = reinterpret_cast<const __half2*>(&g);
      uint4 o4;
      __half2* o = reinterpret_cast<__half2*>(&o4);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __half22float2(h[k]);
        o[k] = __hmul2(gw[k], __floats2half2_rn(f.x * r, f.y * r));
      }
      *reinterpret_cast<uint4*>(yr + i) = o4;
    }
  } else {
    for (int i = threadIdx.x; i < d; i += 256)
      yr[i] = __hmul(w[i], __float2half_rn(__half2float(xr[i]) * r));
  }
}

}  // namespace

// See include/onecomp_b200.h for the contract.
extern "C" int oc_rmsnorm_f16(const void* x, long long ldx, const void* weight, float eps, long long rows,
                              int d, void* y, long long ldy, void* stream) {
  OC_REQUIRE(x && weight && y && d > 0 && rows >= 0 && ldx >= d && ldy >= d, "rmsnorm: bad arguments");
  OC_REQUIRE(rows < (1ll << 31), "rmsnorm: too many rows");
  if (rows == 0) return OC_OK;
  rmsnorm_f16_kernel<<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>(
      (const __half*)x, ldx, (const __half*)weight, eps, d, (__half*)y, ldy);
  OC_CHECK_LAUNCH();
  return OC_OK;
}

// Second-moment helpers and the general-shape moment kernel.
//
//   H <- a_old * H + a_new * Xq^T Xq            (Hessian; reference
//   C <- a_old * C + a_new * (Xf - Xq)^T Xq      onecomp/quantizer/_quantizer.py:764-895,
//                                               onecomp/qep/_quantize_with_qep_arch.py:118-201)
//
// The tensor-core kernel (moment_tc.cu) needs rows of X that are 16-byte
// multiples; this fp32 FMA kernel takes any shape and is also the independent
// cross-check of the tensor-core path in the tests.  fp16 products are exact
// in fp32, accumulation is fp32.
#include "common.cuh"

namespace {

constexpr int T = 64;    // output tile
constexpr int KT = 32;   // tokens per step

__global__ void scale_matrix_kernel(float* __restrict__ M, long long ld, int n, float a) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int i = blockIdx.y;
  if (j < n) {
    float* p = M + (long long)i * ld + j;
    *p = (a == 0.f) ? 0.f : a * (*p);
  }
}

// One CTA: 64x64 tile of the d x d moment over a slice of the tokens; adds a_new * partial
// atomically (the matrix was rescaled by a_old beforehand).
__global__ void __launch_bounds__(256) moment_simt_kernel(const void* __restrict__ xq,
                                                          const void* __restrict__ xf, int bf16,
                                                          long long n_tok, int d, long long ld,
                                                          float* __restrict__ H, float* __restrict__ C,
                                                          long long ldh, float a_new, int tok_per_split) {
  __shared__ float Bq[KT][T + 1];  // xq columns n0..  (right operand of both moments)
  __shared__ float Aq[KT][T + 1];  // xq columns m0..
  __shared__ float Ad[KT][T + 1];  // (xf - xq) columns m0..
  const int m0 = blockIdx.y * T, n0 = blockIdx.x * T;
  const long long t_begin = (long long)blockIdx.z * tok_per_split;
  const long long t_end = min(n_tok, t_begin + tok_per_split);
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const bool cross = (xf != nullptr) && (C != nullptr);
  float hacc[4][4] = {}, cacc[4][4] = {};
  for (long long t0 = t_begin; t0 < t_end; t0 += KT) {
    for (int e = tid; e < KT * T; e += 256) {
      const int k = e / T, c = e % T;
      const long long t = t0 + k;
      float bq = 0.f, aq = 0.f, ad = 0.f;
      if (t < t_end) {
        if (n0 + c < d) bq = oc_ld16(xq, t * ld + n0 + c, bf16);
        if (m0 + c < d) {
          aq = oc_ld16(xq, t * ld + m0 + c, bf16);
          if (cross) ad = oc_ld16(xf, t * ld + m0 + c, bf16) - aq;
        }
      }
      Bq[k][c] = bq; Aq[k][c] = aq; Ad[k][c] = ad;
    }
    __syncthreads();
#pragma unroll 4
    for (int k = 0; k < KT; ++k) {
      float a[4], b[4], dl[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = Aq[k][ty * 4 + i]; b[i] = Bq[k][tx * 4 + i]; dl[i] = Ad[k][ty * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          hacc[i][j] = fmaf(a[i], b[j], hacc[i][j]);
          if (cross) cacc[i][j] = fmaf(dl[i], b[j], cacc[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = m0 + ty * 4 + i, c = n0 + tx * 4 + j;
      if (r < d && c < d) {
        if (H) atomicAdd(H + (long long)r * ldh + c, a_new * hacc[i][j]);
        if (cross) atomicAdd(C + (long long)r * ldh + c, a_new * cacc[i][j]);
      }
    }
}

// D = float(xf) - float(xq) as two planes in the activations' own 16-bit type:
//   hi = round16(D)                 (exact whenever the two values are within a factor of two)
//   lo = round16((D - hi) * lo_up)  (the rounding error of hi, scaled up into the normal range)
// Rows are read ld elements apart and written packed (d elements apart); eight elements per thread.
template <typename T2>
__device__ __forceinline__ float2 oc_cvt2(T2 v);
template <> __device__ __forceinline__ float2 oc_cvt2<__half2>(__half2 v) { return __half22float2(v); }
template <> __device__ __forceinline__ float2 oc_cvt2<__nv_bfloat162>(__nv_bfloat162 v) { return __bfloat1622float2(v); }
template <typename T2>
__device__ __forceinline__ T2 oc_rnd2(float a, float b);
template <> __device__ __forceinline__ __half2 oc_rnd2<__half2>(float a, float b) { return __floats2half2_rn(a, b); }
template <> __device__ __forceinline__ __nv_bfloat162 oc_rnd2<__nv_bfloat162>(float a, float b) { return __floats2bfloat162_rn(a, b); }

template <typename T2>
__global__ void delta_split_kernel(const uint4* __restrict__ xf, const uint4* __restrict__ xq, long long ld8,
                                   uint4* __restrict__ hi, uint4* __restrict__ lo, long long n_tok, int d8,
                                   float lo_up) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_tok * d8) return;
  const long long t = i / d8;
  const int c = (int)(i - t * d8);
  union V { uint4 u; T2 h[4]; };
  V f, q, oh, ol;
  f.u = xf[t * ld8 + c];
  q.u = xq[t * ld8 + c];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 a = oc_cvt2<T2>(f.h[k]), b = oc_cvt2<T2>(q.h[k]);
    const float dx = a.x - b.x, dy = a.y - b.y;
    const T2 h = oc_rnd2<T2>(dx, dy);
    const float2 hf = oc_cvt2<T2>(h);
    oh.h[k] = h;
    ol.h[k] = oc_rnd2<T2>((dx - hf.x) * lo_up, (dy - hf.y) * lo_up);
  }
  hi[i] = oh.u;
  lo[i] = ol.u;
}

// lower <- upper (mirror across the diagonal), 32x32 tiles
__global__ void mirror_upper_kernel(float* __restrict__ M, long long ld, int n) {
  __shared__ float t[32][33];
  const int bi = blockIdx.y, bj = blockIdx.x;
  if (bj < bi) return;  // only tiles on or above the diagonal are sources
  const int tx = threadIdx.x, ty = threadIdx.y;
  for (int k = ty; k < 32; k += 8) {
    const int r = bi * 32 + k, c = bj * 32 + tx;
    t[k][tx] = (r < n && c < n) ? M[(long long)r * ld + c] : 0.f;
  }
  __syncthreads();
  for (int k = ty; k < 32; k += 8) {
    const int r = bj * 32 + k, c = bi * 32 + tx;  // transposed position
    if (r < n && c < n && r > c) M[(long long)r * ld + c] = t[tx][k];
  }
}

}  // namespace

int oc_moment_simt_launch(const void* xq, const void* xf, int bf16, long long n_tok, int d, long long ld,
                          float* H, float* C, long long ldh, float a_old, float a_new,
                          cudaStream_t stream) {
  const int tb = 256;
  dim3 sg(oc_div_up(d, tb), d);
  if (H) scale_matrix_kernel<<<sg, tb, 0, stream>>>(H, ldh, d, a_old);
  if (H && C) oc_count_launches(1);
  if (C) scale_matrix_kernel<<<sg, tb, 0, stream>>>(C, ldh, d, a_old);
  OC_CHECK_LAUNCH();
  if (n_tok <= 0) return OC_OK;
  const int tiles = oc_div_up(d, T);
  // enough token slices to fill the device a few times over, at least 256 tokens each
  long long splits = (148LL * 4 + (long long)tiles * tiles - 1) / ((long long)tiles * tiles);
  splits = max(1LL, min(splits, (n_tok + 255) / 256));
  splits = min(splits, 65535LL);
  long long per = (n_tok + splits - 1) / splits;
  per = (per + KT - 1) / KT * KT;
  splits = (n_tok + per - 1) / per;
  moment_simt_kernel<<<dim3(tiles, tiles, (unsigned)splits), 256, 0, stream>>>(
      xq, xf, bf16, n_tok, d, ld, H, C, ldh, a_new, (int)per);
  OC_CHECK_LAUNCH();
  return OC_OK;
}

// out = [2][n_tok][d]: the hi plane, then the lo plane.  d and ld multiples of 8, all pointers
// 16-byte aligned (the conditions of the tensor-core path).
int oc_delta_split_launch(const void* xf, const void* xq, long long ld, void* out, long long n_tok, int d,
                          int bf16, float lo_up, cudaStream_t stream) {
  OC_REQUIRE(xf && xq && out && n_tok >= 0 && d % 8 == 0 && ld % 8 == 0, "delta_split: bad arguments");
  if (n_tok == 0) return OC_OK;
  const int d8 = d / 8;
  const long long n = n_tok * d8;
  uint4* hi = (uint4*)out;
  uint4* lo = hi + n;
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (bf16)
    delta_split_kernel<__nv_bfloat162><<<grid, 256, 0, stream>>>((const uint4*)xf, (const uint4*)xq, ld / 8, hi, lo,
                                                               n_tok, d8, lo_up);
  else
    delta_split_kernel<__half2><<<grid, 256, 0, stream>>>((const uint4*)xf, (const uint4*)xq, ld / 8, hi, lo, n_tok,
                                                        d8, lo_up);
  OC_CHECK_LAUNCH();
  return OC_OK;
}

extern "C" int oc_mirror_upper(float* M, long long ld, int n, void* stream) {
  OC_REQUIRE(M && n > 0 && ld >= n, "mirror_upper: bad arguments");
  const int t = oc_div_up(n, 32);
  mirror_upper_kernel<<<dim3(t, t), dim3(32, 8), 0, (cudaStream_t)stream>>>(M, ld, n);
  OC_CHECK_LAUNCH();
  return OC_OK;
}

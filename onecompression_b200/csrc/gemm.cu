// fp32 GEMM engine, FMA version: C = beta*C + alpha*opA(A)*opB(B) with exact fp32 FMA
// arithmetic.  Products whose operands are 16-byte aligned go to the tensor-core version
// (gemm_tc.cu, 3xTF32) unless oc_set_gemm_engine(1) pins this one; this kernel takes every
// other shape and is the reference the tensor-core engine is tested against.
//
// One engine serves every fp32 matrix product of the path: the lazy-batch
// trailing update of the GPTQ column loop, the trailing update and panel solve
// of the blocked Cholesky factorisation, the recursive triangular inverse and
// the three products of the QEP weight correction.  128x128x16 tiles, 256
// threads, 8x8 outputs per thread, register-prefetch double buffering.
#include "common.cuh"

namespace {

constexpr int TM = 128, TN = 128, TK = 16, NT = 256;
constexpr int PAD = 4;  // keeps float4 alignment, spreads the transposing stores over banks

template <bool VEC>
__device__ __forceinline__ void load_rows_k(  // source is [rows, K] row-major: 128 rows x 16 k
    const float* __restrict__ src, long long ld, int row0, int nrows, int k0, int kend,
    float (&reg)[2][4], int tid) {
  const int kq = (tid & 3) * 4;
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    const int r = row0 + (tid >> 2) + 64 * p;
    const int k = k0 + kq;
    if (VEC) {
      if (r < nrows && k + 3 < kend) {
        const float4 v = *reinterpret_cast<const float4*>(src + (long long)r * ld + k);
        reg[p][0] = v.x; reg[p][1] = v.y; reg[p][2] = v.z; reg[p][3] = v.w;
        continue;
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
      reg[p][i] = (r < nrows && k + i < kend) ? src[(long long)r * ld + k + i] : 0.f;
  }
}

__device__ __forceinline__ void store_rows_k(float (*dst)[TM + PAD], const float (&reg)[2][4], int tid) {
  const int kq = (tid & 3) * 4;
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    const int r = (tid >> 2) + 64 * p;
#pragma unroll
    for (int i = 0; i < 4; ++i) dst[kq + i][r] = reg[p][i];
  }
}

template <bool VEC>
__device__ __forceinline__ void load_k_rows(  // source is [K, cols] row-major: 16 k x 128 cols
    const float* __restrict__ src, long long ld, int col0, int ncols, int k0, int kend,
    float (&reg)[2][4], int tid) {
  const int c = col0 + (tid & 31) * 4;
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    const int k = k0 + (tid >> 5) + 8 * p;
    if (VEC) {
      if (k < kend && c + 3 < ncols) {
        const float4 v = *reinterpret_cast<const float4*>(src + (long long)k * ld + c);
        reg[p][0] = v.x; reg[p][1] = v.y; reg[p][2] = v.z; reg[p][3] = v.w;
        continue;
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
      reg[p][i] = (k < kend && c + i < ncols) ? src[(long long)k * ld + c + i] : 0.f;
  }
}

__device__ __forceinline__ void store_k_rows(float (*dst)[TM + PAD], const float (&reg)[2][4], int tid) {
  const int c = (tid & 31) * 4;
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    const int k = (tid >> 5) + 8 * p;
    *reinterpret_cast<float4*>(&dst[k][c]) = make_float4(reg[p][0], reg[p][1], reg[p][2], reg[p][3]);
  }
}

template <bool TA, bool TB, bool VEC>
__global__ void __launch_bounds__(NT, 2) gemm_f32_kernel(OcGemm g) {
  __shared__ __align__(16) float As[2][TK][TM + PAD];
  __shared__ __align__(16) float Bs[2][TK][TN + PAD];

  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  if ((g.flags & OC_GEMM_SKIP_UPPER_TILES) && n0 > m0 + TM - 1) return;

  const float* A = g.A + (long long)blockIdx.z * g.strideA;
  const float* B = g.B + (long long)blockIdx.z * g.strideB;
  float* C = g.C + (long long)blockIdx.z * g.strideC;

  int k_lo = 0, k_hi = g.K;
  if (g.flags & OC_GEMM_KLO_FROM_N) k_lo = max(k_lo, n0);
  if (g.flags & OC_GEMM_KLO_FROM_M) k_lo = max(k_lo, m0);
  if (g.flags & OC_GEMM_KHI_FROM_M) k_hi = min(k_hi, m0 + TM);
  if (g.flags & OC_GEMM_KHI_FROM_N) k_hi = min(k_hi, n0 + TN);
  k_lo = (k_lo / TK) * TK;

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  float ra[2][4], rb[2][4];
  auto fetch = [&](int k0) {
    if (TA) load_k_rows<VEC>(A, g.lda, m0, g.M, k0, k_hi, ra, tid);
    else    load_rows_k<VEC>(A, g.lda, m0, g.M, k0, k_hi, ra, tid);
    if (TB) load_rows_k<VEC>(B, g.ldb, n0, g.N, k0, k_hi, rb, tid);
    else    load_k_rows<VEC>(B, g.ldb, n0, g.N, k0, k_hi, rb, tid);
  };
  auto stash = [&](int buf) {
    if (TA) store_k_rows(As[buf], ra, tid); else store_rows_k(As[buf], ra, tid);
    if (TB) store_rows_k(Bs[buf], rb, tid); else store_k_rows(Bs[buf], rb, tid);
  };

  const int tx = tid & 15, ty = tid >> 4;
  if (k_lo < k_hi) {
    fetch(k_lo);
    stash(0);
    __syncthreads();
    int buf = 0;
    for (int k0 = k_lo; k0 < k_hi; k0 += TK) {
      const bool more = k0 + TK < k_hi;
      if (more) fetch(k0 + TK);
#pragma unroll
      for (int k = 0; k < TK; ++k) {
        const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
        const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
        const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
        const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][k][64 + tx * 4]);
        const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
      if (more) {
        stash(buf ^ 1);
        __syncthreads();
        buf ^= 1;
      }
    }
  }

  const float alpha = g.alpha, beta = g.beta;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (r >= g.M) continue;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int c = n0 + h * 64 + tx * 4;
      float* p = C + (long long)r * g.ldc + c;
      if (VEC && c + 3 < g.N) {
        float4 o;
        if (beta != 0.f) {
          const float4 v = *reinterpret_cast<const float4*>(p);
          o.x = fmaf(alpha, acc[i][h * 4 + 0], beta * v.x);
          o.y = fmaf(alpha, acc[i][h * 4 + 1], beta * v.y);
          o.z = fmaf(alpha, acc[i][h * 4 + 2], beta * v.z);
          o.w = fmaf(alpha, acc[i][h * 4 + 3], beta * v.w);
        } else {
          o.x = alpha * acc[i][h * 4 + 0]; o.y = alpha * acc[i][h * 4 + 1];
          o.z = alpha * acc[i][h * 4 + 2]; o.w = alpha * acc[i][h * 4 + 3];
        }
        *reinterpret_cast<float4*>(p) = o;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (c + j < g.N) {
            const float v = (beta != 0.f) ? beta * p[j] : 0.f;
            p[j] = fmaf(alpha, acc[i][h * 4 + j], v);
          }
        }
      }
    }
  }
}

template <bool VEC>
void launch_variant(const OcGemm& g, dim3 grid, cudaStream_t s) {
  if (g.transA) {
    if (g.transB) gemm_f32_kernel<true, true, VEC><<<grid, NT, 0, s>>>(g);
    else          gemm_f32_kernel<true, false, VEC><<<grid, NT, 0, s>>>(g);
  } else {
    if (g.transB) gemm_f32_kernel<false, true, VEC><<<grid, NT, 0, s>>>(g);
    else          gemm_f32_kernel<false, false, VEC><<<grid, NT, 0, s>>>(g);
  }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

bool oc_gemm_tc_eligible(const OcGemm& g);
int oc_gemm_tc_launch(const OcGemm& g, cudaStream_t stream);

static int g_engine_mode = 0;  // 0: tensor cores (3xTF32) when the operands allow it; 1: FMA engine only

extern "C" int oc_set_gemm_engine(int mode) {
  const int old = g_engine_mode;
  if (mode == 0 || mode == 1) g_engine_mode = mode;
  return old;
}

int oc_gemm_f32_launch(const OcGemm& g, cudaStream_t stream) {
  if (g.M <= 0 || g.N <= 0 || g.batch <= 0) return OC_OK;
  OC_REQUIRE(g.A && g.B && g.C && g.K >= 0, "gemm: null operand or negative K");
  if (g_engine_mode == 0 && oc_gemm_tc_eligible(g)) return oc_gemm_tc_launch(g, stream);
  const int tiles_m = oc_div_up(g.M, TM), tiles_n = oc_div_up(g.N, TN);
  OC_REQUIRE(tiles_m <= 65535 && g.batch <= 65535, "gemm: M or batch too large for one launch");
  const bool vec = aligned16(g.A) && aligned16(g.B) && aligned16(g.C) && g.lda % 4 == 0 &&
                   g.ldb % 4 == 0 && g.ldc % 4 == 0 && g.strideA % 4 == 0 &&
                   g.strideB % 4 == 0 && g.strideC % 4 == 0;
  dim3 grid(tiles_n, tiles_m, g.batch);
  if (vec) launch_variant<true>(g, grid, stream);
  else     launch_variant<false>(g, grid, stream);
  OC_CHECK_LAUNCH();
  return OC_OK;
}

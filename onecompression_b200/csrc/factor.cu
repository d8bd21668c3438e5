// Inverse-Hessian factor for GPTQ: U upper triangular with U^T U = (H + damp I)^-1.
//
// Replaces the potrf + potri + potrf sequence of the reference
// (onecomp/quantizer/gptq/_gptq.py:594-643, call sites :693-706) with one
// Cholesky factorisation and one triangular inverse:
//
//   A = J (P H P^T + damp I) J      (J reverses the index order, P is the act-order permutation)
//   A = L L^T                       blocked right-looking Cholesky (two levels: 128 / 512), fp32:
//                                   diagonal block on one SM, panel solve by forward substitution
//                                   (fp32 FMAs, all SMs), updates on the tensor cores (3xTF32)
//   X = L^-1                        diagonal blocks inverted in one launch, then joined level by
//                                   level (recursive blocked triangular inverse), fp32
//   U = J X J                       upper triangular, U^T U = (P H P^T + damp I)^-1
//
// because J L J is the upper factor V of H = V V^T and U = V^-1.
#include "common.cuh"

namespace {

constexpr int NB = 128;  // panel width
constexpr int OB = 512;  // outer block of the two-level Cholesky

// ---- diag statistics: dead columns, damping --------------------------------
// diagv[j] = H[j,j] (1 where it is 0), dead[j], damp_out[0] = percdamp * mean(diagv)
// Batched launches: block index `b` of the batch dimension selects the problem; `sH`, `sW`, ... are
// the element strides between consecutive problems.
__global__ void diag_stats_kernel(const float* __restrict__ H, long long ld, int n, float percdamp,
                                  float* __restrict__ diagv, unsigned char* __restrict__ dead,
                                  float* __restrict__ damp_out, long long sH, long long sW) {
  {
    const long long b = blockIdx.x;
    H += b * sH; diagv += b * sW; dead += b * n; damp_out += b * 2;
  }
  __shared__ double red[32];
  double s = 0.0;
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    float v = H[(long long)j * ld + j];
    const bool dd = (v == 0.f);
    if (dd) v = 1.f;
    diagv[j] = v;
    dead[j] = dd ? 1 : 0;
    s += (double)v;
  }
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < (blockDim.x + 31) / 32; ++w) t += red[w];
    damp_out[0] = percdamp * (float)(t / (double)n);
    damp_out[1] = (float)(t / (double)n);
  }
}

// ---- act-order: stable descending argsort by counting ranks ---------------------
__global__ void rank_sort_kernel(const float* __restrict__ key, int n, int* __restrict__ perm, long long sW) {
  key += (long long)blockIdx.y * sW;
  perm += (long long)blockIdx.y * n;
  __shared__ float tile[1024];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const float ki = (i < n) ? key[i] : 0.f;
  int rank = 0;
  for (int base = 0; base < n; base += 1024) {
    for (int t = threadIdx.x; t < 1024; t += blockDim.x) tile[t] = (base + t < n) ? key[base + t] : 0.f;
    __syncthreads();
    const int lim = min(1024, n - base);
    for (int t = 0; t < lim; ++t) {
      const float kj = tile[t];
      const int j = base + t;
      rank += (kj > ki || (kj == ki && j < i)) ? 1 : 0;
    }
    __syncthreads();
  }
  if (i < n) perm[rank] = i;
}

__global__ void iota_kernel(int* __restrict__ perm, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) perm[(long long)blockIdx.y * n + i] = i;
}

__global__ void invert_perm_kernel(const int* __restrict__ perm, int* __restrict__ inv, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  perm += (long long)blockIdx.y * n;
  inv += (long long)blockIdx.y * n;
  if (i < n) inv[perm[i]] = i;
}

// ---- A = J (P Hfix P^T + shift I) J ------------------------------------------------
__global__ void build_reversed_kernel(const float* __restrict__ H, long long ldh, int n,
                                      const int* __restrict__ perm, const float* __restrict__ diagv,
                                      const float* __restrict__ damp, float rel_shift,
                                      float* __restrict__ A, long long lda, long long sH, long long sW) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int i = blockIdx.y;
  if (j >= n) return;
  {
    const long long b = blockIdx.z;
    H += b * sH; perm += b * n; diagv += b * sW; damp += b * 2; A += b * sW;
  }
  const int pi = perm[n - 1 - i], pj = perm[n - 1 - j];
  float v;
  if (i == j) v = diagv[pi] + rel_shift * damp[0];
  else v = H[(long long)pi * ldh + pj];
  A[(long long)i * lda + j] = v;
}

// ---- U = J X J (upper part), zero below the diagonal ------------------------------------
__global__ void reverse_upper_kernel(const float* __restrict__ X, long long ldx, int n,
                                     float* __restrict__ U, long long ldu, long long sW, long long sU) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int i = blockIdx.y;
  if (j >= n) return;
  X += (long long)blockIdx.z * sW;
  U += (long long)blockIdx.z * sU;
  U[(long long)i * ldu + j] = (j >= i) ? X[(long long)(n - 1 - i) * ldx + (n - 1 - j)] : 0.f;
}

// ---- one diagonal block: Cholesky of a (<=128)^2 block on one SM ----------------------------
// A block (nb x nb, lower part read) -> L written back over the lower part, L^T over the upper.
// A non-positive or non-finite pivot records (global index + 1) in *status (first one wins)
// and continues with pivot 1 so that every later kernel still terminates.
//
// 16 x 16 threads, each holding an 8 x 8 sub-block in registers.  The eight columns of a
// micro-panel are finished inside the one warp that holds that block column (the diagonal 8 x 8
// block on one lane, its factor shuffled to the others), published to shared memory, and every
// thread to the right applies them as eight rank-1 updates to its registers: one barrier per
// eight columns.
constexpr int POTRF_SMEM = (NB * (NB + 4) + 2 * 8 * (NB + 4)) * (int)sizeof(float);
__global__ void __launch_bounds__(256) potrf_block_kernel(float* __restrict__ A, long long lda, int k0, int nb,
                                                          int* __restrict__ status, long long sW) {
  A += (long long)blockIdx.x * sW;
  status += blockIdx.x;
  extern __shared__ __align__(16) float sm[];
  // The block travels between global memory and the register blocks through shared memory, so
  // that global accesses are whole rows.  Row r of the block sits at staging row (r % 8) * 16 + r / 8:
  // the sixteen threads of a block column then read sixteen consecutive staging rows at once.
  float (*St)[NB + 4] = reinterpret_cast<float (*)[NB + 4]>(sm);
  // L of the current 8-column micro-panel, column-major [8][128], double buffered
  float (*Lp)[8][NB + 4] = reinterpret_cast<float (*)[8][NB + 4]>(sm + NB * (NB + 4));
  // block column tx of the 16 x 16 grid of 8 x 8 register blocks lives in one half-warp
  const int tid = threadIdx.x, tx = tid >> 4, ty = tid & 15;
  const int r0 = ty * 8, c0 = tx * 8;
  float* Ab = A + (long long)k0 * lda + k0;

  if (nb == NB) {
#pragma unroll
    for (int it = 0; it < NB * NB / 4 / 256; ++it) {
      const int e = it * 256 + tid, r = e / (NB / 4), c4 = e % (NB / 4);
      *reinterpret_cast<float4*>(&St[(r & 7) * 16 + (r >> 3)][4 * c4]) =
          *reinterpret_cast<const float4*>(Ab + (long long)r * lda + 4 * c4);
    }
  } else {
    for (int e = tid; e < NB * NB; e += 256) {
      const int r = e / NB, c = e % NB;
      St[(r & 7) * 16 + (r >> 3)][c] = (r < nb && c < nb) ? Ab[(long long)r * lda + c] : 0.f;
    }
  }
  __syncthreads();
  float a[8][8];
#pragma unroll
  for (int ii = 0; ii < 8; ++ii) {
    const float4 lo = *reinterpret_cast<const float4*>(&St[ii * 16 + ty][c0]);
    const float4 hi = *reinterpret_cast<const float4*>(&St[ii * 16 + ty][c0 + 4]);
    const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
    for (int cc = 0; cc < 8; ++cc) {
      const int r = r0 + ii, c = c0 + cc;
      a[ii][cc] = (r < nb && c <= r) ? v[cc] : ((r == c) ? 1.f : 0.f);
    }
  }

  for (int jb = 0; jb < NB / 8; ++jb) {
    const int buf = jb & 1;
    if ((tid >> 5) == (jb >> 1)) {
      // ---- the micro-panel's eight columns, inside the one warp that holds them ----
      // The lane with the diagonal 8 x 8 block factors it alone in registers; the factor's 28
      // sub-diagonal entries and 8 reciprocal pivots go round by shuffles, and every other lane of
      // the block column solves X L^T = B for its own 8 x 8 block by forward substitution: eight
      // independent rows per lane, the same operations in the same order as a column-by-column
      // elimination across the lanes, without its eight broadcast-scale-update rounds.
      const int pl = ((jb & 1) << 4) + jb;          // lane that owns the diagonal 8 x 8 block
      const bool mine = (tx == jb) && (ty > jb);
      const bool is_pivot = (tx == jb) && (ty == jb);
      float l[8][8], dinv[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        dinv[i] = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) l[i][j] = 0.f;
      }
      if (is_pivot) {
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          float p = a[jj][jj];
          if (!(p > 0.f) || !isfinite(p)) {
            atomicCAS(status, 0, k0 + jb * 8 + jj + 1);
            p = 1.f;
          }
          // one approximate reciprocal square root, refined once, instead of an IEEE square
          // root followed by IEEE divisions
          float inv = rsqrtf(p);
          inv = inv * fmaf(-0.5f * p * inv, inv, 1.5f);
          dinv[jj] = inv;
          a[jj][jj] = p * inv;
#pragma unroll
          for (int ii = jj + 1; ii < 8; ++ii) a[ii][jj] *= inv;
#pragma unroll
          for (int cc = jj + 1; cc < 8; ++cc)
#pragma unroll
            for (int ii = cc; ii < 8; ++ii) a[ii][cc] = fmaf(-a[ii][jj], a[cc][jj], a[ii][cc]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
          for (int j = 0; j < i; ++j) l[i][j] = a[i][j];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        dinv[i] = __shfl_sync(0xffffffffu, dinv[i], pl);
#pragma unroll
        for (int j = 0; j < i; ++j) l[i][j] = __shfl_sync(0xffffffffu, l[i][j], pl);
      }
      if (mine) {
#pragma unroll
        for (int ii = 0; ii < 8; ++ii)
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float acc = a[ii][j];
#pragma unroll
            for (int k = 0; k < j; ++k) acc = fmaf(-a[ii][k], l[j][k], acc);
            a[ii][j] = acc * dinv[j];
          }
      }
      if (mine || is_pivot) {
#pragma unroll
        for (int jj = 0; jj < 8; ++jj)
#pragma unroll
          for (int ii = 0; ii < 8; ++ii) Lp[buf][jj][r0 + ii] = a[ii][jj];
      }
    }
    __syncthreads();
    // ---- rank-8 update of everything to the right, one column of the panel at a time, in
    // the order of eight successive rank-1 updates ----
    if (tx > jb && ty >= tx) {
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const float4 r_lo = *reinterpret_cast<const float4*>(&Lp[buf][jj][r0]);
        const float4 r_hi = *reinterpret_cast<const float4*>(&Lp[buf][jj][r0 + 4]);
        const float4 c_lo = *reinterpret_cast<const float4*>(&Lp[buf][jj][c0]);
        const float4 c_hi = *reinterpret_cast<const float4*>(&Lp[buf][jj][c0 + 4]);
        const float rc[8] = {r_lo.x, r_lo.y, r_lo.z, r_lo.w, r_hi.x, r_hi.y, r_hi.z, r_hi.w};
        const float cv[8] = {c_lo.x, c_lo.y, c_lo.z, c_lo.w, c_hi.x, c_hi.y, c_hi.z, c_hi.w};
        // (the entries above the diagonal of a diagonal block are updated too: nothing reads them)
#pragma unroll
        for (int ii = 0; ii < 8; ++ii)
#pragma unroll
          for (int cc = 0; cc < 8; ++cc) a[ii][cc] = fmaf(-rc[ii], cv[cc], a[ii][cc]);
      }
    }
  }
  // L goes back over the lower part and, transposed, over the upper part (nothing reads the upper
  // part of a diagonal block of A as matrix data; the panel solve loads L^T from there)
  __syncthreads();
#pragma unroll
  for (int ii = 0; ii < 8; ++ii) {
    float v[8];
#pragma unroll
    for (int cc = 0; cc < 8; ++cc) v[cc] = (c0 + cc <= r0 + ii) ? a[ii][cc] : 0.f;
    *reinterpret_cast<float4*>(&St[ii * 16 + ty][c0]) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(&St[ii * 16 + ty][c0 + 4]) = make_float4(v[4], v[5], v[6], v[7]);
  }
  __syncthreads();
  // row r of the result: L[r][c] for c <= r, L[c][r] for c > r
  for (int e = tid; e < NB * NB; e += 256) {
    const int r = e / NB, c = e % NB;
    if (r < nb && c < nb) {
      const int hi = max(r, c), lo = min(r, c);
      Ab[(long long)r * lda + c] = St[(hi & 7) * 16 + (hi >> 3)][lo];
    }
  }
}

// ---- panel solve: P <- P * L^-T for the rows below a factored diagonal block -----------------
// L = the 128 x 128 lower block at (k0, k0), P = the `rest` rows below it (same columns).  Row r of
// the result is the forward substitution y_j = (p_j - sum_{i<j} y_i L[j][i]) / L[j][j]: rows are
// independent.  A CTA takes 128 rows, two threads per row: eight columns at a time, each thread
// sums over every other earlier column, the pair combines with one shuffle per column and both
// finish the 8 x 8 diagonal step.  The block kernel left L^T in the upper triangle of the
// diagonal block, so the tile loads as it is (coalesced, no transposition) and the inner loop
// reads eight consecutive entries L[j0..j0+7][i] as two broadcast vector loads.  Plain fp32 FMAs:
// this is the step that used to need the explicit inverse of the diagonal block on the critical
// path.
constexpr int TR = 128;                    // rows per CTA
constexpr int TPR = 2;                     // threads per row (four were measured slower: the 8 x 8
                                           // diagonal step is repeated by every thread of a row)
constexpr int TRT = TPR * TR;              // threads per CTA
constexpr int LPITCH = NB + 4, YPITCH = NB + 2;   // YPITCH = 2 mod 32: a warp's rows hit distinct banks
constexpr int TRSM_SMEM = (NB * LPITCH + TR * YPITCH + NB) * (int)sizeof(float);
__global__ void __launch_bounds__(TRT) trsm_panel_kernel(float* __restrict__ A, long long lda, int k0, int rest,
                                                         long long sW) {
  A += (long long)blockIdx.y * sW;
  extern __shared__ __align__(16) float sm[];
  float* Lt = sm;                           // Lt[i * LPITCH + j] = L[j][i] for j >= i
  float* Ys = sm + NB * LPITCH;             // this CTA's rows, YPITCH apart
  float* dinv = Ys + TR * YPITCH;
  const int tid = threadIdx.x;
  const float* Lkk = A + (long long)k0 * lda + k0;
  float* P = A + (long long)(k0 + NB) * lda + k0;
  const int row0 = blockIdx.x * TR;
  const int rows = min(TR, rest - row0);
#pragma unroll
  for (int it = 0; it < NB * NB / 4 / TRT; ++it) {
    const int e = it * TRT + tid, i = e / (NB / 4), j4 = e % (NB / 4);
    const float4 v = *reinterpret_cast<const float4*>(Lkk + (long long)i * lda + 4 * j4);
    *reinterpret_cast<float4*>(Lt + i * LPITCH + 4 * j4) = v;
  }
#pragma unroll
  for (int it = 0; it < TR * NB / 4 / TRT; ++it) {
    const int e = it * TRT + tid, r = e / (NB / 4), c4 = e % (NB / 4);
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (r < rows) v = *reinterpret_cast<const float4*>(P + (long long)(row0 + r) * lda + 4 * c4);
    float2* dst = reinterpret_cast<float2*>(Ys + r * YPITCH + 4 * c4);
    dst[0] = make_float2(v.x, v.y);
    dst[1] = make_float2(v.z, v.w);
  }
  __syncthreads();
  if (tid < NB) dinv[tid] = 1.f / Lt[tid * LPITCH + tid];
  __syncthreads();
  {
    const int r = tid / TPR, part = tid % TPR;
    float* y = Ys + r * YPITCH;
    for (int j0 = 0; j0 < NB; j0 += 8) {
      float acc[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] = part ? 0.f : y[j0 + c];
#pragma unroll 4
      for (int i = part; i < j0; i += TPR) {
        const float yi = y[i];
        const float4 l0 = *reinterpret_cast<const float4*>(Lt + i * LPITCH + j0);
        const float4 l1 = *reinterpret_cast<const float4*>(Lt + i * LPITCH + j0 + 4);
        acc[0] = fmaf(-yi, l0.x, acc[0]); acc[1] = fmaf(-yi, l0.y, acc[1]);
        acc[2] = fmaf(-yi, l0.z, acc[2]); acc[3] = fmaf(-yi, l0.w, acc[3]);
        acc[4] = fmaf(-yi, l1.x, acc[4]); acc[5] = fmaf(-yi, l1.y, acc[5]);
        acc[6] = fmaf(-yi, l1.z, acc[6]); acc[7] = fmaf(-yi, l1.w, acc[7]);
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 1);
        if (TPR == 4) acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], 2);
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const float yc = acc[c] * dinv[j0 + c];
        acc[c] = yc;
        if (c < 7) {
          const float4 l0 = *reinterpret_cast<const float4*>(Lt + (j0 + c) * LPITCH + j0);
          const float4 l1 = *reinterpret_cast<const float4*>(Lt + (j0 + c) * LPITCH + j0 + 4);
          const float lr[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
#pragma unroll
          for (int c2 = c + 1; c2 < 8; ++c2) acc[c2] = fmaf(-yc, lr[c2], acc[c2]);
        }
      }
      if (part == 0) {
#pragma unroll
        for (int c = 0; c < 8; ++c) y[j0 + c] = acc[c];
      }
      __syncwarp();          // the partners read these eight values in the next step
    }
  }
  __syncthreads();
#pragma unroll
  for (int it = 0; it < TR * NB / 4 / TRT; ++it) {
    const int e = it * TRT + tid, r = e / (NB / 4), c4 = e % (NB / 4);
    if (r < rows) {
      const float2* src = reinterpret_cast<const float2*>(Ys + r * YPITCH + 4 * c4);
      const float2 a = src[0], b = src[1];
      *reinterpret_cast<float4*>(P + (long long)(row0 + r) * lda + 4 * c4) = make_float4(a.x, a.y, b.x, b.y);
    }
  }
}

// ---- inverses of all diagonal blocks of L, one CTA per block (off the critical path) ----------
// L block (nb x nb, lower) -> L^-1 written to the matching block of X (lower part; upper part
// zero).  The 8 x 8 diagonal blocks are inverted at once, then neighbouring inverted blocks are
// joined level by level (four levels, two small products each).
constexpr int DINV_SMEM = (2 * NB * (NB + 1) + (NB / 2) * (NB / 2)) * (int)sizeof(float);
__global__ void __launch_bounds__(256) diag_inverse_kernel(const float* __restrict__ A, long long lda,
                                                           float* __restrict__ X, long long ldx, int n,
                                                           long long sW) {
  A += (long long)blockIdx.y * sW;
  X += (long long)blockIdx.y * sW;
  extern __shared__ __align__(16) float sm[];
  float (*S)[NB + 1] = reinterpret_cast<float (*)[NB + 1]>(sm);                    // L
  float (*Y)[NB + 1] = reinterpret_cast<float (*)[NB + 1]>(sm + NB * (NB + 1));    // L^-1
  float* T = sm + 2 * NB * (NB + 1);                                               // [64 * 64]
  const int tid = threadIdx.x;
  const int k0 = blockIdx.x * NB, nb = min(NB, n - k0);
  const float* Ab = A + (long long)k0 * lda + k0;
  float* Xb = X + (long long)k0 * ldx + k0;
  for (int e = tid; e < NB * NB; e += 256) {
    const int r = e / NB, c = e % NB;
    S[r][c] = (r < nb && c <= r) ? Ab[(long long)r * lda + c] : ((r == c) ? 1.f : 0.f);
    Y[r][c] = 0.f;
  }
  __syncthreads();
  if (tid < NB) {
    const int i0 = (tid >> 3) * 8, t = tid & 7;     // column t of the inverse of diagonal block i0
    float x[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      float acc = (r == t) ? 1.f : 0.f;
#pragma unroll
      for (int q = 0; q < 8; ++q)
        if (q < r) acc = fmaf(-S[i0 + r][i0 + q], x[q], acc);
      x[r] = (r >= t) ? acc / S[i0 + r][i0 + r] : 0.f;
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) Y[i0 + r][i0 + t] = x[r];
  }
  __syncthreads();
  for (int sz = 8; sz < NB; sz *= 2) {
    // (NB / (2 sz)) problems of sz x sz elements; a thread takes strips of four rows of one column,
    // i.e. four independent sums per pass over k
    const int strips = (NB / 8) * sz;
    const int lg = 31 - __clz(sz);
    for (int e = tid; e < strips; e += 256) {       // T = L21 * X11 (X11 lower triangular)
      const int j = e & (sz - 1), i = ((e >> lg) & (sz / 4 - 1)) * 4, m = e >> (2 * lg - 2);
      const int q0 = 2 * sz * m, mid = q0 + sz;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
      for (int k = j; k < sz; ++k) {
        const float y = Y[q0 + k][q0 + j];
#pragma unroll
        for (int ii = 0; ii < 4; ++ii) acc[ii] = fmaf(S[mid + i + ii][q0 + k], y, acc[ii]);
      }
#pragma unroll
      for (int ii = 0; ii < 4; ++ii) T[(m << (2 * lg)) + ((i + ii) << lg) + j] = acc[ii];
    }
    __syncthreads();
    for (int e = tid; e < strips; e += 256) {       // X21 = -X22 * T (X22 lower triangular)
      const int j = e & (sz - 1), i = ((e >> lg) & (sz / 4 - 1)) * 4, m = e >> (2 * lg - 2);
      const int q0 = 2 * sz * m, mid = q0 + sz;
      const float* tcol = T + (m << (2 * lg)) + j;
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
      for (int k = 0; k < i + 4; ++k) {              // X22[i + ii][k] = 0 for k > i + ii
        const float t = tcol[k << lg];
#pragma unroll
        for (int ii = 0; ii < 4; ++ii) acc[ii] = fmaf(Y[mid + i + ii][mid + k], t, acc[ii]);
      }
#pragma unroll
      for (int ii = 0; ii < 4; ++ii) Y[mid + i + ii][q0 + j] = -acc[ii];
    }
    __syncthreads();
  }
  for (int e = tid; e < nb * nb; e += blockDim.x) {
    const int i = e / nb, j = e % nb;
    Xb[(long long)i * ldx + j] = (j <= i) ? Y[i][j] : 0.f;
  }
}

}  // namespace

// Workspace layout of one problem (floats): A[n*ld] | X[n*ld] | T[n*ld] | diagv[n] | pad;
// ld = round_up(n,4).  A batch keeps the problems' workspaces one after another.
static long long factor_ws_floats(int n) {
  const long long ld = (n + 3) / 4 * 4;
  return (3 * (long long)n * ld + ((n + 3) / 4 * 4) + 4 + 63) / 64 * 64;
}

extern "C" long long oc_hinv_workspace_bytes(int n) { return factor_ws_floats(n) * 4; }

// Factorisation of `batch` matrices of equal size laid out one after another (H [batch, n, ldh],
// U [batch, n, ldu], perm / invperm / dead [batch, n], damp_out [batch, 2], status [batch]).  The
// panel chain is walked once; every launch covers all problems.
static int hinv_factor_impl(int batch, const float* H, long long ldh, int n, float percdamp, float rel_shift,
                            int actorder, int reuse_perm, float* U, long long ldu, int* perm, int* invperm,
                            unsigned char* dead, float* damp_out, int* status, void* workspace,
                            long long workspace_bytes, cudaStream_t stream) {
  OC_REQUIRE(H && U && perm && invperm && dead && damp_out && status && workspace, "hinv_factor: null pointer");
  OC_REQUIRE(n > 0 && ldh >= n && ldu >= n, "hinv_factor: bad dimensions");
  OC_REQUIRE(batch >= 1 && batch <= 65535, "hinv_factor: batch must be in 1..65535");
  const long long sW = factor_ws_floats(n);
  if (workspace_bytes < sW * 4 * batch) {
    oc_set_last_error("hinv_factor: workspace too small");
    return OC_ERR_WORKSPACE;
  }
  const long long ld = (n + 3) / 4 * 4;
  const long long sH = (long long)n * ldh, sU = (long long)n * ldu;
  float* A = (float*)workspace;
  float* X = A + (long long)n * ld;
  float* T = X + (long long)n * ld;
  float* diagv = T + (long long)n * ld;

  OC_CUDA(cudaMemsetAsync(status, 0, sizeof(int) * batch, stream));
  diag_stats_kernel<<<batch, 1024, 0, stream>>>(H, ldh, n, percdamp, diagv, dead, damp_out, sH, sW);
  OC_CHECK_LAUNCH();
  const int tb = 256, gb = oc_div_up(n, tb);
  if (!reuse_perm) {
    if (actorder) rank_sort_kernel<<<dim3(gb, batch), tb, 0, stream>>>(diagv, n, perm, sW);
    else iota_kernel<<<dim3(gb, batch), tb, 0, stream>>>(perm, n);
    OC_CHECK_LAUNCH();
    invert_perm_kernel<<<dim3(gb, batch), tb, 0, stream>>>(perm, invperm, n);
    OC_CHECK_LAUNCH();
  }
  build_reversed_kernel<<<dim3(gb, n, batch), tb, 0, stream>>>(H, ldh, n, perm, diagv, damp_out, rel_shift, A,
                                                                ld, sH, sW);
  OC_CHECK_LAUNCH();
  for (int b = 0; b < batch; ++b)
    OC_CUDA(cudaMemsetAsync(X + b * sW, 0, (size_t)n * ld * sizeof(float), stream));

  // ---- blocked right-looking Cholesky --------------------------------------------------
  OC_OPT_IN_SMEM(potrf_block_kernel, POTRF_SMEM);
  OC_OPT_IN_SMEM(trsm_panel_kernel, TRSM_SMEM);
  OC_OPT_IN_SMEM(diag_inverse_kernel, DINV_SMEM);
  auto batched = [&](OcGemm& g) { g.batch = batch; g.strideA = sW; g.strideB = sW; g.strideC = sW; };
  // Two levels: inside an outer block of OB columns every 128-column panel updates only the
  // rest of that outer block (full height); the matrix behind the outer block is updated once per
  // outer block with K = OB, so it is read and written n/OB times instead of n/128 times.
  // Per panel the serial chain is: factor the diagonal block (one SM), solve the rows below it
  // against that block (all SMs, fp32 FMAs), update the rest of the outer block (tensor cores).
  for (int K0 = 0; K0 < n; K0 += OB) {
    const int kend = min(n, K0 + OB);
    for (int k0 = K0; k0 < kend; k0 += NB) {
      const int nb = min(NB, n - k0);
      potrf_block_kernel<<<batch, 256, POTRF_SMEM, stream>>>(A, ld, k0, nb, status, sW);
      OC_CHECK_LAUNCH();
      const int rest = n - k0 - nb;
      if (rest <= 0) break;
      float* panel = A + (long long)(k0 + nb) * ld + k0;
      OC_REQUIRE(nb == NB, "hinv_factor: a panel with rows below it is a full panel");
      trsm_panel_kernel<<<dim3(oc_div_up(rest, TR), batch), TRT, TRSM_SMEM, stream>>>(A, ld, k0, rest, sW);
      OC_CHECK_LAUNCH();
      const int inner = kend - (k0 + nb);
      if (inner <= 0) continue;
      // columns [k0+nb, kend) of all rows below the panel's diagonal block (lower tiles only)
      OcGemm s{};
      s.A = panel; s.lda = ld; s.B = panel; s.ldb = ld;
      s.C = A + (long long)(k0 + nb) * ld + (k0 + nb); s.ldc = ld;
      s.M = rest; s.N = inner; s.K = nb; s.alpha = -1.f; s.beta = 1.f; s.transA = 0; s.transB = 1;
      s.flags = OC_GEMM_SKIP_UPPER_TILES;
      batched(s);
      int rc = oc_gemm_f32_launch(s, stream);
      if (rc) return rc;
    }
    const int rest2 = n - kend;
    if (rest2 <= 0) break;
    // trailing <- trailing - P * P^T with P = L[kend.., K0..kend)  (lower tiles only)
    float* P = A + (long long)kend * ld + K0;
    OcGemm t{};
    t.A = P; t.lda = ld; t.B = P; t.ldb = ld;
    t.C = A + (long long)kend * ld + kend; t.ldc = ld;
    t.M = rest2; t.N = rest2; t.K = kend - K0; t.alpha = -1.f; t.beta = 1.f; t.transA = 0; t.transB = 1;
    t.flags = OC_GEMM_SKIP_UPPER_TILES;
    batched(t);
    const int rc2 = oc_gemm_f32_launch(t, stream);
    if (rc2) return rc2;
  }
  // inverses of the diagonal blocks, all at once: the seeds of the blocked inverse below
  diag_inverse_kernel<<<dim3(oc_div_up(n, NB), batch), 256, DINV_SMEM, stream>>>(A, ld, X, ld, n, sW);
  OC_CHECK_LAUNCH();

  // ---- recursive blocked inverse of L: X holds the inverted diagonal blocks -----------------
  // One matrix: the uniform problems of a level form one batched product.  Several matrices: the
  // batch dimension is taken by the matrices and the problems of a level are launched one by one.
  for (long long s = NB; s < n; s *= 2) {
    const int nprob = (int)((n + 2 * s - 1) / (2 * s));
    int nfull = 0;
    for (int m = 0; m < nprob; ++m) {
      const long long mid = 2 * s * m + s, end = 2 * s * m + 2 * s;
      if (mid < n && end <= n) nfull = m + 1;
    }
    // (first problem, count as one launch, rows of the lower block)
    struct Launch { int first, count, rows; };
    Launch list[2 + 1];
    int nl = 0;
    if (batch == 1) {
      if (nfull > 0) list[nl++] = {0, nfull, (int)s};
      const long long mid = 2 * s * nfull + s;
      if (nfull < nprob && mid < n) list[nl++] = {nfull, 1, (int)(n - mid)};
    }
    const int total = (batch == 1) ? nl : nprob;
    for (int li = 0; li < total; ++li) {
      int first, count, rows;
      if (batch == 1) { first = list[li].first; count = list[li].count; rows = list[li].rows; }
      else {
        first = li; count = 1;
        const long long mid = 2 * s * first + s;
        if (mid >= n) continue;
        rows = (int)min((long long)s, n - mid);
      }
      const long long r0 = 2 * s * first, mid = r0 + s;
      const long long stride = (batch == 1) ? 2 * s * (ld + 1) : sW;
      const int nb_launch = (batch == 1) ? count : batch;
      OcGemm g1{};  // T21 = L21 * X11   (X11 lower triangular)
      g1.A = A + mid * ld + r0; g1.lda = ld; g1.strideA = stride;
      g1.B = X + r0 * ld + r0; g1.ldb = ld; g1.strideB = stride;
      g1.C = T + mid * ld + r0; g1.ldc = ld; g1.strideC = stride;
      g1.M = rows; g1.N = (int)s; g1.K = (int)s; g1.alpha = 1.f; g1.beta = 0.f;
      g1.flags = OC_GEMM_KLO_FROM_N; g1.batch = nb_launch;
      int rc = oc_gemm_f32_launch(g1, stream);
      if (rc) return rc;
      OcGemm g2{};  // X21 = -X22 * T21  (X22 lower triangular)
      g2.A = X + mid * ld + mid; g2.lda = ld; g2.strideA = stride;
      g2.B = T + mid * ld + r0; g2.ldb = ld; g2.strideB = stride;
      g2.C = X + mid * ld + r0; g2.ldc = ld; g2.strideC = stride;
      g2.M = rows; g2.N = (int)s; g2.K = rows; g2.alpha = -1.f; g2.beta = 0.f;
      g2.flags = OC_GEMM_KHI_FROM_M; g2.batch = nb_launch;
      rc = oc_gemm_f32_launch(g2, stream);
      if (rc) return rc;
    }
  }
  reverse_upper_kernel<<<dim3(gb, n, batch), tb, 0, stream>>>(X, ld, n, U, ldu, sW, sU);
  OC_CHECK_LAUNCH();
  return OC_OK;
}

// See include/onecomp_b200.h for the contracts.
extern "C" int oc_hinv_factor(const float* H, long long ldh, int n, float percdamp, float rel_shift,
                              int actorder, int reuse_perm, float* U, long long ldu, int* perm,
                              int* invperm, unsigned char* dead, float* damp_out, int* status,
                              void* workspace, long long workspace_bytes, void* stream) {
  return hinv_factor_impl(1, H, ldh, n, percdamp, rel_shift, actorder, reuse_perm, U, ldu, perm, invperm, dead,
                          damp_out, status, workspace, workspace_bytes, (cudaStream_t)stream);
}

extern "C" int oc_hinv_factor_batched(int batch, const float* H, int n, float percdamp, int actorder, float* U,
                                      int* perm, int* invperm, unsigned char* dead, float* damp_out,
                                      int* status, void* workspace, long long workspace_bytes, void* stream) {
  return hinv_factor_impl(batch, H, n, n, percdamp, 1.f, actorder, 0, U, n, perm, invperm, dead, damp_out,
                          status, workspace, workspace_bytes, (cudaStream_t)stream);
}

// Inverse-Hessian factor for GPTQ: U upper triangular with U^T U = (H + damp I)^-1.
//
// Replaces the potrf + potri + potrf sequence of the reference
// (onecomp/quantizer/gptq/_gptq.py:594-643, call sites :693-706) with one
// Cholesky factorisation and one triangular inverse:
//
//   A = J (P H P^T + damp I) J      (J reverses the index order, P is the act-order permutation)
//   A = L L^T                       blocked right-looking Cholesky (two levels: 128 / 512), fp32
//   X = L^-1                        recursive blocked triangular inverse, fp32
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

// ---- one diagonal block: Cholesky and inverse of a (<=128)^2 block on one SM -----------------
// A block (nb x nb, lower part read) -> L written back over the lower part;
// L^-1 written to the matching block of X (lower part; upper part zero).
// A non-positive or non-finite pivot records (global index + 1) in *status (first one wins)
// and continues with pivot 1 so that every later kernel still terminates.
//
// Factorisation: 16 x 16 threads, each holding an 8 x 8 sub-block in registers.  The eight
// columns of a micro-panel are finished inside the one warp that holds that block column
// (shuffles only), published to shared memory, and every thread to the right applies them as
// eight rank-1 updates to its registers: one barrier per eight columns.  Inverse: the 8 x 8
// diagonal blocks are inverted at once, then neighbouring inverted blocks are joined level by
// level (four levels, two small products each).
__global__ void __launch_bounds__(256) potrf_diag_kernel(float* __restrict__ A, long long lda,
                                                         float* __restrict__ X, long long ldx,
                                                         int k0, int nb, int* __restrict__ status,
                                                         long long sW) {
  A += (long long)blockIdx.x * sW;
  X += (long long)blockIdx.x * sW;
  status += blockIdx.x;
  extern __shared__ __align__(16) float sm[];
  float (*S)[NB + 1] = reinterpret_cast<float (*)[NB + 1]>(sm);                    // L
  float (*Y)[NB + 1] = reinterpret_cast<float (*)[NB + 1]>(sm + NB * (NB + 1));    // L^-1
  float* T = sm + 2 * NB * (NB + 1);                                               // [64 * 64]
  // block column tx of the 16 x 16 grid of 8 x 8 register blocks lives in one half-warp
  const int tid = threadIdx.x, tx = tid >> 4, ty = tid & 15;
  const int r0 = ty * 8, c0 = tx * 8;
  float* Ab = A + (long long)k0 * lda + k0;
  float* Xb = X + (long long)k0 * ldx + k0;
  // L of the current 8-column micro-panel, column-major [8][128], double buffered; it overlays
  // Y, which is not used before the inverse phase
  float (*Lp)[8][NB + 4] = reinterpret_cast<float (*)[8][NB + 4]>(&Y[0][0]);

  float a[8][8];
#pragma unroll
  for (int ii = 0; ii < 8; ++ii)
#pragma unroll
    for (int cc = 0; cc < 8; ++cc) {
      const int r = r0 + ii, c = c0 + cc;
      a[ii][cc] = (r < nb && c <= r) ? Ab[(long long)r * lda + c] : ((r == c) ? 1.f : 0.f);
    }

  for (int jb = 0; jb < NB / 8; ++jb) {
    const int buf = jb & 1;
    if ((tid >> 5) == (jb >> 1)) {
      // ---- the micro-panel's eight columns inside one warp (shuffles, no barrier) ----
      const int pl = ((jb & 1) << 4) + jb;          // lane that owns the diagonal 8 x 8 block
      const bool mine = (tx == jb) && (ty >= jb);
      const bool is_pivot = (tx == jb) && (ty == jb);
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        float p = __shfl_sync(0xffffffffu, a[jj][jj], pl);
        if (!(p > 0.f) || !isfinite(p)) {
          if (is_pivot) atomicCAS(status, 0, k0 + jb * 8 + jj + 1);
          p = 1.f;
        }
        // the only serial arithmetic of a column step: one approximate reciprocal square root,
        // refined once, instead of an IEEE square root followed by an IEEE division
        float inv = rsqrtf(p);
        inv = inv * fmaf(-0.5f * p * inv, inv, 1.5f);
        const float piv = p * inv;
        if (is_pivot) a[jj][jj] = piv;
        if (mine) {
#pragma unroll
          for (int ii = 0; ii < 8; ++ii)
            if (!is_pivot || ii > jj) a[ii][jj] *= inv;
        }
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          if (cc <= jj) continue;
          const float lc = __shfl_sync(0xffffffffu, a[cc][jj], pl);   // L[8 jb + cc][8 jb + jj]
          if (mine) {
#pragma unroll
            for (int ii = 0; ii < 8; ++ii)
              if (!is_pivot || ii >= cc) a[ii][cc] = fmaf(-a[ii][jj], lc, a[ii][cc]);
          }
        }
      }
      if (mine) {
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
#pragma unroll
        for (int ii = 0; ii < 8; ++ii)
#pragma unroll
          for (int cc = 0; cc < 8; ++cc)
            if (ty > tx || ii >= cc) a[ii][cc] = fmaf(-rc[ii], cv[cc], a[ii][cc]);
      }
    }
  }
  __syncthreads();          // Lp overlays Y: everyone is done with it before S / Y are written
#pragma unroll
  for (int ii = 0; ii < 8; ++ii)
#pragma unroll
    for (int cc = 0; cc < 8; ++cc) {
      const int r = r0 + ii, c = c0 + cc;
      S[r][c] = (c <= r) ? a[ii][cc] : 0.f;
      if (r < nb && c <= r) Ab[(long long)r * lda + c] = a[ii][cc];
    }
  __syncthreads();

  // ---- inverse of L by doubling: the sixteen 8 x 8 diagonal blocks at once, then four levels
  // that join neighbouring inverted blocks of size s:  X21 = -X22 (L21 X11) ----
  for (int e = tid; e < NB * (NB + 1); e += 256) (&Y[0][0])[e] = 0.f;
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
  const int smem = (2 * NB * (NB + 1) + (NB / 2) * (NB / 2)) * (int)sizeof(float);
  OC_OPT_IN_SMEM(potrf_diag_kernel, smem);
  auto batched = [&](OcGemm& g) { g.batch = batch; g.strideA = sW; g.strideB = sW; g.strideC = sW; };
  // Two levels: inside an outer block of OB columns every 128-column panel updates only the
  // rest of that outer block (full height); the matrix behind the outer block is updated once per
  // outer block with K = OB, so it is read and written n/OB times instead of n/128 times.
  for (int K0 = 0; K0 < n; K0 += OB) {
    const int kend = min(n, K0 + OB);
    for (int k0 = K0; k0 < kend; k0 += NB) {
      const int nb = min(NB, n - k0);
      potrf_diag_kernel<<<batch, 256, smem, stream>>>(A, ld, X, ld, k0, nb, status, sW);
      OC_CHECK_LAUNCH();
      const int rest = n - k0 - nb;
      if (rest <= 0) break;
      float* panel = A + (long long)(k0 + nb) * ld + k0;
      OcGemm g{};
      // panel <- panel * (Lkk^-1)^T  (in place: one column tile, every CTA reads its rows first)
      g.A = panel; g.lda = ld; g.B = X + (long long)k0 * ld + k0; g.ldb = ld; g.C = panel; g.ldc = ld;
      g.M = rest; g.N = nb; g.K = nb; g.alpha = 1.f; g.beta = 0.f; g.transA = 0; g.transB = 1;
      g.flags = 0;
      batched(g);
      int rc = oc_gemm_f32_launch(g, stream);
      if (rc) return rc;
      const int inner = kend - (k0 + nb);
      if (inner <= 0) continue;
      // columns [k0+nb, kend) of all rows below the panel's diagonal block (lower tiles only)
      OcGemm s{};
      s.A = panel; s.lda = ld; s.B = panel; s.ldb = ld;
      s.C = A + (long long)(k0 + nb) * ld + (k0 + nb); s.ldc = ld;
      s.M = rest; s.N = inner; s.K = nb; s.alpha = -1.f; s.beta = 1.f; s.transA = 0; s.transB = 1;
      s.flags = OC_GEMM_SKIP_UPPER_TILES;
      batched(s);
      rc = oc_gemm_f32_launch(s, stream);
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

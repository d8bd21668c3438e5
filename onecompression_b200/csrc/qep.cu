// QEP weight correction  W <- fp16( W + perccorr * (W C) (H + damp I)^-1 )
// (reference: Quantizer.adjust_weight, onecomp/quantizer/_quantizer.py:362-432).
//
// The reference factors H + damp I and solves with potrf + potrs.  Here the
// inverse-Hessian factor U of the same damped matrix (U^T U = (P H P^T + damp I)^-1,
// P the act-order permutation or the identity) is already at hand for the GPTQ
// column loop, so the solve becomes two triangular products on the fp32 GEMM
// engine:   dW P^T = ((W C) P^T) U^T U.
#include "common.cuh"

namespace {

__global__ void qep_load_kernel(const void* __restrict__ W, long long ldw_in, int out, int d,
                                const unsigned char* __restrict__ dead, float* __restrict__ Wf,
                                long long ldw, int bf16) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = blockIdx.y;
  if (c >= d) return;
  const float v = oc_ld16(W, (long long)r * ldw_in + c, bf16);
  Wf[(long long)r * ldw + c] = (dead && dead[c]) ? 0.f : v;
}

__global__ void gather_cols_kernel(const float* __restrict__ src, long long lds, int out, int d,
                                   const int* __restrict__ perm, float* __restrict__ dst, long long ldd) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = blockIdx.y;
  if (i >= d) return;
  dst[(long long)r * ldd + i] = src[(long long)r * lds + (perm ? perm[i] : i)];
}

// W[r][perm[i]] = round16( Wf[r][perm[i]] + perccorr * T[r][i] ) in the weight's own 16-bit type
__global__ void qep_store_kernel(const float* __restrict__ Wf, long long ldw, const float* __restrict__ T,
                                 long long ldt, int out, int d, const int* __restrict__ perm,
                                 float perccorr, void* __restrict__ W, long long ldw_out, int bf16) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = blockIdx.y;
  if (i >= d) return;
  const int c = perm ? perm[i] : i;
  const float v = Wf[(long long)r * ldw + c] + perccorr * T[(long long)r * ldt + i];
  oc_st16(W, (long long)r * ldw_out + c, v, bf16);
}

long long round4(long long x) { return (x + 3) / 4 * 4; }

}  // namespace

extern "C" long long oc_qep_workspace_bytes(int out, int d) {
  return 3 * (long long)out * round4(d) * 4 + 256;
}

// See include/onecomp_b200.h for the contract.
extern "C" int oc_qep_adjust(void* W_, long long ldw_io, int out, int d, const float* C, long long ldc,
                             const float* U, long long ldu, const int* perm, const unsigned char* dead,
                             float perccorr, int w_dtype, void* workspace, long long workspace_bytes, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  void* W = W_;
  OC_REQUIRE(w_dtype == OC_DTYPE_F16 || w_dtype == OC_DTYPE_BF16, "qep_adjust: unknown weight dtype");
  const int bf16 = w_dtype == OC_DTYPE_BF16;
  OC_REQUIRE(W && C && U && workspace && out > 0 && d > 0, "qep_adjust: bad arguments");
  OC_REQUIRE(ldw_io >= d && ldc >= d && ldu >= d, "qep_adjust: bad leading dimension");
  OC_REQUIRE(out <= 65535, "qep_adjust: more than 65535 rows in one call");
  if (workspace_bytes < oc_qep_workspace_bytes(out, d)) {
    oc_set_last_error("qep_adjust: workspace too small");
    return OC_ERR_WORKSPACE;
  }
  const long long ld = round4(d);
  float* Wf = (float*)workspace;
  float* A = Wf + (long long)out * ld;
  float* B = A + (long long)out * ld;
  const int tb = 256;
  dim3 grid(oc_div_up(d, tb), out);
  qep_load_kernel<<<grid, tb, 0, stream>>>(W, ldw_io, out, d, dead, Wf, ld, bf16);
  OC_CHECK_LAUNCH();
  OcGemm g{};
  // A = Wf * C
  g.A = Wf; g.lda = ld; g.B = C; g.ldb = ldc; g.C = A; g.ldc = ld;
  g.M = out; g.N = d; g.K = d; g.alpha = 1.f; g.beta = 0.f; g.batch = 1;
  int rc = oc_gemm_f32_launch(g, stream);
  if (rc) return rc;
  // B = A P^T
  gather_cols_kernel<<<grid, tb, 0, stream>>>(A, ld, out, d, perm, B, ld);
  OC_CHECK_LAUNCH();
  // A = B * U^T      (U upper: U[n][k] = 0 for k < n)
  OcGemm t1{};
  t1.A = B; t1.lda = ld; t1.B = U; t1.ldb = ldu; t1.transB = 1; t1.C = A; t1.ldc = ld;
  t1.M = out; t1.N = d; t1.K = d; t1.alpha = 1.f; t1.beta = 0.f; t1.flags = OC_GEMM_KLO_FROM_N; t1.batch = 1;
  rc = oc_gemm_f32_launch(t1, stream);
  if (rc) return rc;
  // B = A * U        (U[k][n] = 0 for k > n)
  OcGemm t2{};
  t2.A = A; t2.lda = ld; t2.B = U; t2.ldb = ldu; t2.C = B; t2.ldc = ld;
  t2.M = out; t2.N = d; t2.K = d; t2.alpha = 1.f; t2.beta = 0.f; t2.flags = OC_GEMM_KHI_FROM_N; t2.batch = 1;
  rc = oc_gemm_f32_launch(t2, stream);
  if (rc) return rc;
  qep_store_kernel<<<grid, tb, 0, stream>>>(Wf, ld, B, ld, out, d, perm, perccorr, W, ldw_io, bf16);
  OC_CHECK_LAUNCH();
  return OC_OK;
}

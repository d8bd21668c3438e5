#include "common.cuh"
#include <string.h>
#include <atomic>

static thread_local char g_last_error[256] = "";

void oc_set_last_error(const char* msg) {
  strncpy(g_last_error, msg ? msg : "", sizeof(g_last_error) - 1);
  g_last_error[sizeof(g_last_error) - 1] = 0;
}

extern "C" const char* oc_last_error(void) { return g_last_error; }

extern "C" int oc_version(void) { return 100; }

static std::atomic<long long> g_launches{0};
void oc_count_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
extern "C" long long oc_launch_count(void) { return g_launches.load(); }
extern "C" long long oc_launch_count_reset(void) { return g_launches.exchange(0); }

// Thin C entry over the fp32 GEMM engine (used by the host layer for the QEP
// products and by the tests).
extern "C" int oc_gemm_f32(const float* A, long long lda, const float* B, long long ldb, float* C,
                           long long ldc, int M, int N, int K, float alpha, float beta, int transA,
                           int transB, int flags, void* stream) {
  OcGemm g{};
  g.A = A; g.lda = lda; g.B = B; g.ldb = ldb; g.C = C; g.ldc = ldc;
  g.M = M; g.N = N; g.K = K; g.alpha = alpha; g.beta = beta;
  g.transA = transA; g.transB = transB; g.flags = flags; g.batch = 1;
  return oc_gemm_f32_launch(g, (cudaStream_t)stream);
}

// Second moments for callers that cannot allocate device memory.
//
// oc_moment_accum needs a caller-provided 16-bit scratch of 2 x n_tok x d elements whenever the
// cross term C is requested (it holds Xf - Xq as two 16-bit terms for the tensor-core kernel).  Some hosts cannot
// hand one over: a plugin that is called from inside somebody else's CUDA-graph capture or
// from a context whose memory pool is owned and sized by another runtime, or a process that
// is forbidden to grow its device footprint after start-up, cannot call cudaMalloc at that
// point.  For them this file keeps the scratch in a fixed, file-scope device array that is
// part of the library image: every GPU on which the library is loaded holds these 64 MiB
// until the process exits, and in exchange the call below allocates nothing at all.
#include "common.cuh"

// capacity of the built-in scratch: activation elements (n_tok x ld) per call; the array holds
// two 16-bit terms for each (64 MiB)
#define OC_STATIC_SCRATCH_HALFS (16ll * 1024 * 1024)

static __device__ __align__(256) __half g_static_delta_scratch[2 * OC_STATIC_SCRATCH_HALFS];

extern "C" int oc_moment_accum(const void* xq, const void* xf, void* delta_scratch, long long n_tok,
                               int d, long long ld, float* H, float* C, long long ldh, float a_old,
                               float a_new, int chunk_tokens, int sm_count, int engine,
                               int x_dtype, int* status, void* stream_);

namespace {
constexpr int MAX_DEVICES = 64;
void* g_scratch_addr[MAX_DEVICES] = {};
}  // namespace

extern "C" long long oc_moment_static_capacity(void) { return OC_STATIC_SCRATCH_HALFS; }

// See include/onecomp_b200.h for the contract.
extern "C" int oc_moment_accum_static(const void* xq, const void* xf, long long n_tok, int d,
                                      long long ld, float* H, float* C, long long ldh, float a_old,
                                      float a_new, int chunk_tokens, int sm_count, int x_dtype,
                                      int* status, void* stream) {
  OC_REQUIRE(n_tok >= 0 && ld >= 0, "moment_accum_static: negative size");
  if (C != nullptr && n_tok * ld > OC_STATIC_SCRATCH_HALFS) {
    oc_set_last_error(
        "moment_accum_static: n_tok * ld exceeds the built-in scratch (16 Mi fp16 elements); "
        "split the tokens over several calls or use oc_moment_accum with your own scratch");
    return OC_ERR_TOO_LARGE;
  }
  int dev = -1;
  OC_CUDA(cudaGetDevice(&dev));
  OC_REQUIRE(dev >= 0 && dev < MAX_DEVICES, "moment_accum_static: device index out of range");
  if (g_scratch_addr[dev] == nullptr) {
    // The array's name is only a host-side handle; the kernels need its address on the
    // current device.  Resolved once per device, on that device's first call.
    void* p = nullptr;
    OC_CUDA(cudaGetSymbolAddress(&p, g_static_delta_scratch));
    g_scratch_addr[dev] = p;
  }
  return oc_moment_accum(xq, xf, g_scratch_addr[dev], n_tok, d, ld, H, C, ldh, a_old, a_new,
                         chunk_tokens, sm_count, 0, x_dtype, status, stream);
}

// Round-to-nearest group quantization of a weight, used for MoE experts that received no
// calibration token (reference: _rtn_fallback_result, onecomp/qep/_quantize_with_qep_arch.py:290-320,
// which calls run_rtn / pseudo_quantize_tensor, onecomp/quantizer/rtn/quantizer.py:64-181).
// Its parameter rule differs from GPTQ's find_params: the symmetric range is mirrored on both
// sides unconditionally and the scale is clamped to at least 1e-5.
#include "common.cuh"

namespace {

// one warp per (row, group)
__global__ void rtn_kernel(const void* __restrict__ W, int bf16, long long ldw, int out, int d, int gs, int G,
                           int maxq, int sym, float* __restrict__ scales, float* __restrict__ zeros,
                           int* __restrict__ codes, void* __restrict__ deq) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= out * G) return;
  const int row = warp / G, g = warp % G;
  const int c0 = g * gs, n = min(gs, d - c0);
  const long long src0 = (long long)row * ldw + c0;
  float mn = 0.f, mx = 0.f;
  for (int t = lane; t < n; t += 32) { const float v = oc_ld16(W, src0 + t, bf16); mn = fminf(mn, v); mx = fmaxf(mx, v); }
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if (sym) { mx = fmaxf(fabsf(mn), mx); mn = -mx; }
  if (mn == 0.f && mx == 0.f) { mn = -1.f; mx = 1.f; }
  const float scale = fmaxf(__fdiv_rn(__fsub_rn(mx, mn), (float)maxq), 1e-5f);
  const float zero = sym ? (float)(maxq + 1) * 0.5f : rintf(__fdiv_rn(-mn, scale));
  if (lane == 0) { scales[(long long)row * G + g] = scale; zeros[(long long)row * G + g] = zero; }
  for (int t = lane; t < n; t += 32) {
    const float v = oc_ld16(W, src0 + t, bf16);
    float q = __fadd_rn(rintf(__fdiv_rn(v, scale)), zero);
    q = fminf(fmaxf(q, 0.f), (float)maxq);
    codes[(long long)row * d + c0 + t] = (int)q;
    oc_st16(deq, (long long)row * d + c0 + t, __fmul_rn(__fsub_rn(q, zero), scale), bf16);
  }
}

}  // namespace

// See include/onecomp_b200.h for the contract.
extern "C" int oc_rtn_quantize(const void* W, long long ldw, int out, int d, int wbits, int groupsize,
                               int sym, float* scales, float* zeros, int* codes, void* deq,
                               int w_dtype, void* stream) {
  OC_REQUIRE(w_dtype == OC_DTYPE_F16 || w_dtype == OC_DTYPE_BF16, "rtn_quantize: unknown weight dtype");
  OC_REQUIRE(W && scales && zeros && codes && deq && out > 0 && d > 0 && ldw >= d, "rtn_quantize: bad arguments");
  OC_REQUIRE(wbits >= 1 && wbits <= 16, "rtn_quantize: wbits must be in 1..16");
  const int gs = (groupsize == -1) ? d : groupsize;
  OC_REQUIRE(gs >= 1 && d % gs == 0, "rtn_quantize: in_features must be divisible by the group size");
  const int G = d / gs;
  const long long warps = (long long)out * G;
  const int tb = 256;
  rtn_kernel<<<(unsigned)((warps * 32 + tb - 1) / tb), tb, 0, (cudaStream_t)stream>>>(
      W, w_dtype == OC_DTYPE_BF16 ? 1 : 0, ldw, out, d, gs, G, (1 << wbits) - 1, sym, scales, zeros, codes, deq);
  OC_CHECK_LAUNCH();
  return OC_OK;
}

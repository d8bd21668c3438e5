// Fused elementwise chains of the block passes of the QEP driver (HBM bound, fp16 in / fp16 out):
//
//  * rotary position embedding  y = x*cos + rotate_half(x)*sin, which the model code runs as a
//    slice, a negation, a concatenation, two products and a sum (six kernels, ~11 passes over the
//    tensor); here one pass: each thread owns an 8-element vector of the lower half of a head and
//    its partner in the upper half.
//  * SwiGLU  y = silu(gate) * up  (two kernels, five tensor passes -> one kernel, three passes).
//
// Rounding points are those of the unfused fp16 torch operators (every product, the sum and the
// SiLU are rounded to fp16 separately, with fp32 arithmetic in between), so the block passes
// produce the same bits with or without the fusion.
#include "common.cuh"

namespace {

__device__ __forceinline__ __half mul_h(__half a, __half b) {
  return __float2half_rn(__half2float(a) * __half2float(b));
}
__device__ __forceinline__ __half add_h(__half a, __half b) {
  return __float2half_rn(__half2float(a) + __half2float(b));
}

struct Vec8 { __half h[8]; };
static_assert(sizeof(Vec8) == 16, "Vec8 must be 16 bytes");

__device__ __forceinline__ Vec8 load8(const __half* p, bool vec) {
  Vec8 v;
  if (vec) {
    *reinterpret_cast<uint4*>(&v) = *reinterpret_cast<const uint4*>(p);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v.h[i] = p[i];
  }
  return v;
}
__device__ __forceinline__ void store8(__half* p, const Vec8& v, bool vec) {
  if (vec) {
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&v);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) p[i] = v.h[i];
  }
}

// x, y: [B, H, S, D] with element strides (sb, sh, ss, 1); cos, sin: [B or 1, S, D] with strides
// (cb, cs, 1).  Work items are ordered (b, s, h, v) so that neighbouring threads touch neighbouring
// addresses in the usual (b, s, h, d) memory order of a transposed projection output.
__global__ void __launch_bounds__(256) rope_f16_kernel(
    const __half* __restrict__ x, __half* __restrict__ y, const __half* __restrict__ cs_,
    const __half* __restrict__ sn_, int H, int S, int D, long long xsb, long long xsh, long long xss,
    long long ysb, long long ysh, long long yss, long long cb, long long cs, long long total, int vec) {
  const int vpr = D / 16;  // vector pairs per head row
  for (long long idx = blockIdx.x * 256ll + threadIdx.x; idx < total; idx += (long long)gridDim.x * 256ll) {
    const int v = (int)(idx % vpr);
    long long r = idx / vpr;
    const int h = (int)(r % H);
    r /= H;
    const int s = (int)(r % S);
    const long long b = r / S;
    const int half_d = D / 2;
    const __half* xr = x + b * xsb + h * xsh + s * xss + 8 * v;
    __half* yr = y + b * ysb + h * ysh + s * yss + 8 * v;
    const __half* cr = cs_ + b * cb + s * cs + 8 * v;
    const __half* sr = sn_ + b * cb + s * cs + 8 * v;
    const Vec8 lo = load8(xr, vec), hi = load8(xr + half_d, vec);
    const Vec8 c_lo = load8(cr, vec), c_hi = load8(cr + half_d, vec);
    const Vec8 s_lo = load8(sr, vec), s_hi = load8(sr + half_d, vec);
    Vec8 o_lo, o_hi;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      o_lo.h[i] = add_h(mul_h(lo.h[i], c_lo.h[i]), mul_h(__hneg(hi.h[i]), s_lo.h[i]));
      o_hi.h[i] = add_h(mul_h(hi.h[i], c_hi.h[i]), mul_h(lo.h[i], s_hi.h[i]));
    }
    store8(yr, o_lo, vec);
    store8(yr + half_d, o_hi, vec);
  }
}

__global__ void __launch_bounds__(256) swiglu_f16_kernel(const __half* __restrict__ gate,
                                                         const __half* __restrict__ up,
                                                         __half* __restrict__ y, long long n_vec,
                                                         long long n, int vec) {
  for (long long idx = blockIdx.x * 256ll + threadIdx.x; idx < n_vec; idx += (long long)gridDim.x * 256ll) {
    const long long base = idx * 8;
    if (vec || base + 8 <= n) {
      const bool v = vec != 0;
      const Vec8 g = load8(gate + base, v), u = load8(up + base, v);
      Vec8 o;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float gf = __half2float(g.h[i]);
        const __half act = __float2half_rn(gf / (1.0f + expf(-gf)));
        o.h[i] = mul_h(act, u.h[i]);
      }
      store8(y + base, o, v);
    } else {
      for (long long i = base; i < n; ++i) {
        const float gf = __half2float(gate[i]);
        const __half act = __float2half_rn(gf / (1.0f + expf(-gf)));
        y[i] = mul_h(act, up[i]);
      }
    }
  }
}

inline unsigned grid_for(long long items, int sm_count) {
  long long blocks = (items + 255) / 256;
  const long long cap = (long long)(sm_count > 0 ? sm_count : 148) * 16;
  if (blocks > cap) blocks = cap;
  return (unsigned)(blocks < 1 ? 1 : blocks);
}

}  // namespace

// See include/onecomp_b200.h for the contracts.
extern "C" int oc_rope_f16(const void* x, void* y, const void* cos_, const void* sin_, long long B, int H,
                           int S, int D, long long xsb, long long xsh, long long xss, long long ysb,
                           long long ysh, long long yss, long long cb, long long cs, int sm_count,
                           void* stream) {
  OC_REQUIRE(x && y && cos_ && sin_ && B >= 0 && H > 0 && S > 0 && D > 0, "rope: bad arguments");
  OC_REQUIRE(D % 16 == 0, "rope: head_dim must be a multiple of 16");
  if (B == 0) return OC_OK;
  const long long total = B * H * (long long)S * (D / 16);
  const uintptr_t ptrs = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) |
                         reinterpret_cast<uintptr_t>(cos_) | reinterpret_cast<uintptr_t>(sin_);
  const long long strides = xsb | xsh | xss | ysb | ysh | yss | cb | cs;
  const int vec = ((ptrs & 15) == 0 && (strides % 8) == 0) ? 1 : 0;
  rope_f16_kernel<<<grid_for(total, sm_count), 256, 0, (cudaStream_t)stream>>>(
      (const __half*)x, (__half*)y, (const __half*)cos_, (const __half*)sin_, H, S, D, xsb, xsh, xss, ysb,
      ysh, yss, cb, cs, total, vec);
  OC_CHECK_LAUNCH();
  return OC_OK;
}

extern "C" int oc_swiglu_f16(const void* gate, const void* up, void* y, long long n, int sm_count,
                             void* stream) {
  OC_REQUIRE(gate && up && y && n >= 0, "swiglu: bad arguments");
  if (n == 0) return OC_OK;
  const uintptr_t ptrs = reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) |
                         reinterpret_cast<uintptr_t>(y);
  const int vec = ((ptrs & 15) == 0 && n % 8 == 0) ? 1 : 0;
  const long long n_vec = (n + 7) / 8;
  swiglu_f16_kernel<<<grid_for(n_vec, sm_count), 256, 0, (cudaStream_t)stream>>>(
      (const __half*)gate, (const __half*)up, (__half*)y, n_vec, n, vec);
  OC_CHECK_LAUNCH();
  return OC_OK;
}

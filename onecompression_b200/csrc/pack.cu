// Stand-alone packing, unpacking and dequantisation of the AutoGPTQ int32 layout
// (reference: onecomp/quantizer/gptq/gptq_layer.py:36-170 and
// GPTQResult.compute_dequantized_weight, onecomp/quantizer/gptq/_gptq.py:84-168).
// The column loop packs its own results; these entry points serve the callers
// that hold integer codes or a packed result already.
#include "common.cuh"

namespace {

__device__ __forceinline__ void pack3(const unsigned (&v)[32], unsigned (&w)[3]) {
  w[0] = w[1] = w[2] = 0u;
#pragma unroll
  for (int k = 0; k < 32; ++k) {
    const int bit = 3 * k, wi = bit >> 5, off = bit & 31;
    w[wi] |= v[k] << off;
    if (off + 3 > 32) w[wi + 1] |= v[k] >> (32 - off);
  }
}

__device__ __forceinline__ unsigned unpack3(const unsigned (&w)[3], int k) {
  const int bit = 3 * k, wi = bit >> 5, off = bit & 31;
  unsigned v = w[wi] >> off;
  if (off + 3 > 32) v |= w[wi + 1] << (32 - off);
  return v & 7u;
}

// Pack along the strided axis: word (p, c) gathers in[(p*f + k) * stride_k + c * stride_c].
// qweight: in = codes [out][d], k walks d (stride 1), c walks out (stride d)  -> [d*bits/32][out]
// qzeros : in = zeros [G][out], handled per group with k walking out          -> [G][out*bits/32]
__global__ void pack_axis_kernel(const int* __restrict__ in, long long stride_k, long long stride_c,
                                 int nk, int nc, int bits, int add, int* __restrict__ out,
                                 long long out_stride_p, long long out_stride_c) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= nc) return;
  const unsigned mask = (1u << bits) - 1u;
  const int* src = in + (long long)c * stride_c;
  if (bits == 3) {
    const long long k0 = (long long)blockIdx.y * 32;
    unsigned v[32], w[3];
#pragma unroll
    for (int k = 0; k < 32; ++k) v[k] = (unsigned)(src[(k0 + k) * stride_k] + add) & mask;
    pack3(v, w);
#pragma unroll
    for (int t = 0; t < 3; ++t) out[(long long)(blockIdx.y * 3 + t) * out_stride_p + (long long)c * out_stride_c] = (int)w[t];
  } else {
    const int f = 32 / bits;
    const long long k0 = (long long)blockIdx.y * f;
    unsigned word = 0u;
    for (int k = 0; k < f; ++k) word |= ((unsigned)(src[(k0 + k) * stride_k] + add) & mask) << (k * bits);
    out[(long long)blockIdx.y * out_stride_p + (long long)c * out_stride_c] = (int)word;
  }
}

__global__ void unpack_axis_kernel(const int* __restrict__ in, long long in_stride_p, long long in_stride_c,
                                   int nk, int nc, int bits, int add, int* __restrict__ out,
                                   long long stride_k, long long stride_c) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= nc) return;
  const unsigned mask = (1u << bits) - 1u;
  int* dst = out + (long long)c * stride_c;
  if (bits == 3) {
    const long long k0 = (long long)blockIdx.y * 32;
    unsigned w[3];
#pragma unroll
    for (int t = 0; t < 3; ++t) w[t] = (unsigned)in[(long long)(blockIdx.y * 3 + t) * in_stride_p + (long long)c * in_stride_c];
#pragma unroll
    for (int k = 0; k < 32; ++k)
      if (k0 + k < nk) dst[(k0 + k) * stride_k] = (int)((unpack3(w, k) + (unsigned)add) & mask);
  } else {
    const int f = 32 / bits;
    const long long k0 = (long long)blockIdx.y * f;
    const unsigned word = (unsigned)in[(long long)blockIdx.y * in_stride_p + (long long)c * in_stride_c];
    for (int k = 0; k < f; ++k)
      if (k0 + k < nk) dst[(k0 + k) * stride_k] = (int)((((word >> (k * bits)) & mask) + (unsigned)add) & mask);
  }
}

// W^[r][c] = fp16( float(scale16[g][r]) * (q - zero) ), g = g_idx[c]; zero = (stored + 1) & mask
__global__ void dequant_packed_kernel(const int* __restrict__ qweight, const int* __restrict__ qzeros,
                                      const __half* __restrict__ scales, const int* __restrict__ g_idx,
                                      int out, int d, int bits, long long ldz,
                                      __half* __restrict__ w, long long ldw) {
  __shared__ float t[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;
  const unsigned mask = (1u << bits) - 1u;
  for (int k = ty; k < 32; k += 8) {
    const int c = c0 + k, r = r0 + tx;
    if (c < d && r < out) {
      unsigned q, z;
      const int g = g_idx ? g_idx[c] : 0;
      if (bits == 3) {
        unsigned wq[3], wz[3];
        for (int s = 0; s < 3; ++s) {
          wq[s] = (unsigned)qweight[(long long)((c / 32) * 3 + s) * out + r];
          wz[s] = (unsigned)qzeros[(long long)g * ldz + (r / 32) * 3 + s];
        }
        q = unpack3(wq, c % 32);
        z = unpack3(wz, r % 32);
      } else {
        const int f = 32 / bits;
        q = ((unsigned)qweight[(long long)(c / f) * out + r] >> ((c % f) * bits)) & mask;
        z = ((unsigned)qzeros[(long long)g * ldz + r / f] >> ((r % f) * bits)) & mask;
      }
      z = (z + 1u) & mask;
      const float s = __half2float(scales[(long long)g * out + r]);
      t[k][tx] = s * ((float)q - (float)z);
    }
  }
  __syncthreads();
  for (int k = ty; k < 32; k += 8) {
    const int r = r0 + k, c = c0 + tx;
    if (c < d && r < out) w[(long long)r * ldw + c] = __float2half_rn(t[tx][k]);
  }
}

int check_bits(int bits) {
  if (bits == 2 || bits == 3 || bits == 4 || bits == 8) return OC_OK;
  oc_set_last_error("pack: wbits must be one of 2, 3, 4, 8");
  return OC_ERR_UNSUPPORTED;
}

}  // namespace

extern "C" int oc_pack_qweight(const int* codes, int out, int d, int bits, int* qweight, void* stream) {
  if (int rc = check_bits(bits)) return rc;
  const int f = (bits == 3) ? 32 : 32 / bits;
  OC_REQUIRE(codes && qweight && out > 0 && d > 0, "pack_qweight: bad arguments");
  OC_REQUIRE(d % f == 0, "pack_qweight: in_features not divisible by the pack factor");
  pack_axis_kernel<<<dim3(oc_div_up(out, 128), d / f), 128, 0, (cudaStream_t)stream>>>(
      codes, 1, d, d, out, bits, 0, qweight, out, 1);
  OC_CHECK_LAUNCH();
  return OC_OK;
}

extern "C" int oc_unpack_qweight(const int* qweight, int out, int d, int bits, int* codes, void* stream) {
  if (int rc = check_bits(bits)) return rc;
  const int f = (bits == 3) ? 32 : 32 / bits;
  OC_REQUIRE(codes && qweight && out > 0 && d > 0, "unpack_qweight: bad arguments");
  unpack_axis_kernel<<<dim3(oc_div_up(out, 128), oc_div_up(d, f)), 128, 0, (cudaStream_t)stream>>>(
      qweight, out, 1, d, out, bits, 0, codes, 1, d);
  OC_CHECK_LAUNCH();
  return OC_OK;
}

// zeros [G][out] raw zero points; stored value is (zero + add) & mask with add = -1 for the
// v1 checkpoint convention (pass add = 0 for values that carry the offset already).
extern "C" int oc_pack_qzeros(const int* zeros, int G, int out, int bits, int add, int* qzeros, void* stream) {
  if (int rc = check_bits(bits)) return rc;
  const int f = (bits == 3) ? 32 : 32 / bits;
  OC_REQUIRE(zeros && qzeros && G > 0 && out > 0, "pack_qzeros: bad arguments");
  OC_REQUIRE(out % f == 0, "pack_qzeros: out_features not divisible by the pack factor");
  const long long ldz = (bits == 3) ? out / 32 * 3 : out / f;
  pack_axis_kernel<<<dim3(oc_div_up(G, 128), out / f), 128, 0, (cudaStream_t)stream>>>(
      zeros, 1, out, out, G, bits, add, qzeros, 1, ldz);
  OC_CHECK_LAUNCH();
  return OC_OK;
}

extern "C" int oc_unpack_qzeros(const int* qzeros, int G, int out, int bits, int add, int* zeros, void* stream) {
  if (int rc = check_bits(bits)) return rc;
  const int f = (bits == 3) ? 32 : 32 / bits;
  OC_REQUIRE(zeros && qzeros && G > 0 && out > 0, "unpack_qzeros: bad arguments");
  const long long ldz = (bits == 3) ? (long long)oc_div_up(out, 32) * 3 : oc_div_up(out, f);
  unpack_axis_kernel<<<dim3(oc_div_up(G, 128), oc_div_up(out, f)), 128, 0, (cudaStream_t)stream>>>(
      qzeros, 1, ldz, out, G, bits, add, zeros, 1, out);
  OC_CHECK_LAUNCH();
  return OC_OK;
}

extern "C" int oc_dequantize_packed(const int* qweight, const int* qzeros, const void* scales16,
                                    const int* g_idx, int out, int d, int bits, void* w16,
                                    long long ldw, void* stream) {
  if (int rc = check_bits(bits)) return rc;
  const int f = (bits == 3) ? 32 : 32 / bits;
  OC_REQUIRE(qweight && qzeros && scales16 && w16 && out > 0 && d > 0 && ldw >= d, "dequantize_packed: bad arguments");
  OC_REQUIRE(d % f == 0 && out % f == 0, "dequantize_packed: shape not divisible by the pack factor");
  const long long ldz = (bits == 3) ? out / 32 * 3 : out / f;
  dequant_packed_kernel<<<dim3(oc_div_up(d, 32), oc_div_up(out, 32)), dim3(32, 8), 0, (cudaStream_t)stream>>>(
      qweight, qzeros, (const __half*)scales16, g_idx, out, d, bits, ldz, (__half*)w16, ldw);
  OC_CHECK_LAUNCH();
  return OC_OK;
}

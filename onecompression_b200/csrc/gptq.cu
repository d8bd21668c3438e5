// GPTQ column loop for one Linear weight, given the inverse-Hessian factor U.
//
// Follows run_gptq of the reference (onecomp/quantizer/gptq/_gptq.py:646-794)
// operation for operation in fp32: true divides, round-half-to-even, the
// rank-1 update as a rounded product followed by a rounded subtraction (this
// file is compiled with -fmad=false and uses the _rn intrinsics besides).
//
// Rows of W are independent given U, so one thread owns one row for a whole
// block of up to 128 columns: the row's block lives in shared memory, 16
// columns at a time in registers; the in-block error propagation needs no
// inter-thread communication at all.  The lazy-batch trailing update
// W[:, i2:] -= Err * U[i1:i2, i2:] is a launch of the fp32 GEMM engine with
// the error block stored transposed (coalesced stores here, coalesced loads
// there).  Codes are kept transposed ([column][row], 16 bit) until a final
// pass packs them in original column order.
#include "common.cuh"

namespace {

constexpr int BLK = 128;      // maximum GPTQ block size handled by the column kernel
constexpr int SUB = 16;       // columns held in registers at a time
constexpr int WS = BLK + 4;   // shared tile row stride in floats (odd multiple of 16 bytes)
constexpr int SUPER = 4;      // blocks per far trailing update (see oc_gptq_quantize)

struct ColArgs {
  const float* Wf; long long ldw;
  int out, d, i1, count;
  const float* U; long long ldu;
  float* ErrT; long long lde;
  unsigned short* codesT;
  float* scales; float* zeros;  // [G][out] fp32 (G = 1 for per-channel)
  int gs, maxq, sym;
  int mse_steps; float mse_grid, mse_norm;   // mse_steps = 0: plain min/max fit
  // batched problems (blockIdx.y): element strides between consecutive problems, 0 for one problem
  long long sW, sU, sE, sC, sS;
  int batch;
};

// scale / zero over the values v[0..n), reference: GPTQExcecutor.find_params
// (onecomp/quantizer/gptq/_gptq.py:886-972, perchannel=True, mse=False)
__device__ __forceinline__ void params_from_range(float& mn, float& mx, int maxq, int sym,
                                                  float& scale, float& zero) {
  // mn <= 0 <= mx on entry; on exit they hold the range the parameters were derived from
  if (sym) {
    mx = fmaxf(fabsf(mn), mx);
    if (mn < 0.f) mn = -mx;
  }
  if (mn == 0.f && mx == 0.f) { mn = -1.f; mx = 1.f; }
  scale = __fdiv_rn(__fsub_rn(mx, mn), (float)maxq);
  zero = sym ? (float)(maxq + 1) * 0.5f : rintf(__fdiv_rn(-mn, scale));
}

// |scale*(q - zero) - v|^norm for one value under candidate parameters (the error term of the
// reference's shrink search, :928-950)
__device__ __forceinline__ float mse_term(float v, float scale, float zero, float maxqf, float norm) {
  float q = __fadd_rn(rintf(__fdiv_rn(v, scale)), zero);
  q = fminf(fmaxf(q, 0.f), maxqf);
  const float dq = __fmul_rn(scale, __fsub_rn(q, zero));
  return powf(fabsf(__fsub_rn(dq, v)), norm);
}

// candidate i of the shrink search: range scaled by p = 1 - i/grid
__device__ __forceinline__ void mse_candidate(int i, float grid, float mn, float mx, int maxq, int sym,
                                              float zero_sym, float& scale1, float& zero1) {
  const float p = (float)(1.0 - (double)i / (double)grid);
  const float mn1 = __fmul_rn(p, mn), mx1 = __fmul_rn(p, mx);
  scale1 = __fdiv_rn(__fsub_rn(mx1, mn1), (float)maxq);
  zero1 = sym ? zero_sym : rintf(__fdiv_rn(-mn1, scale1));
}

// Group parameters are fitted on the block-entry values of columns col .. col+gs-1 (the
// reference, :737-745, reads the matrix, not the block copy).  Kept out of line: it runs once
// per group and would otherwise be replicated in every unrolled column step.
__device__ __noinline__ void fit_group(const float* __restrict__ src, int n, int maxq, int sym,
                                       int mse_steps, float grid, float norm, float* scale, float* zero) {
  float mn = 0.f, mx = 0.f;
  for (int t = 0; t < n; ++t) { const float v = src[t]; mn = fminf(mn, v); mx = fmaxf(mx, v); }
  float s, z;
  params_from_range(mn, mx, maxq, sym, s, z);
  if (mse_steps > 0) {
    float best = __int_as_float(0x7f800000), bs = s, bz = z;
    for (int i = 0; i < mse_steps; ++i) {
      float s1, z1;
      mse_candidate(i, grid, mn, mx, maxq, sym, z, s1, z1);
      float err = 0.f;
      for (int t = 0; t < n; ++t) err += mse_term(src[t], s1, z1, (float)maxq, norm);
      if (err < best) { best = err; bs = s1; bz = z1; }
    }
    s = bs; z = bz;
  }
  *scale = s; *zero = z;
}

// WARPS*32 rows per CTA; the CTA always has LOADERS threads.  The threads beyond the rows load the
// tiles, and when a CTA owns few rows (WARPS <= 2) they also take over the deferred updates: after
// each window of SUB columns the row owners publish the window's errors, the helper threads first
// bring the next window's columns up to date (the owners wait for that), then the rest of the block
// while the owners already work on the next window.  Every element still receives its updates in
// ascending order of the source column with the same two roundings each, so results do not depend
// on who applies them.
constexpr int LOADERS = 256;

__device__ __forceinline__ void apply_window(float4& t, const float* __restrict__ es, const float* __restrict__ us) {
  // es: this row's SUB errors (stride = rows of the CTA is folded in by the caller); us: U rows of the window
#pragma unroll
  for (int i = 0; i < SUB; ++i) {
    const float e = es[i];
    const float4 u = *reinterpret_cast<const float4*>(us + i * BLK);
    t.x = __fsub_rn(t.x, __fmul_rn(e, u.x)); t.y = __fsub_rn(t.y, __fmul_rn(e, u.y));
    t.z = __fsub_rn(t.z, __fmul_rn(e, u.z)); t.w = __fsub_rn(t.w, __fmul_rn(e, u.w));
  }
}

// ALIGNED: every group starts on a multiple of SUB columns (per-channel, or a group size that is
// a multiple of SUB), so the fit can only fall on the first column of a register window and the
// other fifteen unrolled column steps carry no test and no call site for it.
template <int WARPS, bool ALIGNED>
__global__ void __launch_bounds__(LOADERS) gptq_block_kernel(ColArgs a) {
  extern __shared__ __align__(16) float sm[];
  constexpr int NROWS = WARPS * 32;
  constexpr bool HELPERS = WARPS <= 2;
  float* Us = sm;               // [BLK][BLK], upper triangle of the diagonal block of U
  float* Ws = sm + BLK * BLK;   // [NROWS][WS], block-entry values of the rows' columns
  float* Es = Ws + NROWS * WS;  // [2][SUB][NROWS] errors of the last two windows (helpers only)
  const int tid = threadIdx.x;
  const int row0 = blockIdx.x * NROWS;
  const int count = a.count, i1 = a.i1;
  {
    const long long b = blockIdx.y;      // problem of a batch
    a.Wf += b * a.sW; a.U += b * a.sU; a.ErrT += b * a.sE; a.codesT += b * a.sC;
    a.scales += b * a.sS; a.zeros += b * a.sS;
  }

  // whole block, 16-byte aligned rows: vector loads (the part of U below the diagonal is never used)
  const bool vec = count == BLK && (i1 & 3) == 0 && (a.ldu & 3) == 0 && (a.ldw & 3) == 0 &&
                   ((reinterpret_cast<uintptr_t>(a.U) | reinterpret_cast<uintptr_t>(a.Wf)) & 15) == 0;
  if (vec) {
#pragma unroll
    for (int it = 0; it < BLK * BLK / 4 / LOADERS; ++it) {
      const int e = it * LOADERS + tid, i = e / (BLK / 4), j4 = e % (BLK / 4);
      *reinterpret_cast<float4*>(Us + i * BLK + 4 * j4) =
          *reinterpret_cast<const float4*>(a.U + (long long)(i1 + i) * a.ldu + i1 + 4 * j4);
    }
#pragma unroll
    for (int it = 0; it < NROWS * BLK / 4 / LOADERS; ++it) {
      const int e = it * LOADERS + tid, r = e / (BLK / 4), c4 = e % (BLK / 4);
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row0 + r < a.out) v = *reinterpret_cast<const float4*>(a.Wf + (long long)(row0 + r) * a.ldw + i1 + 4 * c4);
      *reinterpret_cast<float4*>(Ws + r * WS + 4 * c4) = v;
    }
  } else {
    for (int e = tid; e < BLK * BLK; e += LOADERS) {
      const int i = e / BLK, j = e % BLK;
      Us[e] = (i < count && j < count && j >= i) ? a.U[(long long)(i1 + i) * a.ldu + i1 + j] : 0.f;
    }
    for (int e = tid; e < NROWS * BLK; e += LOADERS) {
      const int r = e / BLK, c = e % BLK;
      Ws[r * WS + c] = (row0 + r < a.out && c < count) ? a.Wf[(long long)(row0 + r) * a.ldw + i1 + c] : 0.f;
    }
  }
  __syncthreads();

  const int row = row0 + tid;
  const bool owner = tid < NROWS && row < a.out;
  // helpers take the deferred updates when the block's columns come in whole groups of four
  const bool helped = HELPERS && (count & 3) == 0;
  if (!helped && !owner) return;
  float* wrow = Ws + (owner ? tid : 0) * WS;
  const float* grow = a.Wf + (long long)(owner ? row : 0) * a.ldw;  // block-entry state of the whole row
  const float maxqf = (float)a.maxq;
  const int gs = a.gs;
  unsigned short* code_out = a.codesT + (long long)i1 * a.out + row;   // + column * out
  float* err_out = a.ErrT + row;                                        // + column * lde
  float scale = 1.f, zero = 0.f;
  if (owner) {
    if (gs == -1) { scale = a.scales[row]; zero = a.zeros[row]; }
    else if (i1 % gs != 0) {
      // the block starts inside a group opened by an earlier block: continue with its parameters
      scale = a.scales[(long long)(i1 / gs) * a.out + row];
      zero = a.zeros[(long long)(i1 / gs) * a.out + row];
    }
  }
  // helper thread -> (row, every nsel-th group of four columns)
  constexpr int NSEL = HELPERS ? (LOADERS - NROWS) / NROWS : 1;
  const int hrow = (tid - NROWS) % NROWS, gsel = (tid - NROWS) / NROWS;
  const bool helper = helped && tid >= NROWS && gsel < NSEL;

  for (int cb = 0; cb < count; cb += SUB) {
    float* es_buf = Es + ((cb / SUB) & 1) * SUB * NROWS;
    if (owner) {
      float w[SUB], er[SUB];
#pragma unroll
      for (int v = 0; v < SUB / 4; ++v) {
        const float4 t = *reinterpret_cast<const float4*>(wrow + cb + 4 * v);
        w[4 * v] = t.x; w[4 * v + 1] = t.y; w[4 * v + 2] = t.z; w[4 * v + 3] = t.w;
      }
#pragma unroll
      for (int i = 0; i < SUB; ++i) {
        const int ci = cb + i;
        er[i] = 0.f;
        if (ci < count) {
          const int col = i1 + ci;
          if ((!ALIGNED || i == 0) && gs != -1 && col % gs == 0) {
            const int n = min(gs, a.d - col);
            // the shared tile is still pristine only at the very first column of the block
            fit_group((ci == 0 && n <= count) ? wrow : grow + col, n, a.maxq, a.sym, a.mse_steps,
                      a.mse_grid, a.mse_norm, &scale, &zero);
            const int g = col / gs;
            a.scales[(long long)g * a.out + row] = scale;
            a.zeros[(long long)g * a.out + row] = zero;
          }
          const float x = w[i];
          float q = __fadd_rn(rintf(__fdiv_rn(x, scale)), zero);
          q = fminf(fmaxf(q, 0.f), maxqf);
          const float dq = __fmul_rn(scale, __fsub_rn(q, zero));
          const float e = __fdiv_rn(__fsub_rn(x, dq), Us[ci * BLK + ci]);
          er[i] = e;
          code_out[(long long)ci * a.out] = (unsigned short)q;
          err_out[(long long)ci * a.lde] = e;
          const float4* up = reinterpret_cast<const float4*>(Us + ci * BLK + cb);
#pragma unroll
          for (int j4 = (i + 1) / 4; j4 < SUB / 4; ++j4) {
            const float4 u = up[j4];
            if (4 * j4 + 0 > i) w[4 * j4 + 0] = __fsub_rn(w[4 * j4 + 0], __fmul_rn(e, u.x));
            if (4 * j4 + 1 > i) w[4 * j4 + 1] = __fsub_rn(w[4 * j4 + 1], __fmul_rn(e, u.y));
            if (4 * j4 + 2 > i) w[4 * j4 + 2] = __fsub_rn(w[4 * j4 + 2], __fmul_rn(e, u.z));
            if (4 * j4 + 3 > i) w[4 * j4 + 3] = __fsub_rn(w[4 * j4 + 3], __fmul_rn(e, u.w));
          }
        }
      }
      if (helped) {
#pragma unroll
        for (int i = 0; i < SUB; ++i) es_buf[i * NROWS + tid] = er[i];
      } else {
        // Later columns of the block receive this sub-block's updates now, in the
        // same order (ascending source column) and with the same two roundings each.
        for (int jc = cb + SUB; jc < count; jc += 8) {
          float4 t0 = *reinterpret_cast<const float4*>(wrow + jc);
          float4 t1 = *reinterpret_cast<const float4*>(wrow + jc + 4);
#pragma unroll
          for (int i = 0; i < SUB; ++i) {
            const float e = er[i];
            const float4 u0 = *reinterpret_cast<const float4*>(Us + (cb + i) * BLK + jc);
            const float4 u1 = *reinterpret_cast<const float4*>(Us + (cb + i) * BLK + jc + 4);
            t0.x = __fsub_rn(t0.x, __fmul_rn(e, u0.x)); t0.y = __fsub_rn(t0.y, __fmul_rn(e, u0.y));
            t0.z = __fsub_rn(t0.z, __fmul_rn(e, u0.z)); t0.w = __fsub_rn(t0.w, __fmul_rn(e, u0.w));
            t1.x = __fsub_rn(t1.x, __fmul_rn(e, u1.x)); t1.y = __fsub_rn(t1.y, __fmul_rn(e, u1.y));
            t1.z = __fsub_rn(t1.z, __fmul_rn(e, u1.z)); t1.w = __fsub_rn(t1.w, __fmul_rn(e, u1.w));
          }
          *reinterpret_cast<float4*>(wrow + jc) = t0;
          *reinterpret_cast<float4*>(wrow + jc + 4) = t1;
        }
      }
    }
    if (helped) {
      if (cb + SUB >= count) break;         // the last window has nothing to its right
      __syncthreads();                      // the window's errors are published
      const int g_first = (cb + SUB) / 4, g_urgent = min(count, cb + 2 * SUB) / 4, g_end = count / 4;
      if (helper) {
        // the next window's columns first: the row owners wait for these
        for (int g = g_first; g < g_urgent; ++g) {
          if (g % NSEL != gsel) continue;
          float4 t = *reinterpret_cast<const float4*>(Ws + hrow * WS + 4 * g);
          float er[SUB];
#pragma unroll
          for (int i = 0; i < SUB; ++i) er[i] = es_buf[i * NROWS + hrow];
          apply_window(t, er, Us + cb * BLK + 4 * g);
          *reinterpret_cast<float4*>(Ws + hrow * WS + 4 * g) = t;
        }
      }
      __syncthreads();                      // the next window may start
      if (helper) {
        float er[SUB];
#pragma unroll
        for (int i = 0; i < SUB; ++i) er[i] = es_buf[i * NROWS + hrow];
        for (int g = g_urgent; g < g_end; ++g) {
          if (g % NSEL != gsel) continue;
          float4 t = *reinterpret_cast<const float4*>(Ws + hrow * WS + 4 * g);
          apply_window(t, er, Us + cb * BLK + 4 * g);
          *reinterpret_cast<float4*>(Ws + hrow * WS + 4 * g) = t;
        }
      }
    }
  }
}

// ---- preparation: fp16 -> fp32, act-order gather, dead columns, per-channel parameters ----
// Wf[r][j] = dead[perm[j]] ? 0 : float(W[r][perm[j]]).  Per-channel scale / zero are fitted on
// the whole original row before dead columns are zeroed (reference :690-695).
__global__ void gptq_prepare_kernel(const void* __restrict__ W, int bf16, long long ldw_in, int out, int d,
                                    const int* __restrict__ perm, const unsigned char* __restrict__ dead,
                                    float* __restrict__ Wf, long long ldw, int per_channel, int maxq,
                                    int sym, int mse_steps, float mse_grid, float mse_norm,
                                    float* __restrict__ scales, float* __restrict__ zeros,
                                    long long s_win, long long s_wf, long long s_par) {
  const int row = blockIdx.x;
  {
    const long long b = blockIdx.y;      // problem of a batch
    W = static_cast<const char*>(W) + b * s_win * 2;
    Wf += b * s_wf; scales += b * s_par; zeros += b * s_par;
    if (perm) perm += b * d;
    if (dead) dead += b * d;
  }
  const long long src0 = (long long)row * ldw_in;
  float* dst = Wf + (long long)row * ldw;
  float mn = 0.f, mx = 0.f;
  for (int j = threadIdx.x; j < d; j += blockDim.x) {
    const int pj = perm ? perm[j] : j;
    const float v = oc_ld16(W, src0 + pj, bf16);
    mn = fminf(mn, v); mx = fmaxf(mx, v);
    dst[j] = (dead && dead[pj]) ? 0.f : v;
  }
  if (!per_channel) return;
  __shared__ float smn[32], smx[32], bc[4];
  const int nwarp = (blockDim.x + 31) / 32;
  for (int o = 16; o > 0; o >>= 1) {
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if ((threadIdx.x & 31) == 0) { smn[threadIdx.x >> 5] = mn; smx[threadIdx.x >> 5] = mx; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < nwarp; ++w) { mn = fminf(mn, smn[w]); mx = fmaxf(mx, smx[w]); }
    float s, z;
    params_from_range(mn, mx, maxq, sym, s, z);
    bc[0] = mn; bc[1] = mx; bc[2] = s; bc[3] = z;
  }
  __syncthreads();
  float best_s = bc[2], best_z = bc[3];
  if (mse_steps > 0) {
    // shrink search over the whole (original) row, one block-wide error sum per candidate
    const float rmn = bc[0], rmx = bc[1], zsym = bc[3];
    float best = __int_as_float(0x7f800000);
    for (int i = 0; i < mse_steps; ++i) {
      float s1, z1;
      mse_candidate(i, mse_grid, rmn, rmx, maxq, sym, zsym, s1, z1);
      float err = 0.f;
      for (int j = threadIdx.x; j < d; j += blockDim.x)
        err += mse_term(oc_ld16(W, src0 + j, bf16), s1, z1, (float)maxq, mse_norm);
      for (int o = 16; o > 0; o >>= 1) err += __shfl_xor_sync(0xffffffffu, err, o);
      __syncthreads();
      if ((threadIdx.x & 31) == 0) smn[threadIdx.x >> 5] = err;
      __syncthreads();
      float tot = 0.f;
      for (int w = 0; w < nwarp; ++w) tot += smn[w];
      if (tot < best) { best = tot; best_s = s1; best_z = z1; }
    }
  }
  if (threadIdx.x == 0) {
    scales[row] = best_s;
    zeros[row] = best_z;
  }
}

// ---- final pass: pack, cast, dequantize ---------------------------------------------------
// Packed layout: pack_int_weights / pack_zeros of the reference
// (onecomp/quantizer/gptq/gptq_layer.py:36-83, 129-139, 160-170).
__device__ __forceinline__ void pack3(const unsigned (&v)[32], unsigned (&w)[3]) {
  w[0] = w[1] = w[2] = 0u;
#pragma unroll
  for (int k = 0; k < 32; ++k) {
    const int bit = 3 * k, wi = bit >> 5, off = bit & 31;
    w[wi] |= v[k] << off;
    if (off + 3 > 32) w[wi + 1] |= v[k] >> (32 - off);
  }
}

// qweight[pr][r]: codes of original columns pr*f .. pr*f+f-1 (3 bit: 32 columns -> 3 words)
__global__ void pack_qweight_kernel(const unsigned short* __restrict__ codesT, int out, int d,
                                    const int* __restrict__ invperm, int bits,
                                    int* __restrict__ qweight, long long ldq) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= out) return;
  const unsigned mask = (1u << bits) - 1u;
  if (bits == 3) {
    const int c0 = blockIdx.y * 32;
    unsigned v[32], w[3];
#pragma unroll
    for (int k = 0; k < 32; ++k) {
      const int c = c0 + k;
      const int j = invperm ? invperm[c] : c;
      v[k] = codesT[(long long)j * out + r] & mask;
    }
    pack3(v, w);
#pragma unroll
    for (int t = 0; t < 3; ++t) qweight[(long long)(blockIdx.y * 3 + t) * ldq + r] = (int)w[t];
  } else {
    const int f = 32 / bits;
    const int c0 = blockIdx.y * f;
    unsigned word = 0u;
    for (int k = 0; k < f; ++k) {
      const int c = c0 + k;
      const int j = invperm ? invperm[c] : c;
      word |= ((unsigned)codesT[(long long)j * out + r] & mask) << (k * bits);
    }
    qweight[(long long)blockIdx.y * ldq + r] = (int)word;
  }
}

// qzeros[g][w]: (zero - 1) & mask of rows w*f .. w*f+f-1 (3 bit: 32 rows -> 3 words)
__global__ void pack_qzeros_kernel(const float* __restrict__ zeros, int out, int G, int bits,
                                   int* __restrict__ qzeros, long long ldz) {
  const int g = blockIdx.y;
  const unsigned mask = (1u << bits) - 1u;
  const float* zr = zeros + (long long)g * out;
  if (bits == 3) {
    const int blk = blockIdx.x * blockDim.x + threadIdx.x;
    if (blk * 32 >= out) return;
    unsigned v[32], w[3];
#pragma unroll
    for (int k = 0; k < 32; ++k) v[k] = (unsigned)((int)zr[blk * 32 + k] - 1) & mask;
    pack3(v, w);
#pragma unroll
    for (int t = 0; t < 3; ++t) qzeros[(long long)g * ldz + blk * 3 + t] = (int)w[t];
  } else {
    const int f = 32 / bits;
    const int wi = blockIdx.x * blockDim.x + threadIdx.x;
    if (wi * f >= out) return;
    unsigned word = 0u;
    for (int k = 0; k < f; ++k) word |= ((unsigned)((int)zr[wi * f + k] - 1) & mask) << (k * bits);
    qzeros[(long long)g * ldz + wi] = (int)word;
  }
}

__global__ void cast_params_kernel(const float* __restrict__ scales, const float* __restrict__ zeros,
                                   int out, int G, __half* __restrict__ scales16, long long lds,
                                   float* __restrict__ scales32, int* __restrict__ zeros_i32) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  const int g = blockIdx.y;
  if (r >= out) return;
  const float s = scales[(long long)g * out + r];
  if (scales16) scales16[(long long)g * lds + r] = __float2half_rn(s);
  if (scales32) scales32[(long long)g * lds + r] = s;
  if (zeros_i32) zeros_i32[(long long)g * lds + r] = (int)zeros[(long long)g * out + r];
}

// Original-order outputs through a 32x32 transpose: integer codes [out][d] and the fp16
// dequantised weight  fp16( float(fp16(scale)) * (q - zero) )  (reference :153-168).
__global__ void unpermute_outputs_kernel(const unsigned short* __restrict__ codesT, int out, int d,
                                         const int* __restrict__ invperm, int gs,
                                         const float* __restrict__ scales, const float* __restrict__ zeros,
                                         int* __restrict__ codes, long long ldc,
                                         void* __restrict__ what, long long ldwh, int bf16) {
  __shared__ unsigned short tq[32][33];
  __shared__ float tv[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;  // 32 x 8
  for (int k = ty; k < 32; k += 8) {
    const int c = c0 + k, r = r0 + tx;
    if (c < d && r < out) {
      const int j = invperm ? invperm[c] : c;
      const int g = (gs == -1) ? 0 : j / gs;
      const unsigned short q = codesT[(long long)j * out + r];
      tq[k][tx] = q;
      const float s = __half2float(__float2half_rn(scales[(long long)g * out + r]));
      tv[k][tx] = __fmul_rn(s, __fsub_rn((float)q, zeros[(long long)g * out + r]));
    }
  }
  __syncthreads();
  for (int k = ty; k < 32; k += 8) {
    const int r = r0 + k, c = c0 + tx;
    if (c < d && r < out) {
      if (codes) codes[(long long)r * ldc + c] = (int)tq[tx][k];
      if (what) {
        // the reference rounds to fp16 first and casts to the module's dtype afterwards
        const __half h = __float2half_rn(tv[tx][k]);
        if (bf16) static_cast<__nv_bfloat16*>(what)[(long long)r * ldwh + c] = __float2bfloat16_rn(__half2float(h));
        else static_cast<__half*>(what)[(long long)r * ldwh + c] = h;
      }
    }
  }
}

template <int WARPS, bool ALIGNED>
int launch_block_t(const ColArgs& a, cudaStream_t stream) {
  // tiles, plus the error windows the helper threads read (only CTAs with few rows have helpers)
  const int smem = (BLK * BLK + WARPS * 32 * WS + (WARPS <= 2 ? 2 * SUB * WARPS * 32 : 0)) * (int)sizeof(float);
  OC_OPT_IN_SMEM((gptq_block_kernel<WARPS, ALIGNED>), smem);
  gptq_block_kernel<WARPS, ALIGNED><<<dim3(oc_div_up(a.out, WARPS * 32), a.batch), LOADERS, smem, stream>>>(a);
  OC_CHECK_LAUNCH();
  return OC_OK;
}

template <int WARPS>
int launch_block(const ColArgs& a, cudaStream_t stream) {
  // group starts fall on window starts when the block starts on a multiple of SUB columns and
  // the group size is a multiple of SUB
  const bool aligned = a.gs == -1 || (a.gs % SUB == 0 && a.i1 % SUB == 0);
  return aligned ? launch_block_t<WARPS, true>(a, stream) : launch_block_t<WARPS, false>(a, stream);
}

long long round4(long long x) { return (x + 3) / 4 * 4; }

}  // namespace

extern "C" long long oc_gptq_workspace_bytes(int out, int d, int groupsize) {
  const long long G = (groupsize == -1) ? 1 : (d + groupsize - 1) / groupsize;
  long long b = 0;
  b += (long long)out * round4(d) * 4;       // Wf
  b += (long long)SUPER * BLK * round4(out) * 4;  // ErrT
  b += round4((long long)d * out * 2);       // codesT
  b += 2 * G * (long long)out * 4;           // scales, zeros fp32
  return b + 256;
}

// The column loop for `batch` problems of equal shape laid out one after another (every array of
// problem b starts b times its per-problem size after problem 0).  One chain of launches serves
// all problems: the block kernel and the preparation take the problem from blockIdx.y, the
// trailing updates are batched products.
static int gptq_quantize_impl(int batch, const void* W, long long ldw_in, int out, int d, const float* U,
                              long long ldu, const int* perm, const int* invperm, const unsigned char* dead,
                              int wbits, int groupsize, int sym, int blocksize, int mse, int q_grid,
                              float q_norm, int sm_count, int* qweight, int* qzeros, __half* scales16,
                              float* scales32, int* zeros_i32, long long ld_out, int* codes, void* what,
                              long long ldwh, int w_dtype, void* workspace, long long workspace_bytes,
                              cudaStream_t stream) {
  OC_REQUIRE(w_dtype == OC_DTYPE_F16 || w_dtype == OC_DTYPE_BF16, "gptq_quantize: unknown weight dtype");
  const int bf16 = w_dtype == OC_DTYPE_BF16;
  OC_REQUIRE(W && U && workspace, "gptq_quantize: null pointer");
  OC_REQUIRE(batch >= 1 && batch <= 65535, "gptq_quantize: batch must be in 1..65535");
  OC_REQUIRE(out > 0 && d > 0 && ldw_in >= d && ldu >= d, "gptq_quantize: bad dimensions");
  OC_REQUIRE(wbits >= 1 && wbits <= 15, "gptq_quantize: wbits must be in 1..15");
  OC_REQUIRE(groupsize == -1 || groupsize >= 1, "gptq_quantize: groupsize must be -1 or >= 1");
  if (blocksize < 1 || blocksize > BLK) {
    oc_set_last_error("gptq_quantize: blocksize must be in 1..128");
    return OC_ERR_UNSUPPORTED;
  }
  if (qweight || qzeros) {
    OC_REQUIRE(wbits == 2 || wbits == 3 || wbits == 4 || wbits == 8, "gptq_quantize: packing needs wbits in {2,3,4,8}");
    const int f = (wbits == 3) ? 32 : 32 / wbits;
    if (qweight) OC_REQUIRE(d % f == 0, "gptq_quantize: in_features not divisible by the pack factor");
    if (qzeros) OC_REQUIRE(out % f == 0 && ld_out % f == 0, "gptq_quantize: out_features not divisible by the pack factor");
  }
  const long long ws_one = oc_gptq_workspace_bytes(out, d, groupsize);
  if (workspace_bytes < ws_one * batch) {
    oc_set_last_error("gptq_quantize: workspace too small");
    return OC_ERR_WORKSPACE;
  }
  if (ld_out < out) ld_out = out;
  const int G = (groupsize == -1) ? 1 : (d + groupsize - 1) / groupsize;
  const long long ldw = round4(d), lde = round4(out);
  // workspace: all problems' Wf, then all ErrT, codesT, scales, zeros (each contiguous over the batch)
  const long long nWf = (long long)out * ldw, nErr = (long long)SUPER * BLK * lde;
  const long long nCodes = round4((long long)d * out * 2) / 2, nPar = (long long)G * out;
  char* ws = (char*)workspace;
  float* Wf = (float*)ws;                       ws += nWf * 4 * batch;
  float* ErrT = (float*)ws;                     ws += nErr * 4 * batch;
  unsigned short* codesT = (unsigned short*)ws; ws += nCodes * 2 * batch;
  float* scales = (float*)ws;                   ws += nPar * 4 * batch;
  float* zeros = (float*)ws;
  const int maxq = (1 << wbits) - 1;
  const long long sU = (long long)d * ldu, sWin = (long long)out * ldw_in;

  OC_REQUIRE(!mse || (q_grid >= 1 && q_norm > 0.f), "gptq_quantize: mse needs q_grid >= 1 and q_norm > 0");
  const int mse_steps = mse ? (int)(0.8 * q_grid) : 0;   // maxshrink = 0.8 as in the reference
  gptq_prepare_kernel<<<dim3(out, batch), 256, 0, stream>>>(W, bf16, ldw_in, out, d, perm, dead, Wf, ldw,
                                                            groupsize == -1 ? 1 : 0, maxq, sym, mse_steps,
                                                            (float)q_grid, q_norm, scales, zeros, sWin, nWf, nPar);
  OC_CHECK_LAUNCH();

  if (sm_count <= 0) sm_count = 148;
  const int warps_total = oc_div_up(out, 32) * batch;
  const int per_sm = oc_div_up(warps_total, sm_count);
  // The lazy-batch update is done at two distances.  After each block the columns up to the
  // end of its group of SUPER blocks are updated at once (they are needed next); the columns
  // beyond are updated once per group with the errors of all its blocks, which cuts the
  // read-modify-write traffic on the trailing matrix by SUPER.  Every column still receives
  // the same updates, grouped differently in the fp32 sum.
  // A group's parameters are fitted on columns that must carry every earlier update, so the
  // far update may only be postponed when no group reaches across the end of a block group.
  const bool two_level = (groupsize == -1) || ((SUPER * blocksize) % groupsize == 0);
  const int super_cols = (two_level ? SUPER : 1) * blocksize;
  for (int i1 = 0; i1 < d; i1 += blocksize) {
    const int count = min(blocksize, d - i1);
    const int s0 = (i1 / super_cols) * super_cols;          // first column of the group
    const int s1 = min(d, s0 + super_cols);                 // one past its last column
    float* err_rows = ErrT + (long long)(i1 - s0) * lde;
    ColArgs a{Wf, ldw, out, d, i1, count, U, ldu, err_rows, lde, codesT, scales, zeros, groupsize, maxq, sym,
              mse_steps, (float)q_grid, q_norm, nWf, sU, nErr, nCodes, nPar, batch};
    int rc;
    if (per_sm <= 1) rc = launch_block<1>(a, stream);
    else if (per_sm <= 2) rc = launch_block<2>(a, stream);
    else if (per_sm <= 4) rc = launch_block<4>(a, stream);
    else rc = launch_block<8>(a, stream);
    if (rc) return rc;
    const int i2 = i1 + count;
    OcGemm g{};
    g.lda = lde; g.transA = 1; g.ldb = ldu; g.transB = 0; g.ldc = ldw;
    g.M = out; g.alpha = -1.f; g.beta = 1.f; g.flags = 0;
    g.batch = batch; g.strideA = nErr; g.strideB = sU; g.strideC = nWf;
    if (i2 < s1) {
      g.A = err_rows; g.K = count;
      g.B = U + (long long)i1 * ldu + i2; g.C = Wf + i2; g.N = s1 - i2;
      rc = oc_gemm_f32_launch(g, stream);
      if (rc) return rc;
    } else if (i2 < d) {
      g.A = ErrT; g.K = s1 - s0;
      g.B = U + (long long)s0 * ldu + s1; g.C = Wf + s1; g.N = d - s1;
      rc = oc_gemm_f32_launch(g, stream);
      if (rc) return rc;
    }
  }

  const int tb = 128;
  const int f = (wbits == 3) ? 32 : ((wbits == 2 || wbits == 4 || wbits == 8) ? 32 / wbits : 1);
  const long long ldz = (wbits == 3) ? ld_out / 32 * 3 : ld_out / f;
  const long long prow = (wbits == 3) ? d / 32 * 3 : d / f;     // rows of one problem's packed weight
  for (int b = 0; b < batch; ++b) {
    const unsigned short* cT = codesT + b * nCodes;
    const float* sc = scales + b * nPar;
    const float* zr = zeros + b * nPar;
    const int* ip = invperm ? invperm + (long long)b * d : nullptr;
    if (qweight) {
      const int prow_k = (wbits == 3) ? d / 32 : d / (32 / wbits);
      pack_qweight_kernel<<<dim3(oc_div_up(out, tb), prow_k), tb, 0, stream>>>(cT, out, d, ip, wbits,
                                                                               qweight + b * prow * ld_out, ld_out);
      OC_CHECK_LAUNCH();
    }
    if (qzeros) {
      pack_qzeros_kernel<<<dim3(oc_div_up(out / f, tb), G), tb, 0, stream>>>(zr, out, G, wbits,
                                                                             qzeros + b * G * ldz, ldz);
      OC_CHECK_LAUNCH();
    }
    if (scales16 || scales32 || zeros_i32) {
      cast_params_kernel<<<dim3(oc_div_up(out, tb), G), tb, 0, stream>>>(
          sc, zr, out, G, scales16 ? scales16 + b * G * ld_out : nullptr, ld_out,
          scales32 ? scales32 + b * G * ld_out : nullptr, zeros_i32 ? zeros_i32 + b * G * ld_out : nullptr);
      OC_CHECK_LAUNCH();
    }
    if (codes || what) {
      void* wh = what ? (void*)((char*)what + (long long)b * out * ldwh * 2) : nullptr;
      unpermute_outputs_kernel<<<dim3(oc_div_up(d, 32), oc_div_up(out, 32)), dim3(32, 8), 0, stream>>>(
          cT, out, d, ip, groupsize, sc, zr, codes ? codes + (long long)b * out * d : nullptr, d, wh, ldwh, bf16);
      OC_CHECK_LAUNCH();
    }
  }
  return OC_OK;
}

// See include/onecomp_b200.h for the contracts.
extern "C" int oc_gptq_quantize(const void* W, long long ldw_in, int out, int d, const float* U,
                                long long ldu, const int* perm, const int* invperm,
                                const unsigned char* dead, int wbits, int groupsize, int sym,
                                int blocksize, int mse, int q_grid, float q_norm, int sm_count,
                                int* qweight, int* qzeros, void* scales16,
                                float* scales32, int* zeros_i32, long long ld_out, int* codes,
                                void* what, long long ldwh, int w_dtype, void* workspace,
                                long long workspace_bytes, void* stream) {
  return gptq_quantize_impl(1, W, ldw_in, out, d, U, ldu, perm, invperm, dead, wbits, groupsize, sym, blocksize,
                            mse, q_grid, q_norm, sm_count, qweight, qzeros, (__half*)scales16, scales32,
                            zeros_i32, ld_out, codes, what, ldwh, w_dtype, workspace, workspace_bytes,
                            (cudaStream_t)stream);
}

extern "C" int oc_gptq_quantize_batched(int batch, const void* W, long long ldw_in, int out, int d,
                                        const float* U, long long ldu, const int* perm, const int* invperm,
                                        const unsigned char* dead, int wbits, int groupsize, int sym,
                                        int blocksize, int mse, int q_grid, float q_norm, int sm_count,
                                        int* qweight, int* qzeros, void* scales16, float* scales32,
                                        int* zeros_i32, int* codes, void* what, int w_dtype, void* workspace,
                                        long long workspace_bytes, void* stream) {
  return gptq_quantize_impl(batch, W, ldw_in, out, d, U, ldu, perm, invperm, dead, wbits, groupsize, sym,
                            blocksize, mse, q_grid, q_norm, sm_count, qweight, qzeros, (__half*)scales16,
                            scales32, zeros_i32, out, codes, what, d, w_dtype, workspace, workspace_bytes,
                            (cudaStream_t)stream);
}

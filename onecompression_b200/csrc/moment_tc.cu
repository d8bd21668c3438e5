// Tensor-core second moments on sm_100a: tcgen05.mma with TMEM accumulators, fed by TMA.
//
//   H <- a_old * H + a_new * Xq^T Xq          (upper tiles only; mirror afterwards)
//   C <- a_old * C + a_new * D^T  Xq          (D = Xf - Xq carried as two 16-bit terms, full square)
//
// Reference call sites: onecomp/quantizer/_quantizer.py:824-830 (Hessian),
// onecomp/qep/_quantize_with_qep_arch.py:182-196 (Hessian + cross term).
//
// X is [tokens, d] fp16 row-major, so both MMA operands are "MN-major": for a
// fixed token the d index is contiguous.  A TMA box of 64 columns x 64 tokens
// lands in shared memory as 64 rows of 128 bytes with the 128-byte swizzle,
// which is exactly the canonical MN-major SWIZZLE_128B operand layout of
// tcgen05 (8 x 16-byte chunks along MN, groups of 8 tokens 1024 bytes apart,
// 64-column atoms one box apart).
//
// One persistent CTA per SM walks a static list of 128 x 256 output tiles.
//   warp 0      : TMA producer (4-stage ring, 6 boxes per stage)
//   warp 1      : TMEM allocation, MMA issue (M=128, N=256, K=16; 4 per stage)
//   warps 2..9  : drain.  Tokens are consumed in chunks (default 512); each
//                 chunk accumulates in one of two 256-column TMEM buffers, and
//                 the drain warps add finished chunks into fp32 registers with
//                 round-to-nearest while the next chunk is in flight, so the
//                 length of a tensor-core accumulation chain is bounded
//                 whatever the token count.  (The tensor core truncates when it
//                 accumulates: measured relative bias of a sum of squares is
//                 about -4.7e-9 per token of chain length, so 512 tokens keep
//                 H within 2.2e-6 of the exact moment.)
// The difference D = float(Xf) - float(Xq) is what the reference multiplies (in fp32).  One
// 16-bit value holds it exactly only while the two activations are within a factor of two of
// each other; after a few quantized blocks many are not.  D is therefore carried as
// hi = round16(D) and lo = round16((D - hi) * 2^k) (k = 11 for fp16, 8 for bf16: lo is scaled into
// the normal range).  For the tiles of C every chunk of tokens is accumulated twice, once with hi
// and once with lo as the left operand, each in a TMEM chain of its own, and the drain warps add
// the lo chain times 2^-k.
//
// Work items are ordered so that CTAs running at the same time share operand panels (super-columns
// of eight 256-column panels, swept row by row), first the tiles of C (two chains per chunk), then
// the upper tiles of H.
// Every mbarrier wait is bounded: after about two seconds the CTA raises an
// abort flag, records a code in *status and tears down normally.
#include "tc_common.cuh"

namespace {

using namespace octc;

constexpr int TILE_M = 128, TILE_N = 256, BK = 64, STAGES = 4;
constexpr int ATOM_BYTES = BK * 128;                     // one 64-column x BK-token box
constexpr int A_ATOMS = TILE_M / 64, B_ATOMS = TILE_N / 64;
constexpr int STAGE_BYTES = (A_ATOMS + B_ATOMS) * ATOM_BYTES;
constexpr int SMEM_DYN = STAGES * STAGE_BYTES + 1024;
constexpr int NUM_THREADS = 320;
constexpr uint32_t IDESC = (1u << 4) | (1u << 15) | (1u << 16) | ((TILE_N >> 3) << 17) | ((TILE_M >> 4) << 24);

struct MomentParams {
  float* H; float* C; long long ldh;
  int d; long long n_tok;
  float a_old, a_new;
  int chunk_stages;   // stages (of BK tokens) per TMEM accumulation chunk
  int h_tiles, c_tiles, tiles_m, tiles_n;
  int c_planes;       // 16-bit terms of D (2: hi and scaled lo)
  float lo_scale;     // factor that undoes the scaling of the lo term
  uint32_t idesc;     // IDESC, plus the bf16 operand-format bits for bf16 activations
  int* status;
};

__device__ __forceinline__ uint64_t make_desc(uint32_t addr) {
  // MN-major, SWIZZLE_128B: leading (64-column atom) offset = ATOM_BYTES,
  // stride (8-token group) offset = 1024 bytes, descriptor version 1.
  uint64_t d = (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(ATOM_BYTES >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
      "  tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// work item -> (matrix, first row, first column).  Items 0 .. c_tiles-1 are the tiles of C, the
// rest the tiles of H that touch the upper triangle (row tile tm owns column tiles >= tm/2).
// Both are enumerated super-column by super-column (SCW column tiles wide), row by row inside.
constexpr int SCW = 8;
__device__ __forceinline__ void decode_item(const MomentParams& p, int item, int& is_c, int& m0, int& n0) {
  if (item < p.c_tiles) {
    const int full = p.tiles_n / SCW, per_sc = p.tiles_m * SCW;
    int tm, tn;
    if (item < full * per_sc) {
      const int sc = item / per_sc, r = item - sc * per_sc;
      tm = r / SCW; tn = sc * SCW + r % SCW;
    } else {
      const int k = item - full * per_sc, w = p.tiles_n - full * SCW;
      tm = k / w; tn = full * SCW + k % w;
    }
    is_c = 1; m0 = tm * TILE_M; n0 = tn * TILE_N;
    return;
  }
  int left = item - p.c_tiles;
  is_c = 0; m0 = 0; n0 = 0;
  for (int c_lo = 0; c_lo < p.tiles_n; c_lo += SCW) {
    const int c_hi = min(p.tiles_n, c_lo + SCW);
    const int rows = min(p.tiles_m, 2 * c_hi);          // row tiles that reach this super-column
    for (int tm = 0; tm < rows; ++tm) {
      const int first = max(c_lo, tm >> 1), cnt = c_hi - first;
      if (left < cnt) { m0 = tm * TILE_M; n0 = (first + left) * TILE_N; return; }
      left -= cnt;
    }
  }
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
moment_tc_kernel(const __grid_constant__ CUtensorMap map_xq, const __grid_constant__ CUtensorMap map_delta,
                 const MomentParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[STAGES], bar_empty[STAGES], bar_acc_full[2], bar_acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag_s;
  volatile int* abort_flag = &abort_flag_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t stage_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(smem_u32(&bar_full[s]), 1); mbar_init(smem_u32(&bar_empty[s]), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(smem_u32(&bar_acc_full[b]), 1); mbar_init(smem_u32(&bar_acc_empty[b]), 8); }
    abort_flag_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&tmem_slot)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  const int total_items = p.h_tiles + p.c_tiles;
  const int total_stages = (int)((p.n_tok + BK - 1) / BK);
  const int n_chunks = (total_stages + p.chunk_stages - 1) / p.chunk_stages;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 1;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        int is_c, m0, n0;
        decode_item(p, item, is_c, m0, n0);
        const CUtensorMap* map_a = is_c ? &map_delta : &map_xq;
        const int planes = is_c ? p.c_planes : 1;
        for (int ch = 0; ch < n_chunks && ok; ++ch) {
          const int s_begin = ch * p.chunk_stages;
          const int s_end = min(total_stages, s_begin + p.chunk_stages);
          for (int pl = 0; pl < planes && ok; ++pl) {
            for (int ks = s_begin; ks < s_end; ++ks) {
              ok = mbar_wait(smem_u32(&bar_empty[stage]), phase, abort_flag, p.status, 101);
              if (!ok) break;
              const uint32_t full = smem_u32(&bar_full[stage]);
              const uint32_t sa = stage_base + stage * STAGE_BYTES;
              const uint32_t sb = sa + A_ATOMS * ATOM_BYTES;
              mbar_expect_tx(full, STAGE_BYTES);
#pragma unroll
              for (int a = 0; a < A_ATOMS; ++a) tma_load_3d(sa + a * ATOM_BYTES, map_a, m0 + a * 64, ks * BK, pl, full);
#pragma unroll
              for (int b = 0; b < B_ATOMS; ++b) tma_load_3d(sb + b * ATOM_BYTES, &map_xq, n0 + b * 64, ks * BK, 0, full);
              if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
          }
        }
      }
      if (!ok) {
        // let copies already issued land before the CTA's shared memory is released
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) { }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, cc = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        const int chains = n_chunks * ((item < p.c_tiles) ? p.c_planes : 1);
        const int planes = (item < p.c_tiles) ? p.c_planes : 1;
        for (int chain = 0; chain < chains && ok; ++chain, ++cc) {
          const int ch = chain / planes;
          const uint32_t buf = cc & 1u;
          ok = mbar_wait(smem_u32(&bar_acc_empty[buf]), ((cc >> 1) & 1u) ^ 1u, abort_flag, p.status, 102);
          if (!ok) break;
          tc_fence_after();
          const int s_begin = ch * p.chunk_stages;
          const int s_end = min(total_stages, s_begin + p.chunk_stages);
          const uint32_t tmem_d = tmem_base + buf * TILE_N;
          for (int s = s_begin; s < s_end; ++s) {
            ok = mbar_wait(smem_u32(&bar_full[stage]), phase, abort_flag, p.status, 103);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sa = stage_base + stage * STAGE_BYTES;
            const uint32_t sb = sa + A_ATOMS * ATOM_BYTES;
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk) {
              // 16 tokens = two 8-token groups = 2048 bytes further into every atom
              umma_f16(tmem_d, make_desc(sa + kk * 2048), make_desc(sb + kk * 2048), p.idesc,
                       (s > s_begin || kk > 0) ? 1u : 0u);
            }
            umma_commit(smem_u32(&bar_empty[stage]));
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (ok) umma_commit(smem_u32(&bar_acc_full[buf]));
        }
      }
    }
    __syncwarp();
  } else {
    // drain warps: TMEM lane quarter = warp % 4; columns [half*128, half*128+128)
    const int e = warp - 2;
    const int quarter = warp & 3;
    const int half = e >> 2;
    uint32_t cc = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
      int is_c, m0, n0;
      decode_item(p, item, is_c, m0, n0);
      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = 0.f;
      const int planes = is_c ? p.c_planes : 1;
      const int chains = n_chunks * planes;
      for (int chain = 0; chain < chains; ++chain, ++cc) {
        const uint32_t buf = cc & 1u;
        ok = mbar_wait(smem_u32(&bar_acc_full[buf]), (cc >> 1) & 1u, abort_flag, p.status, 104);
        if (!ok) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * TILE_N + half * 128;
        // chains alternate hi, lo; fmaf(v, 1, acc) rounds exactly like v + acc
        const float scale = (chain % planes) ? p.lo_scale : 1.f;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          float v[64];
          tmem_ld64(taddr + c * 64, v);
#pragma unroll
          for (int i = 0; i < 64; ++i) acc[c * 64 + i] = fmaf(v[i], scale, acc[c * 64 + i]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[buf]));
      }
      if (!ok) break;
      const int row = m0 + quarter * 32 + lane;
      if (row < p.d) {
        float* out = (is_c ? p.C : p.H) + (long long)row * p.ldh;
        const int cbase = n0 + half * 128;
#pragma unroll
        for (int c4 = 0; c4 < 32; ++c4) {
          const int col = cbase + c4 * 4;
          if (col < p.d) {  // d is a multiple of 8, so a float4 is inside or outside as a whole
            float4 o;
            o.x = p.a_new * acc[c4 * 4 + 0]; o.y = p.a_new * acc[c4 * 4 + 1];
            o.z = p.a_new * acc[c4 * 4 + 2]; o.w = p.a_new * acc[c4 * 4 + 3];
            if (p.a_old != 0.f) {
              const float4 old = *reinterpret_cast<const float4*>(out + col);
              o.x = fmaf(p.a_old, old.x, o.x); o.y = fmaf(p.a_old, old.y, o.y);
              o.z = fmaf(p.a_old, old.z, o.z); o.w = fmaf(p.a_old, old.w, o.w);
            }
            *reinterpret_cast<float4*>(out + col) = o;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
}

// [planes][n_tok][d] 16-bit elements, rows ld elements apart, planes n_tok * ld elements apart
int make_map(CUtensorMap* map, const void* x, long long n_tok, int d, long long ld, int planes, int bf16) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) { oc_set_last_error("moment: cuTensorMapEncodeTiled is not available"); return OC_ERR_CUDA; }
  cuuint64_t dims[3] = {(cuuint64_t)d, (cuuint64_t)n_tok, (cuuint64_t)planes};
  cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)n_tok * (cuuint64_t)ld * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)BK, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(x), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { oc_set_last_error("moment: cuTensorMapEncodeTiled failed"); return OC_ERR_CUDA; }
  return OC_OK;
}

}  // namespace

int oc_moment_simt_launch(const void* xq, const void* xf, int bf16, long long n_tok, int d, long long ld,
                          float* H, float* C, long long ldh, float a_old, float a_new, cudaStream_t stream);

int oc_delta_split_launch(const void* xf, const void* xq, long long ld, void* out, long long n_tok, int d,
                          int bf16, float lo_scale, cudaStream_t stream);

int oc_moment_pair_launch(const CUtensorMap& map_xq, const CUtensorMap& map_delta, float* H, float* C,
                          long long ldh, int d, long long n_tok, float a_old, float a_new, int chunk_tokens,
                          int sm_count, int bf16, int c_planes, float lo_scale, int* status,
                          cudaStream_t stream);

// See include/onecomp_b200.h for the contract.
extern "C" int oc_moment_accum(const void* xq, const void* xf, void* delta_scratch, long long n_tok,
                               int d, long long ld, float* H, float* C, long long ldh, float a_old,
                               float a_new, int chunk_tokens, int sm_count, int engine,
                               int x_dtype, int* status, void* stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  OC_REQUIRE(x_dtype == OC_DTYPE_F16 || x_dtype == OC_DTYPE_BF16, "moment_accum: unknown activation dtype");
  const int bf16 = x_dtype == OC_DTYPE_BF16;
  OC_REQUIRE(xq && (H || C) && d > 0 && n_tok >= 0 && ld >= d && ldh >= d, "moment_accum: bad arguments");
  OC_REQUIRE(!C || xf, "moment_accum: the cross term needs the full-precision activations");
  const bool tc_ok = engine != OC_MOMENT_SIMT && d % 8 == 0 && ld % 8 == 0 && ldh % 4 == 0 && n_tok > 0 && status &&
                     ((uintptr_t)xq & 15) == 0 &&
                     (!C || (delta_scratch && ((uintptr_t)delta_scratch & 15) == 0 && ((uintptr_t)xf & 15) == 0)) &&
                     (!H || ((uintptr_t)H & 15) == 0) && (!C || ((uintptr_t)C & 15) == 0);
  if (!tc_ok) {
    // general shapes: fp32 FMA kernel (forms Xf - Xq itself, in fp32)
    return oc_moment_simt_launch(xq, C ? xf : nullptr, bf16, n_tok, d, ld,
                                 H, C, ldh, a_old, a_new, stream);
  }
  // D = Xf - Xq as two 16-bit planes [2][n_tok][d] (rows packed to d elements): hi, then lo * 2^k
  const int c_planes = 2;
  const float lo_up = bf16 ? 256.f : 2048.f;
  if (C) {
    int rcd = oc_delta_split_launch(xf, xq, ld, delta_scratch, n_tok, d, bf16, lo_up, stream);
    if (rcd) return rcd;
  }
  CUtensorMap map_xq, map_delta;
  int rc = make_map(&map_xq, xq, n_tok, d, ld, 1, bf16);
  if (rc) return rc;
  if (C) { rc = make_map(&map_delta, delta_scratch, n_tok, d, d, c_planes, bf16); if (rc) return rc; }
  else map_delta = map_xq;

  if (engine == OC_MOMENT_PAIR || (engine == OC_MOMENT_AUTO && OC_MOMENT_AUTO_USES_PAIRS))
    return oc_moment_pair_launch(map_xq, map_delta, H, C, ldh, d, n_tok, a_old, a_new, chunk_tokens, sm_count,
                                 bf16, c_planes, 1.f / lo_up, status, stream);

  MomentParams p{};
  p.H = H; p.C = C; p.ldh = ldh; p.d = d; p.n_tok = n_tok; p.a_old = a_old; p.a_new = a_new;
  if (chunk_tokens <= 0) chunk_tokens = 512;
  p.chunk_stages = max(1, chunk_tokens / BK);
  const int tiles_m = oc_div_up(d, TILE_M);
  p.tiles_m = tiles_m;
  p.tiles_n = oc_div_up(d, TILE_N);
  int h_tiles = 0;
  if (H) for (int tm = 0; tm < tiles_m; ++tm) h_tiles += max(0, p.tiles_n - (tm >> 1));
  p.h_tiles = h_tiles;
  p.c_tiles = C ? tiles_m * p.tiles_n : 0;
  p.c_planes = c_planes;
  p.lo_scale = 1.f / lo_up;
  p.idesc = IDESC | (bf16 ? ((1u << 7) | (1u << 10)) : 0u);
  p.status = status;

  OC_OPT_IN_SMEM(moment_tc_kernel, SMEM_DYN);
  if (sm_count <= 0) sm_count = 148;
  const int grid = min(sm_count, p.h_tiles + p.c_tiles);
  moment_tc_kernel<<<grid, NUM_THREADS, SMEM_DYN, stream>>>(map_xq, map_delta, p);
  OC_CHECK_LAUNCH();
  return OC_OK;
}

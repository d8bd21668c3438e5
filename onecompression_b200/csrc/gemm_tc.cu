// fp32-accurate GEMM on the tensor cores (3xTF32): C = beta*C + alpha*opA(A)*opB(B).
//
// Every fp32 operand value a is split into hi = tf32(a) (round to nearest, low 13 mantissa
// bits zero) and lo = a - hi (exact in fp32); the product a*b is accumulated as
// hi*hi + hi*lo + lo*hi with tcgen05.mma.kind::tf32 into an fp32 TMEM accumulator.  The
// dropped lo*lo term and the truncation of lo to tf32 are about 2^-22 relative, i.e. the
// result is an fp32-grade product sum.
//
// Pipeline of one persistent CTA:
//   warp 0      TMA: raw fp32 tiles of A and B into shared memory (swizzled)
//   split warps rewrite every raw value in place as hi and store lo at the same offset of a
//               second buffer (elementwise, so the swizzled layout is kept)
//   warp 1      MMA: per 8 k-values three tcgen05.mma (lo*hi, hi*lo, hi*hi), M=128 N=BN K=8
//   drain warps accumulators leave TMEM every 256 k-values and are summed in registers (the
//               tensor core truncates when it accumulates, so chains are kept short); at the
//               end of a tile alpha / beta are applied and C is written while the MMA warp
//               already works on the next tile in the other TMEM buffer.
// Two tile shapes share the code.  Narrow: 128 x 128 tiles, 32 k-values per stage, 3 stages,
// 4 split and 4 drain warps.  Wide: 128 x 256 tiles, 16 k-values per stage, 4 stages, 4 split
// and 8 drain warps.  The kernel is bound by shared-memory bandwidth (TMA write, split read
// and two writes, three operand reads per MMA pair); per flop a wide tile reads the operands
// 1.5 instead of 2 times, so it is chosen when the product has enough tiles to fill the SMs.
// Both shapes cut k into the same chains, so a product gives the same bits with either.
// Operands may be K-major ([rows, K] row-major) or MN-major ([K, rows] row-major); both are
// native tcgen05 layouts, so the four transpose combinations need no data movement.
// All mbarrier waits are bounded (see tc_common.cuh).
#include "tc_common.cuh"

namespace {

using namespace octc;

constexpr int BM = 128;
constexpr int CHAIN_K = 128;                            // k-values per accumulation chain (48 MMAs)

template <int BN_, int BK_, int STAGES_, int FIRST_SPLIT_>
struct Shape {
  static constexpr int BN = BN_, BK = BK_, STAGES = STAGES_, SPLIT_WARPS = 4, FIRST_SPLIT = FIRST_SPLIT_;
  static constexpr int A_BYTES = BM * BK * 4, B_BYTES = BN * BK * 4;   // one operand tile (hi or lo)
  static constexpr int STAGE_BYTES = 2 * (A_BYTES + B_BYTES);          // A hi, A lo, B hi, B lo
  static constexpr int DRAIN_WARPS = 4 * (BN / 128);
  // operand ring, slack for its 1024-byte alignment, 4 KB of epilogue staging per drain warp
  static constexpr int SMEM_DYN = STAGES * STAGE_BYTES + 1024 + DRAIN_WARPS * 4096;
  static constexpr int FIRST_DRAIN = FIRST_SPLIT + SPLIT_WARPS;
  // With 16 warps the register file gives 128 registers per thread at launch, fewer than a drain
  // thread needs for its 128 partial sums: the warpgroups then trade registers (setmaxnreg).
  static constexpr bool TRADE_REGISTERS = FIRST_SPLIT == 4;
  static constexpr int THREADS = 32 * (FIRST_DRAIN + DRAIN_WARPS);
  static constexpr int SPLIT_THREADS = 32 * SPLIT_WARPS;
  static constexpr int TMEM_COLS = 2 * BN;
  static_assert(BK == 32 || BK == 16, "K-major rows are one 128- or 64-byte swizzle span");
  static_assert(BN == 128 || BN == 256, "one or two 128-column halves");
};
using Narrow = Shape<128, 32, 3, 2>;   // warps: TMA, MMA, 4 split, 4 drain
using Wide = Shape<256, 16, 4, 4>;     // warps: TMA, MMA, 2 idle | 4 split | 8 drain (four warpgroups)

struct TcGemmParams {
  float* C; long long ldc; long long strideC;
  int M, N, K;
  float alpha, beta;
  int flags, batch;
  int tiles_m, tiles_n;
  int* status;
};

template <bool A_MN, bool B_MN, int BN>
__host__ __device__ constexpr uint32_t idesc() {
  // c = f32 (1<<4); a, b = tf32 (2<<7, 2<<10); major bits 15 / 16; N>>3 at 17; M>>4 at 24
  return (1u << 4) | (2u << 7) | (2u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
         ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// K-major tile: rows (M or N index) of BK k-values = one swizzle span (128 bytes for BK 32,
//   64 bytes for BK 16); groups of 8 rows are 8 spans apart; the next 8 k-values are 32 bytes
//   further in the row.
// MN-major tile: 32-column atoms of [BK k-rows x 128 bytes], one after another.  32-bit
//   MN-major operands exist only in the "128-byte swizzle, 32-byte atom" layout (TMA mode
//   SWIZZLE_128B_ATOM_32B): the pattern repeats every 4 k-rows (512 bytes), an MMA of 8
//   k-values spans two such groups, the next 8 k-values start 1024 bytes further.
template <bool MN, int BK>
__device__ __forceinline__ uint64_t make_desc(uint32_t addr, int k8) {
  uint64_t d;
  if (MN) {
    d = (uint64_t)(((addr + k8 * 1024) & 0x3FFFFu) >> 4);
    d |= (uint64_t)((BK * 128) >> 4) << 16;   // leading offset: next 32-column atom
    d |= (uint64_t)(512 >> 4) << 32;          // stride offset: next group of 4 k-rows
    d |= 1ull << 61;                          // 128-byte swizzle with 32-byte atoms (the MN-major tf32 layout)
  } else {
    d = (uint64_t)(((addr + k8 * 32) & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;                   // unused for swizzled K-major layouts
    d |= (uint64_t)((8 * BK * 4) >> 4) << 32; // next group of 8 rows
    d |= (BK == 32 ? 2ull : 4ull) << 61;      // 128-byte / 64-byte swizzle
  }
  d |= 1ull << 46;
  return d;
}

// The tensor core reads the upper 19 bits of a 32-bit operand (sign, exponent, 10 mantissa bits),
// so the raw value serves as hi = trunc(v) without being rewritten.  lo = v - hi is exact; half a
// tf32 unit is added to its magnitude so that the tensor core's truncation rounds it to nearest.
__device__ __forceinline__ float split_lo(float v) {
  const float l = v - __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
  return __uint_as_float(__float_as_uint(l) + 0x1000u);
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t id,
                                          uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
      "  tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p; }"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(id), "r"(accumulate) : "memory");
}

template <bool MN, int ROWS, int BK>
__device__ __forceinline__ void load_operand(uint32_t dst, const CUtensorMap* map, int mn0, int k0,
                                             int batch, uint32_t bar) {
  if (MN) {
#pragma unroll
    for (int a = 0; a < ROWS / 32; ++a) tma_load_3d(dst + a * BK * 128, map, mn0 + a * 32, k0, batch, bar);
  } else {
    tma_load_3d(dst, map, k0, mn0, batch, bar);
  }
}

template <int BN, int BK>
__device__ __forceinline__ bool tile_coords(const TcGemmParams& p, int item, int& z, int& m0, int& n0,
                                            int& k_lo, int& k_hi) {
  const int per = p.tiles_m * p.tiles_n;
  z = item / per;
  const int r = item - z * per;
  m0 = (r / p.tiles_n) * BM;
  n0 = (r % p.tiles_n) * BN;
  if ((p.flags & OC_GEMM_SKIP_UPPER_TILES) && n0 > m0 + BM - 1) return false;
  k_lo = 0; k_hi = p.K;
  if (p.flags & OC_GEMM_KLO_FROM_N) k_lo = max(k_lo, n0);
  if (p.flags & OC_GEMM_KLO_FROM_M) k_lo = max(k_lo, m0);
  if (p.flags & OC_GEMM_KHI_FROM_M) k_hi = min(k_hi, m0 + BM);
  if (p.flags & OC_GEMM_KHI_FROM_N) k_hi = min(k_hi, n0 + BN);
  k_lo = (k_lo / BK) * BK;
  return true;
}

// A wide tile of a lower-tiles-only product that straddles the diagonal: its upper 128 columns are
// a tile the narrow shape would skip, so they get no MMA and are not written.
template <int BN>
__device__ __forceinline__ bool upper_half_in_use(const TcGemmParams& p, int m0, int n0) {
  return BN == 128 || !(p.flags & OC_GEMM_SKIP_UPPER_TILES) || n0 + 128 <= m0 + BM - 1;
}

template <bool A_MN, bool B_MN, class S>
__global__ void __launch_bounds__(S::THREADS, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const TcGemmParams p) {
  constexpr int BN = S::BN, BK = S::BK, STAGES = S::STAGES, STAGE_BYTES = S::STAGE_BYTES;
  constexpr int A_BYTES = S::A_BYTES, B_BYTES = S::B_BYTES, CHAIN_STAGES = CHAIN_K / BK;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_raw[STAGES], bar_split[STAGES], bar_empty[STAGES];
  __shared__ __align__(8) uint64_t bar_acc_full[2], bar_acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag_s;
  volatile int* abort_flag = &abort_flag_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  uint8_t* stage_ptr = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const uint32_t stage_base = smem_u32(stage_ptr);

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&bar_raw[s]), 1);
      mbar_init(smem_u32(&bar_split[s]), S::SPLIT_THREADS);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) { mbar_init(smem_u32(&bar_acc_full[b]), 1); mbar_init(smem_u32(&bar_acc_empty[b]), S::DRAIN_WARPS); }
    abort_flag_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_slot)), "r"((uint32_t)S::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  const int total_items = p.batch * p.tiles_m * p.tiles_n;

  if (warp < S::FIRST_SPLIT) {
  if (S::TRADE_REGISTERS) asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 1;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        int z, m0, n0, k_lo, k_hi;
        if (!tile_coords<BN, BK>(p, item, z, m0, n0, k_lo, k_hi)) continue;
        for (int k0 = k_lo; k0 < k_hi; k0 += BK) {
          ok = mbar_wait(smem_u32(&bar_empty[stage]), phase, abort_flag, p.status, 201);
          if (!ok) break;
          const uint32_t bar = smem_u32(&bar_raw[stage]);
          const uint32_t sa = stage_base + stage * STAGE_BYTES;
          mbar_expect_tx(bar, A_BYTES + B_BYTES);
          load_operand<A_MN, BM, BK>(sa, &map_a, m0, k0, z, bar);
          load_operand<B_MN, BN, BK>(sa + 2 * A_BYTES, &map_b, n0, k0, z, bar);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) { }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t ID_FULL = idesc<A_MN, B_MN, BN>(), ID_HALF = idesc<A_MN, B_MN, 128>();
      uint32_t stage = 0, phase = 0, cc = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
        int z, m0, n0, k_lo, k_hi;
        if (!tile_coords<BN, BK>(p, item, z, m0, n0, k_lo, k_hi)) continue;
        const uint32_t ID = upper_half_in_use<BN>(p, m0, n0) ? ID_FULL : ID_HALF;
        const int n_stages = max(0, (k_hi - k_lo + BK - 1) / BK);
        const int n_chunks = max(1, (n_stages + CHAIN_STAGES - 1) / CHAIN_STAGES);
        for (int ch = 0; ch < n_chunks && ok; ++ch, ++cc) {
          const uint32_t buf = cc & 1u;
          ok = mbar_wait(smem_u32(&bar_acc_empty[buf]), ((cc >> 1) & 1u) ^ 1u, abort_flag, p.status, 202);
          if (!ok) break;
          tc_fence_after();
          const int s_begin = ch * CHAIN_STAGES;
          const int s_end = min(n_stages, s_begin + CHAIN_STAGES);
          const uint32_t tmem_d = tmem_base + buf * BN;
          for (int s = s_begin; s < s_end; ++s) {
            ok = mbar_wait(smem_u32(&bar_split[stage]), phase, abort_flag, p.status, 203);
            if (!ok) break;
            tc_fence_after();
            const uint32_t a_hi = stage_base + stage * STAGE_BYTES;
            const uint32_t a_lo = a_hi + A_BYTES, b_hi = a_hi + 2 * A_BYTES, b_lo = b_hi + B_BYTES;
#pragma unroll
            for (int k8 = 0; k8 < BK / 8; ++k8) {
              const uint64_t dah = make_desc<A_MN, BK>(a_hi, k8), dal = make_desc<A_MN, BK>(a_lo, k8);
              const uint64_t dbh = make_desc<B_MN, BK>(b_hi, k8), dbl = make_desc<B_MN, BK>(b_lo, k8);
              umma_tf32(tmem_d, dal, dbh, ID, (s > s_begin || k8 > 0) ? 1u : 0u);
              umma_tf32(tmem_d, dah, dbl, ID, 1u);
              umma_tf32(tmem_d, dah, dbh, ID, 1u);
            }
            umma_commit(smem_u32(&bar_empty[stage]));
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (ok) umma_commit(smem_u32(&bar_acc_full[buf]));
        }
      }
    }
    __syncwarp();
  }  // further warps of the first warpgroup (wide shape) idle
  } else if (warp < S::FIRST_DRAIN) {
    // split warps
    if (S::TRADE_REGISTERS) asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    const int st = tid - 32 * S::FIRST_SPLIT;
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
      int z, m0, n0, k_lo, k_hi;
      if (!tile_coords<BN, BK>(p, item, z, m0, n0, k_lo, k_hi)) continue;
      for (int k0 = k_lo; k0 < k_hi; k0 += BK) {
        ok = mbar_wait(smem_u32(&bar_raw[stage]), phase, abort_flag, p.status, 204);
        if (!ok) break;
        uint8_t* base = stage_ptr + stage * STAGE_BYTES;
#pragma unroll
        for (int op = 0; op < 2; ++op) {
          const int bytes = op ? B_BYTES : A_BYTES;
          float4* hi = reinterpret_cast<float4*>(base + op * 2 * A_BYTES);
          float4* lo = reinterpret_cast<float4*>(base + op * 2 * A_BYTES + bytes);
#pragma unroll 8
          for (int i = 0; i < bytes / 16 / S::SPLIT_THREADS; ++i) {
            const int idx = i * S::SPLIT_THREADS + st;
            const float4 v = hi[idx];
            float4 l;
            l.x = split_lo(v.x); l.y = split_lo(v.y); l.z = split_lo(v.z); l.w = split_lo(v.w);
            lo[idx] = l;
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(smem_u32(&bar_split[stage]));
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // drain warps: TMEM lane quarter = warp % 4; with wide tiles a second set of four warps takes
    // the upper 128 columns
    if (S::TRADE_REGISTERS) asm volatile("setmaxnreg.inc.sync.aligned.u32 184;");
    const int quarter = warp & 3;
    const int half = (warp - S::FIRST_DRAIN) >> 2;
    constexpr int DW = 128;               // columns per drain warp
    uint32_t cc = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < total_items && ok; item += gridDim.x) {
      int z, m0, n0, k_lo, k_hi;
      if (!tile_coords<BN, BK>(p, item, z, m0, n0, k_lo, k_hi)) continue;
      const int n_stages = max(0, (k_hi - k_lo + BK - 1) / BK);
      const int n_chunks = max(1, (n_stages + CHAIN_STAGES - 1) / CHAIN_STAGES);
      const bool in_use = half == 0 || upper_half_in_use<BN>(p, m0, n0);
      float acc[DW];
#pragma unroll
      for (int i = 0; i < DW; ++i) acc[i] = 0.f;
      for (int ch = 0; ch < n_chunks; ++ch, ++cc) {
        const uint32_t buf = cc & 1u;
        ok = mbar_wait(smem_u32(&bar_acc_full[buf]), (cc >> 1) & 1u, abort_flag, p.status, 205);
        if (!ok) break;
        tc_fence_after();
        if (n_stages > 0 && in_use) {
          const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN + half * DW;
#pragma unroll
          for (int c = 0; c < DW / 32; ++c) {
            float v[32];
            tmem_ld32(taddr + c * 32, v);
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[c * 32 + i] += v[i];
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_acc_empty[buf]));
      }
      if (!ok) break;
      if (!in_use) continue;
      // Epilogue.  A drain thread holds one row of the tile, so writing from the registers would
      // touch 32 rows per instruction.  Each warp instead passes 32 x 32 slices through 4 KB of
      // shared memory of its own (16-byte chunks swizzled by row, conflict-free both ways) and
      // reads / writes C with four full 128-byte row segments per instruction.
      float4* stg = reinterpret_cast<float4*>(stage_ptr + STAGES * STAGE_BYTES) + (warp - S::FIRST_DRAIN) * 256;
      float* out_tile = p.C + (long long)z * p.strideC;
      const float alpha = p.alpha, beta = p.beta;
      const int sub = lane >> 3, chunk = lane & 7;
#pragma unroll
      for (int c = 0; c < DW / 32; ++c) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float4 o;
          o.x = alpha * acc[c * 32 + j * 4 + 0]; o.y = alpha * acc[c * 32 + j * 4 + 1];
          o.z = alpha * acc[c * 32 + j * 4 + 2]; o.w = alpha * acc[c * 32 + j * 4 + 3];
          stg[lane * 8 + (j ^ (lane & 7))] = o;
        }
        __syncwarp();
        const int col = n0 + half * DW + c * 32 + chunk * 4;
#pragma unroll
        for (int i0 = 0; i0 < 8; i0 += 4) {
          float4 o[4], old[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int r = (i0 + i) * 4 + sub;
            const int row = m0 + quarter * 32 + r;
            o[i] = stg[r * 8 + (chunk ^ (r & 7))];
            old[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (beta != 0.f && row < p.M && col + 3 < p.N)
              old[i] = *reinterpret_cast<const float4*>(out_tile + (long long)row * p.ldc + col);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int r = (i0 + i) * 4 + sub;
            const int row = m0 + quarter * 32 + r;
            if (row >= p.M) continue;
            float* out = out_tile + (long long)row * p.ldc + col;
            if (col + 3 < p.N) {
              float4 v = o[i];
              if (beta != 0.f) {
                v.x = fmaf(beta, old[i].x, v.x); v.y = fmaf(beta, old[i].y, v.y);
                v.z = fmaf(beta, old[i].z, v.z); v.w = fmaf(beta, old[i].w, v.w);
              }
              *reinterpret_cast<float4*>(out) = v;
            } else {
              const float e[4] = {o[i].x, o[i].y, o[i].z, o[i].w};
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (col + j < p.N) out[j] = (beta != 0.f) ? fmaf(beta, out[j], e[j]) : e[j];
            }
          }
        }
        __syncwarp();
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                 ::"r"(tmem_base), "r"((uint32_t)S::TMEM_COLS) : "memory");
  }
}

// rows x K operand.  K-major storage: [rows, K] row-major (ld); MN-major storage: [K, rows].
// `tile_rows` is the tile's extent along rows (BM for A, BN for B), `bk` its k-extent.
int make_operand_map(CUtensorMap* map, const float* ptr, bool mn_major, int rows, int K, long long ld,
                     long long stride_batch, int batch, int tile_rows, int bk) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) { oc_set_last_error("gemm: cuTensorMapEncodeTiled is not available"); return OC_ERR_CUDA; }
  cuuint64_t dims[3], strides[2];
  cuuint32_t box[3], estr[3] = {1, 1, 1};
  if (mn_major) { dims[0] = (cuuint64_t)rows; dims[1] = (cuuint64_t)K; box[0] = 32; box[1] = (cuuint32_t)bk; }
  else          { dims[0] = (cuuint64_t)K; dims[1] = (cuuint64_t)rows; box[0] = (cuuint32_t)bk; box[1] = (cuuint32_t)tile_rows; }
  dims[2] = (cuuint64_t)batch;
  box[2] = 1;
  strides[0] = (cuuint64_t)ld * 4;
  strides[1] = (cuuint64_t)(batch > 1 ? stride_batch : (long long)dims[1] * ld) * 4;
  const CUtensorMapSwizzle swz = mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                 : (bk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { oc_set_last_error("gemm: cuTensorMapEncodeTiled failed"); return OC_ERR_CUDA; }
  return OC_OK;
}

template <bool A_MN, bool B_MN, class S>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const TcGemmParams& p, int grid, cudaStream_t s) {
  OC_OPT_IN_SMEM((gemm_tf32x3_kernel<A_MN, B_MN, S>), S::SMEM_DYN);
  gemm_tf32x3_kernel<A_MN, B_MN, S><<<grid, S::THREADS, S::SMEM_DYN, s>>>(ma, mb, p);
  OC_CHECK_LAUNCH();
  return OC_OK;
}

int g_sm_count[OC_MAX_DEVICES] = {};
int* g_status[OC_MAX_DEVICES] = {};
int g_tile_shape = 0;   // 0: chosen per product; 1: narrow tiles only; 2: wide tiles wherever allowed

template <class S>
int launch_shape(const OcGemm& g, int dev, cudaStream_t stream) {
  CUtensorMap ma, mb;
  int rc = make_operand_map(&ma, g.A, g.transA != 0, g.M, g.K, g.lda, g.strideA, g.batch, BM, S::BK);
  if (rc) return rc;
  rc = make_operand_map(&mb, g.B, g.transB == 0, g.N, g.K, g.ldb, g.strideB, g.batch, S::BN, S::BK);
  if (rc) return rc;
  TcGemmParams p{};
  p.C = g.C; p.ldc = g.ldc; p.strideC = g.strideC; p.M = g.M; p.N = g.N; p.K = g.K;
  p.alpha = g.alpha; p.beta = g.beta; p.flags = g.flags; p.batch = g.batch;
  p.tiles_m = oc_div_up(g.M, BM); p.tiles_n = oc_div_up(g.N, S::BN);
  p.status = g_status[dev];
  const long long items = (long long)p.batch * p.tiles_m * p.tiles_n;
  OC_REQUIRE(items < (1ll << 30), "gemm: too many tiles");
  const int grid = (int)((items < g_sm_count[dev]) ? items : g_sm_count[dev]);
  const bool a_mn = g.transA != 0, b_mn = g.transB == 0;
  if (a_mn) return b_mn ? launch<true, true, S>(ma, mb, p, grid, stream) : launch<true, false, S>(ma, mb, p, grid, stream);
  return b_mn ? launch<false, true, S>(ma, mb, p, grid, stream) : launch<false, false, S>(ma, mb, p, grid, stream);
}

// Relative cost of a wide tile against a narrow one (twice the flops at 1.5 / 2 of the
// shared-memory traffic per flop).
constexpr double WIDE_TILE_COST = 1.6;

}  // namespace

// The tensor-core engine takes a product when every operand is 16-byte aligned with leading
// dimensions and batch strides that are multiples of 4 floats; the caller falls back to the
// FMA engine otherwise.  `status` is a device int (one per device, owned by the library image)
// that records an expired pipeline wait.
static __device__ int g_gemm_status_word;

bool oc_gemm_tc_eligible(const OcGemm& g) {
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return al(g.A) && al(g.B) && al(g.C) && g.lda % 4 == 0 && g.ldb % 4 == 0 && g.ldc % 4 == 0 &&
         g.strideA % 4 == 0 && g.strideB % 4 == 0 && g.strideC % 4 == 0 && g.K >= 1 &&
         (long long)g.M * g.N >= 64 * 64;
}

// 0: tile shape chosen per product (default); 1: narrow tiles only; 2: wide tiles for every plain
// product.  Returns the previous setting.
extern "C" int oc_set_gemm_tile_shape(int mode) {
  const int old = g_tile_shape;
  if (mode >= 0 && mode <= 2) g_tile_shape = mode;
  return old;
}

// The tile shape a product gets: 1 = 128 x 128, 2 = 128 x 256.  Host arithmetic only.
// Either shape serves every product: the k-range flags state that the operand IS zero outside the
// range, so a wide tile only multiplies a few more exact zeros (its k-range is the union of its two
// halves' ranges, and the chains of both shapes start on the same 128-grid).  Wide tiles are taken
// when they need less time, counted in waves of tiles over `sms` SMs.
extern "C" int oc_gemm_tile_choice(int M, int N, int batch, int flags, int sms) {
  if (g_tile_shape == 1 || g_tile_shape == 2) return g_tile_shape;
  if (M <= 0 || N <= 0 || batch <= 0 || sms <= 0) return 1;
  const long long tm = oc_div_up(M, BM);
  const long long tn_narrow = oc_div_up(N, Narrow::BN), tn_wide = oc_div_up(N, Wide::BN);
  long long n_narrow = tm * tn_narrow, n_wide = tm * tn_wide;
  if (flags & OC_GEMM_SKIP_UPPER_TILES) {
    n_narrow = n_wide = 0;
    for (long long i = 0; i < tm; ++i) {      // tiles of row block i that reach the diagonal or lie below it
      n_narrow += (i + 1 < tn_narrow) ? i + 1 : tn_narrow;
      n_wide += (i / 2 + 1 < tn_wide) ? i / 2 + 1 : tn_wide;
    }
  }
  n_narrow *= batch; n_wide *= batch;
  const double cost_narrow = (double)((n_narrow + sms - 1) / sms);
  const double cost_wide = WIDE_TILE_COST * (double)((n_wide + sms - 1) / sms);
  return cost_wide < cost_narrow ? 2 : 1;
}

int oc_gemm_tc_launch(const OcGemm& g, cudaStream_t stream) {
  OC_CURRENT_DEVICE(dev);
  if (!g_status[dev]) {
    void* p = nullptr;
    OC_CUDA(cudaGetSymbolAddress(&p, g_gemm_status_word));
    g_status[dev] = (int*)p;
  }
  if (g_sm_count[dev] == 0) {
    OC_CUDA(cudaDeviceGetAttribute(&g_sm_count[dev], cudaDevAttrMultiProcessorCount, dev));
  }
  const bool wide = oc_gemm_tile_choice(g.M, g.N, g.batch, g.flags, g_sm_count[dev]) == 2;
  return wide ? launch_shape<Wide>(g, dev, stream) : launch_shape<Narrow>(g, dev, stream);
}

// 0 when no tensor-core GEMM on the current device has recorded an expired wait, else its code.
extern "C" int oc_gemm_tc_status(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_gemm_status_word, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

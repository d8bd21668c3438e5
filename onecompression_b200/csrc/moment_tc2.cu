// Second moments on CTA pairs: the same computation as moment_tc.cu with
// tcgen05.mma.cta_group::2, i.e. one 256 x 256 output tile per pair of SMs.
//
// Why pairs: with one CTA per tile every MMA (M=128, N=256, K=16) reads 12 KB of operands from
// shared memory per 128 tensor-core cycles while TMA writes the same amount, and that traffic, not
// the tensor pipe, bounds the single-CTA kernel at about 70 % of the pipe.  In a pair each CTA
// holds its 128 rows of A and only half of B (128 of the 256 columns), so shared-memory traffic
// per SM drops by a third for the same tensor work.
//
// Roles per CTA (320 threads), rank = position in the pair, rank 0 leads:
//   warp 0      : TMA producer for this CTA's operand halves (6-stage ring, 4 boxes per stage);
//                 all copies of a stage, from both CTAs, complete on the leader's `full` barrier
//   warp 1      : TMEM allocation (both CTAs); in the leader, MMA issue for the pair and commits
//                 that arrive on the barriers of both CTAs
//   warps 2..9  : drain this CTA's 128 x 256 accumulator (chunked accumulation as in
//                 moment_tc.cu) and tell the leader when a TMEM buffer is free again
// Every mbarrier wait is bounded (about two seconds, then abort flag + status code); both CTAs
// always reach the closing cluster barrier, so neither touches the other's shared memory after
// it has gone.  No cluster-multicast loads, no peer-GPU memory.
#include "tc_common.cuh"

namespace {

using namespace octc;

constexpr int PAIR_M = 256, PAIR_N = 256, HALF = 128, BK = 64, STAGES = 6;
constexpr int ATOM_BYTES = BK * 128;                       // one 64-column x BK-token box
constexpr int HALF_ATOMS = HALF / 64;                      // boxes per operand half
constexpr int STAGE_BYTES = 2 * HALF_ATOMS * ATOM_BYTES;   // this CTA's share of a stage (32 KB)
constexpr int SMEM_DYN = STAGES * STAGE_BYTES + 1024;
constexpr int NUM_THREADS = 320;
constexpr uint32_t PEER_MASK = 0xFEFFFFFFu;                // clears the pair-rank bit of a shared address
// kind::f16, fp32 accumulate, A and B MN-major, N = 256, M = 256 (over the pair)
constexpr uint32_t IDESC = (1u << 4) | (1u << 15) | (1u << 16) | ((PAIR_N >> 3) << 17) | ((PAIR_M >> 4) << 24);

struct PairParams {
  float* H; float* C; long long ldh;
  int d; long long n_tok;
  float a_old, a_new;
  int chunk_stages;
  int h_tiles, c_tiles, tiles;   // tiles = tiles per matrix side
  int c_planes;                  // 16-bit terms of Xf - Xq (see moment_tc.cu)
  float lo_scale;
  uint32_t idesc;
  int* status;
};

__device__ __forceinline__ uint64_t make_desc(uint32_t addr) {
  uint64_t d = (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(ATOM_BYTES >> 4) << 16;   // next 64-column atom
  d |= (uint64_t)(1024 >> 4) << 32;         // next 8-token group
  d |= 1ull << 46;
  d |= 2ull << 61;                          // SWIZZLE_128B
  return d;
}

__device__ __forceinline__ void umma_pair_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
      "  tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p; }"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// commit of all earlier MMAs of this thread; arrives on `bar` in both CTAs of the pair
__device__ __forceinline__ void umma_pair_commit(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void tma_pair_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z,
                                                 uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(leader_bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_on_leader(uint32_t bar) {
  asm volatile(
      "{ .reg .b32 ra; mapa.shared::cluster.u32 ra, %0, 0;\n"
      "  mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra]; }" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// work item -> (matrix, first row, first column) of a 256 x 256 tile: first the tiles of C, then
// the tiles of H on or above the diagonal (row tile tm owns column tiles >= tm), both enumerated
// super-column by super-column (SCW column tiles wide), row by row inside, so that pairs running
// at the same time share operand panels.
constexpr int SCW = 8;
__device__ __forceinline__ void decode_item(const PairParams& p, int item, int& is_c, int& m0, int& n0) {
  if (item < p.c_tiles) {
    const int full = p.tiles / SCW, per_sc = p.tiles * SCW;
    int tm, tn;
    if (item < full * per_sc) {
      const int sc = item / per_sc, r = item - sc * per_sc;
      tm = r / SCW; tn = sc * SCW + r % SCW;
    } else {
      const int k = item - full * per_sc, w = p.tiles - full * SCW;
      tm = k / w; tn = full * SCW + k % w;
    }
    is_c = 1; m0 = tm * PAIR_M; n0 = tn * PAIR_N;
    return;
  }
  int left = item - p.c_tiles;
  is_c = 0; m0 = 0; n0 = 0;
  for (int c_lo = 0; c_lo < p.tiles; c_lo += SCW) {
    const int c_hi = min(p.tiles, c_lo + SCW);
    for (int tm = 0; tm < c_hi; ++tm) {
      const int first = max(c_lo, tm), cnt = c_hi - first;
      if (left < cnt) { m0 = tm * PAIR_M; n0 = (first + left) * PAIR_N; return; }
      left -= cnt;
    }
  }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
moment_pair_kernel(const __grid_constant__ CUtensorMap map_xq, const __grid_constant__ CUtensorMap map_delta,
                   const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[STAGES], bar_empty[STAGES], bar_acc_full[2], bar_acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag_s;
  volatile int* abort_flag = &abort_flag_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const uint32_t stage_base = (smem_u32(smem_raw) + 1023u) & ~1023u;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(smem_u32(&bar_full[s]), 1); mbar_init(smem_u32(&bar_empty[s]), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(smem_u32(&bar_acc_full[b]), 1); mbar_init(smem_u32(&bar_acc_empty[b]), 16); }
    abort_flag_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(smem_u32(&tmem_slot)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();          // barriers of both CTAs are initialised before anything remote
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;

  const int total_items = p.h_tiles + p.c_tiles;
  const int total_stages = (int)((p.n_tok + BK - 1) / BK);
  const int n_chunks = (total_stages + p.chunk_stages - 1) / p.chunk_stages;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 1;
      bool ok = true;
      for (int item = pair; item < total_items && ok; item += n_pairs) {
        int is_c, m0, n0;
        decode_item(p, item, is_c, m0, n0);
        const CUtensorMap* map_a = is_c ? &map_delta : &map_xq;
        const int am = m0 + (int)rank * HALF, bn = n0 + (int)rank * HALF;
        const int planes = is_c ? p.c_planes : 1;
        for (int ch = 0; ch < n_chunks && ok; ++ch) {
          const int s_begin = ch * p.chunk_stages;
          const int s_end = min(total_stages, s_begin + p.chunk_stages);
          for (int pl = 0; pl < planes && ok; ++pl) {
            for (int ks = s_begin; ks < s_end; ++ks) {
              ok = mbar_wait(smem_u32(&bar_empty[stage]), phase, abort_flag, p.status, 201);
              if (!ok) break;
              const uint32_t full_local = smem_u32(&bar_full[stage]);
              const uint32_t sa = stage_base + stage * STAGE_BYTES;
              const uint32_t sb = sa + HALF_ATOMS * ATOM_BYTES;
              if (leader) mbar_expect_tx(full_local, 2 * STAGE_BYTES);   // both CTAs' copies
              const uint32_t full_leader = full_local & PEER_MASK;
#pragma unroll
              for (int a = 0; a < HALF_ATOMS; ++a)
                tma_pair_load_3d(sa + a * ATOM_BYTES, map_a, am + a * 64, ks * BK, pl, full_leader);
#pragma unroll
              for (int b = 0; b < HALF_ATOMS; ++b)
                tma_pair_load_3d(sb + b * ATOM_BYTES, &map_xq, bn + b * 64, ks * BK, 0, full_leader);
              if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
          }
        }
      }
      if (!ok) {
        const unsigned long long t0 = globaltimer_ns();   // let copies in flight land
        while (globaltimer_ns() - t0 < 200000ull) { }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (leader && lane == 0) {
      uint32_t stage = 0, phase = 0, cc = 0;
      bool ok = true;
      for (int item = pair; item < total_items && ok; item += n_pairs) {
        const int planes = (item < p.c_tiles) ? p.c_planes : 1;
        const int chains = n_chunks * planes;
        for (int chain = 0; chain < chains && ok; ++chain, ++cc) {
          const int ch = chain / planes;
          const uint32_t buf = cc & 1u;
          ok = mbar_wait(smem_u32(&bar_acc_empty[buf]), ((cc >> 1) & 1u) ^ 1u, abort_flag, p.status, 202);
          if (!ok) break;
          tc_fence_after();
          const int s_begin = ch * p.chunk_stages;
          const int s_end = min(total_stages, s_begin + p.chunk_stages);
          const uint32_t tmem_d = tmem_base + buf * PAIR_N;
          for (int s = s_begin; s < s_end; ++s) {
            ok = mbar_wait(smem_u32(&bar_full[stage]), phase, abort_flag, p.status, 203);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sa = stage_base + stage * STAGE_BYTES;
            const uint32_t sb = sa + HALF_ATOMS * ATOM_BYTES;
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk)
              umma_pair_f16(tmem_d, make_desc(sa + kk * 2048), make_desc(sb + kk * 2048), p.idesc,
                            (s > s_begin || kk > 0) ? 1u : 0u);
            umma_pair_commit(smem_u32(&bar_empty[stage]));
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (ok) umma_pair_commit(smem_u32(&bar_acc_full[buf]));
        }
      }
    }
    __syncwarp();
  } else {
    const int e = warp - 2;
    const int quarter = warp & 3;       // TMEM lane quarter this warp may read
    const int half = e >> 2;            // columns [half*128, half*128+128)
    uint32_t cc = 0;
    bool ok = true;
    for (int item = pair; item < total_items && ok; item += n_pairs) {
      int is_c, m0, n0;
      decode_item(p, item, is_c, m0, n0);
      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = 0.f;
      const int planes = is_c ? p.c_planes : 1;
      const int chains = n_chunks * planes;
      for (int chain = 0; chain < chains; ++chain, ++cc) {
        const uint32_t buf = cc & 1u;
        ok = mbar_wait(smem_u32(&bar_acc_full[buf]), (cc >> 1) & 1u, abort_flag, p.status, 204);
        if (!ok) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * PAIR_N + half * 128;
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
        if (lane == 0) mbar_arrive_on_leader(smem_u32(&bar_acc_empty[buf]));
      }
      if (!ok) break;
      const int row = m0 + (int)rank * HALF + quarter * 32 + lane;
      if (row < p.d) {
        float* out = (is_c ? p.C : p.H) + (long long)row * p.ldh;
        const int cbase = n0 + half * 128;
#pragma unroll
        for (int c4 = 0; c4 < 32; ++c4) {
          const int col = cbase + c4 * 4;
          if (col < p.d) {  // d is a multiple of 8: a float4 is inside or outside as a whole
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
  cluster_sync_all();          // nothing of the peer is in flight towards this CTA any more
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, 512;" ::"r"(tmem_base) : "memory");
  }
}

}  // namespace

// Launches the pair kernel; returns OC_ERR_UNSUPPORTED-like non-zero (without setting an error)
// when pairs cannot be scheduled on this device, so that the caller can fall back.
int oc_moment_pair_launch(const CUtensorMap& map_xq, const CUtensorMap& map_delta, float* H, float* C,
                          long long ldh, int d, long long n_tok, float a_old, float a_new, int chunk_tokens,
                          int sm_count, int bf16, int c_planes, float lo_scale, int* status,
                          cudaStream_t stream) {
  PairParams p{};
  p.H = H; p.C = C; p.ldh = ldh; p.d = d; p.n_tok = n_tok; p.a_old = a_old; p.a_new = a_new;
  if (chunk_tokens <= 0) chunk_tokens = 512;
  p.chunk_stages = max(1, chunk_tokens / BK);
  p.tiles = oc_div_up(d, PAIR_M);
  p.h_tiles = H ? p.tiles * (p.tiles + 1) / 2 : 0;
  p.c_tiles = C ? p.tiles * p.tiles : 0;
  p.c_planes = c_planes;
  p.lo_scale = lo_scale;
  p.idesc = IDESC | (bf16 ? ((1u << 7) | (1u << 10)) : 0u);
  p.status = status;
  OC_OPT_IN_SMEM(moment_pair_kernel, SMEM_DYN);
  if (sm_count <= 0) sm_count = 148;
  const int pairs = min(sm_count / 2, p.h_tiles + p.c_tiles);
  if (pairs < 1) return OC_OK;
  moment_pair_kernel<<<2 * pairs, NUM_THREADS, SMEM_DYN, stream>>>(map_xq, map_delta, p);
  OC_CHECK_LAUNCH();
  return OC_OK;
}

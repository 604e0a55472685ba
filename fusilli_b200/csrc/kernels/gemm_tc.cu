// Batched 16-bit GEMM on the 5th-generation tensor cores:
//   C[b] = epilogue(A[b] * B[b]),  A,B bf16 or f16, fp32 accumulation in TMEM.
//
// Persistent, warp-specialised, one CTA per SM:
//   warp 0      TMA producer: per 64-wide K block one A tile (128 x 64) and one B
//               tile (64 x 256, or 64 x 128 for a half tile) land in a 4-stage ring of 128B-swizzled shared memory
//               (cp.async.bulk.tensor, no multicast, zero fill past the edges).
//   warp 1      MMA issuer: one thread issues tcgen05.mma 128x256x16 (cta_group::1),
//               four per K block, accumulating into one of two 256-column TMEM
//               buffers; tcgen05.commit releases the stage / publishes the tile.
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator (one row per thread),
//               apply the fused pointwise chain (rounding at each declared dtype),
//               convert and store 64-byte runs. Overlaps the next tile's main loop
//               through the second TMEM buffer.
// Operands may be K-major or MN-major (row-major B is MN-major): the layout goes into
// the shared-memory and instruction descriptors, no transposition pass.
// Every mbarrier wait is bounded; on expiry the kernel records an error word and
// drains instead of spinning.
#include <algorithm>
#include <array>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "../common.h"
#include "sm100.cuh"
#include "tc_epilogue.cuh"

namespace fb {

using namespace sm100;

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int NUM_THREADS = 224; // TMA warp, MMA warp, 4 epilogue warps, second TMA warp
constexpr int PRODUCERS = 2;
constexpr int TMEM_COLS = 512;

struct GemmTcParams {
  int32_t M, N, K, batches;
  int32_t a_mn_major, b_mn_major;
  int32_t a_batches, b_batches; // distinct matrices of each operand: batch b reads matrix b % count
  int32_t ab_format;
  int32_t tiles_m, tiles_n, total_tiles;
  // Work items: tiles [0, full_tiles) whole, the rest as two 128-column halves each. The host
  // splits the tiles of a last, less than half full wave, which then takes half a tile's time.
  int32_t full_tiles, total_work;
  void *out;
  int64_t ldc, c_bstride;
  uint32_t *err;
  TcEpilogue epi;
};

struct WorkItem {
  int m0, n0, b, nb; // output origin, batch, columns of this item (BN or BN / 2)
};
__device__ __forceinline__ WorkItem decode_work(const GemmTcParams &p, int w) {
  int tile = w, n_off = 0, nb = BN;
  if (w >= p.full_tiles) {
    const int r = w - p.full_tiles;
    tile = p.full_tiles + (r >> 1);
    n_off = (r & 1) * (BN / 2);
    nb = BN / 2;
  }
  WorkItem it;
  it.m0 = (tile % p.tiles_m) * BM;
  it.n0 = ((tile / p.tiles_m) % p.tiles_n) * BN + n_off;
  it.b = tile / (p.tiles_m * p.tiles_n);
  it.nb = nb;
  return it;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GemmTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  pdl_launch_dependents(); // the next kernel's CTAs may take the SMs this kernel's CTAs leave
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait(); // nothing before this line touches global memory; the kernels before this one are complete after it
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  const int kblocks = (p.K + BK - 1) / BK;

  if (warp == 0 || warp == 6) {
    // Two producer warps take alternate K blocks: waits, expect and the TMA issues of one block
    // are a serial chain of long-latency instructions in the issuing thread.
    const uint32_t pid = warp == 0 ? 0u : 1u;
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x) {
        const WorkItem wi = decode_work(p, w);
        const int m0 = wi.m0, n0 = wi.n0, nb = wi.nb;
        const int ba = wi.b % p.a_batches, bb = wi.b % p.b_batches;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          if ((it % PRODUCERS) != pid) continue;
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(empty_bar(s), ph ^ 1, p.err, ERR_WAIT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(full_bar(s), A_BYTES + nb * BK * 2);
          const uint32_t sa = smem_base + s * STAGE_BYTES, sb = sa + A_BYTES;
          const int k0 = kb * BK;
          if (!p.a_mn_major) {
            tma_load_3d(sa, &tmap_a, full_bar(s), k0, m0, ba);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i)
              tma_load_3d(sa + i * (64 * BK * 2), &tmap_a, full_bar(s), m0 + 64 * i, k0, ba);
          }
          if (!p.b_mn_major) {
            // boxes of BN / 2 rows: one per half
#pragma unroll
            for (int i = 0; i < 2; ++i)
              if (i * (BN / 2) < nb)
                tma_load_3d(sb + i * ((BN / 2) * BK * 2), &tmap_b, full_bar(s), k0, n0 + (BN / 2) * i, bb);
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              if (i * 64 < nb)
                tma_load_3d(sb + i * (64 * BK * 2), &tmap_b, full_bar(s), n0 + 64 * i, k0, bb);
          }
        }
      }
    }
  } else if (warp == 1) {
    // The whole warp runs the loop (addresses and descriptors stay in uniform registers); one
    // elected lane issues the MMAs and the commits, which track the issuing thread.
    const bool leader = elect_one();
    const uint32_t idesc_full = make_idesc_f16(BM, BN, p.ab_format, p.a_mn_major, p.b_mn_major);
    const uint32_t idesc_half = make_idesc_f16(BM, BN / 2, p.ab_format, p.a_mn_major, p.b_mn_major);
    // K-major: rows of 128 B, 8-row groups 1024 B apart; a 16-element K step is 32 B.
    // MN-major: 64-element MN blocks 8 KB apart (LBO), 8-row K groups 1024 B apart;
    // a 16-element K step is two K groups = 2048 B.
    const uint32_t a_lbo = p.a_mn_major ? 64 * BK * 2 : 16, a_kstep = p.a_mn_major ? 2048 : 32;
    const uint32_t b_lbo = p.b_mn_major ? 64 * BK * 2 : 16, b_kstep = p.b_mn_major ? 2048 : 32;
    // descriptors of stage 0, K step 0; stages and K steps add to the 16-byte-unit address field
    const uint64_t a_desc0 = make_smem_desc(smem_base, a_lbo, 1024);
    const uint64_t b_desc0 = make_smem_desc(smem_base + A_BYTES, b_lbo, 1024);
    uint32_t it = 0, lt = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x, ++lt) {
      const uint32_t idesc = w < p.full_tiles ? idesc_full : idesc_half;
      const int acc = lt & 1;
      const uint32_t aph = (lt >> 1) & 1;
      if (!mbar_wait(tempty_bar(acc), aph ^ 1, p.err, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int kb = 0; kb < kblocks; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(full_bar(s), ph, p.err, ERR_WAIT_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint64_t soff = (uint64_t)((s * STAGE_BYTES) >> 4);
        if (leader) {
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            tc_mma_f16(d_tmem, a_desc0 + soff + (uint64_t)((k * a_kstep) >> 4),
                       b_desc0 + soff + (uint64_t)((k * b_kstep) >> 4), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          tc_commit(empty_bar(s)); // stage reusable once these MMAs have read it
        }
      }
      if (ok && leader) tc_commit(tfull_bar(acc)); // accumulator complete
    }
  } else {
    const int q = warp & 3; // TMEM lane quadrant this warp may access
    uint32_t lt = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x, ++lt) {
      const WorkItem wi = decode_work(p, w);
      const int b = wi.b, chunks = wi.nb / 32;
      const int acc = lt & 1;
      const uint32_t aph = (lt >> 1) & 1;
      if (!mbar_wait(tfull_bar(acc), aph, p.err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int m = wi.m0 + q * 32 + lane;
      const int n0 = wi.n0;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
      const int64_t row_off = (int64_t)b * p.c_bstride + (int64_t)m * p.ldc;
#pragma unroll 1
      for (int c = 0; c < chunks; ++c) {
        uint32_t raw[32];
        tmem_ld_32x32(taddr + c * 32, raw);
        tmem_ld_wait();
        if (c == chunks - 1) {
          // all of this warp's reads of the accumulator are done: hand it back
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_bar(acc));
        }
        const int nc = n0 + c * 32;
        if (m < p.M && nc < p.N) {
          const int valid = min(32, p.N - nc);
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
          epi_run32(p.epi, v, row_off, nc, valid);
          epi_store32(p.out, p.epi.out_dtype, row_off + nc, v, valid);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---- paired-CTA variant -----------------------------------------------------------------
// The same GEMM on CTA pairs (clusters of two, tcgen05 cta_group::2): one 256 x 256 output tile per
// pair, each CTA holding its own 128 rows of A and its own 128 of the 256 B columns. Per CTA and K
// block that is 32 KB fetched from L2 instead of the 48 KB of the 128 x 256 single-CTA tile -- L2
// to shared-memory traffic is what paces the single-CTA kernel -- and the ring has six stages.
// Every CTA loads its own operands with ordinary (not multicast) TMA; completions are counted on
// the leader's barrier, MMA completion is committed to both CTAs' barriers, the peer's epilogue
// warps release the accumulator on the leader's barrier.
namespace pair {
constexpr int TM = 256, STAGES = 6;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = (BN / 2) * BK * 2; // per CTA
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
} // namespace pair

__device__ __forceinline__ WorkItem decode_work_pair(const GemmTcParams &p, int w) {
  int tile = w, n_off = 0, nb = BN;
  if (w >= p.full_tiles) {
    const int r = w - p.full_tiles;
    tile = p.full_tiles + (r >> 1);
    n_off = (r & 1) * (BN / 2);
    nb = BN / 2;
  }
  WorkItem it;
  it.m0 = (tile % p.tiles_m) * pair::TM;
  it.n0 = ((tile / p.tiles_m) % p.tiles_n) * BN + n_off;
  it.b = tile / (p.tiles_m * p.tiles_n);
  it.nb = nb;
  return it;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_pair_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const GemmTcParams p) {
  using namespace pair;
  extern __shared__ uint8_t smem_raw[];
  pdl_launch_dependents(); // the next kernel's CTAs may take the SMs this kernel's CTAs leave
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u; // the same offset in both CTAs
  const uint32_t bar_base = smem_base + pair::STAGES * pair::STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (pair::STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * pair::STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * pair::STAGES + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * pair::STAGES + 4);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank(); // 0 = leader
  const int cluster_id = blockIdx.x >> 1, nclusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < pair::STAGES; ++s) {
      mbar_init(full_bar(s), 1);  // leader's: one expect_tx arrival, bytes of both CTAs
      mbar_init(empty_bar(s), 1); // each CTA's own: committed to by the leader's MMA thread
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8); // leader's: four epilogue warps of each CTA
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS); // one warp of each CTA of the pair, collectively
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all(); // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  pdl_wait(); // nothing before this line touches global memory; the kernels before this one are complete after it
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  const int kblocks = (p.K + BK - 1) / BK;

  if (warp == 0 || warp == 6) {
    const uint32_t pid = warp == 0 ? 0u : 1u;
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int w = cluster_id; w < p.total_work && ok; w += nclusters) {
        const WorkItem wi = decode_work_pair(p, w);
        const int m0 = wi.m0 + (int)rank * BM, nh = wi.nb / 2, n0 = wi.n0 + (int)rank * nh;
        const int ba = wi.b % p.a_batches, bb = wi.b % p.b_batches;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          if ((it % PRODUCERS) != pid) continue;
          const int s = it % pair::STAGES;
          const uint32_t ph = (it / pair::STAGES) & 1;
          if (!mbar_wait(empty_bar(s), ph ^ 1, p.err, ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t lead_full = map_to_cta(full_bar(s), 0);
          if (rank == 0) mbar_expect_tx(full_bar(s), 2u * (uint32_t)(pair::A_BYTES + nh * BK * 2));
          const uint32_t sa = smem_base + s * pair::STAGE_BYTES, sb = sa + pair::A_BYTES;
          const int k0 = kb * BK;
          if (!p.a_mn_major) {
            tma_load_3d_pair(sa, &tmap_a, lead_full, k0, m0, ba);
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i)
              tma_load_3d_pair(sa + i * (64 * BK * 2), &tmap_a, lead_full, m0 + 64 * i, k0, ba);
          }
          // this CTA's half of the B columns, in boxes of 64
#pragma unroll
          for (int i = 0; i < BN / 128; ++i)
            if (i * 64 < nh) {
              if (!p.b_mn_major) tma_load_3d_pair(sb + i * (64 * BK * 2), &tmap_b, lead_full, k0, n0 + 64 * i, bb);
              else tma_load_3d_pair(sb + i * (64 * BK * 2), &tmap_b, lead_full, n0 + 64 * i, k0, bb);
            }
        }
      }
    }
  } else if (warp == 1) {
    if (rank == 0) {
      const bool leader = elect_one();
      const uint32_t idesc_full = make_idesc_f16(pair::TM, BN, p.ab_format, p.a_mn_major, p.b_mn_major);
      const uint32_t idesc_half = make_idesc_f16(pair::TM, BN / 2, p.ab_format, p.a_mn_major, p.b_mn_major);
      const uint32_t a_lbo = p.a_mn_major ? 64 * BK * 2 : 16, a_kstep = p.a_mn_major ? 2048 : 32;
      const uint32_t b_lbo = p.b_mn_major ? 64 * BK * 2 : 16, b_kstep = p.b_mn_major ? 2048 : 32;
      const uint64_t a_desc0 = make_smem_desc(smem_base, a_lbo, 1024);
      const uint64_t b_desc0 = make_smem_desc(smem_base + pair::A_BYTES, b_lbo, 1024);
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int w = cluster_id; w < p.total_work && ok; w += nclusters, ++lt) {
        const uint32_t idesc = w < p.full_tiles ? idesc_full : idesc_half;
        const int acc = lt & 1;
        const uint32_t aph = (lt >> 1) & 1;
        if (!mbar_wait(tempty_bar(acc), aph ^ 1, p.err, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % pair::STAGES;
          const uint32_t ph = (it / pair::STAGES) & 1;
          if (!mbar_wait(full_bar(s), ph, p.err, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint64_t soff = (uint64_t)((s * pair::STAGE_BYTES) >> 4);
          if (leader) {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              tc_mma_f16_pair(d_tmem, a_desc0 + soff + (uint64_t)((k * a_kstep) >> 4),
                              b_desc0 + soff + (uint64_t)((k * b_kstep) >> 4), idesc, (kb > 0 || k > 0) ? 1u : 0u);
            // the stage is free in BOTH CTAs once these MMAs have read it
            tc_commit_pair(map_to_cta(empty_bar(s), 0));
            tc_commit_pair(map_to_cta(empty_bar(s), 1));
          }
        }
        if (ok && leader) { // accumulator complete, in both CTAs' TMEM
          tc_commit_pair(map_to_cta(tfull_bar(acc), 0));
          tc_commit_pair(map_to_cta(tfull_bar(acc), 1));
        }
      }
    }
  } else {
    const int q = warp & 3;
    uint32_t lt = 0;
    bool ok = true;
    for (int w = cluster_id; w < p.total_work && ok; w += nclusters, ++lt) {
      const WorkItem wi = decode_work_pair(p, w);
      const int b = wi.b, chunks = wi.nb / 32;
      const int acc = lt & 1;
      const uint32_t aph = (lt >> 1) & 1;
      if (!mbar_wait(tfull_bar(acc), aph, p.err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int m = wi.m0 + (int)rank * BM + q * 32 + lane;
      const int n0 = wi.n0;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
      const int64_t row_off = (int64_t)b * p.c_bstride + (int64_t)m * p.ldc;
      const uint32_t lead_tempty = map_to_cta(tempty_bar(acc), 0);
#pragma unroll 1
      for (int c = 0; c < chunks; ++c) {
        uint32_t raw[32];
        tmem_ld_32x32(taddr + c * 32, raw);
        tmem_ld_wait();
        if (c == chunks - 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(lead_tempty);
        }
        const int nc = n0 + c * 32;
        if (m < p.M && nc < p.N) {
          const int valid = min(32, p.N - nc);
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
          epi_run32(p.epi, v, row_off, nc, valid);
          epi_store32(p.out, p.epi.out_dtype, row_off + nc, v, valid);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all(); // neither CTA leaves while the other may still signal its barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

} // namespace

// ---- host ------------------------------------------------------------------------

namespace sm100 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    else
      cudaGetLastError();
  });
  return fn;
}

// FUSILLI_B200_NO_LAUNCH_CACHE=1 re-encodes every tensor map and sets the shared-memory attribute on
// every launch, as the first version of this library did: the switch exists to measure what the
// caches below save on the host.
static bool launch_cache_enabled() {
  static const bool on = [] {
    const char *e = getenv("FUSILLI_B200_NO_LAUNCH_CACHE");
    return !(e && e[0] == '1');
  }();
  return on;
}

static bool encode_tmap_2byte_now(CUtensorMap *map, const void *base, int rank, const uint64_t *dims,
                                  const uint64_t *strides_bytes, const uint32_t *box, const char **why) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) {
    *why = "cuTensorMapEncodeTiled entry point not available";
    return false;
  }
  cuuint64_t gdims[5], gstr[4];
  cuuint32_t gbox[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, (cuuint32_t)rank, const_cast<void *>(base), gdims, gstr,
                  gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    *why = "cuTensorMapEncodeTiled rejected the tensor map";
    return false;
  }
  return true;
}

// A tensor map is a pure function of (base address, dims, strides, box): a plan executed again on
// the same buffers finds its maps here instead of going through the driver on every launch.
namespace {
struct TmapKey {
  const void *base;
  int32_t rank;
  uint64_t dims[5], strides[4];
  uint32_t box[5];
  bool operator==(const TmapKey &o) const { return memcmp(this, &o, sizeof(TmapKey)) == 0; }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey &k) const {
    uint64_t h = 1469598103934665603ull;
    const unsigned char *p = reinterpret_cast<const unsigned char *>(&k);
    for (size_t i = 0; i < sizeof(TmapKey); ++i) h = (h ^ p[i]) * 1099511628211ull;
    return (size_t)h;
  }
};
std::mutex g_tmap_mutex;
std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmap_cache;
constexpr size_t kTmapCacheMax = 4096;
} // namespace

bool encode_tmap_2byte(CUtensorMap *map, const void *base, int rank, const uint64_t *dims,
                       const uint64_t *strides_bytes, const uint32_t *box, const char **why) {
  if (!launch_cache_enabled()) return encode_tmap_2byte_now(map, base, rank, dims, strides_bytes, box, why);
  TmapKey key;
  memset(&key, 0, sizeof(key)); // padding and unused slots compare equal
  key.base = base;
  key.rank = rank;
  for (int i = 0; i < rank; ++i) {
    key.dims[i] = dims[i];
    key.box[i] = box[i];
  }
  for (int i = 0; i + 1 < rank; ++i) key.strides[i] = strides_bytes[i];
  std::lock_guard<std::mutex> lock(g_tmap_mutex);
  auto it = g_tmap_cache.find(key);
  if (it != g_tmap_cache.end()) {
    *map = it->second;
    return true;
  }
  if (!encode_tmap_2byte_now(map, base, rank, dims, strides_bytes, box, why)) return false;
  if (g_tmap_cache.size() >= kTmapCacheMax) g_tmap_cache.clear();
  g_tmap_cache.emplace(key, *map);
  return true;
}

// cudaFuncAttributeMaxDynamicSharedMemorySize is per function and device: set once, not per launch.
bool pdl_enabled() {
  static const bool on = [] {
    const char *e = getenv("FUSILLI_B200_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

cudaError_t set_max_dynamic_smem(const void *func, int bytes, int device) {
  if (!launch_cache_enabled()) return cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  static std::mutex mu;
  static std::unordered_map<const void *, std::array<int, 64>> set_bytes; // function -> bytes set per device
  std::lock_guard<std::mutex> lock(mu);
  auto it = set_bytes.find(func);
  if (it == set_bytes.end()) it = set_bytes.emplace(func, std::array<int, 64>{}).first;
  const bool tracked = device >= 0 && device < 64;
  if (tracked && it->second[device] >= bytes) return cudaSuccess; // already large enough
  cudaError_t e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess && tracked) it->second[device] = bytes;
  return e;
}

} // namespace sm100

namespace {

struct GemmView {
  int64_t M, N, K, batches;
  int a_mn, b_mn;      // operand is MN-major
  int64_t a_ld, b_ld;  // leading (slow) stride in elements
  int64_t a_bs, b_bs;  // batch strides (0 = broadcast)
  int64_t a_nb, b_nb;  // distinct matrices of A and B (1 = broadcast; a divisor of `batches` otherwise)
  int64_t ldc, c_bs;
};

bool is16(int dt) { return dt == FB_DT_HALF || dt == FB_DT_BFLOAT16; }
bool isfl(int dt) { return dt == FB_DT_HALF || dt == FB_DT_BFLOAT16 || dt == FB_DT_FLOAT; }

// Collapses the batch dims of `t` into (count, stride): `count` distinct matrices `stride` elements
// apart, batch b of the result reading matrix b % count. False if the batch dims are not a dense
// run, a pure broadcast, or (single batch dim only) a proper divisor of the result's batch
// (reference matmul_node.h:140-150 accepts dims that divide one another).
bool batch_collapse(const TensorInfo &t, const TensorInfo &full, int64_t &stride, int64_t &count) {
  int nb = t.rank - 2;
  bool all_one = true;
  count = 1;
  for (int i = 0; i < nb; ++i) {
    if (t.dims[i] != 1) all_one = false;
    count *= t.dims[i];
  }
  if (all_one) {
    stride = 0;
    return true;
  }
  if (nb == 1 && t.dims[0] != full.dims[0]) {
    if (full.dims[0] % t.dims[0] != 0) return false;
    stride = t.strides[0];
    return true;
  }
  for (int i = 0; i < nb; ++i)
    if (t.dims[i] != full.dims[i]) return false; // partial broadcast over several batch dims
  int64_t expect = -1;
  for (int i = nb - 1; i >= 0; --i) {
    if (t.dims[i] == 1) continue;
    if (expect < 0) {
      stride = t.strides[i];
      expect = t.strides[i] * t.dims[i];
    } else {
      if (t.strides[i] != expect) return false;
      expect *= t.dims[i];
    }
  }
  return true;
}

bool gemm_view(const Plan &p, const Step &s, GemmView &g) {
  const fb_node_desc &d = p.nodes[s.node].d;
  const TensorInfo &a = p.tensors[d.inputs[0]], &b = p.tensors[d.inputs[1]];
  const TensorInfo &c0 = p.tensors[d.outputs[0]], &c = p.tensors[s.out_tensor];
  if (!is16(a.dtype) || a.dtype != b.dtype || !isfl(c.dtype) || !isfl(c0.dtype)) return false;
  int r = a.rank;
  g.M = a.dims[r - 2]; g.K = a.dims[r - 1]; g.N = b.dims[r - 1];
  g.batches = 1;
  for (int i = 0; i < r - 2; ++i) g.batches *= c.dims[i];
  // A[m][k]
  if (a.strides[r - 1] == 1 && (g.M == 1 || a.strides[r - 2] >= g.K)) { g.a_mn = 0; g.a_ld = a.strides[r - 2]; }
  else if (a.strides[r - 2] == 1 && a.strides[r - 1] >= g.M) { g.a_mn = 1; g.a_ld = a.strides[r - 1]; }
  else return false;
  // B[k][n]
  if (b.strides[r - 2] == 1 && (g.N == 1 || b.strides[r - 1] >= g.K)) { g.b_mn = 0; g.b_ld = b.strides[r - 1]; }
  else if (b.strides[r - 1] == 1 && b.strides[r - 2] >= g.N) { g.b_mn = 1; g.b_ld = b.strides[r - 2]; }
  else return false;
  if (c.strides[r - 1] != 1) return false;
  g.ldc = c.strides[r - 2];
  int64_t c_nb = 1;
  if (!batch_collapse(a, c, g.a_bs, g.a_nb) || !batch_collapse(b, c, g.b_bs, g.b_nb) ||
      !batch_collapse(c, c, g.c_bs, c_nb))
    return false;
  if (g.batches == 1) g.a_bs = g.b_bs = g.c_bs = 0;
  if (!g.a_bs) g.a_nb = 1;
  if (!g.b_bs) g.b_nb = 1;
  // TMA: 16-byte aligned strides
  if (g.a_ld % 8 || g.b_ld % 8 || g.a_bs % 8 || g.b_bs % 8) return false;
  if (g.M >= (1ll << 31) || g.N >= (1ll << 31) || g.K >= (1ll << 31) || g.batches >= 65536) return false;
  return true;
}

// Epilogue operands the tensor-core epilogue can address.
int epi_kind(const Plan &p, const Step &s, const EpilogueOpInfo &op) {
  if (op.operand < 0) return 0;
  const TensorInfo &o = p.tensors[op.operand];
  const TensorInfo &c = p.tensors[s.out_tensor];
  if (o.role == FB_TENSOR_SCALAR) return 2;
  bool vec = o.dims[o.rank - 1] == c.dims[c.rank - 1] && o.strides[o.rank - 1] == 1;
  for (int i = 0; i + 1 < o.rank; ++i)
    if (o.dims[i] != 1) vec = false;
  if (vec) return 1;
  bool full = o.rank == c.rank;
  for (int i = 0; full && i < c.rank; ++i)
    if (o.dims[i] != c.dims[i] || (c.dims[i] > 1 && o.strides[i] != c.strides[i])) full = false;
  if (full) return 3;
  return -1;
}

} // namespace

bool gemm_tc_eligible(const Plan &p, const Step &s) {
  GemmView g;
  if (!gemm_view(p, s, g)) return false;
  // tiny problems stay on the CUDA-core kernel: a 128x256 tile would be mostly padding
  if (g.M < 64 || g.N < 64 || g.K < 32) return false;
  for (int i = 0; i < s.num_epilogue; ++i) {
    if (epi_kind(p, s, s.epilogue[i]) < 0) return false;
    if (!isfl(p.tensors[s.epilogue[i].out_tensor].dtype)) return false;
    if (s.epilogue[i].operand >= 0 && !isfl(p.tensors[s.epilogue[i].operand].dtype)) return false;
  }
  return true;
}

// Whether clusters of two CTAs of the pair kernel can be resident on this device (asked once per
// device), and whether the caller left the pair kernel enabled.
static bool pair_kernel_usable(int device) {
  static const bool enabled = [] {
    const char *e = getenv("FUSILLI_B200_GEMM_PAIR");
    return !(e && e[0] == '0');
  }();
  if (!enabled || device < 0 || device >= 64) return false;
  static std::mutex mu;
  static int8_t state[64] = {0}; // 0 unknown, 1 usable, -1 not
  std::lock_guard<std::mutex> lock(mu);
  if (state[device] == 0) {
    state[device] = -1;
    if (sm100::set_max_dynamic_smem(reinterpret_cast<const void *>(gemm_pair_tcgen05_kernel), pair::SMEM_BYTES,
                                    device) == cudaSuccess) {
      cudaLaunchConfig_t cfg;
      memset(&cfg, 0, sizeof(cfg));
      cfg.gridDim = dim3(2, 1, 1);
      cfg.blockDim = dim3(NUM_THREADS, 1, 1);
      cfg.dynamicSmemBytes = pair::SMEM_BYTES;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 2;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, reinterpret_cast<const void *>(gemm_pair_tcgen05_kernel), &cfg) ==
              cudaSuccess &&
          n >= 1)
        state[device] = 1;
    }
    (void)cudaGetLastError();
  }
  return state[device] == 1;
}

fb_status launch_gemm_tc(const ExecContext &cx, const Step &s) {
  const Plan &plan = *cx.plan;
  const fb_node_desc &d = plan.nodes[s.node].d;
  GemmView g;
  FB_REQUIRE(gemm_view(plan, s, g), FB_INTERNAL_ERROR, "gemm_tcgen05: step is not eligible");
  const TensorInfo &a = plan.tensors[d.inputs[0]];
  const void *aptr = cx.tensor_ptr(d.inputs[0]);
  const void *bptr = cx.tensor_ptr(d.inputs[1]);
  void *cptr = cx.tensor_ptr(s.out_tensor);
  FB_REQUIRE(aptr && bptr && cptr, FB_INTERNAL_ERROR, "gemm_tcgen05: tensor has no buffer");
  FB_REQUIRE(((uintptr_t)aptr % 16 == 0) && ((uintptr_t)bptr % 16 == 0), FB_INVALID_ARGUMENT,
             "gemm_tcgen05: operand buffers must be 16-byte aligned");

  static thread_local GemmTcParams p;
  memset(&p, 0, sizeof(p));
  p.M = (int)g.M; p.N = (int)g.N; p.K = (int)g.K; p.batches = (int)g.batches;
  p.a_mn_major = g.a_mn; p.b_mn_major = g.b_mn;
  p.a_batches = (int)g.a_nb;
  p.b_batches = (int)g.b_nb;
  p.ab_format = a.dtype == FB_DT_BFLOAT16 ? 1 : 0;
  // CTA pairs (256 x 256 tiles) when the problem has at least one full pair tile of rows and the
  // device can run clusters of two; FUSILLI_B200_GEMM_PAIR=0 keeps the single-CTA kernel.
  const bool use_pair = g.M >= pair::TM && g.N >= BN / 2 && pair_kernel_usable(cx.dev->ordinal);
  const int tile_m = use_pair ? pair::TM : BM;
  p.tiles_m = (p.M + tile_m - 1) / tile_m;
  p.tiles_n = (p.N + BN - 1) / BN;
  int64_t total = (int64_t)p.tiles_m * p.tiles_n * p.batches;
  FB_REQUIRE(total < (1ll << 31), FB_NOT_IMPLEMENTED, "gemm_tcgen05: too many tiles");
  p.total_tiles = (int)total;
  {
    // A last wave that fills at most half of the SMs (or SM pairs) runs as half tiles on twice as many.
    const int sms = use_pair ? cx.dev->sm_count / 2 : cx.dev->sm_count;
    const int tail = p.total_tiles % sms;
    const bool split = tail > 0 && 2 * tail <= sms && p.N > BN / 2;
    p.full_tiles = split ? p.total_tiles - tail : p.total_tiles;
    p.total_work = p.full_tiles + 2 * (p.total_tiles - p.full_tiles);
  }
  p.out = cptr;
  p.ldc = g.ldc;
  p.c_bstride = g.c_bs;
  p.err = cx.dev->error_word;
  p.epi.num_ops = s.num_epilogue;
  p.epi.acc_round_dtype = plan.tensors[d.outputs[0]].dtype;
  p.epi.out_dtype = plan.tensors[s.out_tensor].dtype;
  for (int i = 0; i < s.num_epilogue; ++i) {
    const EpilogueOpInfo &src = s.epilogue[i];
    TcEpiOp &op = p.epi.ops[i];
    op.mode = src.mode;
    op.kind = epi_kind(plan, s, src);
    op.value_is_in1 = src.value_is_in1;
    op.round_dtype = plan.tensors[src.out_tensor].dtype;
    memcpy(op.prm, src.fparams, sizeof(op.prm));
    if (src.operand >= 0) {
      const TensorInfo &o = plan.tensors[src.operand];
      op.dtype = o.dtype;
      if (op.kind == 2) op.scalar = (float)o.scalar;
      else {
        op.ptr = cx.tensor_ptr(src.operand);
        FB_REQUIRE(op.ptr != nullptr, FB_INTERNAL_ERROR, "gemm_tcgen05: epilogue operand has no buffer");
      }
    }
  }

  CUtensorMap tmA, tmB;
  const char *why = "";
  {
    // innermost-first dims; a broadcast operand gets a batch extent of 1
    uint64_t ab = (uint64_t)g.a_nb, bb = (uint64_t)g.b_nb;
    uint64_t a_bstride = g.a_bs ? (uint64_t)g.a_bs * 2 : (uint64_t)g.a_ld * 2 * (g.a_mn ? g.K : g.M);
    uint64_t b_bstride = g.b_bs ? (uint64_t)g.b_bs * 2 : (uint64_t)g.b_ld * 2 * (g.b_mn ? g.K : g.N);
    if (!g.a_mn) {
      uint64_t dims[3] = {(uint64_t)g.K, (uint64_t)g.M, ab}, str[2] = {(uint64_t)g.a_ld * 2, a_bstride};
      uint32_t box[3] = {BK, BM, 1};
      FB_REQUIRE(encode_tmap_2byte(&tmA, aptr, 3, dims, str, box, &why), FB_RUNTIME_FAILURE, why);
    } else {
      uint64_t dims[3] = {(uint64_t)g.M, (uint64_t)g.K, ab}, str[2] = {(uint64_t)g.a_ld * 2, a_bstride};
      uint32_t box[3] = {64, BK, 1};
      FB_REQUIRE(encode_tmap_2byte(&tmA, aptr, 3, dims, str, box, &why), FB_RUNTIME_FAILURE, why);
    }
    if (!g.b_mn) {
      uint64_t dims[3] = {(uint64_t)g.K, (uint64_t)g.N, bb}, str[2] = {(uint64_t)g.b_ld * 2, b_bstride};
      uint32_t box[3] = {BK, use_pair ? 64u : (uint32_t)(BN / 2), 1}; // the pair kernel loads 64-row boxes
      FB_REQUIRE(encode_tmap_2byte(&tmB, bptr, 3, dims, str, box, &why), FB_RUNTIME_FAILURE, why);
    } else {
      uint64_t dims[3] = {(uint64_t)g.N, (uint64_t)g.K, bb}, str[2] = {(uint64_t)g.b_ld * 2, b_bstride};
      uint32_t box[3] = {64, BK, 1};
      FB_REQUIRE(encode_tmap_2byte(&tmB, bptr, 3, dims, str, box, &why), FB_RUNTIME_FAILURE, why);
    }
  }
  if (use_pair) {
    cudaError_t pe = set_max_dynamic_smem(reinterpret_cast<const void *>(gemm_pair_tcgen05_kernel), pair::SMEM_BYTES,
                                          cx.dev->ordinal);
    FB_REQUIRE(pe == cudaSuccess, FB_RUNTIME_FAILURE,
               std::string("gemm_pair_tcgen05: cannot reserve shared memory: ") + cudaGetErrorString(pe));
    const int clusters = std::min<int>(p.total_work, cx.dev->sm_count / 2);
    FB_CUDA_OK(launch_pdl(gemm_pair_tcgen05_kernel, dim3(2 * clusters), dim3(NUM_THREADS), pair::SMEM_BYTES, cx.dev->stream, tmA,
                          tmB, p));
    return FB_OK;
  }
  cudaError_t attr_err =
      set_max_dynamic_smem(reinterpret_cast<const void *>(gemm_tcgen05_kernel), SMEM_BYTES, cx.dev->ordinal);
  FB_REQUIRE(attr_err == cudaSuccess, FB_RUNTIME_FAILURE,
             std::string("gemm_tcgen05: cannot reserve shared memory: ") + cudaGetErrorString(attr_err));
  int grid = std::min<int>(p.total_work, cx.dev->sm_count);
  FB_CUDA_OK(launch_pdl(gemm_tcgen05_kernel, dim3(grid), dim3(NUM_THREADS), SMEM_BYTES, cx.dev->stream, tmA, tmB, p));
  return FB_OK;
}

} // namespace fb

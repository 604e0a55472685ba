// Flash-style scaled-dot-product attention forward on the tensor cores:
//   O = softmax(Q K^T * scale [causal]) V,  Q/K/V/O contiguous [B,H,S,128], bf16 or f16.
//
// Persistent CTAs, one per SM, each working through (256-query block, batch*head) items: two
// 128-query tiles that take turns on the tensor pipe, so the softmax of one tile runs under the MMAs
// of the other. Under a causal mask a CTA takes the query blocks of a head in pairs, the k-th heaviest
// and then the k-th lightest, so every pair costs the same and a static round-robin over the pairs is
// balanced; neighbouring CTAs work on the same head at the same time and share its K/V in L2. Barrier
// phases run on across items, the next item's Q is loaded as soon as the last Q K^T of the current
// one has read it and its first scores are computed while the softmax warps still drain the previous
// output accumulator: TMEM allocation, barrier set-up and the first load latency are paid once per SM
// instead of once per item. Memory stays O(S): K/V
// stream through 2-stage shared-memory rings; scores, probabilities and the output accumulator
// live in TMEM (512 columns: S0 | S1 | O0 | O1, 128 fp32 columns each).
//   warp 0      TMA producer: both Q tiles once, then K_j / V_j tiles (128 keys x 128 dims, two
//               128B-swizzled 64-wide boxes each), separate full/empty barriers for K and V.
//   warp 1      MMA issuer, per key block j and tile t: PV(t,j) then QK(t,j+1).
//               S_t = Q_t K_j^T is tcgen05.mma 128x128x16 x8 with both operands in shared memory;
//               O_t += P_t V_j takes A = P_t from TMEM (16-bit values packed two per column, written
//               by the softmax warps over the first 64 columns of S_t) and B = V_j MN-major.
//   warps 2..9  softmax, four warps per tile, one query row per thread: ONE pass over the 128
//               scores of the row in registers (max, exp2 with scale*log2(e) folded in, row sum,
//               16-bit pack, tcgen05.st). The output accumulator is rescaled in TMEM only when the
//               running maximum has grown by more than 2^8 since the last rescale (decided per
//               warp), so on most blocks the accumulator is never touched by the softmax warps.
// Causal blocks above the diagonal are never loaded or multiplied; the diagonal block and a
// ragged last key block are masked elementwise.
// Every mbarrier wait is bounded.
#include <algorithm>

#include "../common.h"
#include "sm100.cuh"
#include "tc_epilogue.cuh"

namespace fb {

using namespace sm100;

namespace {

constexpr int BQ = 128, BKV = 128, HD = 128, QTILES = 2;
constexpr int TILE_BYTES = 128 * 128 * 2;  // one 128x128 16-bit tile = two 64-wide boxes
constexpr int HALF_BYTES = TILE_BYTES / 2; // one 128-row x 64-col swizzled box
constexpr int SM_Q = 0, SM_K = 2 * TILE_BYTES, SM_V = 4 * TILE_BYTES;
constexpr int SM_BARS = 6 * TILE_BYTES;
constexpr int SMEM_BYTES = 6 * TILE_BYTES + 1024 + 256;
constexpr int NUM_THREADS = 320;
constexpr int TMEM_COLS = 512;
constexpr int TM_S = 0, TM_O = 256; // S_t: cols [128t, 128t+128); O_t: cols [256+128t, ...)
constexpr float RESCALE_LOG2 = 8.f; // the accumulator is rescaled when the row max grew by > 2^8

struct SdpaTcParams {
  int32_t B, Hq, Hk, Sq, Skv;
  int32_t causal, ab_format, out_dtype;
  int32_t q_blocks;
  int32_t pairs_per_head, total_pairs;   // work units: (head, k) -> query blocks q_blocks-1-k and k
  float scale_log2e;
  void *out;
  uint32_t *err;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// packed fp32 pairs: one instruction per pair on sm_100
__device__ __forceinline__ float2 f2_fma(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(*reinterpret_cast<uint64_t *>(&d))
      : "l"(*reinterpret_cast<uint64_t *>(&a)), "l"(*reinterpret_cast<uint64_t *>(&b)),
        "l"(*reinterpret_cast<uint64_t *>(&c)));
  return d;
}
__device__ __forceinline__ float2 f2_add(float2 a, float2 b) {
  float2 d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(*reinterpret_cast<uint64_t *>(&d))
      : "l"(*reinterpret_cast<uint64_t *>(&a)), "l"(*reinterpret_cast<uint64_t *>(&b)));
  return d;
}
// 2^x for a pair on the FMA and integer pipes instead of the special-function unit, which is the
// busiest pipe of the softmax warps: x = j + f with j = round(x) taken from the mantissa of
// x + 1.5 * 2^23, 2^f for f in [-0.5, 0.5] from a cubic (relative error 7.5e-5, far inside the
// 16-bit rounding of P), and j added into the exponent field. x is clamped at -125 so that the
// exponent cannot wrap: masked scores (-inf) come out as 2^-125, which no sum or product sees.
// One pair in eight takes this path: measured on 8 x 32 x 4096 x 128 causal, none 1.089 ms, one in
// eight 1.063 ms, one in four 1.075 ms, one in two 1.174 ms (the extra FMA / integer work then
// costs more than the special-function slots it frees).
#ifndef SDPA_POLY_AND
#define SDPA_POLY_AND 7 // pairs with (i & AND) == EQ take this path
#define SDPA_POLY_EQ 7
#endif
__device__ __forceinline__ float2 ex2_poly(float2 x) {
  x.x = fmaxf(x.x, -125.f);
  x.y = fmaxf(x.y, -125.f);
  const float2 t = f2_add(x, make_float2(12582912.f, 12582912.f));
  const float2 j = f2_add(t, make_float2(-12582912.f, -12582912.f));
  const float2 f = f2_fma(j, make_float2(-1.f, -1.f), x);
  float2 q = f2_fma(f, make_float2(0.0551716685f, 0.0551716685f), make_float2(0.242611125f, 0.242611125f));
  q = f2_fma(q, f, make_float2(0.693260968f, 0.693260968f));
  q = f2_fma(q, f, make_float2(0.999928057f, 0.999928057f));
  float2 r;
  r.x = __int_as_float(__float_as_int(q.x) + (__float_as_int(t.x) << 23));
  r.y = __int_as_float(__float_as_int(q.y) + (__float_as_int(t.y) << 23));
  return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ void tmem_st_32x16(uint32_t addr, const uint32_t *v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
sdpa_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const SdpaTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  pdl_launch_dependents(); // the next kernel's CTAs may take the SMs this kernel's CTAs leave
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + SM_BARS;
  // barrier slots
  const uint32_t q_full = bar_base;
  auto k_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bar_base + 8u * (3 + s); };
  auto v_full = [&](int s) { return bar_base + 8u * (5 + s); };
  auto v_empty = [&](int s) { return bar_base + 8u * (7 + s); };
  auto s_full = [&](int t) { return bar_base + 8u * (9 + t); };
  // P_t is published in two halves (keys 0..63, 64..127) so that P V starts under the second half's exp
  auto p_half = [&](int t, int hf) { return bar_base + 8u * (11 + 2 * t + hf); };
  auto pv_done = [&](int t) { return bar_base + 8u * (15 + t); };
  const uint32_t q_free = bar_base + 8u * 17;                              // Q tiles read by the item's last Q K^T
  auto o_free = [&](int t) { return bar_base + 8u * (18 + t); };          // O_t drained by the softmax warps
  const uint32_t tmem_slot = bar_base + 8u * 20;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  const int nblk_all = (p.Skv + BKV - 1) / BKV;
  // Item n of this CTA: pair u = blockIdx.x + (n / 2) * gridDim.x is (head u / pairs_per_head, k = u %
  // pairs_per_head); its first half is query block q_blocks-1-k, its second half block k (no second
  // half when both are the same block).
  struct Item { bool any, valid; int bh, kvh, q0, nt0, nt1, nmax; };
  auto item_of = [&](int n) {
    Item it;
    const int64_t u = (int64_t)blockIdx.x + (int64_t)(n >> 1) * gridDim.x;
    it.any = u < p.total_pairs;
    it.valid = false; it.bh = it.kvh = it.q0 = it.nt0 = it.nt1 = it.nmax = 0;
    if (!it.any) return it;
    const int bh = (int)(u / p.pairs_per_head), k = (int)(u % p.pairs_per_head);
    const int qb = (n & 1) ? k : p.q_blocks - 1 - k;
    if ((n & 1) && k == p.q_blocks - 1 - k) return it; // the middle block of an odd count: first half only
    it.valid = true;
    it.bh = bh;
    const int b = bh / p.Hq, h = bh % p.Hq;
    it.kvh = b * p.Hk + h / (p.Hq / p.Hk);
    it.q0 = qb * (BQ * QTILES);
    // key blocks each tile needs; a tile that starts beyond Sq does nothing
    auto blocks_of = [&](int t) {
      const int qt = it.q0 + t * BQ;
      return qt >= p.Sq ? 0 : (p.causal ? min(nblk_all, (qt + BQ - 1) / BKV + 1) : nblk_all);
    };
    it.nt0 = blocks_of(0); it.nt1 = blocks_of(1);
    it.nmax = max(it.nt0, it.nt1);
    return it;
  };

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(k_empty(s), 1);
      mbar_init(v_full(s), 1);
      mbar_init(v_empty(s), 1);
      mbar_init(s_full(s), 1);
      mbar_init(p_half(s, 0), 4);
      mbar_init(p_half(s, 1), 4);
      mbar_init(pv_done(s), 1);
      mbar_init(o_free(s), 4);
    }
    mbar_init(q_free, 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
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

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      uint32_t g = 0;     // key blocks loaded so far: ring stage g & 1, phase (g >> 1) & 1
      uint32_t items = 0; // valid items so far: phase of q_full / q_free
      for (int n = 0; ok; ++n) {
        const Item it = item_of(n);
        if (!it.any) break;
        if (!it.valid) continue;
        // the previous item's last Q K^T has read the Q tiles
        if (!mbar_wait(q_free, (items & 1) ^ 1, p.err, ERR_WAIT_EMPTY)) { ok = false; break; }
        mbar_expect_tx(q_full, QTILES * TILE_BYTES);
#pragma unroll
        for (int t = 0; t < QTILES; ++t) {
          tma_load_3d(smem_base + SM_Q + t * TILE_BYTES, &tmap_q, q_full, 0, it.q0 + t * BQ, it.bh);
          tma_load_3d(smem_base + SM_Q + t * TILE_BYTES + HALF_BYTES, &tmap_q, q_full, 64, it.q0 + t * BQ, it.bh);
        }
        ++items;
        for (int j = 0; j < it.nmax && ok; ++j, ++g) {
          const int s = g & 1;
          const uint32_t ph = (g >> 1) & 1;
          if (!mbar_wait(k_empty(s), ph ^ 1, p.err, ERR_WAIT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(k_full(s), TILE_BYTES);
          const uint32_t sk = smem_base + SM_K + s * TILE_BYTES;
          tma_load_3d(sk, &tmap_k, k_full(s), 0, j * BKV, it.kvh);
          tma_load_3d(sk + HALF_BYTES, &tmap_k, k_full(s), 64, j * BKV, it.kvh);
          if (!mbar_wait(v_empty(s), ph ^ 1, p.err, ERR_WAIT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(v_full(s), TILE_BYTES);
          const uint32_t sv = smem_base + SM_V + s * TILE_BYTES;
          tma_load_3d(sv, &tmap_v, v_full(s), 0, j * BKV, it.kvh);
          tma_load_3d(sv + HALF_BYTES, &tmap_v, v_full(s), 64, j * BKV, it.kvh);
        }
      }
    }
  } else if (warp == 1) {
    // The whole warp runs the loop so that addresses and descriptors stay in uniform registers;
    // one elected lane issues the MMAs and the commits (a commit tracks the issuing thread).
    const bool leader = elect_one();
    // scores: A = Q_t (K-major), B = K_j (K-major, N = keys)
    // output: A = P_t (TMEM), B = V_j (MN-major: 64-wide head-dim blocks HALF_BYTES apart,
    //         8-key groups 1024 B apart)
    const uint32_t idesc_qk = make_idesc_f16(BQ, BKV, p.ab_format, 0, 0);
    const uint32_t idesc_pv = make_idesc_f16(BQ, HD, p.ab_format, 0, 1);
    // descriptor of the first K-step of each operand; later K-steps add a constant to the
    // 16-byte-unit address field
    const uint64_t q_desc0 = make_smem_desc(smem_base + SM_Q, 16, 1024);
    const uint64_t k_desc0 = make_smem_desc(smem_base + SM_K, 16, 1024);
    const uint64_t v_desc0 = make_smem_desc(smem_base + SM_V, HALF_BYTES, 1024);
    auto issue_qk = [&](int t, uint32_t stage) {
      const uint64_t qd = q_desc0 + (uint64_t)((t * TILE_BYTES) >> 4);
      const uint64_t kd = k_desc0 + (uint64_t)((stage * TILE_BYTES) >> 4);
      if (leader) {
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t off = (uint64_t)(((k >> 2) * HALF_BYTES + (k & 3) * 32) >> 4);
          tc_mma_f16(tmem_base + TM_S + t * BKV, qd + off, kd + off, idesc_qk, k > 0 ? 1u : 0u);
        }
        tc_commit(s_full(t));
      }
    };
    auto issue_pv = [&](int t, uint32_t stage, int j, int hf) {
      const uint64_t vd = v_desc0 + (uint64_t)((stage * TILE_BYTES) >> 4);
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < BKV / 32; ++kk) {
          const int k = hf * (BKV / 32) + kk;
          tc_mma_f16_ts(tmem_base + TM_O + t * HD, tmem_base + TM_S + t * BKV + k * 8,
                        vd + (uint64_t)((k * 2048) >> 4), idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
        }
        if (hf == 1) tc_commit(pv_done(t));
      }
    };
    bool ok = true;
    uint32_t g = 0, items = 0;        // key blocks / valid items so far
    uint32_t blk[QTILES] = {0, 0};    // key blocks of tile t so far: phase of s_full / p_half / pv_done
    uint32_t drained[QTILES] = {0, 0}; // items of tile t so far: phase of o_free
    for (int n = 0; ok; ++n) {
      const Item it = item_of(n);
      if (!it.any) break;
      if (!it.valid) continue;
      const int nt[QTILES] = {it.nt0, it.nt1};
      if (!mbar_wait(q_full, items & 1, p.err, ERR_WAIT_FULL)) { ok = false; break; }
      ++items;
      if (it.nmax > 0) {
        if (!mbar_wait(k_full(g & 1), (g >> 1) & 1, p.err, ERR_WAIT_FULL)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int t = 0; t < QTILES; ++t)
          if (nt[t] > 0) issue_qk(t, g & 1);
        if (leader) {
          tc_commit(k_empty(g & 1));
          if (it.nmax == 1) tc_commit(q_free); // the only Q K^T of the item
        }
      } else if (leader) {
        tc_commit(q_free);
      }
      for (int j = 0; j < it.nmax && ok; ++j, ++g) {
        const uint32_t s = g & 1;
        const uint32_t ph = (g >> 1) & 1;
        if (!mbar_wait(v_full(s), ph, p.err, ERR_WAIT_FULL)) { ok = false; break; }
        if (j + 1 < it.nmax && !mbar_wait(k_full(s ^ 1), ((g + 1) >> 1) & 1, p.err, ERR_WAIT_FULL)) { ok = false; break; }
#pragma unroll
        for (int t = 0; t < QTILES; ++t) {
          if (j < nt[t]) {
            // the item's first P V overwrites O_t: the previous item's output has been drained
            if (j == 0 && !mbar_wait(o_free(t), (drained[t] & 1) ^ 1, p.err, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
            if (!mbar_wait(p_half(t, 0), blk[t] & 1, p.err, ERR_WAIT_OTHER)) { ok = false; break; }
            tc_fence_after();
            issue_pv(t, s, j, 0);
            if (!mbar_wait(p_half(t, 1), blk[t] & 1, p.err, ERR_WAIT_OTHER)) { ok = false; break; }
            tc_fence_after();
            issue_pv(t, s, j, 1);
            ++blk[t];
          }
          if (j + 1 < nt[t]) issue_qk(t, s ^ 1);
        }
        if (!ok) break;
        if (leader) {
          tc_commit(v_empty(s));
          if (j + 1 < it.nmax) tc_commit(k_empty(s ^ 1));
          if (j + 2 == it.nmax) tc_commit(q_free); // the item's last Q K^T is among the MMAs issued so far
        }
      }
#pragma unroll
      for (int t = 0; t < QTILES; ++t)
        if (nt[t] > 0) ++drained[t];
    }
  } else {
    const int t = (warp - 2) >> 2;     // query tile of this warp
    const int q = warp & 3;            // TMEM lane quarter this warp may access
    const int row = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t s_addr = tmem_base + TM_S + t * BKV + lane_addr;
    const uint32_t o_addr = tmem_base + TM_O + t * HD + lane_addr;
    const float c = p.scale_log2e;
    bool ok = true;
    uint32_t blk = 0; // key blocks of this tile so far: phase of s_full / pv_done
    for (int n = 0; ok; ++n) {
      const Item it = item_of(n);
      if (!it.any) break;
      if (!it.valid) continue;
      const int bh = it.bh;
      const int q0t = it.q0 + t * BQ;
      const int qi = q0t + row;
      const int n_blocks = t ? it.nt1 : it.nt0;
      float m_ref = -INFINITY, l_run = 0.f;
      for (int j = 0; j < n_blocks && ok; ++j, ++blk) {
        if (!mbar_wait(s_full(t), blk & 1, p.err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        const int k0 = j * BKV;
        const bool need_mask = (k0 + BKV > p.Skv) || (p.causal && k0 + BKV - 1 > q0t);
        const int k_lim = p.causal ? min(p.Skv, qi + 1) : p.Skv; // keys >= k_lim are masked for this row
        // the whole score row of this block, one pass
        uint32_t raw[BKV];
  #pragma unroll
        for (int cc = 0; cc < BKV / 32; ++cc) tmem_ld_32x32(s_addr + cc * 32, raw + cc * 32);
        tmem_ld_wait();
        if (need_mask) {
  #pragma unroll
          for (int i = 0; i < BKV; ++i)
            if (k0 + i >= k_lim) raw[i] = 0xff800000u; // -inf
        }
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
  #pragma unroll
        for (int i = 0; i < BKV; i += 8) {
          mx0 = max3(mx0, __uint_as_float(raw[i]), __uint_as_float(raw[i + 1]));
          mx1 = max3(mx1, __uint_as_float(raw[i + 2]), __uint_as_float(raw[i + 3]));
          mx2 = max3(mx2, __uint_as_float(raw[i + 4]), __uint_as_float(raw[i + 5]));
          mx3 = max3(mx3, __uint_as_float(raw[i + 6]), __uint_as_float(raw[i + 7]));
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        // Rescale only when some row of the warp moved its maximum by more than 2^RESCALE_LOG2
        // (always on the first block): until then probabilities are taken against the stale
        // maximum and stay below 2^RESCALE_LOG2, which fp32 sums and 16-bit P hold exactly as well.
        const bool grow = mx > m_ref && ((mx - m_ref) * c > RESCALE_LOG2 || m_ref == -INFINITY);
        if (__any_sync(0xffffffffu, grow)) {
          const float m_new = fmaxf(m_ref, mx);
          const float m_use = (m_new == -INFINITY) ? 0.f : m_new; // a fully masked row so far
          const float alpha = (m_ref == -INFINITY) ? 0.f : ex2_approx((m_ref - m_use) * c);
          if (j > 0) {
            if (!mbar_wait(pv_done(t), (blk - 1) & 1, p.err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
            tc_fence_after();
  #pragma unroll 1
            for (int cc = 0; cc < HD / 32; ++cc) {
              uint32_t acc[32];
              tmem_ld_32x32(o_addr + cc * 32, acc);
              tmem_ld_wait();
  #pragma unroll
              for (int i = 0; i < 32; ++i) acc[i] = __float_as_uint(__uint_as_float(acc[i]) * alpha);
              tmem_st_32x32(o_addr + cc * 32, acc);
            }
          }
          l_run *= alpha;
          m_ref = (m_new == -INFINITY) ? -INFINITY : m_use;
        }
        const float mc = (m_ref == -INFINITY) ? 0.f : m_ref * c;
        // probabilities -> 16-bit pairs -> TMEM (the A operand of P V), 32 keys at a time
        // probabilities -> 16-bit pairs -> TMEM (the A operand of P V), 32 keys at a time
        const float2 c2 = make_float2(c, c), nmc2 = make_float2(-mc, -mc);
        float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
  #pragma unroll
        for (int cc = 0; cc < BKV / 32; ++cc) {
          uint32_t packed[16];
  #pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float2 x = f2_fma(make_float2(__uint_as_float(raw[cc * 32 + 2 * i]), __uint_as_float(raw[cc * 32 + 2 * i + 1])),
                                    c2, nmc2);
            float2 pr;
            if ((i & SDPA_POLY_AND) == SDPA_POLY_EQ) {
              pr = ex2_poly(x);
            } else {
              pr.x = ex2_approx(x.x);
              pr.y = ex2_approx(x.y);
            }
            if (i & 1) lb = f2_add(lb, pr);
            else la = f2_add(la, pr);
            if (p.ab_format) {
              __nv_bfloat162 hh = __floats2bfloat162_rn(pr.x, pr.y);
              packed[i] = *reinterpret_cast<uint32_t *>(&hh);
            } else {
              __half2 hh = __floats2half2_rn(pr.x, pr.y);
              packed[i] = *reinterpret_cast<uint32_t *>(&hh);
            }
          }
          tmem_st_32x16(s_addr + cc * 16, packed);
          if (cc & 1) {
            // half of P (and, the first time, a rescaled accumulator) is in TMEM: let the MMA warp
            // issue that half of P V
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_half(t, cc >> 1));
          }
        }
        l_run += (la.x + la.y) + (lb.x + lb.y);
      }
      if (ok && n_blocks > 0) {
        if (mbar_wait(pv_done(t), (blk - 1) & 1, p.err, ERR_WAIT_TMEM_FULL)) {
          tc_fence_after();
          const float inv = 1.f / l_run;
          const int64_t row_off = ((int64_t)bh * p.Sq + qi) * HD;
  #pragma unroll 1
          for (int cc = 0; cc < HD / 32; ++cc) {
            uint32_t acc[32];
            tmem_ld_32x32(o_addr + cc * 32, acc);
            tmem_ld_wait();
            float v[32];
  #pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(acc[i]) * inv;
            if (qi < p.Sq) epi_store32(p.out, p.out_dtype, row_off + cc * 32, v, 32);
          }
        }
      }
      // O_t may be overwritten by the next item's first P V
      if (n_blocks > 0) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(o_free(t));
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

bool is16(int dt) { return dt == FB_DT_HALF || dt == FB_DT_BFLOAT16; }

bool dense_bhsd(const TensorInfo &t) {
  if (t.rank != 4) return false;
  const int64_t H = t.dims[1], S = t.dims[2], D = t.dims[3];
  return t.strides[3] == 1 && t.strides[2] == D && t.strides[1] == S * D && t.strides[0] == H * S * D;
}

} // namespace

bool sdpa_tc_eligible(const Plan &p, const Step &s) {
  const fb_node_desc &d = p.nodes[s.node].d;
  if (d.inputs[3] >= 0) return false; // additive masks: CUDA-core kernel
  const TensorInfo &q = p.tensors[d.inputs[0]], &k = p.tensors[d.inputs[1]], &v = p.tensors[d.inputs[2]];
  const TensorInfo &o = p.tensors[d.outputs[0]];
  if (!is16(q.dtype) || k.dtype != q.dtype || v.dtype != q.dtype || o.dtype != q.dtype) return false;
  if (q.dims[3] != HD || v.dims[3] != HD) return false;
  if (!dense_bhsd(q) || !dense_bhsd(k) || !dense_bhsd(v) || !dense_bhsd(o)) return false;
  if (k.dims[1] != v.dims[1] || q.dims[1] % k.dims[1] != 0) return false;
  if (q.dims[2] < 128 || k.dims[2] < 128) return false; // short sequences: CUDA-core kernel
  if (q.dims[0] * q.dims[1] > 65535) return false;
  if (d.fparams[1] != 0.f) return false;
  if ((d.flags & FB_FLAG_SDPA_HAS_SCALE) && !(d.fparams[0] > 0.f)) return false; // max(s) must be max(s*scale)
  return true;
}

fb_status launch_sdpa_tc(const ExecContext &cx, const Step &s) {
  const Plan &plan = *cx.plan;
  const fb_node_desc &d = plan.nodes[s.node].d;
  const TensorInfo &q = plan.tensors[d.inputs[0]], &k = plan.tensors[d.inputs[1]];
  const void *qp = cx.tensor_ptr(d.inputs[0]), *kp = cx.tensor_ptr(d.inputs[1]), *vp = cx.tensor_ptr(d.inputs[2]);
  void *op = cx.tensor_ptr(d.outputs[0]);
  FB_REQUIRE(qp && kp && vp && op, FB_INTERNAL_ERROR, "sdpa_tcgen05: tensor has no buffer");
  FB_REQUIRE(((uintptr_t)qp % 16 == 0) && ((uintptr_t)kp % 16 == 0) && ((uintptr_t)vp % 16 == 0) &&
                 ((uintptr_t)op % 16 == 0),
             FB_INVALID_ARGUMENT, "sdpa_tcgen05: buffers must be 16-byte aligned");
  SdpaTcParams p;
  memset(&p, 0, sizeof(p));
  p.B = (int)q.dims[0]; p.Hq = (int)q.dims[1]; p.Sq = (int)q.dims[2];
  p.Hk = (int)k.dims[1]; p.Skv = (int)k.dims[2];
  p.causal = (d.flags & FB_FLAG_SDPA_CAUSAL) ? 1 : 0;
  p.ab_format = q.dtype == FB_DT_BFLOAT16 ? 1 : 0;
  p.out_dtype = q.dtype;
  p.q_blocks = (p.Sq + BQ * QTILES - 1) / (BQ * QTILES);
  const float scale = (d.flags & FB_FLAG_SDPA_HAS_SCALE) ? d.fparams[0] : 1.f / sqrtf((float)HD);
  p.scale_log2e = scale * 1.4426950408889634f;
  p.out = op;
  p.err = cx.dev->error_word;
  CUtensorMap tq, tk, tv;
  const char *why = "";
  uint32_t box[3] = {64, 128, 1};
  {
    uint64_t dims[3] = {HD, (uint64_t)p.Sq, (uint64_t)p.B * p.Hq};
    uint64_t str[2] = {HD * 2, (uint64_t)p.Sq * HD * 2};
    FB_REQUIRE(encode_tmap_2byte(&tq, qp, 3, dims, str, box, &why), FB_RUNTIME_FAILURE, why);
  }
  {
    uint64_t dims[3] = {HD, (uint64_t)p.Skv, (uint64_t)p.B * p.Hk};
    uint64_t str[2] = {HD * 2, (uint64_t)p.Skv * HD * 2};
    FB_REQUIRE(encode_tmap_2byte(&tk, kp, 3, dims, str, box, &why), FB_RUNTIME_FAILURE, why);
    FB_REQUIRE(encode_tmap_2byte(&tv, vp, 3, dims, str, box, &why), FB_RUNTIME_FAILURE, why);
  }
  cudaError_t ae = set_max_dynamic_smem(reinterpret_cast<const void *>(sdpa_tcgen05_kernel), SMEM_BYTES, cx.dev->ordinal);
  FB_REQUIRE(ae == cudaSuccess, FB_RUNTIME_FAILURE,
             std::string("sdpa_tcgen05: cannot reserve shared memory: ") + cudaGetErrorString(ae));
  p.pairs_per_head = (p.q_blocks + 1) / 2;
  const int64_t pairs = (int64_t)p.pairs_per_head * p.B * p.Hq;
  FB_REQUIRE(pairs < (1ll << 31), FB_NOT_IMPLEMENTED, "sdpa_tcgen05: too many query blocks");
  p.total_pairs = (int)pairs;
  const int grid = (int)std::min<int64_t>(pairs, cx.dev->sm_count);
  FB_CUDA_OK(launch_pdl(sdpa_tcgen05_kernel, dim3(grid), dim3(NUM_THREADS), SMEM_BYTES, cx.dev->stream, tq, tk, tv, p));
  return FB_OK;
}

} // namespace fb

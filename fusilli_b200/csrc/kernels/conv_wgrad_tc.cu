// Weight gradient of 2-D, stride-1, channels-last convolutions on the tensor cores:
//   DW[ko,r,s,c] = sum_{n,p,q} DY[n,p,q,ko] * X[n, p-pad+r*dil, q-pad+s*dil, c]
//
// Per filter tap this is a GEMM with M = ko, N = c and the reduction over output pixels.
// Both operands are read straight from the NHWC tensors as MN-major tiles: a K block is
// a patch of 64 output pixels (bw x bh x bn), DY's patch [64 pixels][ko] is the A tile
// and X's patch shifted by the tap offset [64 pixels][c] is the B tile, each fetched by
// tiled 4-D TMA with zero fill outside the image (= the padding, and the ragged edge of
// the pixel space). The A patch is loaded once and reused for every tap of the CTA's tap
// group; each tap accumulates into its own TMEM columns (taps x BN <= 512). On narrow layers
// (BN <= 128) the shifted X boxes of up to 256 / BN taps land side by side in one B stage and are
// one MMA operand, N = taps x BN, writing those taps' adjacent column ranges at once.
// On 64-channel layers with R x S > 1 (unit dilation) the X operand comes from a haloed patch instead:
// a CTA owns one filter COLUMN s, loads per 8 x 8 pixel patch ONE box of 8 x (8+R-1) input pixels
// shifted by s, and the R taps of the column are the 64-channel blocks of a single B operand whose
// blocks are 1024 bytes (one image row of the patch) apart: one MMA of N = 64 R per 16 pixels, 10 KB of
// X per patch instead of R boxes of 8 KB.
// The pixel reduction is split across CTAs: a CTA owns (ko tile, c tile, tap group, pixel
// slice), writes its fp32 partial filter to the workspace, and a second kernel adds the
// slices in a fixed order and converts -- deterministic, no atomics.
#include <algorithm>

#include "../common.h"
#include "sm100.cuh"

namespace fb {

using namespace sm100;

namespace {

constexpr int BM = 128, KPIX = 64, MAX_BN = 256;
constexpr int HALF = 64 * KPIX * 2;              // one [64 pixels][64 channels] box, 8 KB
// The dY ring gets 48 KB and the X ring 128 KB; a stage is as large as the layer's tiles need
// (dY: one or two boxes; X: up to four), so narrow layers keep more loads in flight: 6 + 12 stages
// of 8 KB on a 1x1 C64 layer against 3 + 4 stages of 16 / 32 KB on the wide ones.
constexpr int A_RING_BYTES = 3 * BM * KPIX * 2, B_RING_BYTES = 4 * MAX_BN * KPIX * 2;
constexpr int MAX_A_STAGES = 6, MAX_B_STAGES = 12;
// With haloed X patches the two rings share 220 KB and are split per layer (p.a_ring_bytes).
constexpr int HALO_RING_BYTES = 220 * 1024;
constexpr int SMEM_BYTES = HALO_RING_BYTES + 1024 + 512;
constexpr int NUM_THREADS = 224; // warps 0, 3, 4, 5: X producers; 1 (and 6 with haloed patches): MMA issue; 2: dY producer; 2..5 drain the accumulators
constexpr int B_PRODUCERS = 4; // warps 0, 3, 4, 5 take every fourth B stage each
constexpr int TMEM_COLS = 512;

struct WgradTcParams {
  int32_t ab_format;
  int32_t Kout, C, R, S;
  int32_t N, P, Q;          // DY pixel space
  int32_t pad_h, pad_w, dil_h, dil_w;
  int32_t bw, bh, bn, tiles_w, tiles_h, tiles_nb;
  int32_t patches_total, patches_per_slice, slices;
  int32_t k_tiles, c_tiles, ngroups, taps_per_group, BN, a_halves;
  int32_t tpack;            // filter taps that share one B stage and one MMA (tpack * BN <= 256)
  int32_t halo;             // haloed X patches: the CTA's tap group is filter column `grp`, its taps the R rows
  int32_t issuers;          // MMA-issuing warps (2 with haloed patches and R >= 2: they split the column's taps)
  int32_t a_stages, b_stages, a_stage_bytes, b_stage_bytes;
  int32_t a_ring_bytes;     // bytes of the dY ring; the X ring follows
  float *partial;           // [slices][Kout][R*S][C] fp32
  uint32_t *err;
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
conv_wgrad_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_dy, const __grid_constant__ CUtensorMap tmap_x,
                          const WgradTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  pdl_launch_dependents(); // the next kernel's CTAs may take the SMs this kernel's CTAs leave
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int A_STAGES = p.a_stages, B_STAGES = p.b_stages;
  const uint32_t A_STAGE_BYTES = (uint32_t)p.a_stage_bytes, B_STAGE_BYTES = (uint32_t)p.b_stage_bytes;
  const uint32_t sb_base = smem_base + (uint32_t)p.a_ring_bytes;
  const uint32_t bar_base = smem_base + HALO_RING_BYTES;
  auto a_full = [&](int s) { return bar_base + 8u * s; };
  auto a_empty = [&](int s) { return bar_base + 8u * (MAX_A_STAGES + s); };
  auto b_full = [&](int s) { return bar_base + 8u * (2 * MAX_A_STAGES + s); };
  auto b_empty = [&](int s) { return bar_base + 8u * (2 * MAX_A_STAGES + MAX_B_STAGES + s); };
  const uint32_t acc_full = bar_base + 8u * (2 * MAX_A_STAGES + 2 * MAX_B_STAGES);
  const uint32_t tmem_slot = acc_full + 8u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // unit decomposition: ko tile fastest, then c tile, tap group, pixel slice
  int u = blockIdx.x;
  const int kt = u % p.k_tiles; u /= p.k_tiles;
  const int ct = u % p.c_tiles; u /= p.c_tiles;
  const int grp = u % p.ngroups;
  const int slice = u / p.ngroups;
  const int tap0 = p.halo ? 0 : grp * p.taps_per_group;
  const int ntaps = p.halo ? p.R : min(p.taps_per_group, p.R * p.S - tap0);
  const int patch0 = slice * p.patches_per_slice;
  const int npatch = min(p.patches_per_slice, p.patches_total - patch0);
  const uint32_t img = p.halo ? (uint32_t)p.bn : 1u; // images per stage (haloed patches take two)
  const uint32_t a_bytes = (uint32_t)p.a_halves * HALF * img, b_bytes = (uint32_t)p.BN * KPIX * 2;

  if (threadIdx.x == 0) {
    // every issuing warp releases a stage and reports its accumulators
    for (int s = 0; s < A_STAGES; ++s) { mbar_init(a_full(s), 1); mbar_init(a_empty(s), p.issuers); }
    for (int s = 0; s < B_STAGES; ++s) { mbar_init(b_full(s), 1); mbar_init(b_empty(s), p.issuers); }
    mbar_init(acc_full, p.issuers);
    fence_barrier_init();
    tma_prefetch_desc(&tmap_dy);
    tma_prefetch_desc(&tmap_x);
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

  // Three warps feed the rings, each with its own copy of the patch and tap counters: one loads
  // the dY patches, two take alternate B stages. A single producer warp was the pace of the whole
  // kernel: every elected wait / expect / TMA issue costs it 100-300 clk one after the other
  // (1113 clk per 64-pixel patch on a 1x1 layer that needs two boxes), while the MMA warp waited.
  // Whole warp in the loop, every issue predicated on an in-line election: coordinates stay in
  // uniform registers and the tap counters advance without divisions.
  auto produce_a = [&]() {
    int sa_i = 0;
    uint32_t pha = 0;
    int tw = patch0 % p.tiles_w, th = (patch0 / p.tiles_w) % p.tiles_h, tb = patch0 / (p.tiles_w * p.tiles_h);
    for (int pi = 0; pi < npatch; ++pi) {
      const int w0 = tw * p.bw, h0 = th * p.bh, n0 = tb * p.bn;
      if (!mbar_wait_warp(a_empty(sa_i), pha ^ 1, p.err, ERR_WAIT_EMPTY)) break;
      mbar_expect_tx_elect(a_full(sa_i), a_bytes);
      const uint32_t sa = smem_base + (uint32_t)sa_i * A_STAGE_BYTES;
      for (int hh = 0; hh < p.a_halves; ++hh)
        tma_load_4d_elect(sa + hh * HALF * img, &tmap_dy, a_full(sa_i), kt * BM + 64 * hh, w0, h0, n0);
      sa_i = (sa_i + 1 == A_STAGES) ? 0 : sa_i + 1;
      pha ^= (sa_i == 0);
      if (++tw == p.tiles_w) {
        tw = 0;
        if (++th == p.tiles_h) {
          th = 0;
          ++tb;
        }
      }
    }
  };
  auto produce_b = [&](int id) {
    int sb_i = 0, chunk = 0;
    uint32_t phb = 0;
    bool ok = true;
    if (p.halo) {
      // one stage per patch: the 8 x (bh+R-1) input pixels under the patch for filter column grp
      // No more producer warps than stages: a warp's consecutive loads must be consecutive uses of their
      // stage. (With four warps on three stages a warp's second load was the THIRD use of its stage, its
      // parity wait passed on the barrier's initial phase, and the stage's full barrier got a second
      // arrival in one phase: a launch failure.)
      const int nprod = min(B_PRODUCERS, B_STAGES);
      if (id >= nprod) return;
      int tw = patch0 % p.tiles_w, th = (patch0 / p.tiles_w) % p.tiles_h, tb = patch0 / (p.tiles_w * p.tiles_h);
      for (int pi = 0; pi < npatch && ok; ++pi) {
        if (pi % nprod == id) {
          if (!mbar_wait_warp(b_empty(sb_i), phb ^ 1, p.err, ERR_WAIT_EMPTY)) { ok = false; break; }
          mbar_expect_tx_elect(b_full(sb_i), B_STAGE_BYTES);
          tma_load_4d_elect(sb_base + (uint32_t)sb_i * B_STAGE_BYTES, &tmap_x, b_full(sb_i), ct * p.BN,
                            tw * p.bw - p.pad_w + grp, th * p.bh - p.pad_h, tb * p.bn);
        }
        sb_i = (sb_i + 1 == B_STAGES) ? 0 : sb_i + 1;
        phb ^= (sb_i == 0);
        if (++tw == p.tiles_w) {
          tw = 0;
          if (++th == p.tiles_h) {
            th = 0;
            ++tb;
          }
        }
      }
      return;
    }
    const int ts0 = tap0 % p.S, tr0 = tap0 / p.S;
    int tw = patch0 % p.tiles_w, th = (patch0 / p.tiles_w) % p.tiles_h, tb = patch0 / (p.tiles_w * p.tiles_h);
    for (int pi = 0; pi < npatch && ok; ++pi) {
      const int w0 = tw * p.bw, h0 = th * p.bh, n0 = tb * p.bn;
      int ts = ts0, tr = tr0;
      // a stage takes the shifted X boxes of up to tpack taps side by side: they become the
      // column blocks of ONE B operand, so narrow layers issue a quarter of the MMAs
      for (int t = 0; t < ntaps; t += p.tpack, ++chunk) {
        const int nt = min(p.tpack, ntaps - t);
        const bool mine = (chunk & (B_PRODUCERS - 1)) == id;
        if (mine) {
          if (!mbar_wait_warp(b_empty(sb_i), phb ^ 1, p.err, ERR_WAIT_EMPTY)) { ok = false; break; }
          mbar_expect_tx_elect(b_full(sb_i), (uint32_t)nt * b_bytes);
        }
        const uint32_t sb = sb_base + (uint32_t)sb_i * B_STAGE_BYTES;
        for (int u = 0; u < nt; ++u) {
          if (mine)
            for (int i = 0; i < p.BN / 64; ++i)
              tma_load_4d_elect(sb + (u * (p.BN / 64) + i) * HALF, &tmap_x, b_full(sb_i), ct * p.BN + 64 * i,
                                w0 - p.pad_w + ts * p.dil_w, h0 - p.pad_h + tr * p.dil_h, n0);
          if (++ts == p.S) {
            ts = 0;
            ++tr;
          }
        }
        sb_i = (sb_i + 1 == B_STAGES) ? 0 : sb_i + 1;
        phb ^= (sb_i == 0);
      }
      if (++tw == p.tiles_w) {
        tw = 0;
        if (++th == p.tiles_h) {
          th = 0;
          ++tb;
        }
      }
    }
  };

  if (warp == 0) {
    produce_b(0);
  } else if (warp == 1 || warp == 6) {
    // The whole warp runs the loop (addresses and descriptors stay in uniform registers); one
    // elected lane issues the MMAs and the commits, which track the issuing thread.
    // one instruction descriptor per number of taps in a stage (N = taps * BN)
    uint32_t idesc_n[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) idesc_n[u] = make_idesc_f16(BM, min((u + 1) * p.BN, MAX_BN), p.ab_format, 1, 1);
    // both tiles MN-major: 64-channel blocks HALF apart (LBO), 8-pixel groups 1024 B apart,
    // a 16-pixel K step is 2048 B
    const uint64_t a_desc0 = make_smem_desc(smem_base, HALF, 1024);
    const uint64_t b_desc0 = make_smem_desc(sb_base, HALF, 1024);
    int sa_i = 0, sb_i = 0;
    uint32_t pha = 0, phb = 0;
    bool ok = warp == 1 || p.issuers == 2, npatch_done = false;
    if (p.halo && ok) {
      // The taps of the column are ONE B operand: N = 64 x taps, the taps' 64-channel blocks one patch row
      // (1024 B) apart. With two issuing warps the first takes the upper half of the rows and the second
      // the rest, each into TMEM columns of its own (one issuing thread and a fixed order of sums per
      // accumulator): four MMAs per patch are ~400 clk of tensor time between two barrier waits of ~200
      // clk each, and the pipe queues only two or three instructions.
      const int r_first = p.issuers == 2 ? (p.R + 1) / 2 : p.R;
      const int r0 = warp == 1 ? 0 : r_first, nr = warp == 1 ? r_first : p.R - r_first;
      const uint32_t idesc_h = make_idesc_f16(BM, nr * 64, p.ab_format, 1, 1);
      const uint64_t bh_desc0 = make_smem_desc(sb_base + (uint32_t)r0 * 1024u, 1024, 1024);
      const uint64_t ah_desc0 = make_smem_desc(smem_base, HALF * img, 1024); // 64-channel blocks of dY: img boxes apart
      const uint32_t d_tmem = tmem_base + (uint32_t)(r0 * 64);
      const uint32_t x_img = (uint32_t)(p.bh + p.R - 1) * 1024u; // one image's rows of the X box
      const int ksteps = (KPIX / 16) * (int)img;
      for (int pi = 0; pi < npatch && ok; ++pi) {
        if (!mbar_wait_warp(a_full(sa_i), pha, p.err, ERR_WAIT_FULL)) { ok = false; break; }
        if (!mbar_wait_warp(b_full(sb_i), phb, p.err, ERR_WAIT_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint64_t ad = ah_desc0 + (uint64_t)(((uint32_t)sa_i * A_STAGE_BYTES) >> 4);
        const uint64_t bd = bh_desc0 + (uint64_t)(((uint32_t)sb_i * B_STAGE_BYTES) >> 4);
        for (int k = 0; k < ksteps; ++k) // 16 pixels = two patch rows per step; the images' X rows are x_img apart
          tc_mma_f16_elect(d_tmem, ad + (uint64_t)((k * 2048) >> 4),
                           bd + (uint64_t)(((uint32_t)(k >> 2) * x_img + (uint32_t)(k & 3) * 2048u) >> 4), idesc_h,
                           (pi > 0 || k > 0) ? 1u : 0u);
        tc_commit_elect(b_empty(sb_i));
        tc_commit_elect(a_empty(sa_i));
        sb_i = (sb_i + 1 == B_STAGES) ? 0 : sb_i + 1;
        phb ^= (sb_i == 0);
        sa_i = (sa_i + 1 == A_STAGES) ? 0 : sa_i + 1;
        pha ^= (sa_i == 0);
      }
      npatch_done = true;
    }
    if (warp != 1) npatch_done = true;
    for (int pi = 0; pi < npatch && ok && !npatch_done; ++pi) {
      if (!mbar_wait_warp(a_full(sa_i), pha, p.err, ERR_WAIT_FULL)) { ok = false; break; }
      const uint64_t ad = a_desc0 + (uint64_t)(((uint32_t)sa_i * A_STAGE_BYTES) >> 4);
      for (int t = 0; t < ntaps; t += p.tpack) {
        const int nt = min(p.tpack, ntaps - t);
        const uint32_t idesc = nt == 1 ? idesc_n[0] : (nt == 2 ? idesc_n[1] : (nt == 3 ? idesc_n[2] : idesc_n[3]));
        if (!mbar_wait_warp(b_full(sb_i), phb, p.err, ERR_WAIT_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint64_t bd = b_desc0 + (uint64_t)(((uint32_t)sb_i * B_STAGE_BYTES) >> 4);
#pragma unroll
        for (int k = 0; k < KPIX / 16; ++k)
          tc_mma_f16_elect(tmem_base + t * p.BN, ad + (uint64_t)((k * 2048) >> 4), bd + (uint64_t)((k * 2048) >> 4),
                           idesc, (pi > 0 || k > 0) ? 1u : 0u);
        tc_commit_elect(b_empty(sb_i));
        sb_i = (sb_i + 1 == B_STAGES) ? 0 : sb_i + 1;
        phb ^= (sb_i == 0);
      }
      if (ok) tc_commit_elect(a_empty(sa_i));
      sa_i = (sa_i + 1 == A_STAGES) ? 0 : sa_i + 1;
      pha ^= (sa_i == 0);
    }
    if (ok && (warp == 1 || p.issuers == 2)) tc_commit_elect(acc_full);
  } else {
    if (warp == 2) produce_a();
    if (warp >= 3) produce_b(warp - 2);
    __syncwarp();
    const int q = warp & 3;
    const int ko = kt * BM + q * 32 + lane;
    const int taps_all = p.R * p.S;
    bool have = npatch > 0;
    if (have) have = mbar_wait(acc_full, 0, p.err, ERR_WAIT_TMEM_FULL);
    tc_fence_after();
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    for (int t = 0; t < ntaps; ++t) {
      for (int cc = 0; cc < p.BN / 32; ++cc) {
        uint32_t raw[32];
        if (have) {
          tmem_ld_32x32(tmem_base + lane_addr + t * p.BN + cc * 32, raw);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) raw[j] = 0u;
        }
        const int c0 = ct * p.BN + cc * 32;
        if (ko < p.Kout && c0 < p.C) {
          const int tap = p.halo ? t * p.S + grp : tap0 + t; // halo: row t of filter column grp
          float *dst = p.partial + (((int64_t)slice * p.Kout + ko) * taps_all + tap) * p.C + c0;
          if (c0 + 32 <= p.C && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              reinterpret_cast<float4 *>(dst)[j] =
                  make_float4(__uint_as_float(raw[4 * j]), __uint_as_float(raw[4 * j + 1]),
                              __uint_as_float(raw[4 * j + 2]), __uint_as_float(raw[4 * j + 3]));
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (c0 + j < p.C) dst[j] = __uint_as_float(raw[j]);
          }
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

// out[i] = sum over slices of partial[s][i] in a fixed order: four threads per element take every
// fourth slice each (eight loads in flight per thread: one dependent load per slice made this pass
// latency-bound) and their sums are combined pairwise, (g0 + g1) + (g2 + g3).
__global__ void __launch_bounds__(256)
wgrad_slice_reduce_kernel(const float *__restrict__ partial, void *out, int out_dtype, int64_t elems, int slices) {
  pdl_launch_dependents();
  pdl_wait(); // the partials are complete and visible after this
  const int g = threadIdx.x & 3;
  const int64_t per_block = blockDim.x / 4;
  for (int64_t i0 = (int64_t)blockIdx.x * per_block; i0 < elems; i0 += (int64_t)gridDim.x * per_block) {
    const int64_t i = i0 + (threadIdx.x >> 2);
    float acc = 0.f;
    if (i < elems) {
      int s = g;
      for (; s + 28 < slices; s += 32) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) v[u] = __ldg(partial + (int64_t)(s + 4 * u) * elems + i);
#pragma unroll
        for (int u = 0; u < 8; ++u) acc += v[u];
      }
      for (; s < slices; s += 4) acc += __ldg(partial + (int64_t)s * elems + i);
    }
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    if (g == 0 && i < elems) store_f(out, out_dtype, i, acc);
  }
}

// The same with one thread per element: few slices and a large filter (coalesced rows, nothing to
// spread).
__global__ void __launch_bounds__(256)
wgrad_slice_reduce1_kernel(const float *__restrict__ partial, void *out, int out_dtype, int64_t elems, int slices) {
  pdl_launch_dependents();
  pdl_wait(); // the partials are complete and visible after this
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < elems; i += (int64_t)gridDim.x * blockDim.x) {
    float acc = 0.f;
    int s = 0;
    for (; s + 8 <= slices; s += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldg(partial + (int64_t)(s + u) * elems + i);
#pragma unroll
      for (int u = 0; u < 8; ++u) acc += v[u];
    }
    for (; s < slices; ++s) acc += __ldg(partial + (int64_t)s * elems + i);
    store_f(out, out_dtype, i, acc);
  }
}

bool is16(int dt) { return dt == FB_DT_HALF || dt == FB_DT_BFLOAT16; }
bool isfl(int dt) { return dt == FB_DT_HALF || dt == FB_DT_BFLOAT16 || dt == FB_DT_FLOAT; }

bool cl_dense(const TensorInfo &t) {
  if (t.rank != 4) return false;
  const int64_t C = t.dims[1], H = t.dims[2], W = t.dims[3];
  return t.strides[1] == 1 && t.strides[3] == C && t.strides[2] == W * C && t.strides[0] == H * W * C;
}

struct WgradView {
  int N, P, Q, XH, XW, Kout, C, R, S, pad_h, pad_w, dil_h, dil_w;
};

bool wgrad_view(const Plan &p, const Step &s, WgradView &v) {
  const fb_node_desc &d = p.nodes[s.node].d;
  if (d.op != FB_OP_CONV_WGRAD || d.num_spatial != 2) return false;
  if (d.stride[0] != 1 || d.stride[1] != 1) return false;
  if (s.num_epilogue != 0) return false;
  const TensorInfo &dy = p.tensors[d.inputs[0]], &x = p.tensors[d.inputs[1]], &dw = p.tensors[d.outputs[0]];
  if (!is16(dy.dtype) || x.dtype != dy.dtype || !isfl(dw.dtype)) return false;
  if (!cl_dense(dy) || !cl_dense(x) || !cl_dense(dw)) return false;
  if (dw.dims[1] != x.dims[1]) return false; // groups == 1
  v.N = (int)dy.dims[0]; v.Kout = (int)dy.dims[1]; v.P = (int)dy.dims[2]; v.Q = (int)dy.dims[3];
  v.C = (int)x.dims[1]; v.XH = (int)x.dims[2]; v.XW = (int)x.dims[3];
  v.R = (int)dw.dims[2]; v.S = (int)dw.dims[3];
  v.pad_h = (int)d.padding[0]; v.pad_w = (int)d.padding[1];
  v.dil_h = (int)d.dilation[0]; v.dil_w = (int)d.dilation[1];
  if (v.C % 8 || v.Kout % 8 || v.C < 64 || v.Kout < 64) return false;
  // at least 16 patches of 64 pixels to reduce over (a rank's shard of the 7x7 layer at N = 256 / 8 is 1568 pixels)
  if ((int64_t)v.N * v.P * v.Q < 1024) return false;
  return true;
}

struct WgradTiling {
  int bw, bh, bn, tiles_w, tiles_h, tiles_nb, patches;
  int k_tiles, c_tiles, BN, ngroups, taps_per_group, slices, per_slice;
  int halo;
};

// FUSILLI_B200_WGRAD_HALO=0 at plan build AND execute keeps the per-tap X boxes.
bool wgrad_halo_off() {
  static const bool off = [] {
    const char *e = getenv("FUSILLI_B200_WGRAD_HALO");
    return e && e[0] == '0';
  }();
  return off;
}

int wgrad_halo_max_c() {
  static const int c = [] {
    const char *e = getenv("FUSILLI_B200_WGRAD_HALO_MAXC");
    return e ? atoi(e) : 128;
  }();
  return c;
}

int wgrad_halo_min_taps() {
  static const int c = [] {
    const char *e = getenv("FUSILLI_B200_WGRAD_HALO_MINTAPS");
    return e ? atoi(e) : 1;
  }();
  return c;
}

void wgrad_tiling(const WgradView &v, WgradTiling &t, bool allow_halo = true) {
  // 64-pixel patches with power-of-two sides (the K block must be exactly 64 rows)
  double best = -1.0;
  t.bw = 8; t.bh = 8; t.bn = 1;
  for (int w = 1; w <= 64; w *= 2)
    for (int h = 1; w * h <= 64; h *= 2) {
      const int n = 64 / (w * h);
      if (n > v.N && n > 1) continue;
      const int64_t tiles = (int64_t)((v.Q + w - 1) / w) * ((v.P + h - 1) / h) * ((v.N + n - 1) / n);
      const double eff = (double)v.N * v.P * v.Q / ((double)tiles * 64.0);
      if (eff > best + 1e-9 || (eff > best - 1e-9 && w > t.bw)) {
        best = eff; t.bw = w; t.bh = h; t.bn = n;
      }
    }
  t.tiles_w = (v.Q + t.bw - 1) / t.bw;
  t.tiles_h = (v.P + t.bh - 1) / t.bh;
  t.tiles_nb = (v.N + t.bn - 1) / t.bn;
  t.patches = t.tiles_w * t.tiles_h * t.tiles_nb;
  t.k_tiles = (v.Kout + BM - 1) / BM;
  t.BN = v.C > 128 ? 256 : (v.C > 64 ? 128 : 64);
  t.c_tiles = (v.C + t.BN - 1) / t.BN;
  const int taps = v.R * v.S;
  t.ngroups = (taps * t.BN + TMEM_COLS - 1) / TMEM_COLS;
  t.taps_per_group = (taps + t.ngroups - 1) / t.ngroups;
  t.ngroups = (taps + t.taps_per_group - 1) / t.taps_per_group;
  // Haloed X patches (one CTA per filter column): 64-channel tiles, unit dilation, R taps = N <= 256, and
  // an image that 8 x 8 patches tile without much waste
  t.halo = 0;
  if (allow_halo && taps >= wgrad_halo_min_taps() && v.C <= wgrad_halo_max_c() && v.dil_h == 1 && v.dil_w == 1 && v.R <= 4 && v.S <= 8 && !wgrad_halo_off()) {
    const int64_t tiles = (int64_t)((v.Q + 7) / 8) * ((v.P + 7) / 8) * v.N;
    if ((double)v.N * v.P * v.Q / ((double)tiles * 64.0) >= 0.75) {
      t.halo = 1;
      t.BN = 64; // a CTA takes 64 input channels of one filter column
      t.c_tiles = (v.C + 63) / 64;
      // Several images per stage: 4 MMAs per image between two barrier waits (~200 clk each even on a
      // completed barrier; 120 -> 103 us on 56x56 C64 3x3 with two images). The most images that leave
      // three stages of both rings.
      const int a_halves = v.Kout > 64 ? 2 : 1;
      t.bw = 8; t.bh = 8; t.bn = 1;
      for (int n = 4; n > 1; n /= 2)
        if (n <= v.N && 3 * n * (a_halves * HALF + (8 + v.R - 1) * 1024) <= HALO_RING_BYTES) {
          t.bn = n;
          break;
        }
      t.tiles_w = (v.Q + 7) / 8; t.tiles_h = (v.P + 7) / 8; t.tiles_nb = (v.N + t.bn - 1) / t.bn;
      t.patches = t.tiles_w * t.tiles_h * t.tiles_nb;
      t.ngroups = v.S;
      t.taps_per_group = v.R;
    }
  }
  const int units = t.k_tiles * t.c_tiles * t.ngroups;
  // One CTA per SM: with two per SM (which run one after the other: shared memory and TMEM admit
  // one) every layer was 7-15 % slower, each CTA paying its own prologue, first-load latency and
  // accumulator drain, and the slice reduction reading twice the partials.
  int slices = std::max(1, 148 / units);
  // at least eight stages per slice; counted in image patches where a stage holds several images, so that
  // the slice count (and the workspace) never shrinks when the batch grows
  slices = std::min(slices, std::max(1, t.halo ? (t.tiles_w * t.tiles_h * v.N) / 32 : t.patches / 8));
  t.per_slice = (t.patches + slices - 1) / slices;
  t.slices = (t.patches + t.per_slice - 1) / t.per_slice;
}

} // namespace

bool conv_wgrad_tc_eligible(const Plan &p, const Step &s) {
  WgradView v;
  return wgrad_view(p, s, v);
}

// Workspace bytes of the fp32 slice partials (device independent: the plan is built without a device).
int64_t conv_wgrad_tc_scratch_bytes(const Plan &p, const Step &s, int32_t *slices) {
  WgradView v;
  if (!wgrad_view(p, s, v)) return 0;
  WgradTiling t, plain;
  wgrad_tiling(v, t);
  wgrad_tiling(v, plain, false);
  *slices = t.slices;
  // A plan with dynamic dims is specialised per shape and a smaller shape may take the other tiling: the
  // workspace of the representative shape covers both.
  return (int64_t)std::max(t.slices, plain.slices) * v.Kout * v.R * v.S * v.C * 4;
}

fb_status launch_conv_wgrad_tc(const ExecContext &cx, const Step &s) {
  const Plan &plan = *cx.plan;
  const fb_node_desc &d = plan.nodes[s.node].d;
  WgradView v;
  FB_REQUIRE(wgrad_view(plan, s, v), FB_INTERNAL_ERROR, "conv_wgrad_tcgen05: step is not eligible");
  WgradTiling t;
  wgrad_tiling(v, t);
  const TensorInfo &dy = plan.tensors[d.inputs[0]], &dw = plan.tensors[d.outputs[0]];
  const void *dyp = cx.tensor_ptr(d.inputs[0]), *xp = cx.tensor_ptr(d.inputs[1]);
  void *dwp = cx.tensor_ptr(s.out_tensor);
  FB_REQUIRE(dyp && xp && dwp, FB_INTERNAL_ERROR, "conv_wgrad_tcgen05: tensor has no buffer");
  FB_REQUIRE(((uintptr_t)dyp % 16 == 0) && ((uintptr_t)xp % 16 == 0), FB_INVALID_ARGUMENT,
             "conv_wgrad_tcgen05: operand buffers must be 16-byte aligned");
  FB_REQUIRE(cx.workspace && s.scratch_offset >= 0, FB_INTERNAL_ERROR, "conv_wgrad_tcgen05: scratch missing");
  const int64_t elems = (int64_t)v.Kout * v.R * v.S * v.C;
  FB_REQUIRE(s.scratch_bytes >= (int64_t)t.slices * elems * 4, FB_INTERNAL_ERROR,
             "conv_wgrad_tcgen05: scratch smaller than the tiling needs");
  WgradTcParams p;
  memset(&p, 0, sizeof(p));
  p.ab_format = dy.dtype == FB_DT_BFLOAT16 ? 1 : 0;
  p.Kout = v.Kout; p.C = v.C; p.R = v.R; p.S = v.S;
  p.N = v.N; p.P = v.P; p.Q = v.Q;
  p.pad_h = v.pad_h; p.pad_w = v.pad_w; p.dil_h = v.dil_h; p.dil_w = v.dil_w;
  p.bw = t.bw; p.bh = t.bh; p.bn = t.bn;
  p.tiles_w = t.tiles_w; p.tiles_h = t.tiles_h; p.tiles_nb = t.tiles_nb;
  p.patches_total = t.patches; p.patches_per_slice = t.per_slice; p.slices = t.slices;
  p.k_tiles = t.k_tiles; p.c_tiles = t.c_tiles; p.ngroups = t.ngroups; p.taps_per_group = t.taps_per_group;
  p.BN = t.BN;
  p.a_halves = (v.Kout - 0 > 64) ? 2 : 1;
  p.tpack = std::max(1, std::min(4, MAX_BN / t.BN));
  p.halo = t.halo;
  p.issuers = 1; // a second issuing warp on the column's lower taps was slower (140 against 120 us on 56x56 C64 3x3)
  p.a_stage_bytes = p.a_halves * HALF * (t.halo ? t.bn : 1);
  p.b_stage_bytes = t.halo ? t.bn * (t.bh + v.R - 1) * 1024 : std::min(p.tpack, t.taps_per_group) * (t.BN / 64) * HALF;
  if (t.halo) {
    const int st = std::min(MAX_A_STAGES, HALO_RING_BYTES / (p.a_stage_bytes + p.b_stage_bytes));
    p.a_stages = p.b_stages = st;
    p.a_ring_bytes = st * p.a_stage_bytes;
  } else {
    p.a_stages = std::min(MAX_A_STAGES, A_RING_BYTES / p.a_stage_bytes);
    p.b_stages = std::min(MAX_B_STAGES, B_RING_BYTES / p.b_stage_bytes);
    p.a_ring_bytes = A_RING_BYTES;
  }
  p.partial = reinterpret_cast<float *>(cx.workspace + s.scratch_offset);
  p.err = cx.dev->error_word;
  CUtensorMap tmDy, tmX;
  const char *why = "";
  {
    uint64_t dims[4] = {(uint64_t)v.Kout, (uint64_t)v.Q, (uint64_t)v.P, (uint64_t)v.N};
    uint64_t str[3] = {(uint64_t)v.Kout * 2, (uint64_t)v.Q * v.Kout * 2, (uint64_t)v.P * v.Q * v.Kout * 2};
    uint32_t box[4] = {64, (uint32_t)t.bw, (uint32_t)t.bh, (uint32_t)t.bn};
    FB_REQUIRE(encode_tmap_2byte(&tmDy, dyp, 4, dims, str, box, &why), FB_RUNTIME_FAILURE, why);
  }
  {
    uint64_t dims[4] = {(uint64_t)v.C, (uint64_t)v.XW, (uint64_t)v.XH, (uint64_t)v.N};
    uint64_t str[3] = {(uint64_t)v.C * 2, (uint64_t)v.XW * v.C * 2, (uint64_t)v.XH * v.XW * v.C * 2};
    uint32_t box[4] = {64, (uint32_t)t.bw, (uint32_t)(t.halo ? t.bh + v.R - 1 : t.bh), (uint32_t)t.bn};
    FB_REQUIRE(encode_tmap_2byte(&tmX, xp, 4, dims, str, box, &why), FB_RUNTIME_FAILURE, why);
  }
  cudaError_t ae =
      set_max_dynamic_smem(reinterpret_cast<const void *>(conv_wgrad_tcgen05_kernel), SMEM_BYTES, cx.dev->ordinal);
  FB_REQUIRE(ae == cudaSuccess, FB_RUNTIME_FAILURE,
             std::string("conv_wgrad_tcgen05: cannot reserve shared memory: ") + cudaGetErrorString(ae));
  const int grid = t.k_tiles * t.c_tiles * t.ngroups * t.slices;
  FB_CUDA_OK(launch_pdl(conv_wgrad_tcgen05_kernel, dim3(grid), dim3(NUM_THREADS), SMEM_BYTES, cx.dev->stream, tmDy, tmX, p));
  if (t.slices >= 16) {
    const int rblocks = (int)std::min<int64_t>((elems + 63) / 64, (int64_t)cx.dev->sm_count * 8);
    FB_CUDA_OK(launch_pdl(wgrad_slice_reduce_kernel, dim3(rblocks), dim3(256), 0, cx.dev->stream, (const float *)p.partial, dwp,
                          (int)dw.dtype, elems, (int)t.slices));
  } else {
    const int rblocks = (int)std::min<int64_t>((elems + 255) / 256, (int64_t)cx.dev->sm_count * 8);
    FB_CUDA_OK(launch_pdl(wgrad_slice_reduce1_kernel, dim3(rblocks), dim3(256), 0, cx.dev->stream, (const float *)p.partial, dwp,
                          (int)dw.dtype, elems, (int)t.slices));
  }
  return FB_OK;
}

} // namespace fb

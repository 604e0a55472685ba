// Implicit-GEMM convolution on the tensor cores: fprop and dgrad of 2-D, stride-1,
// channels-last (NHWC / KRSC) convolutions with 16-bit operands.
//
//   fprop  Y[n,p,q,ko]  = sum_{r,s,c}  X[n, p-pad+r*dil, q-pad+s*dil, c] * W[ko,r,s,c]
//   dgrad  DX[n,h,w,c]  = sum_{r,s,ko} DY[n, h+pad-r*dil, w+pad-s*dil, ko] * W[ko,r,s,c]
//
// No im2col buffer exists anywhere. The GEMM M tile is a rectangular patch of output
// pixels (bw x bh x bn <= 128 rows); for every filter tap and 64-channel block the TMA
// producer loads the same patch of the input shifted by the tap offset with ONE tiled
// 4-D cp.async.bulk.tensor (channels innermost, 128-byte swizzle). Coordinates that
// fall outside the image are zero-filled by the TMA unit, which is exactly the
// convolution's padding. 1x1 / pad-0 convolutions collapse (n,h,w) into one axis and
// run at full tile occupancy. Everything else -- 4-stage ring, one MMA-issuing thread,
// fp32 accumulators double-buffered in TMEM, register epilogue with the fused pointwise
// chain, bounded mbarrier waits -- is the batched-GEMM kernel's structure.
// fprop's filter tile is K-major (c contiguous); dgrad's is MN-major (W[ko][c] rows).
#include <algorithm>
#include <mutex>
#include <unordered_map>

#include "../common.h"
#include "sm100.cuh"
#include "tc_epilogue.cuh"

namespace fb {

using namespace sm100;

namespace {

constexpr int BM = 128, BK = 64, MAX_BN = 256;
constexpr int A_BYTES = BM * BK * 2;
// The ring takes all of shared memory: a stage is the patch tile plus BN filter rows, so narrow
// layers (BN = 64) get 9 stages, BN = 128 gets 7 and BN = 256 gets 4. What bounds these kernels on narrow
// layers is bytes in flight per SM against L2 latency, not bandwidth.
constexpr int MAX_STAGES = 12;
constexpr int RING_BYTES = 229376; // 9 x 24 KB, 7 x 32 KB or 4 x 48 KB fit
// With 16-bit outputs the last 32 KB of that space are the epilogue's staging tiles (two boxes of
// 128 rows x 64 channels, 128-byte swizzled) and the operand ring gets the 192 KB before them.
constexpr int STAGING_BYTES = 32768, BOX_BYTES = 16384;
constexpr int RING_BYTES_STAGED = RING_BYTES - STAGING_BYTES; // 8 x 24 KB, 6 x 32 KB or 4 x 48 KB
constexpr int SMEM_BYTES = RING_BYTES + 1024 + 512;
constexpr int NUM_THREADS = 320; // TMA warp, MMA warp, 8 epilogue warps (two per TMEM lane quarter)
constexpr int TMEM_COLS = 512;

#ifdef FB_CONV_TRACE
// Instrumented build only: cycles block 0 spends in each phase (index meanings in fb_debug_conv_trace's caller).
__device__ unsigned long long g_conv_trace[32];
#define TR_BEGIN long long _tr0 = clock64()
#define TR_ADD(i) do { if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) { long long _t = clock64(); atomicAdd(&g_conv_trace[i], (unsigned long long)(_t - _tr0)); _tr0 = _t; } } while (0)
#else
#define TR_BEGIN
#define TR_ADD(i)
#endif

struct ConvTcParams {
  int32_t dgrad;        // 0 fprop, 1 dgrad
  int32_t ab_format;    // 0 f16, 1 bf16
  int32_t N, H, W;      // extents of the OUTPUT pixel space that is tiled
  int32_t Cred, Nout;   // contraction channels, output channels
  int32_t R, S;
  int32_t off_h, off_w, step_h, step_w; // input coord = output coord + off + tap * step
  int32_t bw, bh, bn, rows;             // patch shape, rows = bw*bh*bn
  int32_t tiles_w, tiles_h, tiles_nb, tiles_nout, total_tiles;
  int32_t BN;                            // 64, 128 or 256
  int32_t cblocks;                       // ceil(Cred / 64)
  uint32_t a_bytes, b_bytes;
  int32_t stages, stage_bytes;           // ring depth and bytes per stage (patch tile + BN filter rows)
  // halo mode (conv_halo_tcgen05_kernel): the (bw+S-1) x (bh+R-1) input patch of a tile is loaded
  // once per channel block and every tap reads a shifted window of it
  int32_t pw, phh;                       // patch width / height in pixels
  int32_t org_w, org_h;                  // input coordinate of the patch origin minus the tile origin
  int32_t a_slot_bytes, a_slots;         // patch slots
  int32_t b_resident;                    // whole filter slice resident in shared memory
  int32_t b_stages;                      // filter ring depth when it is streamed
  void *out;
  int64_t out_sn, out_sh, out_sw;        // element strides of the output (channel stride 1)
  int32_t tma_store;                     // 16-bit output: stage tiles in shared memory, store them by TMA
  int32_t nacc, nacc_log2, acc_cols;     // TMEM accumulator ring: 2 or 4 tiles, acc_cols columns apart
  int32_t epi_alt;                       // epilogue groups of four warps take alternate tiles (BN = 64, staged stores)
  int32_t pair_stages, pair_stage_bytes; // CTA-pair kernel: ring depth, bytes per stage (pixel box + half the filter rows)
  uint32_t *err;
  TcEpilogue epi;
};

// Epilogue warps (2..9) of both convolution kernels: accumulator tile -> registers -> fused
// pointwise chain -> global memory, one output pixel (row) per thread. Two warps share a TMEM lane
// quarter (warp index mod 4) and split the tile's columns in halves: on layers with few channel
// blocks per tile the epilogue, not the MMAs, sets the pace. tfull0 / tempty0 are the barriers of
// accumulator 0; accumulator 1's follow 8 bytes later.
// `pair_rank` < 0: this CTA's tiles are blockIdx.x, + gridDim.x, ... and tempty0 is its own barrier. In the
// CTA-pair kernel (`pair_rank` 0 or 1) cluster c takes the pairs c, c + clusters, ...; pair j is the pixel
// tiles 2j and 2j+1 (the second may lie past the last image: nothing is loaded or stored for it) of one
// channel tile, this CTA drains tile 2j + rank, and the accumulator is released on the LEADER's barrier.
__device__ __forceinline__ void conv_epilogue_warps(const ConvTcParams &p, const CUtensorMap *tmap_c,
                                                    uint32_t staging, uint32_t tmem_base, uint32_t tfull0,
                                                    uint32_t tempty0, int warp, int lane, int pair_rank = -1) {
  const int tiles_pix = p.tiles_w * p.tiles_h * p.tiles_nb;
  const bool paired = pair_rank >= 0;
  const int pairs_pix = (tiles_pix + 1) / 2;
  const int q = warp & 3;
  const int set = (warp - 2) >> 2; // 0 or 1: which group of four warps this one belongs to
  // 64-channel tiles with staged stores: the two groups take alternate tiles, each warp all 64 columns
  // of its 32 rows (the per-tile chain of wait, TMEM load, conversion, staging writes, barriers and
  // store is latency, not throughput: two chains in flight halve its cost per tile). Otherwise both
  // groups work on every tile and split its columns in halves.
  const bool alt = p.epi_alt != 0;
  bool ok = true;
  // This thread's pixel within a tile, and the tile coordinates as mixed-radix digits (w, h, image
  // block, channel tile) that advance by the grid stride with carries: no division inside the loop.
  const int row = q * 32 + lane;
  const int dw = row % p.bw, dh = (row / p.bw) % p.bh, dn = row / (p.bw * p.bh);
  const int64_t row_off0 = (int64_t)dn * p.out_sn + (int64_t)dh * p.out_sh + (int64_t)dw * p.out_sw;
  const uint32_t lt0 = alt ? (uint32_t)set : 0u, lt_step = alt ? 2u : 1u;
  int64_t tile = paired ? (int64_t)(blockIdx.x >> 1) + (int64_t)lt0 * (gridDim.x >> 1) : (int64_t)blockIdx.x + (int64_t)lt0 * gridDim.x;
  const int64_t tile_step = (int64_t)lt_step * (paired ? (gridDim.x >> 1) : gridDim.x);
  const int64_t tile_end = paired ? (int64_t)pairs_pix * p.tiles_nout : (int64_t)p.total_tiles;
  int tw = 0, th = 0, tb = 0, tno = 0, sw = 0, sh = 0, sb = 0, sno = 0;
  if (!paired) {
    const int64_t tp = tile % tiles_pix, sp = tile_step % tiles_pix;
    tno = (int)(tile / tiles_pix); sno = (int)(tile_step / tiles_pix);
    tw = (int)(tp % p.tiles_w); th = (int)((tp / p.tiles_w) % p.tiles_h); tb = (int)(tp / (p.tiles_w * p.tiles_h));
    sw = (int)(sp % p.tiles_w); sh = (int)((sp / p.tiles_w) % p.tiles_h); sb = (int)(sp / (p.tiles_w * p.tiles_h));
  }
  for (uint32_t lt = lt0; ok && tile < tile_end; lt += lt_step, tile += tile_step) {
    const int acc = (int)(lt & (uint32_t)(p.nacc - 1));
    const uint32_t aph = (lt >> p.nacc_log2) & 1;
    if (paired) {
      // long reductions per tile: the divisions are not what bounds these layers
      const int tp = 2 * (int)(tile % pairs_pix) + pair_rank;
      tno = (int)(tile / pairs_pix);
      tw = tp % p.tiles_w; th = (tp / p.tiles_w) % p.tiles_h; tb = tp / (p.tiles_w * p.tiles_h); // tb == tiles_nb: past the end
    }
    const int w = tw * p.bw + dw, h = th * p.bh + dh, n = tb * p.bn + dn;
    const bool row_ok = row < p.rows && w < p.W && h < p.H && n < p.N;
    const int64_t row_off = row_off0 + (int64_t)(tb * p.bn) * p.out_sn + (int64_t)(th * p.bh) * p.out_sh +
                            (int64_t)(tw * p.bw) * p.out_sw;
    const int tw_c = tw, th_c = th, tb_c = tb, tno_c = tno; // this tile's digits; advance for the next one
    const bool tile_ok = tb_c < p.tiles_nb;
    if (!paired) {
      tw += sw; if (tw >= p.tiles_w) { tw -= p.tiles_w; ++th; }
      th += sh; if (th >= p.tiles_h) { th -= p.tiles_h; ++tb; }
      tb += sb; if (tb >= p.tiles_nb) { tb -= p.tiles_nb; ++tno; }
      tno += sno;
    }
    TR_BEGIN;
    if (!mbar_wait(tfull0 + 8u * acc, aph, p.err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
    if (warp == 2) TR_ADD(5); // epilogue: waiting for a finished accumulator
    tc_fence_after();
    const int no0 = tno_c * p.BN;
    const uint32_t taddr = tmem_base + acc * p.acc_cols + ((uint32_t)(q * 32) << 16);
    const int nchunks = p.BN / 32;
    const int c_begin = alt ? 0 : set * (nchunks / 2), c_end = alt ? nchunks : c_begin + nchunks / 2;
    if (p.tma_store) {
      // Converted rows go to a 128-byte-swizzled staging box (128 rows x 64 channels) and leave by
      // ONE tiled TMA store per box: whole 128-byte lines, clipped at the tensor's edges by the TMA
      // unit. (One 16-byte store per lane straight from registers touches 32 different lines per
      // instruction, two instructions per 32-byte sector: those stores alone kept the load/store
      // unit busy for more than half of the kernel on the layers with few K blocks per tile.)
      // Warps that share a box meet at a named barrier. BN = 64: one box per tile shared by all
      // eight warps, the two staging buffers alternate between tiles and ONE barrier per tile says
      // both "this tile is written" and "the other buffer has been read" (the issuing thread waits
      // for its previous store's read before it arrives). Otherwise the four warps of a column half
      // own one buffer and BN / 128 boxes per tile, with a barrier before and after the writes.
      const bool whole = p.BN == 64 && !alt;
      const int bar_id = whole ? 1 : 1 + set, bar_threads = whole ? 256 : 128;
      const bool issuer = lane == 0 && warp == (whole ? 2 : 2 + 4 * set);
      const uint32_t buf = staging + (whole ? (lt & 1u) : (uint32_t)set) * BOX_BYTES;
      const int boxes = whole || alt ? 1 : p.BN / 128;
      const bool bf = p.epi.out_dtype == FB_DT_BFLOAT16;
      // 32 accumulator columns of this thread's row -> fused chain -> 16-bit -> four 16-byte chunks of
      // the row's 128-byte line in the staging box (chunk index XOR row: the 128-byte swizzle)
      auto stage_chunk = [&](uint32_t (&raw)[32], int c, int box_col0) {
        const int nc = no0 + c * 32;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
        if (row_ok && nc < p.Nout) epi_run32(p.epi, v, row_off, nc, min(32, p.Nout - nc));
        const int chunk0 = ((c * 32 - box_col0) >> 3); // 0 or 4
        const uint32_t row_addr = buf + (uint32_t)row * 128u;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t wv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float lo = v[8 * j + 2 * e], hi = v[8 * j + 2 * e + 1];
            if (bf) {
              __nv_bfloat162 h2 = __floats2bfloat162_rn(lo, hi);
              wv[e] = *reinterpret_cast<uint32_t *>(&h2);
            } else {
              __half2 h2 = __floats2half2_rn(lo, hi);
              wv[e] = *reinterpret_cast<uint32_t *>(&h2);
            }
          }
          st_shared_v4(row_addr + (uint32_t)(((chunk0 + j) ^ (row & 7)) << 4), wv[0], wv[1], wv[2], wv[3]);
        }
      };
      auto release_accumulator = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (paired) mbar_arrive_cluster(map_to_cta(tempty0 + 8u * acc, 0));
          else mbar_arrive(tempty0 + 8u * acc);
        }
      };
      uint32_t raw_a[32], raw_b[32];
      tmem_ld_32x32(taddr + c_begin * 32, raw_a);
      if (whole) {
        tmem_ld_wait();
        release_accumulator();
        if (warp == 2) TR_ADD(6);
        stage_chunk(raw_a, c_begin, 0);
        if (warp == 2) TR_ADD(7); // epilogue: convert, staging writes
        fence_proxy_async(); // generic-proxy writes above, async-proxy reads below
        if (issuer) tma_store_wait_read(); // frees the buffer the NEXT tile writes
        if (warp == 2) TR_ADD(8);
        named_barrier_sync(bar_id, bar_threads);
        if (warp == 2) TR_ADD(9);
        if (issuer && tile_ok) {
          tma_store_4d(tmap_c, buf, no0, tw_c * p.bw, th_c * p.bh, tb_c * p.bn);
          tma_store_commit();
        }
        continue;
      }
      // Two chunks per box; the TMEM load of the next chunk is in flight while this one is converted.
      for (int bx = 0; bx < boxes; ++bx) {
        const int box_col0 = ((alt ? 0 : set * boxes) + bx) * 64; // first channel of the box within the tile
        const int c0 = c_begin + bx * 2;
        tmem_ld_wait();
        tmem_ld_32x32(taddr + (c0 + 1) * 32, raw_b);
        if (issuer) tma_store_wait_read(); // the previous store has read this buffer
        named_barrier_sync(bar_id, bar_threads);
        if (warp == 2) TR_ADD(6); // epilogue: set-up + first barrier
        stage_chunk(raw_a, c0, box_col0);
        tmem_ld_wait();
        if (bx + 1 < boxes) tmem_ld_32x32(taddr + (c0 + 2) * 32, raw_a);
        else release_accumulator();
        stage_chunk(raw_b, c0 + 1, box_col0);
        if (warp == 2) TR_ADD(7); // epilogue: convert, staging writes
        fence_proxy_async();
        named_barrier_sync(bar_id, bar_threads);
        if (warp == 2) TR_ADD(9); // epilogue: barrier
        if (issuer && tile_ok) {
          tma_store_4d(tmap_c, buf, no0 + box_col0, tw_c * p.bw, th_c * p.bh, tb_c * p.bn);
          tma_store_commit();
        }
      }
      continue;
    }
#pragma unroll 1
    for (int c = c_begin; c < c_end; ++c) {
      uint32_t raw[32];
      tmem_ld_32x32(taddr + c * 32, raw);
      tmem_ld_wait();
      if (c == c_end - 1) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (paired) mbar_arrive_cluster(map_to_cta(tempty0 + 8u * acc, 0));
          else mbar_arrive(tempty0 + 8u * acc);
        }
      }
      const int nc = no0 + c * 32;
      if (row_ok && nc < p.Nout) {
        const int valid = min(32, p.Nout - nc);
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
        epi_run32(p.epi, v, row_off, nc, valid);
        epi_store32(p.out, p.epi.out_dtype, row_off + nc, v, valid);
      }
    }
  }
  if (p.tma_store && lane == 0 && (warp == 2 || warp == 6)) tma_store_wait_all(); // before the CTA's memory goes away
}

// The per-tap kernel runs one more warp than the halo kernel: a second TMA producer.
constexpr int NUM_THREADS_TAP = NUM_THREADS + 32;
__global__ void __launch_bounds__(NUM_THREADS_TAP, 1)
conv_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_c, const ConvTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  pdl_launch_dependents(); // the next kernel's CTAs may take the SMs this kernel's CTAs leave
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int STAGES = p.stages;
  const uint32_t STAGE_BYTES = (uint32_t)p.stage_bytes;
  const uint32_t bar_base = smem_base + RING_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (MAX_STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * MAX_STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * MAX_STAGES + 2 + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * MAX_STAGES + 4);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), p.epi_alt ? 4 : 8);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (p.tma_store) tma_prefetch_desc(&tmap_c);
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

  const int kblocks = p.R * p.S * p.cblocks;
  const int tiles_pix = p.tiles_w * p.tiles_h * p.tiles_nb;

  if (warp == 0 || warp == NUM_THREADS / 32) {
    // Two producer warps take alternate K blocks (the wait, the expect and the TMA issues of a
    // block are a serial chain of long-latency instructions in the issuing warp; one warp set the
    // pace of the kernel on narrow layers). Both run the whole loop so that slot, phase and tap
    // counters stay in step; whole warp in the loop, one elected lane issues: coordinates and
    // addresses stay in uniform registers, the counters advance without divisions.
    const uint32_t pid = warp == 0 ? 0u : 1u;
    uint32_t it = 0;
    const bool leader = elect_one();
    int s = 0;       // ring slot and its phase, advanced together (the depth is a run-time value)
    uint32_t ph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
      // pixel tiles fastest so that concurrently running CTAs share the filter slice in L2
      const int tp = tile % tiles_pix, tno = tile / tiles_pix;
      const int tw = tp % p.tiles_w, th = (tp / p.tiles_w) % p.tiles_h, tb = tp / (p.tiles_w * p.tiles_h);
      const int w0 = tw * p.bw + p.off_w, h0 = th * p.bh + p.off_h, n0 = tb * p.bn, no0 = tno * p.BN;
      int cb = 0, ts = 0, tr = 0; // channel block (fastest), filter column, filter row
      for (int kb = 0; kb < kblocks; ++kb, ++it, s = (s + 1 == STAGES) ? 0 : s + 1, ph ^= (s == 0)) {
        if ((it & 1u) == pid) {
          if (!mbar_wait_warp(empty_bar(s), ph ^ 1, p.err, ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t sa = smem_base + (uint32_t)s * STAGE_BYTES, sb = sa + A_BYTES;
          const int c0 = cb * BK;
          mbar_expect_tx_elect(full_bar(s), p.a_bytes + p.b_bytes);
          tma_load_4d_elect(sa, &tmap_a, full_bar(s), c0, w0 + ts * p.step_w, h0 + tr * p.step_h, n0);
          if (!p.dgrad) {
            // filter rows ko, contraction channel c contiguous: one K-major box
            tma_load_4d_elect(sb, &tmap_b, full_bar(s), c0, ts, tr, no0);
          } else {
            // filter rows ko (contraction), output channel c contiguous: MN-major 64-wide blocks
            for (int i = 0; i < p.BN / 64; ++i)
              tma_load_4d_elect(sb + i * (64 * BK * 2), &tmap_b, full_bar(s), no0 + 64 * i, ts, tr, c0);
          }
        }
        if (++cb == p.cblocks) {
          cb = 0;
          if (++ts == p.S) {
            ts = 0;
            ++tr;
          }
        }
      }
    }
  } else if (warp == 1) {
    // The whole warp runs the loop (addresses and descriptors stay in uniform registers); one
    // elected lane issues the MMAs and the commits, which track the issuing thread.
    const bool leader = elect_one();
    const uint32_t idesc = make_idesc_f16(BM, p.BN, p.ab_format, 0, p.dgrad);
    const uint32_t b_lbo = p.dgrad ? 64 * BK * 2 : 16, b_kstep = p.dgrad ? 2048 : 32;
    const uint64_t a_desc0 = make_smem_desc(smem_base, 16, 1024);
    const uint64_t b_desc0 = make_smem_desc(smem_base + A_BYTES, b_lbo, 1024);
    uint32_t lt = 0, ph = 0;
    int s = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x, ++lt) {
      const int acc = lt & 1;
      const uint32_t aph = (lt >> 1) & 1;
      if (!mbar_wait_warp(tempty_bar(acc), aph ^ 1, p.err, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * MAX_BN;
      for (int kb = 0; kb < kblocks; ++kb, s = (s + 1 == STAGES) ? 0 : s + 1, ph ^= (s == 0)) {
        if (!mbar_wait_warp(full_bar(s), ph, p.err, ERR_WAIT_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint64_t soff = (uint64_t)(((uint32_t)s * STAGE_BYTES) >> 4);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          tc_mma_f16_elect(d_tmem, a_desc0 + soff + (uint64_t)((k * 32) >> 4),
                           b_desc0 + soff + (uint64_t)((k * b_kstep) >> 4), idesc, (kb > 0 || k > 0) ? 1u : 0u);
        tc_commit_elect(empty_bar(s));
      }
      if (ok) tc_commit_elect(tfull_bar(acc));
    }
  } else {
    conv_epilogue_warps(p, &tmap_c, smem_base + RING_BYTES_STAGED, tmem_base, tfull_bar(0), tempty_bar(0), warp, lane);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}


// CTA-pair variant of the per-tap kernel for tiles of 128 or 256 output channels (cta_group::2): the two
// CTAs of a cluster work on two neighbouring 128-pixel tiles of one channel tile. Each loads its own
// pixel boxes and only ITS HALF of the filter rows of a K block; one MMA of 256 x BN x 16, issued by the
// even CTA, reads both halves and writes each CTA's 128 accumulator rows into that CTA's TMEM. Per CTA and
// K block that is 16 KB + BN/2 x 128 bytes instead of 16 KB + BN x 128 for the same math: six or eight ring
// stages instead of four or six, and one issuing warp (whose barrier waits cost 230-320 clk each even when
// the barrier is complete) for two tiles. No load is multicast: every CTA fetches its own operands; only
// barrier arrivals cross between the two CTAs.
constexpr int PAIR_MAX_STAGES = 8;
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS_TAP, 1)
conv_pair_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ CUtensorMap tmap_c, const ConvTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  pdl_launch_dependents(); // the next kernel's CTAs may take the SMs this kernel's CTAs leave
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u; // the same offset in both CTAs
  const int STAGES = p.pair_stages;
  const uint32_t STAGE_BYTES = (uint32_t)p.pair_stage_bytes;
  const uint32_t bar_base = smem_base + RING_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };                       // used in the leader only
  auto empty_bar = [&](int s) { return bar_base + 8u * (PAIR_MAX_STAGES + s); };  // each CTA's own
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * PAIR_MAX_STAGES + a); };      // each CTA's own
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * PAIR_MAX_STAGES + 2 + a); }; // the leader's
  const uint32_t tmem_slot = bar_base + 8u * (2 * PAIR_MAX_STAGES + 4);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank(); // 0 = leader
  const int cluster_id = blockIdx.x >> 1, nclusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);  // one expect_tx arrival, the bytes of both CTAs
      mbar_init(empty_bar(s), 1); // committed to by the leader's MMA thread
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 16); // eight epilogue warps of each CTA
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (p.tma_store) tma_prefetch_desc(&tmap_c);
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

  const int kblocks = p.R * p.S * p.cblocks;
  const int tiles_pix = p.tiles_w * p.tiles_h * p.tiles_nb;
  const int pairs_pix = (tiles_pix + 1) / 2;
  const int total_pairs = pairs_pix * p.tiles_nout;
  const int half_n = p.BN / 2;
  const uint32_t stage_tx = 2u * (p.a_bytes + (uint32_t)half_n * BK * 2);

  if (warp == 0 || warp == NUM_THREADS / 32) {
    // two producer warps on alternate K blocks, as in the single-CTA kernel: whole warp in the loop,
    // elected lane issues
    const uint32_t pid = warp == 0 ? 0u : 1u;
    uint32_t it = 0;
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int w = cluster_id; w < total_pairs && ok; w += nclusters) {
      const int tp = 2 * (w % pairs_pix) + (int)rank, tno = w / pairs_pix;
      // a pixel tile past the last image (odd tile count) has tb == tiles_nb: its boxes lie outside
      // the tensor and arrive as zeros
      const int tw = tp % p.tiles_w, th = (tp / p.tiles_w) % p.tiles_h, tb = tp / (p.tiles_w * p.tiles_h);
      const int w0 = tw * p.bw + p.off_w, h0 = th * p.bh + p.off_h, n0 = tb * p.bn;
      const int no0 = tno * p.BN + (int)rank * half_n; // this CTA's half of the channel tile
      int cb = 0, ts = 0, tr = 0;
      for (int kb = 0; kb < kblocks; ++kb, ++it, s = (s + 1 == STAGES) ? 0 : s + 1, ph ^= (s == 0)) {
        if ((it & 1u) == pid) {
          TR_BEGIN;
          if (!mbar_wait_warp(empty_bar(s), ph ^ 1, p.err, ERR_WAIT_EMPTY)) { ok = false; break; }
          if (warp == 0) TR_ADD(10);
          const uint32_t lead_full = map_to_cta(full_bar(s), 0);
          if (rank == 0) mbar_expect_tx_elect(full_bar(s), stage_tx);
          const uint32_t sa = smem_base + (uint32_t)s * STAGE_BYTES, sb = sa + A_BYTES;
          const int c0 = cb * BK;
          tma_load_4d_pair_elect(sa, &tmap_a, lead_full, c0, w0 + ts * p.step_w, h0 + tr * p.step_h, n0);
          if (!p.dgrad) {
            tma_load_4d_pair_elect(sb, &tmap_b, lead_full, c0, ts, tr, no0); // box of BN/2 filter rows
          } else {
            for (int i = 0; i < half_n / 64; ++i)
              tma_load_4d_pair_elect(sb + i * (64 * BK * 2), &tmap_b, lead_full, no0 + 64 * i, ts, tr, c0);
          }
          if (warp == 0) TR_ADD(11);
        }
        if (++cb == p.cblocks) {
          cb = 0;
          if (++ts == p.S) {
            ts = 0;
            ++tr;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (rank == 0) {
      const uint32_t idesc = make_idesc_f16(2 * BM, p.BN, p.ab_format, 0, p.dgrad);
      const uint32_t b_lbo = p.dgrad ? 64 * BK * 2 : 16, b_kstep = p.dgrad ? 2048 : 32;
      const uint64_t a_desc0 = make_smem_desc(smem_base, 16, 1024);
      const uint64_t b_desc0 = make_smem_desc(smem_base + A_BYTES, b_lbo, 1024);
      uint32_t lt = 0, ph = 0;
      int s = 0;
      bool ok = true;
      // The NEXT stage's barrier is tested before a stage's MMAs are issued and the answer looked at after
      // them: a wait costs the warp 230-320 clk even on a completed barrier.
      uint32_t peek = mbar_peek_elect(full_bar(0), 0);
      for (int w = cluster_id; w < total_pairs && ok; w += nclusters, ++lt) {
        const int acc = lt & 1;
        const uint32_t aph = (lt >> 1) & 1;
        TR_BEGIN;
        if (!mbar_wait_warp(tempty_bar(acc), aph ^ 1, p.err, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        TR_ADD(12);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * MAX_BN;
        for (int kb = 0; kb < kblocks; ++kb, s = (s + 1 == STAGES) ? 0 : s + 1, ph ^= (s == 0)) {
          if (!__any_sync(0xffffffffu, peek != 0) && !mbar_wait_warp(full_bar(s), ph, p.err, ERR_WAIT_FULL)) { ok = false; break; }
          TR_ADD(13);
          tc_fence_after();
          {
            const int sn = (s + 1 == STAGES) ? 0 : s + 1;
            peek = mbar_peek_elect(full_bar(sn), ph ^ (uint32_t)(sn == 0));
          }
          const uint64_t soff = (uint64_t)(((uint32_t)s * STAGE_BYTES) >> 4);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            tc_mma_f16_pair_elect(d_tmem, a_desc0 + soff + (uint64_t)((k * 32) >> 4),
                                  b_desc0 + soff + (uint64_t)((k * b_kstep) >> 4), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          // the stage is free in BOTH CTAs once these MMAs have read it
          tc_commit_pair_elect(map_to_cta(empty_bar(s), 0));
          tc_commit_pair_elect(map_to_cta(empty_bar(s), 1));
          TR_ADD(14);
        }
        if (ok) { // accumulator complete, in both CTAs' TMEM
          tc_commit_pair_elect(map_to_cta(tfull_bar(acc), 0));
          tc_commit_pair_elect(map_to_cta(tfull_bar(acc), 1));
        }
      }
    }
  } else {
    conv_epilogue_warps(p, &tmap_c, smem_base + RING_BYTES_STAGED, tmem_base, tfull_bar(0), tempty_bar(0), warp, lane,
                        (int)rank);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all(); // neither CTA leaves while the other may still signal its barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// Halo variant for R x S > 1 (unit stride and dilation): the tile is 8 x 16 output pixels of one
// image. Per 64-channel block the producer loads S column-shifted patches of 8 x (16+R-1) input
// pixels (one tiled TMA box each); the window of filter tap (r, s) is then patch s starting r
// image rows (r * 1024 bytes) further down: an ordinary 1024-byte-aligned K-major tile, read
// straight out of shared memory. That cuts the rows the TMA unit moves per tile from R*S*128 to
// S*(16+R-1)*8, which is what bounds the per-tap kernel above on narrow layers. (A single
// (8+S-1)-wide patch with windows shifted by whole pixels also computes the right result but its
// 8-row groups straddle swizzle atoms and the MMAs run ~1.5x slower.) When the whole filter slice
// fits (narrow layers) it is loaded once per CTA and stays resident; otherwise it streams through
// a ring, one (tap, channel block) box per step.
constexpr int HALO_BW = 8, HALO_BH = 16;
constexpr int HALO_MAX_A_SLOTS = 4, HALO_MAX_B_STAGES = 12;
// The halo kernel's eleventh warp is a second MMA issuer (resident filter only).
constexpr int NUM_THREADS_HALO = NUM_THREADS + 32;
__global__ void __launch_bounds__(NUM_THREADS_HALO, 1)
conv_halo_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ CUtensorMap tmap_c, const ConvTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  pdl_launch_dependents(); // the next kernel's CTAs may take the SMs this kernel's CTAs leave
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sb_base = smem_base + (uint32_t)(p.a_slots * p.a_slot_bytes);
  const uint32_t bar_base = smem_base + RING_BYTES;
  auto a_full = [&](int s) { return bar_base + 8u * s; };
  auto a_empty = [&](int s) { return bar_base + 8u * (HALO_MAX_A_SLOTS + s); };
  auto b_full = [&](int s) { return bar_base + 8u * (2 * HALO_MAX_A_SLOTS + s); };
  auto b_empty = [&](int s) { return bar_base + 8u * (2 * HALO_MAX_A_SLOTS + HALO_MAX_B_STAGES + s); };
  const uint32_t tfull0 = bar_base + 8u * (2 * HALO_MAX_A_SLOTS + 2 * HALO_MAX_B_STAGES);
  const uint32_t tempty0 = tfull0 + 32u; // up to four accumulators
  const uint32_t tmem_slot = tfull0 + 64u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int taps = p.R * p.S;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.a_slots; ++s) {
      mbar_init(a_full(s), 1);
      mbar_init(a_empty(s), 1);
    }
    for (int s = 0; s < HALO_MAX_B_STAGES; ++s) {
      mbar_init(b_full(s), 1);
      mbar_init(b_empty(s), 1);
    }
    for (int a = 0; a < 4; ++a) {
      mbar_init(tfull0 + 8u * a, 1);
      mbar_init(tempty0 + 8u * a, p.epi_alt ? 4 : 8);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (p.tma_store) tma_prefetch_desc(&tmap_c);
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

  const int tiles_pix = p.tiles_w * p.tiles_h * p.tiles_nb;
  const uint32_t patch_bytes = (uint32_t)(HALO_BW * p.phh) * 128u; // one column-shifted patch

  // one filter box: rows of output channels (fprop, K-major) or of contraction channels (dgrad,
  // MN-major 64-wide blocks), for tap (tr, ts) and channel block cb
  auto load_filter = [&](uint32_t dst, uint32_t bar, int cb, int tr, int ts, int no0) {
    const int c0 = cb * BK;
    if (!p.dgrad) {
      tma_load_4d(dst, &tmap_b, bar, c0, ts, tr, no0);
    } else {
      for (int i = 0; i < p.BN / 64; ++i) tma_load_4d(dst + i * (64 * BK * 2), &tmap_b, bar, no0 + 64 * i, ts, tr, c0);
    }
  };

  if (warp == 0) {
    const bool leader = elect_one();
    bool ok = true;
    if (p.b_resident && leader) {
      // the whole filter slice, (cb, tap) boxes back to back; completion on b_full(0)
      mbar_expect_tx(b_full(0), (uint32_t)(p.cblocks * taps) * p.b_bytes);
      for (int cb = 0; cb < p.cblocks; ++cb)
        for (int t = 0; t < taps; ++t)
          load_filter(sb_base + (uint32_t)(cb * taps + t) * p.b_bytes, b_full(0), cb, t / p.S, t % p.S, 0);
    }
    int sa = 0, sbs = 0;
    uint32_t pha = 0, phb = 0;
    for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
      const int tp = tile % tiles_pix, tno = tile / tiles_pix;
      const int tw = tp % p.tiles_w, th = (tp / p.tiles_w) % p.tiles_h, tb = tp / (p.tiles_w * p.tiles_h);
      const int w0 = tw * p.bw + p.org_w, h0 = th * p.bh + p.org_h, no0 = tno * p.BN;
      for (int cb = 0; cb < p.cblocks && ok; ++cb) {
        TR_BEGIN;
        if (!mbar_wait_warp(a_empty(sa), pha ^ 1, p.err, ERR_WAIT_EMPTY)) { ok = false; break; }
        TR_ADD(0); // producer: waiting for a free patch slot
        if (leader) {
          mbar_expect_tx(a_full(sa), (uint32_t)p.S * patch_bytes);
          for (int ss = 0; ss < p.S; ++ss)
            tma_load_4d(smem_base + (uint32_t)(sa * p.a_slot_bytes) + (uint32_t)ss * patch_bytes, &tmap_a, a_full(sa),
                        cb * BK, w0 + ss, h0, tb);
        }
        __syncwarp();
        TR_ADD(1); // producer: expect + TMA issue
        sa = (sa + 1 == p.a_slots) ? 0 : sa + 1;
        pha ^= (sa == 0);
        if (!p.b_resident) {
          for (int t = 0; t < taps; ++t) {
            if (!mbar_wait_warp(b_empty(sbs), phb ^ 1, p.err, ERR_WAIT_EMPTY)) { ok = false; break; }
            if (leader) {
              mbar_expect_tx(b_full(sbs), p.b_bytes);
              load_filter(sb_base + (uint32_t)sbs * p.b_bytes, b_full(sbs), cb, t / p.S, t % p.S, no0);
            }
            sbs = (sbs + 1 == p.b_stages) ? 0 : sbs + 1;
            phb ^= (sbs == 0);
          }
        }
      }
    }
  } else if (warp == 1 || warp == NUM_THREADS / 32) {
    // MMA issue. The tensor pipe queues only a few instructions: while the issuing warp sits in the
    // barrier waits between two tiles (a few hundred cycles even when both are already complete) the
    // pipe runs dry, and a 128 x 64 x 16 MMA lasts only 48 clk. With the filter resident, two warps
    // therefore issue alternate tiles (each its own accumulators and patch slots), so that one of
    // them is always issuing; MMAs of different tiles may interleave in the pipe. With a streamed
    // filter the ring is consumed in tile order and warp 1 issues alone.
    const bool two = p.b_resident != 0;
    const uint32_t first = (two && warp != 1) ? 1u : 0u, step = two ? 2u : 1u;
    const uint32_t idesc = make_idesc_f16(BM, p.BN, p.ab_format, 0, p.dgrad);
    const uint32_t b_lbo = p.dgrad ? 64 * BK * 2 : 16, b_kstep = p.dgrad ? 2048 : 32;
    const uint64_t a_desc0 = make_smem_desc(smem_base, 16, 1024);
    const uint64_t b_desc0 = make_smem_desc(sb_base, b_lbo, 1024);
    bool ok = warp == 1 || two;
    const bool lean = p.b_resident && p.R == 3 && p.S == 3;
    const uint32_t a_hi = (uint32_t)(a_desc0 >> 32), b_hi = (uint32_t)(b_desc0 >> 32);
    uint32_t a_off[9]; // descriptor offset (16-byte units) of each tap's window within a patch slot
#pragma unroll
    for (int t = 0; t < 9; ++t) {
      const int tr = t / 3, ts = t % 3;
      const int rr = p.dgrad ? 2 - tr : tr, ss = p.dgrad ? 2 - ts : ts;
      a_off[t] = ((uint32_t)ss * patch_bytes + (uint32_t)rr * 1024u) >> 4;
    }
    if (ok && p.b_resident) ok = mbar_wait_warp(b_full(0), 0, p.err, ERR_WAIT_FULL);
    int sbs = 0;
    uint32_t phb = 0;
    // patch slot and phase of this warp's first tile (channel blocks are numbered through the tiles)
    int sa_next = (int)((first * (uint32_t)p.cblocks) % (uint32_t)p.a_slots);
    uint32_t pha_next = ((first * (uint32_t)p.cblocks) / (uint32_t)p.a_slots) & 1u;
    for (uint32_t lt = first; ok; lt += step) {
      const int64_t tile = (int64_t)blockIdx.x + (int64_t)lt * gridDim.x;
      if (tile >= p.total_tiles) break;
      const int acc = (int)(lt & (uint32_t)(p.nacc - 1));
      const uint32_t aph = (lt >> p.nacc_log2) & 1;
      int sa = sa_next;
      uint32_t pha = pha_next;
      // the slot of this warp's next tile: `step` tiles of cblocks blocks further round the ring
      for (uint32_t adv = step * (uint32_t)p.cblocks; adv > 0; --adv) {
        sa_next = (sa_next + 1 == p.a_slots) ? 0 : sa_next + 1;
        pha_next ^= (sa_next == 0);
      }
      TR_BEGIN;
      if (!mbar_wait_warp(tempty0 + 8u * acc, aph ^ 1, p.err, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
      TR_ADD(2); // MMA warp: waiting for a drained accumulator
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * p.acc_cols;
      for (int cb = 0; cb < p.cblocks && ok; ++cb) {
        if (!mbar_wait_warp(a_full(sa), pha, p.err, ERR_WAIT_FULL)) { ok = false; break; }
        TR_ADD(3); // MMA warp: waiting for the patch to land
        tc_fence_after();
        const uint64_t ad = a_desc0 + (uint64_t)((uint32_t)(sa * p.a_slot_bytes) >> 4);
        if (lean) {
          // 3 x 3 taps, resident filter: the 36 MMAs straight-line, window and tap offsets from registers.
          // The issue rate matters: each instruction lasts 48 clk on a 64-channel layer and only a few
          // are queued, so address arithmetic between two of them is tensor time lost.
          const uint32_t a_lo = (uint32_t)ad, b_lo = (uint32_t)b_desc0 + (uint32_t)cb * 9u * (p.b_bytes >> 4);
#pragma unroll
          for (int t = 0; t < 9; ++t) {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              tc_mma_f16_elect(d_tmem, ((uint64_t)a_hi << 32) | (a_lo + a_off[t] + (uint32_t)(k * 2)),
                               ((uint64_t)b_hi << 32) | (b_lo + (uint32_t)t * (p.b_bytes >> 4) + (uint32_t)k * (b_kstep >> 4)),
                               idesc, (cb > 0 || t > 0 || k > 0) ? 1u : 0u);
          }
        } else {
        int tr = 0, ts = 0;
        for (int t = 0; t < taps; ++t) {
          uint64_t bd;
          if (p.b_resident) {
            bd = b_desc0 + (uint64_t)(((uint32_t)(cb * taps + t) * p.b_bytes) >> 4);
          } else {
            if (!mbar_wait_warp(b_full(sbs), phb, p.err, ERR_WAIT_FULL)) { ok = false; break; }
            tc_fence_after();
            bd = b_desc0 + (uint64_t)(((uint32_t)sbs * p.b_bytes) >> 4);
          }
          // window of tap (tr, ts): fprop reads input (h + tr, w + ts) relative to the patch
          // origin, dgrad reads (h + R-1-tr, w + S-1-ts)
          const int rr = p.dgrad ? p.R - 1 - tr : tr, ss = p.dgrad ? p.S - 1 - ts : ts;
          const uint64_t aw = ad + (uint64_t)(((uint32_t)ss * patch_bytes + (uint32_t)rr * 1024u) >> 4);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)
            tc_mma_f16_elect(d_tmem, aw + (uint64_t)((k * 32) >> 4), bd + (uint64_t)((k * b_kstep) >> 4), idesc,
                             (cb > 0 || t > 0 || k > 0) ? 1u : 0u);
          if (!p.b_resident) {
            tc_commit_elect(b_empty(sbs));
            sbs = (sbs + 1 == p.b_stages) ? 0 : sbs + 1;
            phb ^= (sbs == 0);
          }
          if (++ts == p.S) {
            ts = 0;
            ++tr;
          }
        }
        }
        tc_commit_elect(a_empty(sa));
        TR_ADD(4); // MMA warp: issuing the taps' MMAs
        sa = (sa + 1 == p.a_slots) ? 0 : sa + 1;
        pha ^= (sa == 0);
      }
      if (ok) tc_commit_elect(tfull0 + 8u * acc);
    }
  } else {
    conv_epilogue_warps(p, &tmap_c, smem_base + RING_BYTES_STAGED, tmem_base, tfull0, tempty0, warp, lane);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Whether clusters of two CTAs of the pair kernel can be resident on this device (asked once per device),
// and whether the caller left the pair kernel enabled.
static bool conv_pair_usable(int device) {
  static const bool enabled = [] {
    const char *e = getenv("FUSILLI_B200_CONV_PAIR");
    return !(e && e[0] == '0');
  }();
  if (!enabled || device < 0 || device >= 64) return false;
  static std::mutex mu;
  static int8_t state[64] = {0}; // 0 unknown, 1 usable, -1 not
  std::lock_guard<std::mutex> lock(mu);
  if (state[device] == 0) {
    state[device] = -1;
    if (set_max_dynamic_smem(reinterpret_cast<const void *>(conv_pair_tcgen05_kernel), SMEM_BYTES, device) ==
        cudaSuccess) {
      cudaLaunchConfig_t cfg;
      memset(&cfg, 0, sizeof(cfg));
      cfg.gridDim = dim3(2, 1, 1);
      cfg.blockDim = dim3(NUM_THREADS_TAP, 1, 1);
      cfg.dynamicSmemBytes = SMEM_BYTES;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 2;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, reinterpret_cast<const void *>(conv_pair_tcgen05_kernel), &cfg) ==
              cudaSuccess &&
          n >= 1)
        state[device] = 1;
    }
    (void)cudaGetLastError();
  }
  return state[device] == 1;
}

// ---- host -----------------------------------------------------------------------------

struct ConvView {
  int dgrad;
  int N, H, W;          // tiled (output) pixel space
  int IH, IW;           // spatial extent of the tensor the A patches are read from
  int Cred, Nout, R, S, pad_h, pad_w, dil_h, dil_w;
  int in_id, w_id;      // tensor ids: activation-like input, filter
  bool pointwise_1x1;
};

bool is16(int dt) { return dt == FB_DT_HALF || dt == FB_DT_BFLOAT16; }
bool isfl(int dt) { return dt == FB_DT_HALF || dt == FB_DT_BFLOAT16 || dt == FB_DT_FLOAT; }

bool channels_last_dense(const TensorInfo &t) {
  if (t.rank != 4) return false;
  const int64_t C = t.dims[1], H = t.dims[2], W = t.dims[3];
  return t.strides[1] == 1 && t.strides[3] == C && t.strides[2] == W * C && t.strides[0] == H * W * C;
}

bool conv_view(const Plan &p, const Step &s, ConvView &v) {
  const fb_node_desc &d = p.nodes[s.node].d;
  if (d.op != FB_OP_CONV_FPROP && d.op != FB_OP_CONV_DGRAD) return false;
  if (d.num_spatial != 2) return false;
  if (d.stride[0] != 1 || d.stride[1] != 1) return false;
  const TensorInfo &in = p.tensors[d.inputs[0]], &w = p.tensors[d.inputs[1]];
  const TensorInfo &o0 = p.tensors[d.outputs[0]], &out = p.tensors[s.out_tensor];
  if (!is16(in.dtype) || in.dtype != w.dtype || !isfl(out.dtype) || !isfl(o0.dtype)) return false;
  if (!channels_last_dense(in) || !channels_last_dense(w) || !channels_last_dense(out)) return false;
  v.dgrad = d.op == FB_OP_CONV_DGRAD;
  v.in_id = d.inputs[0];
  v.w_id = d.inputs[1];
  v.R = (int)w.dims[2]; v.S = (int)w.dims[3];
  v.pad_h = (int)d.padding[0]; v.pad_w = (int)d.padding[1];
  v.dil_h = (int)d.dilation[0]; v.dil_w = (int)d.dilation[1];
  v.N = (int)out.dims[0]; v.H = (int)out.dims[2]; v.W = (int)out.dims[3];
  v.IH = (int)in.dims[2]; v.IW = (int)in.dims[3];
  const int64_t K = w.dims[0], Cf = w.dims[1];
  if (!v.dgrad) {
    if (in.dims[1] != Cf) return false; // groups == 1 only
    v.Cred = (int)Cf; v.Nout = (int)K;
  } else {
    if (out.dims[1] != Cf) return false;
    v.Cred = (int)K; v.Nout = (int)Cf;
  }
  if (v.Cred % 8 || v.Nout % 8) return false; // TMA: 16-byte strides
  if (v.Cred < 64 || v.Nout < 32) return false;
  if ((int64_t)v.N * v.H * v.W < 128) return false;
  if (out.dims[0] >= (1 << 30) || (int64_t)v.N * v.H * v.W >= (1ll << 31)) return false;
  v.pointwise_1x1 = v.R == 1 && v.S == 1 && v.pad_h == 0 && v.pad_w == 0 && v.IH == v.H && v.IW == v.W;
  return true;
}

int conv_epi_kind(const Plan &p, const Step &s, const EpilogueOpInfo &op) {
  if (op.operand < 0) return 0;
  const TensorInfo &o = p.tensors[op.operand];
  const TensorInfo &c = p.tensors[s.out_tensor];
  if (o.role == FB_TENSOR_SCALAR) return 2;
  if (o.rank == 4 && o.dims[0] == 1 && o.dims[2] == 1 && o.dims[3] == 1 && o.dims[1] == c.dims[1] &&
      o.strides[1] == 1)
    return 1;
  bool full = o.rank == c.rank;
  for (int i = 0; full && i < c.rank; ++i)
    if (o.dims[i] != c.dims[i] || (c.dims[i] > 1 && o.strides[i] != c.strides[i])) full = false;
  return full ? 3 : -1;
}

// Patch shape (bw, bh, bn) with bw*bh*bn <= 128 that wastes the fewest tile rows.
void choose_patch_search(int N, int H, int W, int &bw, int &bh, int &bn);
void choose_patch(int N, int H, int W, int &bw, int &bh, int &bn) {
  // asked on every launch: remember the answer per (N, H, W)
  struct Shape { int bw, bh, bn; };
  static std::mutex mu;
  static std::unordered_map<uint64_t, Shape> memo;
  const uint64_t key = ((uint64_t)(uint32_t)N << 42) ^ ((uint64_t)(uint32_t)H << 21) ^ (uint64_t)(uint32_t)W;
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = memo.find(key);
    if (it != memo.end()) {
      bw = it->second.bw; bh = it->second.bh; bn = it->second.bn;
      return;
    }
  }
  choose_patch_search(N, H, W, bw, bh, bn);
  std::lock_guard<std::mutex> lock(mu);
  if (memo.size() > 4096) memo.clear();
  memo[key] = Shape{bw, bh, bn};
}

void choose_patch_search(int N, int H, int W, int &bw, int &bh, int &bn) {
  double best = -1.0;
  bw = std::min(W, 128); bh = 1; bn = 1;
  for (int w = 1; w <= std::min(W, 128); ++w) {
    for (int h = 1; h <= std::min(H, 128 / w); ++h) {
      // the box may span several images: a (w x h) window of n consecutive images
      const int n = std::max(1, std::min(N, 128 / (w * h)));
      const int64_t tiles = (int64_t)((W + w - 1) / w) * ((H + h - 1) / h) * ((N + n - 1) / n);
      const double eff = (double)N * H * W / ((double)tiles * 128.0);
      // prefer wider patches on ties: longer contiguous runs per TMA row
      if (eff > best + 1e-9 || (eff > best - 1e-9 && w > bw)) {
        best = eff; bw = w; bh = h; bn = n;
      }
    }
  }
}

} // namespace

bool conv_tc_eligible(const Plan &p, const Step &s) {
  ConvView v;
  if (!conv_view(p, s, v)) return false;
  for (int i = 0; i < s.num_epilogue; ++i) {
    if (conv_epi_kind(p, s, s.epilogue[i]) < 0) return false;
    if (!isfl(p.tensors[s.epilogue[i].out_tensor].dtype)) return false;
    if (s.epilogue[i].operand >= 0 && !isfl(p.tensors[s.epilogue[i].operand].dtype)) return false;
  }
  return true;
}

fb_status launch_conv_tc(const ExecContext &cx, const Step &s) {
  const Plan &plan = *cx.plan;
  const fb_node_desc &d = plan.nodes[s.node].d;
  ConvView v;
  FB_REQUIRE(conv_view(plan, s, v), FB_INTERNAL_ERROR, "conv_tcgen05: step is not eligible");
  const TensorInfo &in = plan.tensors[v.in_id], &wt = plan.tensors[v.w_id];
  const TensorInfo &out = plan.tensors[s.out_tensor];
  const void *inptr = cx.tensor_ptr(v.in_id);
  const void *wptr = cx.tensor_ptr(v.w_id);
  void *optr = cx.tensor_ptr(s.out_tensor);
  FB_REQUIRE(inptr && wptr && optr, FB_INTERNAL_ERROR, "conv_tcgen05: tensor has no buffer");
  FB_REQUIRE(((uintptr_t)inptr % 16 == 0) && ((uintptr_t)wptr % 16 == 0), FB_INVALID_ARGUMENT,
             "conv_tcgen05: operand buffers must be 16-byte aligned");

  static thread_local ConvTcParams p;
  memset(&p, 0, sizeof(p));
  p.dgrad = v.dgrad;
  p.ab_format = in.dtype == FB_DT_BFLOAT16 ? 1 : 0;
  p.Cred = v.Cred; p.Nout = v.Nout; p.R = v.R; p.S = v.S;
  p.cblocks = (v.Cred + BK - 1) / BK;
  p.BN = v.Nout > 128 ? 256 : (v.Nout > 64 ? 128 : 64);
  // tiled pixel space and the activation tensor as TMA sees it: (C, W, H, N)
  uint64_t a_dims[4], a_str[3];
  const int64_t inC = in.dims[1];
  if (v.pointwise_1x1) {
    // no halo: (n,h,w) collapses into one axis and every tile is full
    const int64_t pix = (int64_t)v.N * v.H * v.W;
    p.N = 1; p.H = 1; p.W = (int32_t)pix;
    p.bw = 128; p.bh = 1; p.bn = 1;
    a_dims[0] = inC; a_dims[1] = pix; a_dims[2] = 1; a_dims[3] = 1;
    a_str[0] = inC * 2; a_str[1] = pix * inC * 2; a_str[2] = pix * inC * 2;
    p.out_sn = 0; p.out_sh = 0; p.out_sw = out.strides[3];
  } else {
    p.N = v.N; p.H = v.H; p.W = v.W;
    choose_patch(v.N, v.H, v.W, p.bw, p.bh, p.bn);
    a_dims[0] = inC; a_dims[1] = v.IW; a_dims[2] = v.IH; a_dims[3] = in.dims[0];
    a_str[0] = inC * 2; a_str[1] = (uint64_t)v.IW * inC * 2; a_str[2] = (uint64_t)v.IH * v.IW * inC * 2;
    p.out_sn = out.strides[0]; p.out_sh = out.strides[2]; p.out_sw = out.strides[3];
  }
  // Halo path: taps read shifted windows of one patch per channel block. Taken when the fixed
  // 8 x 16 tile wastes little of the image.
  // 16-bit outputs leave through staged TMA stores; the staging tiles come out of the ring's space
  p.tma_store = is16(out.dtype) ? 1 : 0;
  p.nacc = 2; p.nacc_log2 = 1; p.acc_cols = MAX_BN;
  p.epi_alt = (p.tma_store && p.BN == 64) ? 1 : 0;
  const int ring_bytes = p.tma_store ? RING_BYTES_STAGED : RING_BYTES;
  bool halo = false;
  if (!v.pointwise_1x1 && v.R * v.S > 1 && v.dil_h == 1 && v.dil_w == 1 && v.R <= 7 && v.S <= 7) {
    const int64_t tiles = (int64_t)((v.W + HALO_BW - 1) / HALO_BW) * ((v.H + HALO_BH - 1) / HALO_BH) * v.N;
    halo = (double)v.N * v.H * v.W / ((double)tiles * 128.0) >= 0.6;
    // Measured: with the filter streamed (one box per tap) the halo kernel is slower than the
    // per-tap kernel (522 against 747 TFLOP/s on 28x28 C128), with the filter resident faster
    // (494 against 431 on 56x56 C64), so it is taken only when the filter slice stays resident.
    const int64_t filter_bytes = (int64_t)p.cblocks * v.R * v.S * p.BN * BK * 2;
    const int64_t slot_bytes = (int64_t)v.S * HALO_BW * (HALO_BH + v.R - 1) * 128;
    halo = halo && v.Nout <= p.BN && filter_bytes + 2 * slot_bytes <= ring_bytes;
  }
  if (halo) {
    p.bw = HALO_BW; p.bh = HALO_BH; p.bn = 1;
    p.pw = HALO_BW + v.S - 1; p.phh = HALO_BH + v.R - 1;
    // fprop: input = output - pad + tap; dgrad: input(dY) = output(dX) + pad - tap, so the patch
    // starts (R-1, S-1) earlier and the taps are read mirrored
    p.org_w = v.dgrad ? v.pad_w - (v.S - 1) : -v.pad_w;
    p.org_h = v.dgrad ? v.pad_h - (v.R - 1) : -v.pad_h;
    p.a_slot_bytes = v.S * HALO_BW * p.phh * 128; // S column-shifted patches of 8 x phh pixels
    // two accumulators per issuing warp, so that neither waits for the tile it just finished to drain
    if (p.BN <= 128) { p.nacc = 4; p.nacc_log2 = 2; p.acc_cols = 128; }
  }
  p.rows = p.bw * p.bh * p.bn;
  if (!v.dgrad) { p.off_h = -v.pad_h; p.off_w = -v.pad_w; p.step_h = v.dil_h; p.step_w = v.dil_w; }
  else          { p.off_h = v.pad_h;  p.off_w = v.pad_w;  p.step_h = -v.dil_h; p.step_w = -v.dil_w; }
  p.tiles_w = (p.W + p.bw - 1) / p.bw;
  p.tiles_h = (p.H + p.bh - 1) / p.bh;
  p.tiles_nb = (p.N + p.bn - 1) / p.bn;
  p.tiles_nout = (p.Nout + p.BN - 1) / p.BN;
  const int64_t total = (int64_t)p.tiles_w * p.tiles_h * p.tiles_nb * p.tiles_nout;
  FB_REQUIRE(total < (1ll << 31), FB_NOT_IMPLEMENTED, "conv_tcgen05: too many tiles");
  p.total_tiles = (int)total;
  p.a_bytes = (uint32_t)p.rows * BK * 2;
  p.b_bytes = (uint32_t)p.BN * BK * 2;
  p.stage_bytes = A_BYTES + p.BN * BK * 2;
  p.stages = std::min(MAX_STAGES, ring_bytes / p.stage_bytes);
  if (halo) {
    const int64_t filter_bytes = (int64_t)p.cblocks * v.R * v.S * p.b_bytes;
    p.b_resident = p.tiles_nout == 1 && filter_bytes + 2 * p.a_slot_bytes <= ring_bytes;
    if (p.b_resident) {
      p.a_slots = (int)std::min<int64_t>(HALO_MAX_A_SLOTS, (ring_bytes - filter_bytes) / p.a_slot_bytes);
      p.b_stages = 1;
    } else {
      p.a_slots = 2;
      p.b_stages = (int)std::min<int64_t>(HALO_MAX_B_STAGES, (ring_bytes - 2 * p.a_slot_bytes) / p.b_bytes);
    }
  }
  // CTA pairs on tiles of 128 / 256 channels with at least eight K blocks per tile: a stage is 24 / 32 KB per
  // CTA instead of 32 / 48 KB (more stages round the ring, whose round trip sets the pace of the single-CTA
  // kernel on these layers) and one issuing warp serves two tiles. Measured: 28x28 C128 3x3 68.6 -> 64.5 us
  // fprop, 72.7 -> 66.6 dgrad; 7x7 C512 3x3 62.4 -> 58.4 / 60.4; 14x14 1024 -> 256 dgrad 35.8 -> 33.8; with only
  // four K blocks (14x14 256 -> 1024 fprop) the pair is slower (56 against 46 us) and is not taken.
  // FUSILLI_B200_CONV_PAIR=0 keeps the single-CTA kernel.
  const int tiles_pix_all = p.tiles_w * p.tiles_h * p.tiles_nb;
  const bool use_pair = !halo && p.BN >= 128 && p.R * p.S * p.cblocks >= 8 && tiles_pix_all >= 2 &&
                        conv_pair_usable(cx.dev->ordinal);
  p.pair_stage_bytes = A_BYTES + (p.BN / 2) * BK * 2;
  p.pair_stages = std::min(PAIR_MAX_STAGES, ring_bytes / p.pair_stage_bytes);
  p.out = optr;
  p.err = cx.dev->error_word;
  p.epi.num_ops = s.num_epilogue;
  p.epi.acc_round_dtype = plan.tensors[d.outputs[0]].dtype;
  p.epi.out_dtype = out.dtype;
  for (int i = 0; i < s.num_epilogue; ++i) {
    const EpilogueOpInfo &src = s.epilogue[i];
    TcEpiOp &op = p.epi.ops[i];
    op.mode = src.mode;
    op.kind = conv_epi_kind(plan, s, src);
    op.value_is_in1 = src.value_is_in1;
    op.round_dtype = plan.tensors[src.out_tensor].dtype;
    memcpy(op.prm, src.fparams, sizeof(op.prm));
    if (src.operand >= 0) {
      const TensorInfo &o = plan.tensors[src.operand];
      op.dtype = o.dtype;
      if (op.kind == 2) op.scalar = (float)o.scalar;
      else {
        op.ptr = cx.tensor_ptr(src.operand);
        FB_REQUIRE(op.ptr != nullptr, FB_INTERNAL_ERROR, "conv_tcgen05: epilogue operand has no buffer");
      }
    }
  }
  CUtensorMap tmA, tmB, tmC;
  const char *why = "";
  {
    uint32_t box[4] = {BK, (uint32_t)p.bw, (uint32_t)(halo ? p.phh : p.bh), (uint32_t)p.bn};
    FB_REQUIRE(encode_tmap_2byte(&tmA, inptr, 4, a_dims, a_str, box, &why), FB_RUNTIME_FAILURE, why);
    // filter KRSC as (C, S, R, K)
    const int64_t Cf = wt.dims[1];
    uint64_t w_dims[4] = {(uint64_t)Cf, (uint64_t)v.S, (uint64_t)v.R, (uint64_t)wt.dims[0]};
    uint64_t w_str[3] = {(uint64_t)Cf * 2, (uint64_t)v.S * Cf * 2, (uint64_t)v.R * v.S * Cf * 2};
    uint32_t wbox_f[4] = {BK, 1, 1, (uint32_t)(use_pair ? p.BN / 2 : p.BN)}; // a CTA of a pair loads half the rows
    uint32_t wbox_d[4] = {64, 1, 1, BK};
    FB_REQUIRE(encode_tmap_2byte(&tmB, wptr, 4, w_dims, w_str, v.dgrad ? wbox_d : wbox_f, &why),
               FB_RUNTIME_FAILURE, why);
    if (p.tma_store) {
      // the output as (channels, W, H, N) -- or (channels, pixels, 1, 1) for a collapsed 1x1 layer --
      // stored in boxes of 64 channels by the tile's pixel patch
      const uint64_t oc = (uint64_t)out.dims[1];
      uint64_t c_dims[4], c_str[3];
      if (v.pointwise_1x1) {
        const uint64_t pix = (uint64_t)v.N * v.H * v.W;
        c_dims[0] = oc; c_dims[1] = pix; c_dims[2] = 1; c_dims[3] = 1;
        c_str[0] = oc * 2; c_str[1] = pix * oc * 2; c_str[2] = pix * oc * 2;
      } else {
        c_dims[0] = oc; c_dims[1] = (uint64_t)v.W; c_dims[2] = (uint64_t)v.H; c_dims[3] = (uint64_t)v.N;
        c_str[0] = oc * 2; c_str[1] = (uint64_t)v.W * oc * 2; c_str[2] = (uint64_t)v.H * v.W * oc * 2;
      }
      uint32_t cbox[4] = {64, (uint32_t)p.bw, (uint32_t)p.bh, (uint32_t)p.bn};
      FB_REQUIRE(((uintptr_t)optr % 16) == 0, FB_INVALID_ARGUMENT, "conv_tcgen05: output buffer must be 16-byte aligned");
      FB_REQUIRE(encode_tmap_2byte(&tmC, optr, 4, c_dims, c_str, cbox, &why), FB_RUNTIME_FAILURE, why);
    } else {
      tmC = tmA; // unused by the kernel
    }
  }
  if (use_pair) {
    cudaError_t pe = set_max_dynamic_smem(reinterpret_cast<const void *>(conv_pair_tcgen05_kernel), SMEM_BYTES, cx.dev->ordinal);
    FB_REQUIRE(pe == cudaSuccess, FB_RUNTIME_FAILURE,
               std::string("conv_pair_tcgen05: cannot reserve shared memory: ") + cudaGetErrorString(pe));
    const int total_pairs = ((tiles_pix_all + 1) / 2) * p.tiles_nout;
    const int clusters = std::min<int>(total_pairs, cx.dev->sm_count / 2);
    FB_CUDA_OK(launch_pdl(conv_pair_tcgen05_kernel, dim3(2 * clusters), dim3(NUM_THREADS_TAP), SMEM_BYTES, cx.dev->stream, tmA, tmB,
                          tmC, p));
    return FB_OK;
  }
  cudaError_t ae = set_max_dynamic_smem(reinterpret_cast<const void *>(conv_tcgen05_kernel), SMEM_BYTES, cx.dev->ordinal);
  FB_REQUIRE(ae == cudaSuccess, FB_RUNTIME_FAILURE,
             std::string("conv_tcgen05: cannot reserve shared memory: ") + cudaGetErrorString(ae));
  int grid = std::min<int>(p.total_tiles, cx.dev->sm_count);
  if (halo) {
    ae = set_max_dynamic_smem(reinterpret_cast<const void *>(conv_halo_tcgen05_kernel), SMEM_BYTES, cx.dev->ordinal);
    FB_REQUIRE(ae == cudaSuccess, FB_RUNTIME_FAILURE,
               std::string("conv_halo_tcgen05: cannot reserve shared memory: ") + cudaGetErrorString(ae));
    FB_CUDA_OK(launch_pdl(conv_halo_tcgen05_kernel, dim3(grid), dim3(NUM_THREADS_HALO), SMEM_BYTES, cx.dev->stream, tmA, tmB, tmC, p));
    return FB_OK;
  }
  FB_CUDA_OK(launch_pdl(conv_tcgen05_kernel, dim3(grid), dim3(NUM_THREADS_TAP), SMEM_BYTES, cx.dev->stream, tmA, tmB, tmC, p));
  return FB_OK;
}

} // namespace fb

#ifdef FB_CONV_TRACE
FB_EXPORT fb_status fb_debug_conv_trace(unsigned long long *out, int reset) {
  cudaMemcpyFromSymbol(out, fb::g_conv_trace, sizeof(unsigned long long) * 32);
  if (reset) {
    unsigned long long z[32] = {0};
    cudaMemcpyToSymbol(fb::g_conv_trace, z, sizeof(z));
  }
  return FB_OK;
}
#endif

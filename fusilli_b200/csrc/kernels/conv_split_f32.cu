// fp32 forward convolution on the tensor cores with fp32-grade results: 2-D, stride-1,
// channels-last (NHWC / KRSC), groups = 1, C a multiple of 64.
//
// bf16 tensor-core products are exact in fp32, so an fp32 value written as the sum of three bf16
// pieces (x = x0 + x1 + x2, 8 significant bits each) multiplies exactly piece by piece. Of the nine
// piece products of x * w the three below 2^-24 of the result are dropped; the other six are six
// "channel blocks" of one implicit GEMM whose contraction axis is (tap, piece pair, channel):
//   a pre-pass writes X' = [x0 | x1 | x2] and W' = [w0 | w1 | w2] in bf16 (3C channels each);
//   a ring stage holds, for one (tap, 64-channel block), the three X' piece tiles and the three W'
//   piece tiles, and the MMA warp multiplies the six pairs out of that one stage (each X' tile is
//   fetched once for up to three products).
// What is NOT exact on the tensor pipe is the running fp32 accumulation: every MMA adds its 16
// products into the accumulator with less than a correctly rounded fp32 add, and the error grows
// with the length of the chain and the size of the running sum. The accumulation in TMEM is
// therefore kept SHORT: after the 24 MMAs of one stage (or of `chunk_steps` stages) the MMA warp
// publishes the accumulator and starts the next chunk from zero in another TMEM buffer; the
// epilogue warps add the chunks into fp32 registers (correctly rounded adds) and run the fused
// pointwise chain after the last one. Within a stage the small piece products come first and
// x0*w0 last, so most of the chain runs while the accumulator is still small. Measured on the
// benchmarked 3x3 C64 layer against a float64 oracle: worst error 7.6e-6 with one tap per chain,
// 1.8e-4 with the whole 216-MMA reduction in one chain, 4.2e-5 for a plain fp32 FMA kernel.
//
// Structure otherwise as the 16-bit per-tap kernel: one 4-D TMA box per (tap, K block) with zero
// fill as padding, two producer warps, one MMA warp, eight epilogue warps, bounded waits.
#include <algorithm>
#include <mutex>
#include <unordered_map>
#include <cstdlib>
#include <cstring>

#include "../common.h"
#include "sm100.cuh"
#include "tc_epilogue.cuh"

namespace fb {

using namespace sm100;

namespace {

constexpr int BM = 128, BK = 64;
constexpr int A_BYTES = BM * BK * 2;
constexpr int MAX_STAGES = 3, MAX_ACC = 8;
constexpr int RING_BYTES = 221184; // 3 x 72 KB (BN = 64) or 2 x 96 KB (BN = 128) fit
constexpr int SMEM_BYTES = RING_BYTES + 1024 + 512;
constexpr int NUM_THREADS = 384; // TMA warp, MMA warp, 8 epilogue warps, second TMA warp, second MMA warp
constexpr int TMEM_COLS = 512;
constexpr int PAIRS = 6;

struct SplitParams {
  int32_t N, H, W;      // output pixel space
  int32_t C, Nout;      // channels of the fp32 tensors
  int32_t R, S;
  int32_t off_h, off_w, step_h, step_w;
  int32_t bw, bh, bn, rows;
  int32_t tiles_w, tiles_h, tiles_nb, tiles_nout, total_tiles;
  int32_t BN, cb_per;   // output-channel tile, 64-channel blocks per piece
  int32_t steps, chunk_steps, nchunks, nacc; // steps = taps x channel blocks, each one ring stage
  uint32_t a_bytes, b_bytes;
  int32_t stages, stage_bytes;
  void *out;
  int64_t out_sn, out_sh, out_sw;
  uint32_t *err;
  TcEpilogue epi;
};

// rows x C fp32 -> rows x 3C bf16: piece p of channel c at [row][p*C + c]. One launch splits both
// operands: the rows of X first, then the rows of W.
__global__ void __launch_bounds__(256)
split3_bf16_kernel(const float *__restrict__ x, __nv_bfloat16 *__restrict__ xs, int64_t x_rows,
                   const float *__restrict__ w, __nv_bfloat16 *__restrict__ ws, int64_t w_rows, int C) {
  pdl_launch_dependents();
  pdl_wait(); // (the scratch this kernel overwrites may still be read by the launch before it)
  const int64_t vec_per_row = C / 4;
  const int64_t x_total = x_rows * vec_per_row, total = x_total + w_rows * vec_per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const bool is_x = i < x_total;
    const int64_t li = is_x ? i : i - x_total;
    const float *in = is_x ? x : w;
    __nv_bfloat16 *out = is_x ? xs : ws;
    const int64_t row = li / vec_per_row;
    const int c = (int)(li - row * vec_per_row) * 4;
    const float4 v = __ldg(reinterpret_cast<const float4 *>(in + row * C + c));
    const float f[4] = {v.x, v.y, v.z, v.w};
    __nv_bfloat16 p0[4], p1[4], p2[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      p0[j] = __float2bfloat16_rn(f[j]);
      const float r1 = f[j] - __bfloat162float(p0[j]); // exact: the difference fits in fp32
      p1[j] = __float2bfloat16_rn(r1);
      const float r2 = r1 - __bfloat162float(p1[j]);
      p2[j] = __float2bfloat16_rn(r2);
    }
    __nv_bfloat16 *o = out + row * 3 * C + c;
    *reinterpret_cast<uint2 *>(o) = *reinterpret_cast<uint2 *>(p0);
    *reinterpret_cast<uint2 *>(o + C) = *reinterpret_cast<uint2 *>(p1);
    *reinterpret_cast<uint2 *>(o + 2 * C) = *reinterpret_cast<uint2 *>(p2);
  }
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
conv_split_f32_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                              const SplitParams p) {
  extern __shared__ uint8_t smem_raw[];
  pdl_launch_dependents(); // the next kernel's CTAs may take the SMs this kernel's CTAs leave
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int STAGES = p.stages;
  const uint32_t STAGE_BYTES = (uint32_t)p.stage_bytes;
  const uint32_t bar_base = smem_base + RING_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (MAX_STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * MAX_STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * MAX_STAGES + MAX_ACC + a); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * MAX_STAGES + 2 * MAX_ACC);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < p.nacc; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);
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

  const int tiles_pix = p.tiles_w * p.tiles_h * p.tiles_nb;

  if (warp == 0 || warp == 10) {
    // two producer warps on alternate K blocks, whole warp in the loop, elected lane issues
    const uint32_t pid = warp == 0 ? 0u : 1u;
    uint32_t it = 0;
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
      const int tp = tile % tiles_pix, tno = tile / tiles_pix;
      const int tw = tp % p.tiles_w, th = (tp / p.tiles_w) % p.tiles_h, tb = tp / (p.tiles_w * p.tiles_h);
      const int w0 = tw * p.bw + p.off_w, h0 = th * p.bh + p.off_h, n0 = tb * p.bn, no0 = tno * p.BN;
      int cbi = 0, ts = 0, tr = 0; // channel block (fastest), filter column, filter row
      for (int st = 0; st < p.steps; ++st, ++it, s = (s + 1 == STAGES) ? 0 : s + 1, ph ^= (s == 0)) {
        if ((it & 1u) == pid) {
          if (!mbar_wait_warp(empty_bar(s), ph ^ 1, p.err, ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t sa = smem_base + (uint32_t)s * STAGE_BYTES, sb = sa + 3 * A_BYTES;
          mbar_expect_tx_elect(full_bar(s), 3 * (p.a_bytes + p.b_bytes));
#pragma unroll
          for (int pc = 0; pc < 3; ++pc) {
            const int c0 = pc * p.C + cbi * BK;
            tma_load_4d_elect(sa + pc * A_BYTES, &tmap_a, full_bar(s), c0, w0 + ts * p.step_w, h0 + tr * p.step_h, n0);
            tma_load_4d_elect(sb + pc * p.b_bytes, &tmap_b, full_bar(s), c0, ts, tr, no0);
          }
        }
        if (++cbi == p.cb_per) {
          cbi = 0;
          if (++ts == p.S) {
            ts = 0;
            ++tr;
          }
        }
      }
    }
  } else if (warp == 1 || warp == 11) {
    // Two warps issue alternate chunks (each chunk has its own accumulator and ring stages): the tensor
    // pipe queues only a few instructions and a 128 x 64 x 16 MMA lasts 48 clk, so with one issuer the
    // pipe ran dry during the barrier waits between two chunks.
    const uint32_t which = warp == 1 ? 0u : 1u;
    const uint32_t idesc = make_idesc_f16(BM, p.BN, /*bf16*/ 1, 0, 0);
    const uint64_t a_desc0 = make_smem_desc(smem_base, 16, 1024);
    const uint64_t b_desc0 = make_smem_desc(smem_base + 3 * A_BYTES, 16, 1024);
    uint32_t ph = 0, g = 0; // g: chunks so far in this CTA
    int s = 0, acc = 0; // accumulator ring position and its phase
    uint32_t aph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
      for (int ch = 0; ch < p.nchunks && ok; ++ch, ++g) {
        if ((g & 1u) != which) {
          // the other warp's chunk: step over its stages
          for (int j = 0; j < p.chunk_steps; ++j) {
            s = (s + 1 == STAGES) ? 0 : s + 1;
            ph ^= (s == 0);
          }
        } else {
          if (!mbar_wait_warp(tempty_bar(acc), aph ^ 1, p.err, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * p.BN);
          for (int j = 0; j < p.chunk_steps; ++j, s = (s + 1 == STAGES) ? 0 : s + 1, ph ^= (s == 0)) {
            if (!mbar_wait_warp(full_bar(s), ph, p.err, ERR_WAIT_FULL)) { ok = false; break; }
            tc_fence_after();
            const uint64_t soff = (uint64_t)(((uint32_t)s * STAGE_BYTES) >> 4);
#pragma unroll
            for (int pr = 0; pr < PAIRS; ++pr) {
              // X piece / W piece of product `pr`, smallest products first: (0,2) (2,0) (1,1) (0,1) (1,0) (0,0)
              const int pa = pr == 1 ? 2 : ((pr == 2 || pr == 4) ? 1 : 0);
              const int pb = pr == 0 ? 2 : ((pr == 2 || pr == 3) ? 1 : 0);
              const uint64_t ad = a_desc0 + soff + (uint64_t)((uint32_t)(pa * A_BYTES) >> 4);
              const uint64_t bd = b_desc0 + soff + (uint64_t)(((uint32_t)pb * p.b_bytes) >> 4);
#pragma unroll
              for (int k = 0; k < BK / 16; ++k)
                tc_mma_f16_elect(d_tmem, ad + (uint64_t)((k * 32) >> 4), bd + (uint64_t)((k * 32) >> 4), idesc,
                                 (j > 0 || pr > 0 || k > 0) ? 1u : 0u);
            }
            tc_commit_elect(empty_bar(s));
          }
          if (ok) tc_commit_elect(tfull_bar(acc));
        }
        acc = (acc + 1 == p.nacc) ? 0 : acc + 1;
        aph ^= (acc == 0);
      }
    }
  } else {
    // epilogue warps 2..9: two per TMEM lane quarter, each half of the tile's columns
    const int q = warp & 3;
    const int nchunks32 = p.BN / 32;                  // 2 or 4 column chunks per tile
    const int per_warp = nchunks32 / 2;               // 1 or 2 per warp
    const int c_begin = ((warp - 2) >> 2) * per_warp;
    int acc = 0;
    uint32_t aph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
      const int tp = tile % tiles_pix, tno = tile / tiles_pix;
      const int tw = tp % p.tiles_w, th = (tp / p.tiles_w) % p.tiles_h, tb = tp / (p.tiles_w * p.tiles_h);
      float sum[2][32];
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int j = 0; j < 32; ++j) sum[u][j] = 0.f;
      for (int ch = 0; ch < p.nchunks && ok; ++ch) {
        if (!mbar_wait(tfull_bar(acc), aph, p.err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (uint32_t)(acc * p.BN) + ((uint32_t)(q * 32) << 16);
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (u < per_warp) {
            uint32_t raw[32];
            tmem_ld_32x32(taddr + (c_begin + u) * 32, raw);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) sum[u][j] += __uint_as_float(raw[j]); // correctly rounded fp32 adds
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
        acc = (acc + 1 == p.nacc) ? 0 : acc + 1;
        aph ^= (acc == 0);
      }
      if (!ok) break;
      const int row = q * 32 + lane;
      const int dw = row % p.bw, dh = (row / p.bw) % p.bh, dn = row / (p.bw * p.bh);
      const int w = tw * p.bw + dw, h = th * p.bh + dh, n = tb * p.bn + dn;
      const bool row_ok = row < p.rows && w < p.W && h < p.H && n < p.N;
      const int64_t row_off = (int64_t)n * p.out_sn + (int64_t)h * p.out_sh + (int64_t)w * p.out_sw;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (u < per_warp) {
          const int nc = tno * p.BN + (c_begin + u) * 32;
          if (row_ok && nc < p.Nout) {
            const int valid = min(32, p.Nout - nc);
            epi_run32(p.epi, sum[u], row_off, nc, valid);
            epi_store32(p.out, p.epi.out_dtype, row_off + nc, sum[u], valid);
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

// ---- host -------------------------------------------------------------------------------

struct SplitView {
  int N, H, W, IH, IW, C, Nout, R, S, pad_h, pad_w, dil_h, dil_w;
};

bool cl_dense4(const TensorInfo &t) {
  if (t.rank != 4) return false;
  const int64_t C = t.dims[1], H = t.dims[2], W = t.dims[3];
  return t.strides[1] == 1 && t.strides[3] == C && t.strides[2] == W * C && t.strides[0] == H * W * C;
}

bool split_view(const Plan &p, const Step &s, SplitView &v) {
  const fb_node_desc &d = p.nodes[s.node].d;
  if (d.op != FB_OP_CONV_FPROP || d.num_spatial != 2) return false;
  if (d.stride[0] != 1 || d.stride[1] != 1) return false;
  const TensorInfo &in = p.tensors[d.inputs[0]], &w = p.tensors[d.inputs[1]];
  const TensorInfo &o0 = p.tensors[d.outputs[0]], &out = p.tensors[s.out_tensor];
  if (in.dtype != FB_DT_FLOAT || w.dtype != FB_DT_FLOAT || o0.dtype != FB_DT_FLOAT || out.dtype != FB_DT_FLOAT)
    return false;
  if (!cl_dense4(in) || !cl_dense4(w) || !cl_dense4(out)) return false;
  if (in.dims[1] != w.dims[1]) return false; // groups == 1
  v.C = (int)in.dims[1]; v.Nout = (int)w.dims[0];
  v.R = (int)w.dims[2]; v.S = (int)w.dims[3];
  v.pad_h = (int)d.padding[0]; v.pad_w = (int)d.padding[1];
  v.dil_h = (int)d.dilation[0]; v.dil_w = (int)d.dilation[1];
  v.N = (int)out.dims[0]; v.H = (int)out.dims[2]; v.W = (int)out.dims[3];
  v.IH = (int)in.dims[2]; v.IW = (int)in.dims[3];
  if (v.C % 64 || v.C > 1024 || v.Nout % 8 || v.Nout < 32) return false;
  if ((int64_t)v.N * v.H * v.W < 4096) return false; // small problems stay on the CUDA cores
  if ((int64_t)v.N * v.IH * v.IW * 3 * v.C >= (1ll << 40)) return false;
  return true;
}

int split_epi_kind(const Plan &p, const Step &s, const EpilogueOpInfo &op) {
  if (op.operand < 0) return 0;
  const TensorInfo &o = p.tensors[op.operand];
  const TensorInfo &c = p.tensors[s.out_tensor];
  if (o.role == FB_TENSOR_SCALAR) return 2;
  if (o.rank == 4 && o.dims[0] == 1 && o.dims[2] == 1 && o.dims[3] == 1 && o.dims[1] == c.dims[1] && o.strides[1] == 1)
    return 1;
  bool full = o.rank == c.rank;
  for (int i = 0; full && i < c.rank; ++i)
    if (o.dims[i] != c.dims[i] || (c.dims[i] > 1 && o.strides[i] != c.strides[i])) full = false;
  return full ? 3 : -1;
}

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
  for (int w = 1; w <= std::min(W, 128); ++w)
    for (int h = 1; h <= std::min(H, 128 / w); ++h) {
      const int n = std::max(1, std::min(N, 128 / (w * h)));
      const int64_t tiles = (int64_t)((W + w - 1) / w) * ((H + h - 1) / h) * ((N + n - 1) / n);
      const double eff = (double)N * H * W / ((double)tiles * 128.0);
      if (eff > best + 1e-9 || (eff > best - 1e-9 && w > bw)) {
        best = eff; bw = w; bh = h; bn = n;
      }
    }
}

int64_t align256(int64_t v) { return (v + 255) & ~(int64_t)255; }

} // namespace

// FUSILLI_B200_F32_CONV=simt keeps fp32 convolutions on the CUDA-core kernel (read when the plan is
// built): the switch exists to compare the two paths.
bool conv_split_f32_eligible(const Plan &p, const Step &s) {
  const char *e = getenv("FUSILLI_B200_F32_CONV");
  if (e && strcmp(e, "simt") == 0) return false;
  SplitView v;
  if (!split_view(p, s, v)) return false;
  for (int i = 0; i < s.num_epilogue; ++i) {
    if (split_epi_kind(p, s, s.epilogue[i]) < 0) return false;
    if (p.tensors[s.epilogue[i].out_tensor].dtype != FB_DT_FLOAT) return false;
    if (s.epilogue[i].operand >= 0 && p.tensors[s.epilogue[i].operand].dtype != FB_DT_FLOAT) return false;
  }
  return true;
}

// Workspace: X' and W' (bf16, three pieces per channel).
int64_t conv_split_f32_scratch_bytes(const Plan &p, const Step &s) {
  SplitView v;
  if (!split_view(p, s, v)) return 0;
  return align256((int64_t)v.N * v.IH * v.IW * 3 * v.C * 2) + align256((int64_t)v.Nout * v.R * v.S * 3 * v.C * 2);
}

fb_status launch_conv_split_f32(const ExecContext &cx, const Step &s) {
  const Plan &plan = *cx.plan;
  const fb_node_desc &d = plan.nodes[s.node].d;
  SplitView v;
  FB_REQUIRE(split_view(plan, s, v), FB_INTERNAL_ERROR, "conv_split_f32: step is not eligible");
  const TensorInfo &out = plan.tensors[s.out_tensor];
  const float *xptr = static_cast<const float *>(cx.tensor_ptr(d.inputs[0]));
  const float *wptr = static_cast<const float *>(cx.tensor_ptr(d.inputs[1]));
  void *optr = cx.tensor_ptr(s.out_tensor);
  FB_REQUIRE(xptr && wptr && optr, FB_INTERNAL_ERROR, "conv_split_f32: tensor has no buffer");
  FB_REQUIRE(((uintptr_t)xptr % 16 == 0) && ((uintptr_t)wptr % 16 == 0), FB_INVALID_ARGUMENT,
             "conv_split_f32: operand buffers must be 16-byte aligned");
  FB_REQUIRE(cx.workspace && s.scratch_offset >= 0 && s.scratch_bytes >= conv_split_f32_scratch_bytes(plan, s),
             FB_INTERNAL_ERROR, "conv_split_f32: scratch missing");
  const int64_t x_rows = (int64_t)v.N * v.IH * v.IW, w_rows = (int64_t)v.Nout * v.R * v.S;
  __nv_bfloat16 *xs = reinterpret_cast<__nv_bfloat16 *>(cx.workspace + s.scratch_offset);
  __nv_bfloat16 *ws = reinterpret_cast<__nv_bfloat16 *>(cx.workspace + s.scratch_offset + align256(x_rows * 3 * v.C * 2));
  {
    const int64_t vecs = (x_rows + w_rows) * (v.C / 4);
    const int blocks = (int)std::min<int64_t>((vecs + 255) / 256, (int64_t)cx.dev->sm_count * 16);
    split3_bf16_kernel<<<blocks, 256, 0, cx.dev->stream>>>(xptr, xs, x_rows, wptr, ws, w_rows, v.C);
  }

  static thread_local SplitParams p;
  memset(&p, 0, sizeof(p));
  p.C = v.C; p.Nout = v.Nout; p.R = v.R; p.S = v.S;
  p.cb_per = v.C / BK;
  p.BN = v.Nout > 64 ? 128 : 64;
  p.N = v.N; p.H = v.H; p.W = v.W;
  choose_patch(v.N, v.H, v.W, p.bw, p.bh, p.bn);
  p.rows = p.bw * p.bh * p.bn;
  p.off_h = -v.pad_h; p.off_w = -v.pad_w; p.step_h = v.dil_h; p.step_w = v.dil_w;
  p.tiles_w = (p.W + p.bw - 1) / p.bw;
  p.tiles_h = (p.H + p.bh - 1) / p.bh;
  p.tiles_nb = (p.N + p.bn - 1) / p.bn;
  p.tiles_nout = (p.Nout + p.BN - 1) / p.BN;
  const int64_t total = (int64_t)p.tiles_w * p.tiles_h * p.tiles_nb * p.tiles_nout;
  FB_REQUIRE(total < (1ll << 31), FB_NOT_IMPLEMENTED, "conv_split_f32: too many tiles");
  p.total_tiles = (int)total;
  p.steps = v.R * v.S * p.cb_per;
  // Length of one accumulation in TMEM, in ring stages of 24 MMAs (six piece products of one tap
  // and 64-channel block): one stage by default. FUSILLI_B200_F32_CHUNK = tap | tile lengthens it
  // (for measurements of the error against the chain length).
  p.chunk_steps = 1;
  if (const char *e = getenv("FUSILLI_B200_F32_CHUNK")) {
    if (strcmp(e, "tap") == 0) p.chunk_steps = p.cb_per;
    else if (strcmp(e, "tile") == 0) p.chunk_steps = p.steps;
  }
  p.nchunks = p.steps / p.chunk_steps;
  p.nacc = std::min(MAX_ACC, TMEM_COLS / p.BN);
  p.a_bytes = (uint32_t)p.rows * BK * 2;
  p.b_bytes = (uint32_t)p.BN * BK * 2;
  p.stage_bytes = 3 * (A_BYTES + p.BN * BK * 2);
  p.stages = std::min(MAX_STAGES, RING_BYTES / p.stage_bytes);
  p.out = optr;
  p.out_sn = out.strides[0]; p.out_sh = out.strides[2]; p.out_sw = out.strides[3];
  p.err = cx.dev->error_word;
  p.epi.num_ops = s.num_epilogue;
  p.epi.acc_round_dtype = FB_DT_FLOAT;
  p.epi.out_dtype = FB_DT_FLOAT;
  for (int i = 0; i < s.num_epilogue; ++i) {
    const EpilogueOpInfo &src = s.epilogue[i];
    TcEpiOp &op = p.epi.ops[i];
    op.mode = src.mode;
    op.kind = split_epi_kind(plan, s, src);
    op.value_is_in1 = src.value_is_in1;
    op.round_dtype = FB_DT_FLOAT;
    memcpy(op.prm, src.fparams, sizeof(op.prm));
    if (src.operand >= 0) {
      const TensorInfo &o = plan.tensors[src.operand];
      op.dtype = o.dtype;
      if (op.kind == 2) op.scalar = (float)o.scalar;
      else {
        op.ptr = cx.tensor_ptr(src.operand);
        FB_REQUIRE(op.ptr != nullptr, FB_INTERNAL_ERROR, "conv_split_f32: epilogue operand has no buffer");
      }
    }
  }
  CUtensorMap tmA, tmB;
  const char *why = "";
  {
    const uint64_t c3 = (uint64_t)3 * v.C;
    uint64_t a_dims[4] = {c3, (uint64_t)v.IW, (uint64_t)v.IH, (uint64_t)v.N};
    uint64_t a_str[3] = {c3 * 2, (uint64_t)v.IW * c3 * 2, (uint64_t)v.IH * v.IW * c3 * 2};
    uint32_t box[4] = {BK, (uint32_t)p.bw, (uint32_t)p.bh, (uint32_t)p.bn};
    FB_REQUIRE(encode_tmap_2byte(&tmA, xs, 4, a_dims, a_str, box, &why), FB_RUNTIME_FAILURE, why);
    uint64_t w_dims[4] = {c3, (uint64_t)v.S, (uint64_t)v.R, (uint64_t)v.Nout};
    uint64_t w_str[3] = {c3 * 2, (uint64_t)v.S * c3 * 2, (uint64_t)v.R * v.S * c3 * 2};
    uint32_t wbox[4] = {BK, 1, 1, (uint32_t)p.BN};
    FB_REQUIRE(encode_tmap_2byte(&tmB, ws, 4, w_dims, w_str, wbox, &why), FB_RUNTIME_FAILURE, why);
  }
  cudaError_t ae = set_max_dynamic_smem(reinterpret_cast<const void *>(conv_split_f32_tcgen05_kernel), SMEM_BYTES,
                                        cx.dev->ordinal);
  FB_REQUIRE(ae == cudaSuccess, FB_RUNTIME_FAILURE,
             std::string("conv_split_f32: cannot reserve shared memory: ") + cudaGetErrorString(ae));
  const int grid = std::min<int>(p.total_tiles, cx.dev->sm_count);
  FB_CUDA_OK(launch_pdl(conv_split_f32_tcgen05_kernel, dim3(grid), dim3(NUM_THREADS), SMEM_BYTES, cx.dev->stream, tmA, tmB, p));
  return FB_OK;
}

} // namespace fb

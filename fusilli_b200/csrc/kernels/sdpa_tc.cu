// Flash-style scaled-dot-product attention forward on the tensor cores:
//   O = softmax(Q K^T * scale [causal]) V,  Q/K/V/O contiguous [B,H,S,128], bf16 or f16.
//
// One CTA per (128-query block, batch*head). Memory stays O(S): K/V stream through a
// 2-stage shared-memory ring and the 128x128 score tile never leaves the SM.
//   warp 0      TMA producer: Q once, then K_j / V_j tiles (128 keys x 128 dims, two
//               128B-swizzled 64-wide boxes each), separate full/empty barriers for K and V.
//   warp 1      MMA issuer: S_j = Q K_j^T (tcgen05.mma 128x128x16 x8) into one of two TMEM
//               score buffers -- issued one block ahead so the tensor pipe works while the
//               softmax of the previous block runs -- then PV_j = P_j V_j into a third
//               TMEM buffer (V is the MN-major operand: no transposition).
//   warps 2..5  softmax, one query row per thread: pass 1 reads S_j from TMEM for the row
//               max; the previous block's PV tile is folded into the fp32 output row kept
//               in registers and rescaled by exp2((m_old-m_new)*c); pass 2 re-reads S_j,
//               p = exp2(s*c - m*c) with c = scale*log2(e), accumulates the row sum in
//               fp32 and writes P_j as 16-bit values into 128B-swizzled shared memory, the
//               A operand of the PV product.
// Causal blocks above the diagonal are never loaded or multiplied; the diagonal block and
// a ragged last key block are masked elementwise. Heavy (late) query blocks are scheduled
// first. Every mbarrier wait is bounded.
#include <algorithm>

#include "../common.h"
#include "sm100.cuh"
#include "tc_epilogue.cuh"

namespace fb {

using namespace sm100;

namespace {

constexpr int BQ = 128, BKV = 128, HD = 128;
constexpr int TILE_BYTES = 128 * 128 * 2;  // one 128x128 16-bit tile = two 64-wide boxes
constexpr int HALF_BYTES = TILE_BYTES / 2; // one 128-row x 64-col swizzled box
constexpr int SM_Q = 0, SM_K = TILE_BYTES, SM_V = 3 * TILE_BYTES, SM_P = 5 * TILE_BYTES;
constexpr int SM_BARS = 6 * TILE_BYTES;
constexpr int SMEM_BYTES = 6 * TILE_BYTES + 1024 + 256;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int TM_PV = 0, TM_S = 128; // PV tile: cols [0,128); score buffers: [128,256), [256,384)

struct SdpaTcParams {
  int32_t B, Hq, Hk, Sq, Skv;
  int32_t causal, ab_format, out_dtype;
  int32_t q_blocks;
  float scale_log2e;
  void *out;
  uint32_t *err;
};

__global__ void __launch_bounds__(NUM_THREADS, 1)
sdpa_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const SdpaTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + SM_BARS;
  // barrier slots
  const uint32_t q_full = bar_base;
  auto k_full = [&](int s) { return bar_base + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bar_base + 8u * (3 + s); };
  auto v_full = [&](int s) { return bar_base + 8u * (5 + s); };
  auto v_empty = [&](int s) { return bar_base + 8u * (7 + s); };
  auto s_full = [&](int s) { return bar_base + 8u * (9 + s); };
  auto s_empty = [&](int s) { return bar_base + 8u * (11 + s); };
  const uint32_t p_full = bar_base + 8u * 13, pv_full = bar_base + 8u * 14;
  const uint32_t tmem_slot = bar_base + 8u * 15;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // heavy query blocks (late rows under a causal mask) first
  const int qb = p.q_blocks - 1 - (int)blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / p.Hq, h = bh % p.Hq;
  const int kvh = b * p.Hk + h / (p.Hq / p.Hk);
  const int q0 = qb * BQ;
  int nblk = (p.Skv + BKV - 1) / BKV;
  if (p.causal) nblk = min(nblk, (q0 + BQ - 1) / BKV + 1);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(k_empty(s), 1);
      mbar_init(v_full(s), 1);
      mbar_init(v_empty(s), 1);
      mbar_init(s_full(s), 1);
      mbar_init(s_empty(s), 4);
    }
    mbar_init(p_full, 4);
    mbar_init(pv_full, 1);
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
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, TILE_BYTES);
      tma_load_3d(smem_base + SM_Q, &tmap_q, q_full, 0, q0, bh);
      tma_load_3d(smem_base + SM_Q + HALF_BYTES, &tmap_q, q_full, 64, q0, bh);
      bool ok = true;
      for (int j = 0; j < nblk && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(k_empty(s), ph ^ 1, p.err, ERR_WAIT_EMPTY)) { ok = false; break; }
        mbar_expect_tx(k_full(s), TILE_BYTES);
        const uint32_t sk = smem_base + SM_K + s * TILE_BYTES;
        tma_load_3d(sk, &tmap_k, k_full(s), 0, j * BKV, kvh);
        tma_load_3d(sk + HALF_BYTES, &tmap_k, k_full(s), 64, j * BKV, kvh);
        if (!mbar_wait(v_empty(s), ph ^ 1, p.err, ERR_WAIT_EMPTY)) { ok = false; break; }
        mbar_expect_tx(v_full(s), TILE_BYTES);
        const uint32_t sv = smem_base + SM_V + s * TILE_BYTES;
        tma_load_3d(sv, &tmap_v, v_full(s), 0, j * BKV, kvh);
        tma_load_3d(sv + HALF_BYTES, &tmap_v, v_full(s), 64, j * BKV, kvh);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // scores: A = Q (K-major), B = K_j (K-major, N = keys); output: A = P (K-major), B = V_j (MN-major)
      const uint32_t idesc_qk = make_idesc_f16(BQ, BKV, p.ab_format, 0, 0);
      const uint32_t idesc_pv = make_idesc_f16(BQ, HD, p.ab_format, 0, 1);
      const uint32_t sq = smem_base + SM_Q, sp = smem_base + SM_P;
      bool ok = mbar_wait(q_full, 0, p.err, ERR_WAIT_FULL);
      auto issue_scores = [&](int j) -> bool {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(k_full(s), ph, p.err, ERR_WAIT_FULL)) return false;
        if (!mbar_wait(s_empty(s), ph ^ 1, p.err, ERR_WAIT_TMEM_EMPTY)) return false;
        tc_fence_after();
        const uint32_t sk = smem_base + SM_K + s * TILE_BYTES;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
          tc_mma_f16(tmem_base + TM_S + s * BKV, make_smem_desc(sq + off, 16, 1024),
                     make_smem_desc(sk + off, 16, 1024), idesc_qk, k > 0 ? 1u : 0u);
        }
        tc_commit(k_empty(s));
        tc_commit(s_full(s));
        return true;
      };
      if (ok && nblk > 0) ok = issue_scores(0);
      for (int j = 0; j < nblk && ok; ++j) {
        if (j + 1 < nblk) {
          if (!issue_scores(j + 1)) { ok = false; break; }
        }
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(v_full(s), ph, p.err, ERR_WAIT_FULL)) { ok = false; break; }
        if (!mbar_wait(p_full, j & 1, p.err, ERR_WAIT_OTHER)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sv = smem_base + SM_V + s * TILE_BYTES;
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          const uint32_t a_off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
          // V_j: 64-wide head-dim blocks HALF_BYTES apart (LBO), 8-key groups 1024 B apart
          tc_mma_f16(tmem_base + TM_PV, make_smem_desc(sp + a_off, 16, 1024),
                     make_smem_desc(sv + k * 2048, HALF_BYTES, 1024), idesc_pv, k > 0 ? 1u : 0u);
        }
        tc_commit(v_empty(s));
        tc_commit(pv_full);
      }
    }
  } else {
    const int q = warp & 3;
    const int row = q * 32 + lane;
    const int qi = q0 + row;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const float c = p.scale_log2e;
    float m_run = -INFINITY, l_run = 0.f;
    float o_acc[HD];
#pragma unroll
    for (int d = 0; d < HD; ++d) o_acc[d] = 0.f;
    bool ok = true;
    const uint32_t p_row = smem_base + SM_P + (uint32_t)row * 128u;
    for (int j = 0; j < nblk && ok; ++j) {
      const int s = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait(s_full(s), ph, p.err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const uint32_t s_addr = tmem_base + TM_S + s * BKV + lane_addr;
      const int k0 = j * BKV;
      const bool need_mask = (k0 + BKV > p.Skv) || (p.causal && k0 + BKV - 1 > q0);
      const int k_lim = p.causal ? min(p.Skv, qi + 1) : p.Skv; // keys >= k_lim are masked for this row
      // pass 1: row maximum of the raw scores
      float mx = -INFINITY;
#pragma unroll 1
      for (int cc = 0; cc < BKV / 32; ++cc) {
        uint32_t raw[32];
        tmem_ld_32x32(s_addr + cc * 32, raw);
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int t = 0; t < 32; ++t)
            if (k0 + cc * 32 + t < k_lim) mx = fmaxf(mx, __uint_as_float(raw[t]));
        } else {
#pragma unroll
          for (int t = 0; t < 32; ++t) mx = fmaxf(mx, __uint_as_float(raw[t]));
        }
      }
      const float m_new = fmaxf(m_run, mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = exp2f((m_run - m_use) * c); // exp2(-inf) = 0 on the first block
      // fold in the previous block's P*V (computed against m_run), then rescale to m_new
      if (j > 0) {
        if (!mbar_wait(pv_full, (j - 1) & 1, p.err, ERR_WAIT_TMEM_FULL)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int cc = 0; cc < HD / 32; ++cc) {
          uint32_t raw[32];
          tmem_ld_32x32(tmem_base + TM_PV + lane_addr + cc * 32, raw);
          tmem_ld_wait();
#pragma unroll
          for (int t = 0; t < 32; ++t) o_acc[cc * 32 + t] = (o_acc[cc * 32 + t] + __uint_as_float(raw[t])) * alpha;
        }
      }
      l_run *= alpha;
      m_run = m_new;
      const float mc = m_use * c;
      // pass 2: probabilities -> 16-bit -> swizzled shared memory
      float lsum = 0.f;
#pragma unroll 1
      for (int cc = 0; cc < BKV / 32; ++cc) {
        uint32_t raw[32];
        tmem_ld_32x32(s_addr + cc * 32, raw);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int t = 0; t < 16; ++t) {
          float p0 = exp2f(fmaf(__uint_as_float(raw[2 * t]), c, -mc));
          float p1 = exp2f(fmaf(__uint_as_float(raw[2 * t + 1]), c, -mc));
          if (need_mask) {
            if (k0 + cc * 32 + 2 * t >= k_lim) p0 = 0.f;
            if (k0 + cc * 32 + 2 * t + 1 >= k_lim) p1 = 0.f;
          }
          lsum += p0 + p1;
          if (p.ab_format) {
            __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
            packed[t] = *reinterpret_cast<uint32_t *>(&hh);
          } else {
            __half2 hh = __floats2half2_rn(p0, p1);
            packed[t] = *reinterpret_cast<uint32_t *>(&hh);
          }
        }
        // 32 keys = four 16-byte chunks of this row; chunk index XOR (row % 8) is the 128B swizzle
        const uint32_t half_base = p_row + (uint32_t)(cc >> 1) * HALF_BYTES;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          const uint32_t chunk = (uint32_t)((cc & 1) * 4 + ch) ^ (uint32_t)(row & 7);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(half_base + chunk * 16u),
                       "r"(packed[4 * ch]), "r"(packed[4 * ch + 1]), "r"(packed[4 * ch + 2]), "r"(packed[4 * ch + 3])
                       : "memory");
        }
      }
      l_run += lsum;
      // scores consumed: the score buffer may be overwritten; P written: publish to the tensor proxy
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(s_empty(s));
        mbar_arrive(p_full);
      }
    }
    if (ok && nblk > 0) {
      if (mbar_wait(pv_full, (nblk - 1) & 1, p.err, ERR_WAIT_TMEM_FULL)) {
        tc_fence_after();
        const float inv = 1.f / l_run;
        const int64_t row_off = ((int64_t)bh * p.Sq + qi) * HD;
#pragma unroll
        for (int cc = 0; cc < HD / 32; ++cc) {
          uint32_t raw[32];
          tmem_ld_32x32(tmem_base + TM_PV + lane_addr + cc * 32, raw);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int t = 0; t < 32; ++t) v[t] = (o_acc[cc * 32 + t] + __uint_as_float(raw[t])) * inv;
          if (qi < p.Sq) epi_store32(p.out, p.out_dtype, row_off + cc * 32, v, 32);
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
  p.q_blocks = (p.Sq + BQ - 1) / BQ;
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
  cudaError_t ae = cudaFuncSetAttribute(sdpa_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  FB_REQUIRE(ae == cudaSuccess, FB_RUNTIME_FAILURE,
             std::string("sdpa_tcgen05: cannot reserve shared memory: ") + cudaGetErrorString(ae));
  dim3 grid((unsigned)p.q_blocks, (unsigned)(p.B * p.Hq));
  sdpa_tcgen05_kernel<<<grid, NUM_THREADS, SMEM_BYTES, cx.dev->stream>>>(tq, tk, tv, p);
  return FB_OK;
}

} // namespace fb

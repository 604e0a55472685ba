// CUDA-core scaled-dot-product attention for the cases the tensor-core kernel does
// not take: additive masks, GQA, cross attention, f16/f32 tensors, head dims other
// than 128, short or ragged sequences, arbitrary strides.
//
// One warp per query row, streaming over keys 32 at a time with an online softmax
// (running max and sum in fp32), so memory is O(S) like the tensor-core kernel.
// Lane j scores key j0+j; the output row is spread over lanes (dim d = lane + 32*i).
#include "../common.h"

namespace fb {

struct SdpaSimtParams {
  const void *q, *k, *v, *mask;
  void *o;
  int32_t q_dt, k_dt, v_dt, m_dt, o_dt;
  int32_t B, Hq, Hk, Hv, Sq, Skv, D, Dv;
  int32_t causal;
  float scale;
  int64_t qs[4], ks[4], vs[4], os[4], ms[4];
};

constexpr int kSdpaWarps = 4;
constexpr int kSdpaMaxD = 256;

__global__ void __launch_bounds__(kSdpaWarps * 32) sdpa_simt_kernel(const SdpaSimtParams p) {
  __shared__ float qsm[kSdpaWarps][kSdpaMaxD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kSdpaWarps + warp;
  const int64_t nrows = (int64_t)p.B * p.Hq * p.Sq;
  if (row >= nrows) return; // whole warp leaves together; no block-wide barrier below
  const int i = (int)(row % p.Sq);
  const int h = (int)((row / p.Sq) % p.Hq);
  const int b = (int)(row / ((int64_t)p.Sq * p.Hq));
  const int hk = h / (p.Hq / p.Hk), hv = h / (p.Hq / p.Hv);
  const int64_t qoff = b * p.qs[0] + h * p.qs[1] + i * p.qs[2];
  const int64_t koff = b * p.ks[0] + hk * p.ks[1];
  const int64_t voff = b * p.vs[0] + hv * p.vs[1];
  for (int d = lane; d < p.D; d += 32) qsm[warp][d] = load_f(p.q, p.q_dt, qoff + d * p.qs[3]) * p.scale;
  __syncwarp();
  const int jend = p.causal ? min(i + 1, p.Skv) : p.Skv;
  float m_run = -INFINITY, l_run = 0.f;
  float acc[kSdpaMaxD / 32];
#pragma unroll
  for (int t = 0; t < kSdpaMaxD / 32; ++t) acc[t] = 0.f;
  for (int j0 = 0; j0 < jend; j0 += 32) {
    const int j = j0 + lane;
    float sc = -INFINITY;
    if (j < jend) {
      const int64_t kr = koff + j * p.ks[2];
      float dot = 0.f;
      for (int d = 0; d < p.D; ++d) dot = fmaf(qsm[warp][d], load_f(p.k, p.k_dt, kr + d * p.ks[3]), dot);
      if (p.mask) dot += load_f(p.mask, p.m_dt, b * p.ms[0] + h * p.ms[1] + i * p.ms[2] + j * p.ms[3]);
      sc = dot;
    }
    float cmax = sc;
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, s));
    const float m_new = fmaxf(m_run, cmax);
    const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
    const float alpha = expf(m_run - m_use); // exp(-inf) = 0 on the first chunk
    const float pj = (j < jend) ? expf(sc - m_use) : 0.f;
    float psum = pj;
#pragma unroll
    for (int s = 16; s >= 1; s >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, s);
    l_run = l_run * alpha + psum;
    m_run = m_new;
#pragma unroll
    for (int t = 0; t < kSdpaMaxD / 32; ++t) acc[t] *= alpha;
    const int cnt = min(32, jend - j0);
    for (int jj = 0; jj < cnt; ++jj) {
      const float pv = __shfl_sync(0xffffffffu, pj, jj);
      const int64_t vr = voff + (int64_t)(j0 + jj) * p.vs[2];
#pragma unroll
      for (int t = 0; t < kSdpaMaxD / 32; ++t) {
        const int d = lane + 32 * t;
        if (d < p.Dv) acc[t] = fmaf(pv, load_f(p.v, p.v_dt, vr + d * p.vs[3]), acc[t]);
      }
    }
  }
  const float inv = 1.f / l_run;
  const int64_t ooff = b * p.os[0] + h * p.os[1] + i * p.os[2];
#pragma unroll
  for (int t = 0; t < kSdpaMaxD / 32; ++t) {
    const int d = lane + 32 * t;
    if (d < p.Dv) store_f(p.o, p.o_dt, ooff + d * p.os[3], acc[t] * inv);
  }
}

fb_status launch_sdpa_simt(const ExecContext &cx, const Step &s) {
  const Plan &plan = *cx.plan;
  const fb_node_desc &d = plan.nodes[s.node].d;
  const TensorInfo &q = plan.tensors[d.inputs[0]], &k = plan.tensors[d.inputs[1]];
  const TensorInfo &v = plan.tensors[d.inputs[2]], &o = plan.tensors[d.outputs[0]];
  SdpaSimtParams p;
  memset(&p, 0, sizeof(p));
  p.q = cx.tensor_ptr(d.inputs[0]);
  p.k = cx.tensor_ptr(d.inputs[1]);
  p.v = cx.tensor_ptr(d.inputs[2]);
  p.o = cx.tensor_ptr(d.outputs[0]);
  FB_REQUIRE(p.q && p.k && p.v && p.o, FB_INTERNAL_ERROR, "sdpa: tensor has no buffer");
  p.q_dt = q.dtype; p.k_dt = k.dtype; p.v_dt = v.dtype; p.o_dt = o.dtype;
  p.B = (int)q.dims[0]; p.Hq = (int)q.dims[1]; p.Sq = (int)q.dims[2]; p.D = (int)q.dims[3];
  p.Hk = (int)k.dims[1]; p.Skv = (int)k.dims[2];
  p.Hv = (int)v.dims[1]; p.Dv = (int)v.dims[3];
  FB_REQUIRE(p.D <= kSdpaMaxD && p.Dv <= kSdpaMaxD, FB_NOT_IMPLEMENTED,
             "sdpa: head dims above 256 are not supported");
  FB_REQUIRE(p.Hq % p.Hk == 0 && p.Hq % p.Hv == 0, FB_INVALID_ARGUMENT,
             "sdpa: query heads must be a multiple of key and value heads");
  p.causal = (d.flags & FB_FLAG_SDPA_CAUSAL) ? 1 : 0;
  p.scale = (d.flags & FB_FLAG_SDPA_HAS_SCALE) ? d.fparams[0] : 1.f / sqrtf((float)p.D);
  for (int i = 0; i < 4; ++i) {
    p.qs[i] = q.strides[i]; p.ks[i] = k.strides[i]; p.vs[i] = v.strides[i]; p.os[i] = o.strides[i];
  }
  if (d.inputs[3] >= 0) {
    const TensorInfo &m = plan.tensors[d.inputs[3]];
    p.mask = cx.tensor_ptr(d.inputs[3]);
    FB_REQUIRE(p.mask != nullptr, FB_INTERNAL_ERROR, "sdpa: mask has no buffer");
    p.m_dt = m.dtype;
    for (int i = 0; i < 4; ++i) p.ms[i] = m.dims[i] == 1 ? 0 : m.strides[i];
  }
  int64_t rows = (int64_t)p.B * p.Hq * p.Sq;
  int64_t blocks = (rows + kSdpaWarps - 1) / kSdpaWarps;
  FB_REQUIRE(blocks <= 0x7fffffff, FB_NOT_IMPLEMENTED, "sdpa: too many query rows for one launch");
  sdpa_simt_kernel<<<(unsigned)blocks, kSdpaWarps * 32, 0, cx.dev->stream>>>(p);
  return FB_OK;
}

} // namespace fb

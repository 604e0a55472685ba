// Batch normalisation over [N, C, spatial...] tensors, contiguous or channels-last.
//
// The reference lowers BatchNormNode to torch.aten.native_batch_norm on value tensors
// (include/fusilli/support/asm_emitter.h:1232-1307): inference normalises with the running MEAN and
// VAR, training with the statistics of the batch (biased variance) and also returns them as
// SAVED_MEAN and SAVED_INV_VARIANCE = 1 / sqrt(var + eps); being functional, it returns no updated
// running statistics, and momentum has no effect on any output.
//
// Training is three launches: per (channel, slice) partial sums of (x - K) and (x - K)^2 with
// K = the channel's first element (the shift keeps the one-pass variance from cancelling), a merge
// in a fixed order (deterministic, no atomics), and the elementwise apply. Inference is the apply
// alone. Threads run along whichever of the spatial or the channel axis is contiguous in X, so
// loads coalesce in both layouts. These are HBM-bound passes with scalar accesses.
#include "../common.h"
#include "device_types.h"

namespace fb {

namespace {

struct BnParams {
  const void *x, *scale, *bias, *mean, *var;
  void *y, *saved_mean, *saved_invstd;
  int32_t x_dtype, y_dtype, scale_dtype, bias_dtype, mean_dtype, var_dtype, sm_dtype, si_dtype;
  int64_t N, C, S;          // batch, channels, spatial volume
  int64_t xs_n, xs_c, xs_s; // element strides of X along batch, channel, flattened spatial index
  int64_t ys_n, ys_c, ys_s;
  float eps;
  int32_t splits, training, channel_fast;
  float *partial; // [C][splits][2]: sum(x - K), sum((x - K)^2)
  float *stats;   // [2][C]: mean, 1 / sqrt(var + eps)
};

constexpr int BN_THREADS = 256;

__device__ __forceinline__ float2 block_sum2(float2 v, float2 *sh) {
  for (int o = 16; o > 0; o >>= 1) {
    v.x += __shfl_xor_sync(0xffffffffu, v.x, o);
    v.y += __shfl_xor_sync(0xffffffffu, v.y, o);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float2 r = make_float2(0.f, 0.f);
  if (warp == 0) {
    r = lane < BN_THREADS / 32 ? sh[lane] : make_float2(0.f, 0.f);
    for (int o = 4; o > 0; o >>= 1) {
      r.x += __shfl_xor_sync(0xffffffffu, r.x, o);
      r.y += __shfl_xor_sync(0xffffffffu, r.y, o);
    }
  }
  return r; // valid in thread 0
}

// Spatial axis contiguous (NCHW): one CTA per (channel, slice of the N*S elements).
__global__ void __launch_bounds__(BN_THREADS) bn_partial_spatial_kernel(const BnParams p) {
  __shared__ float2 sh[BN_THREADS / 32];
  const int64_t c = blockIdx.x;
  const int64_t total = p.N * p.S;
  const int64_t per = (total + p.splits - 1) / p.splits;
  const int64_t begin = (int64_t)blockIdx.y * per, end = min(total, begin + per);
  const float K = load_f(p.x, p.x_dtype, c * p.xs_c);
  float2 acc = make_float2(0.f, 0.f);
  for (int64_t i = begin + threadIdx.x; i < end; i += BN_THREADS) {
    const int64_t n = i / p.S, s = i - n * p.S;
    const float d = load_f(p.x, p.x_dtype, n * p.xs_n + c * p.xs_c + s * p.xs_s) - K;
    acc.x += d;
    acc.y = fmaf(d, d, acc.y);
  }
  const float2 r = block_sum2(acc, sh);
  if (threadIdx.x == 0) {
    p.partial[(c * p.splits + blockIdx.y) * 2 + 0] = r.x;
    p.partial[(c * p.splits + blockIdx.y) * 2 + 1] = r.y;
  }
}

// Channel axis contiguous (channels-last): a CTA takes 32 channels (threadIdx.x) and walks a
// slice of the N*S positions with 8 rows of threads (threadIdx.y).
__global__ void __launch_bounds__(BN_THREADS) bn_partial_channel_kernel(const BnParams p) {
  __shared__ float2 sh[8][33];
  const int64_t c = (int64_t)blockIdx.x * 32 + threadIdx.x;
  const int64_t total = p.N * p.S;
  const int64_t per = (total + p.splits - 1) / p.splits;
  const int64_t begin = (int64_t)blockIdx.y * per, end = min(total, begin + per);
  float2 acc = make_float2(0.f, 0.f);
  if (c < p.C) {
    const float K = load_f(p.x, p.x_dtype, c * p.xs_c);
    for (int64_t i = begin + threadIdx.y; i < end; i += 8) {
      const int64_t n = i / p.S, s = i - n * p.S;
      const float d = load_f(p.x, p.x_dtype, n * p.xs_n + c * p.xs_c + s * p.xs_s) - K;
      acc.x += d;
      acc.y = fmaf(d, d, acc.y);
    }
  }
  sh[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && c < p.C) {
    float2 r = sh[0][threadIdx.x];
    for (int j = 1; j < 8; ++j) {
      r.x += sh[j][threadIdx.x].x;
      r.y += sh[j][threadIdx.x].y;
    }
    p.partial[(c * p.splits + blockIdx.y) * 2 + 0] = r.x;
    p.partial[(c * p.splits + blockIdx.y) * 2 + 1] = r.y;
  }
}

__global__ void bn_finalize_kernel(const BnParams p) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= p.C) return;
  const float K = load_f(p.x, p.x_dtype, c * p.xs_c);
  double sd = 0.0, sq = 0.0;
  for (int j = 0; j < p.splits; ++j) {
    sd += (double)p.partial[(c * p.splits + j) * 2 + 0];
    sq += (double)p.partial[(c * p.splits + j) * 2 + 1];
  }
  const double cnt = (double)(p.N * p.S);
  const double md = sd / cnt;
  double var = sq / cnt - md * md; // biased, about the shifted mean
  if (var < 0.0) var = 0.0;
  const float mean = (float)((double)K + md);
  const float invstd = rsqrtf((float)var + p.eps);
  p.stats[c] = mean;
  p.stats[p.C + c] = invstd;
  if (p.saved_mean) store_f(p.saved_mean, p.sm_dtype, c, mean);
  if (p.saved_invstd) store_f(p.saved_invstd, p.si_dtype, c, invstd);
}

// y = (x - mean[c]) * invstd[c] * scale[c] + bias[c]; the linear index runs in X's physical order.
__global__ void __launch_bounds__(BN_THREADS) bn_apply_kernel(const BnParams p) {
  const int64_t total = p.N * p.C * p.S;
  for (int64_t i = (int64_t)blockIdx.x * BN_THREADS + threadIdx.x; i < total; i += (int64_t)gridDim.x * BN_THREADS) {
    int64_t n, c, s;
    if (p.channel_fast) {
      c = i % p.C;
      const int64_t r = i / p.C;
      s = r % p.S;
      n = r / p.S;
    } else {
      s = i % p.S;
      const int64_t r = i / p.S;
      c = r % p.C;
      n = r / p.C;
    }
    float mean, invstd;
    if (p.training) {
      mean = p.stats[c];
      invstd = p.stats[p.C + c];
    } else {
      mean = load_f(p.mean, p.mean_dtype, c);
      invstd = rsqrtf(load_f(p.var, p.var_dtype, c) + p.eps);
    }
    const float g = p.scale ? load_f(p.scale, p.scale_dtype, c) : 1.f;
    const float b = p.bias ? load_f(p.bias, p.bias_dtype, c) : 0.f;
    const float x = load_f(p.x, p.x_dtype, n * p.xs_n + c * p.xs_c + s * p.xs_s);
    store_f(p.y, p.y_dtype, n * p.ys_n + c * p.ys_c + s * p.ys_s, (x - mean) * invstd * g + b);
  }
}

// (batch, channel, flattened spatial) strides of a contiguous or channels-last tensor; false for
// any other layout.
bool ncs_strides(const TensorInfo &t, int64_t &sn, int64_t &sc, int64_t &ss) {
  int64_t S = 1;
  for (int i = 2; i < t.rank; ++i) S *= t.dims[i];
  const int64_t C = t.dims[1];
  bool contiguous = true, channels_last = true;
  int64_t run = 1;
  for (int i = t.rank - 1; i >= 0; --i) { // N, C, spatial... row-major
    if (t.dims[i] != 1 && t.strides[i] != run) contiguous = false;
    run *= t.dims[i];
  }
  run = C;
  for (int i = t.rank - 1; i >= 2; --i) { // N, spatial..., C
    if (t.dims[i] != 1 && t.strides[i] != run) channels_last = false;
    run *= t.dims[i];
  }
  if (C != 1 && t.strides[1] != 1) channels_last = false;
  if (t.dims[0] != 1 && t.strides[0] != C * S) channels_last = false;
  if (contiguous) {
    sn = C * S; sc = S; ss = 1;
    return true;
  }
  if (channels_last) {
    sn = C * S; sc = 1; ss = C;
    return true;
  }
  return false;
}

int pick_splits(const TensorInfo &x, bool channel_fast) {
  int64_t S = 1;
  for (int i = 2; i < x.rank; ++i) S *= x.dims[i];
  const int64_t total = x.dims[0] * S, C = x.dims[1];
  const int64_t groups = channel_fast ? (C + 31) / 32 : C;
  const int64_t min_per = channel_fast ? 64 : 1024; // positions per slice worth a CTA
  int64_t want = (4 * 148 + groups - 1) / groups;
  int64_t cap = total / min_per;
  if (cap < 1) cap = 1;
  if (want > cap) want = cap;
  if (want > 1024) want = 1024;
  return (int)(want < 1 ? 1 : want);
}

} // namespace

int64_t batchnorm_scratch_bytes(const Plan &plan, const Step &s, int32_t *splits) {
  const fb_node_desc &d = plan.nodes[s.node].d;
  *splits = 1;
  if (!(d.flags & FB_FLAG_NORM_TRAINING)) return 0;
  const TensorInfo &x = plan.tensors[d.inputs[0]];
  int64_t sn, sc, ss;
  if (!ncs_strides(x, sn, sc, ss)) return 0;
  *splits = pick_splits(x, sc == 1 && x.dims[1] > 1);
  const int64_t C = x.dims[1];
  return (C * (int64_t)*splits * 2 + 2 * C) * (int64_t)sizeof(float);
}

fb_status launch_batchnorm(const ExecContext &cx, const Step &s) {
  const Plan &plan = *cx.plan;
  const fb_node_desc &d = plan.nodes[s.node].d;
  const TensorInfo &x = plan.tensors[d.inputs[0]], &y = plan.tensors[d.outputs[0]];
  BnParams p;
  memset(&p, 0, sizeof(p));
  p.training = (d.flags & FB_FLAG_NORM_TRAINING) ? 1 : 0;
  p.N = x.dims[0];
  p.C = x.dims[1];
  p.S = 1;
  for (int i = 2; i < x.rank; ++i) p.S *= x.dims[i];
  FB_REQUIRE(ncs_strides(x, p.xs_n, p.xs_c, p.xs_s) && ncs_strides(y, p.ys_n, p.ys_c, p.ys_s), FB_INTERNAL_ERROR,
             "batchnorm: X and Y must be contiguous or channels-last");
  p.channel_fast = (p.xs_c == 1 && p.C > 1) ? 1 : 0;
  p.x = cx.tensor_ptr(d.inputs[0]);
  p.y = cx.tensor_ptr(d.outputs[0]);
  FB_REQUIRE(p.x && p.y, FB_INTERNAL_ERROR, "batchnorm: tensor has no buffer");
  p.x_dtype = x.dtype;
  p.y_dtype = y.dtype;
  auto bind = [&](int id, const void *&ptr, int32_t &dt) {
    if (id < 0) return;
    ptr = cx.tensor_ptr(id);
    dt = plan.tensors[id].dtype;
  };
  bind(d.inputs[1], p.scale, p.scale_dtype);
  bind(d.inputs[2], p.bias, p.bias_dtype);
  bind(d.inputs[3], p.mean, p.mean_dtype);
  bind(d.inputs[4], p.var, p.var_dtype);
  p.eps = (float)plan.tensors[d.inputs[5]].scalar;
  const int64_t total = p.N * p.C * p.S;
  const int apply_grid = (int)std::min<int64_t>((total + BN_THREADS - 1) / BN_THREADS, (int64_t)cx.dev->sm_count * 16);
  if (p.training) {
    if (d.outputs[1] >= 0) {
      p.saved_mean = cx.tensor_ptr(d.outputs[1]);
      p.sm_dtype = plan.tensors[d.outputs[1]].dtype;
    }
    if (d.outputs[2] >= 0) {
      p.saved_invstd = cx.tensor_ptr(d.outputs[2]);
      p.si_dtype = plan.tensors[d.outputs[2]].dtype;
    }
    FB_REQUIRE(s.scratch_offset >= 0 && cx.workspace != nullptr, FB_INTERNAL_ERROR,
               "batchnorm: training needs its statistics scratch in the workspace");
    p.splits = s.split_k;
    p.partial = reinterpret_cast<float *>(cx.workspace + s.scratch_offset);
    p.stats = p.partial + p.C * p.splits * 2;
    if (p.channel_fast) {
      dim3 grid((unsigned)((p.C + 31) / 32), (unsigned)p.splits), block(32, 8);
      bn_partial_channel_kernel<<<grid, block, 0, cx.dev->stream>>>(p);
    } else {
      FB_REQUIRE(p.C <= 0x7fffffff, FB_NOT_IMPLEMENTED, "batchnorm: too many channels");
      dim3 grid((unsigned)p.C, (unsigned)p.splits);
      bn_partial_spatial_kernel<<<grid, BN_THREADS, 0, cx.dev->stream>>>(p);
    }
    bn_finalize_kernel<<<(unsigned)((p.C + 127) / 128), 128, 0, cx.dev->stream>>>(p);
  } else {
    FB_REQUIRE(p.mean && p.var, FB_INTERNAL_ERROR, "batchnorm: inference needs MEAN and VAR");
  }
  bn_apply_kernel<<<apply_grid, BN_THREADS, 0, cx.dev->stream>>>(p);
  return FB_OK;
}

} // namespace fb

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
// loads coalesce in both layouts. These are HBM-bound passes: X and Y of one type and layout take
// the 16-byte vector kernels, anything else the strided scalar ones.
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

// ---- 16-byte vector paths -------------------------------------------------------------------
// X and Y of one 16- or 32-bit float type and one layout. A thread keeps its channel(s) for the
// whole kernel, so the per-channel coefficients are computed once and the inner loop is one
// 16-byte load, N fused multiply-adds and one 16-byte store, with no index division.

template <typename T> struct V16 {
  static constexpr int N = 16 / sizeof(T);
};
template <typename T> __device__ __forceinline__ void unpack16(const uint4 &r, float *v);
template <> __device__ __forceinline__ void unpack16<float>(const uint4 &r, float *v) {
  v[0] = __uint_as_float(r.x); v[1] = __uint_as_float(r.y); v[2] = __uint_as_float(r.z); v[3] = __uint_as_float(r.w);
}
template <> __device__ __forceinline__ void unpack16<__half>(const uint4 &r, float *v) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
template <> __device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4 &r, float *v) {
  const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <typename T> __device__ __forceinline__ uint4 pack16(const float *v);
template <> __device__ __forceinline__ uint4 pack16<float>(const float *v) {
  return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
}
template <> __device__ __forceinline__ uint4 pack16<__half>(const float *v) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t *>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
template <> __device__ __forceinline__ uint4 pack16<__nv_bfloat16>(const float *v) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t *>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// y = x * a + b for channel c
__device__ __forceinline__ void bn_coeff(const BnParams &p, int64_t c, float &a, float &b) {
  float mean, invstd;
  if (p.training) {
    mean = p.stats[c];
    invstd = p.stats[p.C + c];
  } else {
    mean = load_f(p.mean, p.mean_dtype, c);
    invstd = rsqrtf(load_f(p.var, p.var_dtype, c) + p.eps);
  }
  const float g = p.scale ? load_f(p.scale, p.scale_dtype, c) : 1.f;
  const float bt = p.bias ? load_f(p.bias, p.bias_dtype, c) : 0.f;
  // (x - mean) * invstd * g + bt folded into one multiply-add per element
  a = invstd * g;
  b = bt - mean * a;
}

// Channels-last: the tensor is one linear run of 16-byte vectors, vector i holds channels
// (i % cols) * N ...; blockDim.x is a multiple of cols, so a thread's column never changes.
template <typename T> __global__ void __launch_bounds__(1024) bn_apply_cl_kernel(const BnParams p, int cols) {
  constexpr int N = V16<T>::N;
  extern __shared__ float coeff[]; // [2][C]: the CTA computes every channel's (a, b) once
  for (int64_t c = threadIdx.x; c < p.C; c += blockDim.x) bn_coeff(p, c, coeff[c], coeff[p.C + c]);
  __syncthreads();
  const int col = threadIdx.x % cols;
  float a[N], b[N];
#pragma unroll
  for (int j = 0; j < N; ++j) {
    a[j] = coeff[col * N + j];
    b[j] = coeff[p.C + col * N + j];
  }
  const int64_t total = p.N * p.S * cols;
  const uint4 *x4 = static_cast<const uint4 *>(p.x);
  uint4 *y4 = static_cast<uint4 *>(p.y);
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  // four loads in flight per thread: one per iteration leaves the memory system idle
  for (; i + 3 * step < total; i += 4 * step) {
    uint4 r[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) r[u] = x4[i + u * step];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float v[N];
      unpack16<T>(r[u], v);
#pragma unroll
      for (int j = 0; j < N; ++j) v[j] = fmaf(v[j], a[j], b[j]);
      y4[i + u * step] = pack16<T>(v);
    }
  }
  for (; i < total; i += step) {
    float v[N];
    unpack16<T>(x4[i], v);
#pragma unroll
    for (int j = 0; j < N; ++j) v[j] = fmaf(v[j], a[j], b[j]);
    y4[i] = pack16<T>(v);
  }
}

// Contiguous: plane (n, c) is S consecutive elements; a CTA walks whole planes.
template <typename T> __global__ void __launch_bounds__(BN_THREADS) bn_apply_plane_kernel(const BnParams p) {
  constexpr int N = V16<T>::N;
  const int64_t planes = p.N * p.C;
  const T *x = static_cast<const T *>(p.x);
  T *y = static_cast<T *>(p.y);
  const bool vec = p.S % N == 0;
  for (int64_t pl = blockIdx.x; pl < planes; pl += gridDim.x) {
    float a, b;
    bn_coeff(p, pl % p.C, a, b);
    const int64_t base = pl * p.S;
    if (vec) {
      const uint4 *x4 = reinterpret_cast<const uint4 *>(x + base);
      uint4 *y4 = reinterpret_cast<uint4 *>(y + base);
      const int64_t nv = p.S / N;
      int64_t i = threadIdx.x;
      for (; i + 3 * BN_THREADS < nv; i += 4 * BN_THREADS) {
        uint4 r[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) r[u] = x4[i + u * BN_THREADS];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          float v[N];
          unpack16<T>(r[u], v);
#pragma unroll
          for (int j = 0; j < N; ++j) v[j] = fmaf(v[j], a, b);
          y4[i + u * BN_THREADS] = pack16<T>(v);
        }
      }
      for (; i < nv; i += BN_THREADS) {
        float v[N];
        unpack16<T>(x4[i], v);
#pragma unroll
        for (int j = 0; j < N; ++j) v[j] = fmaf(v[j], a, b);
        y4[i] = pack16<T>(v);
      }
    } else {
      for (int64_t i = threadIdx.x; i < p.S; i += BN_THREADS)
        store_f(y, p.y_dtype, base + i, fmaf(load_f(x, p.x_dtype, base + i), a, b));
    }
  }
}

// Channels-last statistics: CTA `blockIdx.x` of `splits` takes every splits-th group of rows.
template <typename T> __global__ void __launch_bounds__(1024) bn_partial_cl_kernel(const BnParams p, int cols) {
  constexpr int N = V16<T>::N;
  extern __shared__ float2 red[]; // [blockDim.x]
  const int col = threadIdx.x % cols, row = threadIdx.x / cols, rpb = blockDim.x / cols;
  const uint4 *x4 = static_cast<const uint4 *>(p.x);
  float K[N], s1[N], s2[N];
  unpack16<T>(x4[col], K); // first position of each channel
#pragma unroll
  for (int j = 0; j < N; ++j) s1[j] = s2[j] = 0.f;
  const int64_t rows = p.N * p.S;
  const int64_t rstep = (int64_t)gridDim.x * rpb;
  int64_t r = (int64_t)blockIdx.x * rpb + row;
  for (; r + 3 * rstep < rows; r += 4 * rstep) {
    uint4 raw[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) raw[u] = x4[(r + u * rstep) * cols + col];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float v[N];
      unpack16<T>(raw[u], v);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        const float d = v[j] - K[j];
        s1[j] += d;
        s2[j] = fmaf(d, d, s2[j]);
      }
    }
  }
  for (; r < rows; r += rstep) {
    float v[N];
    unpack16<T>(x4[r * cols + col], v);
#pragma unroll
    for (int j = 0; j < N; ++j) {
      const float d = v[j] - K[j];
      s1[j] += d;
      s2[j] = fmaf(d, d, s2[j]);
    }
  }
#pragma unroll
  for (int j = 0; j < N; ++j) {
    red[threadIdx.x] = make_float2(s1[j], s2[j]);
    __syncthreads();
    if (row == 0) {
      float2 t = red[col];
      for (int k = 1; k < rpb; ++k) {
        t.x += red[k * cols + col].x;
        t.y += red[k * cols + col].y;
      }
      const int64_t c = (int64_t)col * N + j;
      p.partial[(c * p.splits + blockIdx.x) * 2 + 0] = t.x;
      p.partial[(c * p.splits + blockIdx.x) * 2 + 1] = t.y;
    }
    __syncthreads();
  }
}

// Contiguous statistics: CTA (c, slice) walks the planes (n, c) of its batch slice.
template <typename T> __global__ void __launch_bounds__(BN_THREADS) bn_partial_plane_kernel(const BnParams p) {
  constexpr int N = V16<T>::N;
  __shared__ float2 sh[BN_THREADS / 32];
  const int64_t c = blockIdx.x;
  const T *x = static_cast<const T *>(p.x);
  const float K = load_f(p.x, p.x_dtype, c * p.S);
  const int64_t per = (p.N + p.splits - 1) / p.splits;
  const int64_t n0 = (int64_t)blockIdx.y * per, n1 = min(p.N, n0 + per);
  const bool vec = p.S % N == 0;
  float2 acc = make_float2(0.f, 0.f);
  for (int64_t n = n0; n < n1; ++n) {
    const int64_t base = (n * p.C + c) * p.S;
    if (vec) {
      const uint4 *x4 = reinterpret_cast<const uint4 *>(x + base);
      const int64_t nv = p.S / N;
      int64_t i = threadIdx.x;
      for (; i + 3 * BN_THREADS < nv; i += 4 * BN_THREADS) {
        uint4 raw[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) raw[u] = x4[i + u * BN_THREADS];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          float v[N];
          unpack16<T>(raw[u], v);
#pragma unroll
          for (int j = 0; j < N; ++j) {
            const float d = v[j] - K;
            acc.x += d;
            acc.y = fmaf(d, d, acc.y);
          }
        }
      }
      for (; i < nv; i += BN_THREADS) {
        float v[N];
        unpack16<T>(x4[i], v);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          const float d = v[j] - K;
          acc.x += d;
          acc.y = fmaf(d, d, acc.y);
        }
      }
    } else {
      for (int64_t i = threadIdx.x; i < p.S; i += BN_THREADS) {
        const float d = load_f(x, p.x_dtype, base + i) - K;
        acc.x += d;
        acc.y = fmaf(d, d, acc.y);
      }
    }
  }
  const float2 r = block_sum2(acc, sh);
  if (threadIdx.x == 0) {
    p.partial[(c * p.splits + blockIdx.y) * 2 + 0] = r.x;
    p.partial[(c * p.splits + blockIdx.y) * 2 + 1] = r.y;
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

// How a node runs: which kernels, how many slices the statistics pass cuts the reduction into.
struct BnChoice {
  bool ok = false;       // X and Y are contiguous or channels-last
  bool channel_fast = false;
  int vec = 0;           // 0 scalar kernels, 1 vector channels-last, 2 vector planes
  int cols = 0, threads = 0; // vector channels-last: 16-byte columns per row, CTA size (multiple of cols)
  int splits = 1;
  int64_t xs[3], ys[3];
};

BnChoice bn_choose(const TensorInfo &x, const TensorInfo &y) {
  BnChoice ch;
  if (!ncs_strides(x, ch.xs[0], ch.xs[1], ch.xs[2]) || !ncs_strides(y, ch.ys[0], ch.ys[1], ch.ys[2])) return ch;
  ch.ok = true;
  int64_t S = 1;
  for (int i = 2; i < x.rank; ++i) S *= x.dims[i];
  const int64_t N = x.dims[0], C = x.dims[1], rows = N * S;
  ch.channel_fast = ch.xs[1] == 1 && C > 1;
  const bool same = x.dtype == y.dtype && ch.xs[1] == ch.ys[1] && ch.xs[2] == ch.ys[2] &&
                    (x.dtype == FB_DT_FLOAT || x.dtype == FB_DT_HALF || x.dtype == FB_DT_BFLOAT16);
  const int per_vec = x.dtype == FB_DT_FLOAT ? 4 : 8;
  if (same && ch.channel_fast && C % per_vec == 0 && C / per_vec <= 1024 && C <= 4096) {
    ch.vec = 1;
    ch.cols = (int)(C / per_vec);
    int rpb = 512 / ch.cols;
    if (rpb < 1) rpb = 1;
    ch.threads = ch.cols * rpb;
    int64_t want = rows / ((int64_t)rpb * 8); // at least 8 rows per thread
    if (want > 2 * 148) want = 2 * 148;
    ch.splits = (int)(want < 1 ? 1 : want);
  } else if (same && !ch.channel_fast && (S * (x.dtype == FB_DT_FLOAT ? 4 : 2)) % 16 == 0) {
    ch.vec = 2;
    int64_t want = (4 * 148 + C - 1) / C;
    if (want > N) want = N;
    ch.splits = (int)(want < 1 ? 1 : want);
  } else {
    const int64_t groups = ch.channel_fast ? (C + 31) / 32 : C;
    const int64_t min_per = ch.channel_fast ? 64 : 1024; // positions per slice worth a CTA
    int64_t want = (4 * 148 + groups - 1) / groups;
    int64_t cap = rows / min_per;
    if (cap < 1) cap = 1;
    if (want > cap) want = cap;
    if (want > 1024) want = 1024;
    ch.splits = (int)(want < 1 ? 1 : want);
  }
  return ch;
}

template <typename T> void launch_vec(const BnParams &p, const BnChoice &ch, bool stats, int sm_count, cudaStream_t st) {
  constexpr int N = V16<T>::N;
  if (ch.vec == 1) {
    if (stats) {
      bn_partial_cl_kernel<T><<<p.splits, ch.threads, ch.threads * sizeof(float2), st>>>(p, ch.cols);
    } else {
      const int64_t total = p.N * p.S * ch.cols;
      // a CTA per SM pair of waves is enough: each thread then streams several vectors
      const int grid = (int)std::min<int64_t>((total + (int64_t)ch.threads * 4 - 1) / ((int64_t)ch.threads * 4),
                                              (int64_t)sm_count * 4);
      bn_apply_cl_kernel<T><<<grid, ch.threads, 2 * p.C * sizeof(float), st>>>(p, ch.cols);
    }
  } else {
    if (stats) {
      dim3 grid((unsigned)p.C, (unsigned)p.splits);
      bn_partial_plane_kernel<T><<<grid, BN_THREADS, 0, st>>>(p);
    } else {
      const int grid = (int)std::min<int64_t>(p.N * p.C, (int64_t)sm_count * 16);
      bn_apply_plane_kernel<T><<<grid, BN_THREADS, 0, st>>>(p);
    }
  }
  (void)N;
}

void launch_vec_any(const BnParams &p, const BnChoice &ch, bool stats, int sm_count, cudaStream_t st) {
  if (p.x_dtype == FB_DT_FLOAT) launch_vec<float>(p, ch, stats, sm_count, st);
  else if (p.x_dtype == FB_DT_HALF) launch_vec<__half>(p, ch, stats, sm_count, st);
  else launch_vec<__nv_bfloat16>(p, ch, stats, sm_count, st);
}

} // namespace

int64_t batchnorm_scratch_bytes(const Plan &plan, const Step &s, int32_t *splits) {
  const fb_node_desc &d = plan.nodes[s.node].d;
  *splits = 1;
  if (!(d.flags & FB_FLAG_NORM_TRAINING)) return 0;
  const TensorInfo &x = plan.tensors[d.inputs[0]];
  const BnChoice ch = bn_choose(x, plan.tensors[d.outputs[0]]);
  if (!ch.ok) return 0;
  *splits = ch.splits;
  const int64_t C = x.dims[1];
  return (C * (int64_t)ch.splits * 2 + 2 * C) * (int64_t)sizeof(float);
}

fb_status launch_batchnorm(const ExecContext &cx, const Step &s) {
  const Plan &plan = *cx.plan;
  const fb_node_desc &d = plan.nodes[s.node].d;
  const TensorInfo &x = plan.tensors[d.inputs[0]], &y = plan.tensors[d.outputs[0]];
  BnChoice ch = bn_choose(x, y);
  FB_REQUIRE(ch.ok, FB_INTERNAL_ERROR, "batchnorm: X and Y must be contiguous or channels-last");
  BnParams p;
  memset(&p, 0, sizeof(p));
  p.training = (d.flags & FB_FLAG_NORM_TRAINING) ? 1 : 0;
  p.N = x.dims[0];
  p.C = x.dims[1];
  p.S = 1;
  for (int i = 2; i < x.rank; ++i) p.S *= x.dims[i];
  p.xs_n = ch.xs[0]; p.xs_c = ch.xs[1]; p.xs_s = ch.xs[2];
  p.ys_n = ch.ys[0]; p.ys_c = ch.ys[1]; p.ys_s = ch.ys[2];
  p.channel_fast = ch.channel_fast ? 1 : 0;
  p.x = cx.tensor_ptr(d.inputs[0]);
  p.y = cx.tensor_ptr(d.outputs[0]);
  FB_REQUIRE(p.x && p.y, FB_INTERNAL_ERROR, "batchnorm: tensor has no buffer");
  // buffers that are not 16-byte aligned take the scalar kernels (same slices, same scratch layout)
  if (((uintptr_t)p.x | (uintptr_t)p.y) % 16 != 0) ch.vec = 0;
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
  cudaStream_t st = cx.dev->stream;
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
    FB_REQUIRE(p.C <= 0x7fffffff, FB_NOT_IMPLEMENTED, "batchnorm: too many channels");
    if (ch.vec) {
      launch_vec_any(p, ch, /*stats=*/true, cx.dev->sm_count, st);
    } else if (p.channel_fast) {
      dim3 grid((unsigned)((p.C + 31) / 32), (unsigned)p.splits), block(32, 8);
      bn_partial_channel_kernel<<<grid, block, 0, st>>>(p);
    } else {
      dim3 grid((unsigned)p.C, (unsigned)p.splits);
      bn_partial_spatial_kernel<<<grid, BN_THREADS, 0, st>>>(p);
    }
    bn_finalize_kernel<<<(unsigned)((p.C + 127) / 128), 128, 0, st>>>(p);
  } else {
    FB_REQUIRE(p.mean && p.var, FB_INTERNAL_ERROR, "batchnorm: inference needs MEAN and VAR");
  }
  if (ch.vec) {
    launch_vec_any(p, ch, /*stats=*/false, cx.dev->sm_count, st);
  } else {
    const int64_t total = p.N * p.C * p.S;
    const int grid = (int)std::min<int64_t>((total + BN_THREADS - 1) / BN_THREADS, (int64_t)cx.dev->sm_count * 16);
    bn_apply_kernel<<<grid, BN_THREADS, 0, st>>>(p);
  }
  return FB_OK;
}

} // namespace fb

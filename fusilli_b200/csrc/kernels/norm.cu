// LayerNorm (inference and training outputs) and RMSNorm over all non-batch dims.
//
// X is contiguous or channels-last, so each sample is one dense run of R elements ("row").
// HBM-bound: every kernel reads a row once and writes it once -- 2 * R * sizeof(T) bytes per
// row, the algorithmic minimum -- and takes the statistics in ONE block reduction through shifted
// moments: d = x - x0 (x0 = first element of the row), mean = x0 + sum(d)/R,
// var = sum(d*d)/R - (sum(d)/R)^2, which has none of the cancellation of E[x^2] - mean^2.
//   norm_rows_staged_kernel  LayerNorm on long rows with many samples: persistent CTAs, rows
//                            staged through a shared-memory ring by bulk copies, scale and bias
//                            in registers;
//   norm_rows_kernel         one row per CTA, the row packed in registers, parameters through L1;
//   norm_generic_kernel      any row length and layouts where scale/bias/Y are ordered
//                            differently from X (re-reads the row from L2).
#include <cstdlib>

#include "../common.h"
#include "sm100.cuh"

namespace fb {

struct NormParams {
  const void *x, *scale, *bias;
  void *y, *mean, *rstd;
  int32_t x_dtype, y_dtype, scale_dtype, bias_dtype, mean_dtype, rstd_dtype;
  int32_t is_rms;
  int32_t n_inner;   // rank - 1
  float eps;
  int64_t batch, row;
  int64_t x_bstride, y_bstride;
  int64_t inner_dims[FB_MAX_RANK]; // non-batch dims in X's physical order, slowest first
  int64_t y_istr[FB_MAX_RANK], s_istr[FB_MAX_RANK], b_istr[FB_MAX_RANK];
  int32_t same_order; // Y, scale, bias are all laid out like X within a row
  uint32_t *err;      // device error word for bounded waits
};

__device__ __forceinline__ float block_sum(float v, float *smem) {
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  int warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  __syncthreads(); // smem may still be read from a previous call
  if ((threadIdx.x & 31) == 0) smem[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < nwarp; ++w) t += smem[w];
  return t;
}

__global__ void __launch_bounds__(256) norm_generic_kernel(const NormParams p) {
  __shared__ float smem[8];
  for (int64_t b = blockIdx.x; b < p.batch; b += gridDim.x) {
    const int64_t xb = b * p.x_bstride;
    float mean = 0.f;
    if (!p.is_rms) {
      float s = 0.f;
      for (int64_t i = threadIdx.x; i < p.row; i += blockDim.x) s += load_f(p.x, p.x_dtype, xb + i);
      mean = block_sum(s, smem) / (float)p.row;
    }
    float ss = 0.f;
    for (int64_t i = threadIdx.x; i < p.row; i += blockDim.x) {
      float dlt = load_f(p.x, p.x_dtype, xb + i) - mean;
      ss += dlt * dlt;
    }
    float rstd = rsqrtf(block_sum(ss, smem) / (float)p.row + p.eps);
    for (int64_t i = threadIdx.x; i < p.row; i += blockDim.x) {
      int64_t yo = i, so = i, bo = i;
      if (!p.same_order) {
        int64_t rem = i;
        yo = so = bo = 0;
        for (int d = p.n_inner - 1; d >= 0; --d) {
          int64_t c = rem % p.inner_dims[d];
          rem /= p.inner_dims[d];
          yo += c * p.y_istr[d];
          so += c * p.s_istr[d];
          bo += c * p.b_istr[d];
        }
      }
      float v = (load_f(p.x, p.x_dtype, xb + i) - mean) * rstd;
      if (p.scale) v *= load_f(p.scale, p.scale_dtype, so);
      if (p.bias) v += load_f(p.bias, p.bias_dtype, bo);
      store_f(p.y, p.y_dtype, b * p.y_bstride + yo, v);
    }
    if (threadIdx.x == 0) {
      if (p.mean) store_f(p.mean, p.mean_dtype, b, mean);
      if (p.rstd) store_f(p.rstd, p.rstd_dtype, b, rstd);
    }
  }
}

template <typename T> __device__ __forceinline__ float nelem_f(T x);
template <> __device__ __forceinline__ float nelem_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float nelem_f<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float nelem_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T nelem_from(float x);
template <> __device__ __forceinline__ float nelem_from<float>(float x) { return x; }
template <> __device__ __forceinline__ __half nelem_from<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 nelem_from<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// Loads N consecutive parameters (scale or bias) as floats; P = parameter type.
template <typename P, int N> __device__ __forceinline__ void load_params(const void *base, int64_t off, float *out) {
  const P *q = static_cast<const P *>(base) + off;
  constexpr int BYTES = N * sizeof(P);
  if constexpr (BYTES == 16) {
    uint4 r = __ldg(reinterpret_cast<const uint4 *>(q));
    const P *e = reinterpret_cast<const P *>(&r);
#pragma unroll
    for (int j = 0; j < N; ++j) out[j] = nelem_f<P>(e[j]);
  } else if constexpr (BYTES == 32) {
    uint4 r0 = __ldg(reinterpret_cast<const uint4 *>(q)), r1 = __ldg(reinterpret_cast<const uint4 *>(q) + 1);
    const P *e0 = reinterpret_cast<const P *>(&r0), *e1 = reinterpret_cast<const P *>(&r1);
#pragma unroll
    for (int j = 0; j < N / 2; ++j) {
      out[j] = nelem_f<P>(e0[j]);
      out[N / 2 + j] = nelem_f<P>(e1[j]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < N; ++j) out[j] = nelem_f<P>(q[j]);
  }
}

// ---- packed fp32x2 arithmetic (sm_100: one instruction per pair) ---------------------------
__device__ __forceinline__ float2 f2_fma(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(*reinterpret_cast<uint64_t *>(&d))
      : "l"(*reinterpret_cast<uint64_t *>(&a)), "l"(*reinterpret_cast<uint64_t *>(&b)),
        "l"(*reinterpret_cast<uint64_t *>(&c)));
  return d;
}
__device__ __forceinline__ float2 f2_mul(float2 a, float2 b) {
  float2 d;
  asm("mul.rn.f32x2 %0, %1, %2;"
      : "=l"(*reinterpret_cast<uint64_t *>(&d))
      : "l"(*reinterpret_cast<uint64_t *>(&a)), "l"(*reinterpret_cast<uint64_t *>(&b)));
  return d;
}
__device__ __forceinline__ float2 f2_add(float2 a, float2 b) {
  float2 d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(*reinterpret_cast<uint64_t *>(&d))
      : "l"(*reinterpret_cast<uint64_t *>(&a)), "l"(*reinterpret_cast<uint64_t *>(&b)));
  return d;
}

// Element pair `i` of a 16-byte vector as two floats.
template <typename T> __device__ __forceinline__ float2 vec_pair(const uint4 &r, int i);
template <> __device__ __forceinline__ float2 vec_pair<float>(const uint4 &r, int i) {
  const float *f = reinterpret_cast<const float *>(&r);
  return make_float2(f[2 * i], f[2 * i + 1]);
}
template <> __device__ __forceinline__ float2 vec_pair<__nv_bfloat16>(const uint4 &r, int i) {
  const uint32_t w = reinterpret_cast<const uint32_t *>(&r)[i];
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 vec_pair<__half>(const uint4 &r, int i) {
  return __half22float2(reinterpret_cast<const __half2 *>(&r)[i]);
}
template <typename T> __device__ __forceinline__ void vec_set_pair(uint4 &r, int i, float2 v);
template <> __device__ __forceinline__ void vec_set_pair<float>(uint4 &r, int i, float2 v) {
  float *f = reinterpret_cast<float *>(&r);
  f[2 * i] = v.x;
  f[2 * i + 1] = v.y;
}
template <> __device__ __forceinline__ void vec_set_pair<__nv_bfloat16>(uint4 &r, int i, float2 v) {
  reinterpret_cast<__nv_bfloat162 *>(&r)[i] = __floats2bfloat162_rn(v.x, v.y);
}
template <> __device__ __forceinline__ void vec_set_pair<__half>(uint4 &r, int i, float2 v) {
  reinterpret_cast<__half2 *>(&r)[i] = __floats2half2_rn(v.x, v.y);
}

// Sums two values across the CTA with one pair of barriers.
__device__ __forceinline__ float2 block_sum2(float2 v, float2 *smem) {
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) {
    v.x += __shfl_xor_sync(0xffffffffu, v.x, m);
    v.y += __shfl_xor_sync(0xffffffffu, v.y, m);
  }
  const int warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  __syncthreads();
  if ((threadIdx.x & 31) == 0) smem[warp] = v;
  __syncthreads();
  float2 t = make_float2(0.f, 0.f);
  for (int w = 0; w < nwarp; ++w) {
    t.x += smem[w].x;
    t.y += smem[w].y;
  }
  return t;
}

// Row kernel: T = X and Y element type, P = scale/bias element type, THREADS threads per
// row, V 16-byte vectors per thread (row == THREADS * V * (16 / sizeof(T))). The row stays
// PACKED in registers (V uint4). Two sweeps over the registers, both in packed fp32x2:
//   1. shifted moments: d = x - x0 (x0 = first element of the row), s += d, ss += d*d, one
//      block reduction for both; mean = x0 + s/n, var = (ss - s*s/n)/n. Shifting by a sample
//      of the row removes the cancellation of the raw E[x^2] - mean^2 form.
//   2. y = x * (rstd*gamma) + (beta - mean*rstd*gamma).
// The kernel is instruction-issue sensitive at HBM speed (64 values per thread): the packed
// ops and the two-sweep form are what keep it on the bandwidth roof.
template <typename T, typename P, int V, int THREADS>
__global__ void __launch_bounds__(THREADS) norm_rows_kernel(const NormParams p) {
  constexpr int N = 16 / sizeof(T);
  constexpr int NP = N / 2;
  __shared__ float2 smem[8];
  const float inv_row = 1.f / (float)p.row;
  for (int64_t b = blockIdx.x; b < p.batch; b += gridDim.x) {
    const T *xrow = static_cast<const T *>(p.x) + b * p.x_bstride;
    const uint4 *xr = reinterpret_cast<const uint4 *>(xrow);
    uint4 raw[V];
#pragma unroll
    for (int v = 0; v < V; ++v) raw[v] = __ldg(xr + threadIdx.x + v * THREADS);
    const float x0 = p.is_rms ? 0.f : nelem_f<T>(__ldg(xrow));
    const float2 shift = make_float2(-x0, -x0);
    float2 s2 = make_float2(0.f, 0.f), ss2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int v = 0; v < V; ++v) {
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        const float2 d = f2_add(vec_pair<T>(raw[v], j), shift);
        s2 = f2_add(s2, d);
        ss2 = f2_fma(d, d, ss2);
      }
    }
    const float2 tot = block_sum2(make_float2(s2.x + s2.y, ss2.x + ss2.y), smem);
    float mean = 0.f, var;
    if (p.is_rms) {
      var = tot.y * inv_row;
    } else {
      const float ds = tot.x * inv_row;
      mean = x0 + ds;
      var = fmaxf(tot.y * inv_row - ds * ds, 0.f);
    }
    const float rstd = rsqrtf(var + p.eps);
    const float2 rs2 = make_float2(rstd, rstd), nm2 = make_float2(-mean, -mean);
    uint4 *yr = reinterpret_cast<uint4 *>(static_cast<T *>(p.y) + b * p.y_bstride);
#pragma unroll
    for (int v = 0; v < V; ++v) {
      const int64_t col = ((int64_t)threadIdx.x + v * THREADS) * N;
      float g[N], bt[N];
      if (p.scale) load_params<P, N>(p.scale, col, g);
      if (p.bias) load_params<P, N>(p.bias, col, bt);
      uint4 o;
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        float2 a = rs2;
        if (p.scale) a = f2_mul(make_float2(g[2 * j], g[2 * j + 1]), rs2);
        float2 c = f2_mul(nm2, a);
        if (p.bias) c = f2_add(c, make_float2(bt[2 * j], bt[2 * j + 1]));
        vec_set_pair<T>(o, j, f2_fma(vec_pair<T>(raw[v], j), a, c));
      }
      yr[threadIdx.x + v * THREADS] = o;
    }
    if (threadIdx.x == 0) {
      if (p.mean) store_f(p.mean, p.mean_dtype, b, mean);
      if (p.rstd) store_f(p.rstd, p.rstd_dtype, b, rstd);
    }
  }
}

// Staged row kernel for the large-row case (HBM-bound at full speed): persistent CTAs of 256
// threads, each walking rows blockIdx.x, blockIdx.x + gridDim.x, ... The rows arrive through a
// ring of STAGES shared-memory slots filled by bulk copies (cp.async.bulk, one elected thread,
// completion on an mbarrier), so STAGES rows per CTA are in flight whatever the threads are
// doing; scale and bias live in registers for the whole kernel (no per-row parameter traffic);
// one barrier per row (partial sums double-buffered). T = X and Y element type, P = scale/bias
// element type, V 16-byte vectors per thread (row == 256 * V * (16 / sizeof(T))).
constexpr int kStagedStages = 4;
template <typename T, typename P, int V, int THREADS>
__global__ void __launch_bounds__(THREADS, 2) norm_rows_staged_kernel(const NormParams p) {
  using namespace sm100;
  constexpr int STAGES = kStagedStages;
  constexpr int N = 16 / sizeof(T), NP = N / 2, NW = THREADS / 32;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  const uint32_t row_bytes = (uint32_t)(p.row * sizeof(T));
  const uint32_t smem0 = smem_u32(smem_raw);
  const uint32_t bar0 = smem0 + STAGES * row_bytes;
  float2 *partial = reinterpret_cast<float2 *>(smem_raw + STAGES * row_bytes + 64); // [2][NW]
  const int64_t first = blockIdx.x, step = gridDim.x;
  const int64_t my_rows = first < p.batch ? (p.batch - first + step - 1) / step : 0;
  auto issue = [&](int64_t k) { // row k of this CTA into slot k % STAGES
    const uint32_t bar = bar0 + 8u * (uint32_t)(k % STAGES);
    mbar_expect_tx(bar, row_bytes);
    tma_bulk_load(smem0 + (uint32_t)(k % STAGES) * row_bytes,
                  static_cast<const T *>(p.x) + (first + k * step) * p.x_bstride, row_bytes, bar);
  };
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) mbar_init(bar0 + 8u * s, 1);
    fence_barrier_init();
    for (int64_t k = 0; k < STAGES && k < my_rows; ++k) issue(k);
  }
  // parameters of this thread's columns, once
  float2 g[V * NP], bt[V * NP];
#pragma unroll
  for (int v = 0; v < V; ++v) {
    const int64_t col = ((int64_t)threadIdx.x + v * THREADS) * N;
    float gf[N], bf[N];
#pragma unroll
    for (int j = 0; j < N; ++j) {
      gf[j] = 1.f;
      bf[j] = 0.f;
    }
    if (p.scale) load_params<P, N>(p.scale, col, gf);
    if (p.bias) load_params<P, N>(p.bias, col, bf);
#pragma unroll
    for (int j = 0; j < NP; ++j) {
      g[v * NP + j] = make_float2(gf[2 * j], gf[2 * j + 1]);
      bt[v * NP + j] = make_float2(bf[2 * j], bf[2 * j + 1]);
    }
  }
  __syncthreads(); // barriers initialised
  const float inv_row = 1.f / (float)p.row;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int64_t k = 0; k < my_rows; ++k) {
    const int slot = (int)(k % STAGES);
    if (!mbar_wait(bar0 + 8u * slot, (uint32_t)((k / STAGES) & 1), p.err, ERR_WAIT_FULL)) break;
    const uint4 *xr = reinterpret_cast<const uint4 *>(smem_raw + (size_t)slot * row_bytes);
    uint4 raw[V];
#pragma unroll
    for (int v = 0; v < V; ++v) raw[v] = xr[threadIdx.x + v * THREADS];
    const float x0 = p.is_rms ? 0.f : nelem_f<T>(*reinterpret_cast<const T *>(xr));
    const float2 shift = make_float2(-x0, -x0);
    float2 s2 = make_float2(0.f, 0.f), ss2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int v = 0; v < V; ++v) {
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        const float2 d = f2_add(vec_pair<T>(raw[v], j), shift);
        s2 = f2_add(s2, d);
        ss2 = f2_fma(d, d, ss2);
      }
    }
    float2 tot = make_float2(s2.x + s2.y, ss2.x + ss2.y);
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) {
      tot.x += __shfl_xor_sync(0xffffffffu, tot.x, m);
      tot.y += __shfl_xor_sync(0xffffffffu, tot.y, m);
    }
    float2 *part = partial + (k & 1) * NW;
    if (lane == 0) part[warp] = tot;
    __syncthreads(); // partial sums visible; every thread has also finished reading the slot
    // The slot's reads have completed (their values fed the sums above) and the barrier orders
    // them before this point, so the slot can be handed back to the copy engine.
    if (threadIdx.x == 0 && k + STAGES < my_rows) issue(k + STAGES);
    tot = part[lane & (NW - 1)]; // NW is a power of two: every group of NW lanes holds all partials
#pragma unroll
    for (int m = NW / 2; m >= 1; m >>= 1) {
      tot.x += __shfl_xor_sync(0xffffffffu, tot.x, m);
      tot.y += __shfl_xor_sync(0xffffffffu, tot.y, m);
    }
    float mean = 0.f, var;
    if (p.is_rms) {
      var = tot.y * inv_row;
    } else {
      const float ds = tot.x * inv_row;
      mean = x0 + ds;
      var = fmaxf(tot.y * inv_row - ds * ds, 0.f);
    }
    const float rstd = rsqrtf(var + p.eps);
    const float2 rs2 = make_float2(rstd, rstd), nmr2 = make_float2(-mean * rstd, -mean * rstd);
    const int64_t b = first + k * step;
    uint4 *yr = reinterpret_cast<uint4 *>(static_cast<T *>(p.y) + b * p.y_bstride);
#pragma unroll
    for (int v = 0; v < V; ++v) {
      uint4 o;
#pragma unroll
      for (int j = 0; j < NP; ++j) {
        // y = ((x - mean) * rstd) * gamma + beta, with (x*rstd - mean*rstd) as one fma
        const float2 nrm = f2_fma(vec_pair<T>(raw[v], j), rs2, nmr2);
        vec_set_pair<T>(o, j, f2_fma(nrm, g[v * NP + j], bt[v * NP + j]));
      }
      yr[threadIdx.x + v * THREADS] = o;
    }
    if (threadIdx.x == 0) {
      if (p.mean) store_f(p.mean, p.mean_dtype, b, mean);
      if (p.rstd) store_f(p.rstd, p.rstd_dtype, b, rstd);
    }
  }
}

template <typename T, typename P, int V, int THREADS>
static bool launch_staged_v(const NormParams &p, int sm_count, cudaStream_t st) {
  const size_t smem = (size_t)kStagedStages * p.row * sizeof(T) + 64 + 2 * (THREADS / 32) * sizeof(float2);
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      sm100::set_max_dynamic_smem(reinterpret_cast<const void *>(norm_rows_staged_kernel<T, P, V, THREADS>), (int)smem,
                                  device) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  const int blocks = (int)std::min<int64_t>(p.batch, (int64_t)sm_count * 2);
  norm_rows_staged_kernel<T, P, V, THREADS><<<blocks, THREADS, smem, st>>>(p);
  return true;
}

// Rows of exactly 256 * V vectors with V in {2, 4} and at least a few rows per CTA.
template <typename T, typename P>
static bool launch_staged(const NormParams &p, int sm_count, cudaStream_t st) {
  constexpr int N = 16 / sizeof(T);
  if (p.batch < (int64_t)sm_count * 4) return false;
  if ((size_t)kStagedStages * p.row * sizeof(T) > 100 * 1024) return false; // two CTAs per SM
  if (p.row % (256 * N) != 0) return false;
  switch (p.row / (256 * N)) {
  case 2: return launch_staged_v<T, P, 2, 256>(p, sm_count, st);
  case 4: return launch_staged_v<T, P, 4, 256>(p, sm_count, st);
  default: return false;
  }
}

template <typename T, typename P>
static bool launch_rows(const NormParams &p, int sm_count, cudaStream_t st) {
  constexpr int N = 16 / sizeof(T);
  // Many long rows: the staged kernel (rows through a bulk-copy ring, parameters in registers) for both
  // norms. Measured on 32768 x 8192 bf16 with the host's enqueue latency hidden: LayerNorm 0.177 ms,
  // RMSNorm 0.180 ms staged against 0.188 ms on the one-row-per-CTA kernel below.
  if (launch_staged<T, P>(p, sm_count, st)) return true;
  const int blocks = (int)std::min<int64_t>(p.batch, (int64_t)sm_count * 64);
  if (p.row % (128 * N) == 0 && p.row / (128 * N) <= 8) {
    switch (p.row / (128 * N)) {
    case 1: norm_rows_kernel<T, P, 1, 128><<<blocks, 128, 0, st>>>(p); return true;
    case 2: norm_rows_kernel<T, P, 2, 128><<<blocks, 128, 0, st>>>(p); return true;
    case 3: norm_rows_kernel<T, P, 3, 128><<<blocks, 128, 0, st>>>(p); return true;
    case 4: norm_rows_kernel<T, P, 4, 128><<<blocks, 128, 0, st>>>(p); return true;
    case 6: norm_rows_kernel<T, P, 6, 128><<<blocks, 128, 0, st>>>(p); return true;
    case 8: norm_rows_kernel<T, P, 8, 128><<<blocks, 128, 0, st>>>(p); return true;
    default: break;
    }
  }
  if (p.row % (256 * N) == 0) {
    switch (p.row / (256 * N)) {
    case 8: norm_rows_kernel<T, P, 8, 256><<<blocks, 256, 0, st>>>(p); return true;
    case 6: norm_rows_kernel<T, P, 6, 256><<<blocks, 256, 0, st>>>(p); return true;
    default: break;
    }
  }
  return false;
}

fb_status launch_norm(const ExecContext &cx, const Step &s) {
  const Plan &plan = *cx.plan;
  const fb_node_desc &d = plan.nodes[s.node].d;
  const bool is_ln = d.op == FB_OP_LAYERNORM;
  const int xi = d.inputs[0], si = d.inputs[1], bi = is_ln ? d.inputs[2] : -1;
  const int ei = is_ln ? d.inputs[3] : d.inputs[2];
  const TensorInfo &x = plan.tensors[xi];
  const TensorInfo &y = plan.tensors[d.outputs[0]];
  NormParams p;
  memset(&p, 0, sizeof(p));
  p.is_rms = !is_ln;
  p.eps = (float)plan.tensors[ei].scalar;
  p.x = cx.tensor_ptr(xi);
  p.y = cx.tensor_ptr(d.outputs[0]);
  FB_REQUIRE(p.x && p.y, FB_INTERNAL_ERROR, "norm: tensor has no buffer");
  p.x_dtype = x.dtype;
  p.y_dtype = y.dtype;
  if (si >= 0) {
    p.scale = cx.tensor_ptr(si);
    p.scale_dtype = plan.tensors[si].dtype;
  }
  if (bi >= 0) {
    p.bias = cx.tensor_ptr(bi);
    p.bias_dtype = plan.tensors[bi].dtype;
  }
  if (is_ln && (d.flags & FB_FLAG_NORM_TRAINING)) {
    if (d.outputs[1] >= 0) {
      p.mean = cx.tensor_ptr(d.outputs[1]);
      p.mean_dtype = plan.tensors[d.outputs[1]].dtype;
    }
    if (d.outputs[2] >= 0) {
      p.rstd = cx.tensor_ptr(d.outputs[2]);
      p.rstd_dtype = plan.tensors[d.outputs[2]].dtype;
    }
  }
  p.batch = x.dims[0];
  p.row = 1;
  for (int i = 1; i < x.rank; ++i) p.row *= x.dims[i];
  p.x_bstride = p.row;
  p.y_bstride = p.row;
  // inner dims in X's physical order (slowest first)
  int order[FB_MAX_RANK];
  int n = 0;
  for (int i = 1; i < x.rank; ++i) order[n++] = i;
  for (int i = 1; i < n; ++i)
    for (int j = i; j > 0 && x.strides[order[j - 1]] < x.strides[order[j]]; --j) {
      int t = order[j - 1];
      order[j - 1] = order[j];
      order[j] = t;
    }
  p.n_inner = n;
  p.same_order = 1;
  for (int i = 0; i < n; ++i) {
    int dd = order[i];
    p.inner_dims[i] = x.dims[dd];
    p.y_istr[i] = y.strides[dd];
    if (x.dims[dd] > 1 && y.strides[dd] != x.strides[dd]) p.same_order = 0;
    if (si >= 0) {
      p.s_istr[i] = plan.tensors[si].strides[dd];
      if (x.dims[dd] > 1 && p.s_istr[i] != x.strides[dd]) p.same_order = 0;
    }
    if (bi >= 0) {
      p.b_istr[i] = plan.tensors[bi].strides[dd];
      if (x.dims[dd] > 1 && p.b_istr[i] != x.strides[dd]) p.same_order = 0;
    }
  }
  p.err = cx.dev->error_word;
  cudaStream_t st = cx.dev->stream;
  int blocks = (int)std::min<int64_t>(p.batch, (int64_t)cx.dev->sm_count * 32);
  bool aligned = ((uintptr_t)p.x % 16 == 0) && ((uintptr_t)p.y % 16 == 0) &&
                 (!p.scale || (uintptr_t)p.scale % 16 == 0) && (!p.bias || (uintptr_t)p.bias % 16 == 0);
  bool params_same = (!p.scale || !p.bias || p.scale_dtype == p.bias_dtype);
  int pdt = p.scale ? p.scale_dtype : (p.bias ? p.bias_dtype : x.dtype);
  if (p.same_order && aligned && params_same && x.dtype == y.dtype && (pdt == x.dtype || pdt == FB_DT_FLOAT)) {
    bool done = false;
    if (x.dtype == FB_DT_BFLOAT16)
      done = (pdt == FB_DT_FLOAT) ? launch_rows<__nv_bfloat16, float>(p, cx.dev->sm_count, st)
                                  : launch_rows<__nv_bfloat16, __nv_bfloat16>(p, cx.dev->sm_count, st);
    else if (x.dtype == FB_DT_HALF)
      done = (pdt == FB_DT_FLOAT) ? launch_rows<__half, float>(p, cx.dev->sm_count, st)
                                  : launch_rows<__half, __half>(p, cx.dev->sm_count, st);
    else if (x.dtype == FB_DT_FLOAT)
      done = launch_rows<float, float>(p, cx.dev->sm_count, st);
    if (done) return FB_OK;
  }
  norm_generic_kernel<<<blocks, 256, 0, st>>>(p);
  return FB_OK;
}

} // namespace fb

// Keep-dim reductions (ADD/SUM, MUL, MIN, MAX, AMAX, AVG, NORM1, NORM2,
// MUL_NO_ZEROS) over {i : Y[i]==1 && X[i]>1}.
//
// HBM-bound. The row kernel (reduction over the contiguous trailing extent of a
// dense tensor) streams each row once with 128-bit loads, several loads in flight
// per thread, fp32 accumulation, warp-shuffle + shared-memory combine. The general
// kernel handles any set of reduced dims and any strides; a group of 1, 32 or 256
// threads owns one output element. Integer inputs accumulate in int64 and stay
// exact.
#include "../common.h"

namespace fb {

struct RedParams {
  const void *x;
  void *y;
  int32_t x_dtype, y_dtype, mode, integer_math;
  int32_t n_keep, n_red;
  int64_t keep_dims[FB_MAX_RANK], keep_xstr[FB_MAX_RANK], keep_ystr[FB_MAX_RANK];
  int64_t red_dims[FB_MAX_RANK], red_xstr[FB_MAX_RANK]; // fastest stride first
  int64_t n_out, n_red_elems;
};

template <typename A> __device__ __forceinline__ A red_identity(int mode);
template <> __device__ __forceinline__ float red_identity<float>(int mode) {
  switch (mode) {
  case FB_RED_MUL:
  case FB_RED_MUL_NO_ZEROS: return 1.f;
  case FB_RED_MIN: return INFINITY;
  case FB_RED_MAX: return -INFINITY;
  default: return 0.f;
  }
}
template <> __device__ __forceinline__ int64_t red_identity<int64_t>(int mode) {
  switch (mode) {
  case FB_RED_MUL:
  case FB_RED_MUL_NO_ZEROS: return 1;
  case FB_RED_MIN: return INT64_MAX;
  case FB_RED_MAX: return INT64_MIN;
  default: return 0;
  }
}

// Folds one input element into an accumulator.
__device__ __forceinline__ float red_accum(int mode, float a, float v) {
  switch (mode) {
  case FB_RED_ADD:
  case FB_RED_SUM:
  case FB_RED_AVG: return a + v;
  case FB_RED_MUL: return a * v;
  case FB_RED_MUL_NO_ZEROS: return v != 0.f ? a * v : a;
  case FB_RED_MIN: return (v < a || v != v) ? v : a;
  case FB_RED_MAX: return (v > a || v != v) ? v : a;
  case FB_RED_AMAX: return (fabsf(v) > a || v != v) ? fabsf(v) : a;
  case FB_RED_NORM1: return a + fabsf(v);
  case FB_RED_NORM2: return a + v * v;
  default: return a;
  }
}
__device__ __forceinline__ int64_t red_accum(int mode, int64_t a, int64_t v) {
  int64_t av = v < 0 ? -v : v;
  switch (mode) {
  case FB_RED_ADD:
  case FB_RED_SUM: return a + v;
  case FB_RED_MUL: return a * v;
  case FB_RED_MUL_NO_ZEROS: return v != 0 ? a * v : a;
  case FB_RED_MIN: return v < a ? v : a;
  case FB_RED_MAX: return v > a ? v : a;
  case FB_RED_AMAX: return av > a ? av : a;
  case FB_RED_NORM1: return a + av;
  case FB_RED_NORM2: return a + v * v;
  default: return a;
  }
}
// Merges two partial accumulators.
__device__ __forceinline__ float red_merge(int mode, float a, float b) {
  switch (mode) {
  case FB_RED_MUL:
  case FB_RED_MUL_NO_ZEROS: return a * b;
  case FB_RED_MIN: return (b < a || b != b) ? b : a;
  case FB_RED_MAX:
  case FB_RED_AMAX: return (b > a || b != b) ? b : a;
  default: return a + b;
  }
}
__device__ __forceinline__ int64_t red_merge(int mode, int64_t a, int64_t b) {
  switch (mode) {
  case FB_RED_MUL:
  case FB_RED_MUL_NO_ZEROS: return a * b;
  case FB_RED_MIN: return b < a ? b : a;
  case FB_RED_MAX:
  case FB_RED_AMAX: return b > a ? b : a;
  default: return a + b;
  }
}
__device__ __forceinline__ float red_finish(int mode, float a, int64_t count) {
  if (mode == FB_RED_AVG) return a / (float)count;
  if (mode == FB_RED_NORM2) return sqrtf(a);
  return a;
}
__device__ __forceinline__ int64_t red_finish(int mode, int64_t a, int64_t) {
  if (mode == FB_RED_NORM2) return (int64_t)sqrt((double)a);
  return a;
}

template <typename A> __device__ __forceinline__ A shfl_xor_t(A v, int m);
template <> __device__ __forceinline__ float shfl_xor_t<float>(float v, int m) {
  return __shfl_xor_sync(0xffffffffu, v, m);
}
template <> __device__ __forceinline__ int64_t shfl_xor_t<int64_t>(int64_t v, int m) {
  return __shfl_xor_sync(0xffffffffu, (long long)v, m);
}

template <typename A> __device__ __forceinline__ A red_load(const void *p, int dt, int64_t i);
template <> __device__ __forceinline__ float red_load<float>(const void *p, int dt, int64_t i) { return load_f(p, dt, i); }
template <> __device__ __forceinline__ int64_t red_load<int64_t>(const void *p, int dt, int64_t i) { return load_i(p, dt, i); }
template <typename A> __device__ __forceinline__ void red_store(void *p, int dt, int64_t i, A v);
template <> __device__ __forceinline__ void red_store<float>(void *p, int dt, int64_t i, float v) { store_f(p, dt, i, v); }
template <> __device__ __forceinline__ void red_store<int64_t>(void *p, int dt, int64_t i, int64_t v) { store_i(p, dt, i, v); }

// G threads (1, 32 or 256 = one CTA) per output element.
template <typename A, int G>
__global__ void __launch_bounds__(256) reduce_generic_kernel(const RedParams p) {
  __shared__ A smem[8];
  const int per_block = 256 / G;
  int64_t out = (int64_t)blockIdx.x * per_block + threadIdx.x / G;
  int lane = threadIdx.x % G;
  bool active = out < p.n_out;
  int64_t xbase = 0, yoff = 0;
  if (active) {
    int64_t rem = out;
    for (int d = p.n_keep - 1; d >= 0; --d) {
      int64_t c = rem % p.keep_dims[d];
      rem /= p.keep_dims[d];
      xbase += c * p.keep_xstr[d];
      yoff += c * p.keep_ystr[d];
    }
  }
  A acc = red_identity<A>(p.mode);
  if (active) {
    for (int64_t r = lane; r < p.n_red_elems; r += G) {
      int64_t rem = r, off = xbase;
      for (int d = 0; d < p.n_red; ++d) {
        off += (rem % p.red_dims[d]) * p.red_xstr[d];
        rem /= p.red_dims[d];
      }
      acc = red_accum(p.mode, acc, red_load<A>(p.x, p.x_dtype, off));
    }
  }
  if (G >= 32) {
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) acc = red_merge(p.mode, acc, shfl_xor_t<A>(acc, m));
  }
  if (G == 256) {
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      A t = smem[0];
      for (int w = 1; w < 8; ++w) t = red_merge(p.mode, t, smem[w]);
      acc = t;
    }
  }
  if (active && lane == 0) red_store<A>(p.y, p.y_dtype, yoff, red_finish(p.mode, acc, p.n_red_elems));
}

// Row reduction of a dense [rows, cols] view, T in {float, __half, __nv_bfloat16};
// cols * sizeof(T) a multiple of 16 and rows 16-byte aligned. One CTA per row.
template <typename T> __device__ __forceinline__ float elem_f(T x);
template <> __device__ __forceinline__ float elem_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float elem_f<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float elem_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

// 128 threads per row; every thread issues all of its 16-byte loads (up to 8) before it
// touches the data, so a 16 KB row is completely in flight at once and up to 16 rows per SM.
template <typename T>
__global__ void __launch_bounds__(128) reduce_rows_kernel(const T *__restrict__ x, void *y, int y_dtype,
                                                          int64_t y_stride, int64_t rows, int64_t cols,
                                                          int mode) {
  constexpr int N = 16 / sizeof(T);
  constexpr int TH = 128, U = 8;
  __shared__ float smem[4];
  const int64_t nvec = cols / N;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4 *xr = reinterpret_cast<const uint4 *>(x + row * cols);
    float acc = red_identity<float>(mode);
    for (int64_t base = 0; base < nvec; base += (int64_t)TH * U) {
      uint4 r[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t i = base + threadIdx.x + (int64_t)u * TH;
        r[u] = i < nvec ? __ldg(xr + i) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t i = base + threadIdx.x + (int64_t)u * TH;
        if (i < nvec) {
          const T *e = reinterpret_cast<const T *>(&r[u]);
#pragma unroll
          for (int j = 0; j < N; ++j) acc = red_accum(mode, acc, elem_f<T>(e[j]));
        }
      }
    }
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) acc = red_merge(mode, acc, __shfl_xor_sync(0xffffffffu, acc, m));
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = smem[0];
      for (int w = 1; w < TH / 32; ++w) t = red_merge(mode, t, smem[w]);
      store_f(y, y_dtype, row * y_stride, red_finish(mode, t, cols));
    }
    __syncthreads();
  }
}

static bool is_float_dt(int dt) { return dt == FB_DT_HALF || dt == FB_DT_BFLOAT16 || dt == FB_DT_FLOAT; }

fb_status launch_reduction(const ExecContext &cx, const Step &s) {
  const Plan &plan = *cx.plan;
  const fb_node_desc &d = plan.nodes[s.node].d;
  const TensorInfo &x = plan.tensors[d.inputs[0]];
  const TensorInfo &y = plan.tensors[d.outputs[0]];
  RedParams p;
  memset(&p, 0, sizeof(p));
  p.x = cx.tensor_ptr(d.inputs[0]);
  p.y = cx.tensor_ptr(d.outputs[0]);
  FB_REQUIRE(p.x && p.y, FB_INTERNAL_ERROR, "reduction: tensor has no buffer");
  p.x_dtype = x.dtype;
  p.y_dtype = y.dtype;
  p.mode = d.mode;
  p.integer_math = !is_float_dt(x.dtype);
  p.n_out = 1;
  p.n_red_elems = 1;
  int red_idx[FB_MAX_RANK];
  for (int i = 0; i < x.rank; ++i) {
    bool reduced = y.dims[i] == 1 && x.dims[i] > 1;
    if (reduced) {
      red_idx[p.n_red++] = i;
      p.n_red_elems *= x.dims[i];
    } else if (x.dims[i] > 1) {
      p.keep_dims[p.n_keep] = x.dims[i];
      p.keep_xstr[p.n_keep] = x.strides[i];
      p.keep_ystr[p.n_keep] = y.strides[i];
      p.n_keep++;
      p.n_out *= x.dims[i];
    }
  }
  // reduced dims ordered by ascending x stride so neighbouring lanes read neighbouring elements
  for (int i = 1; i < p.n_red; ++i)
    for (int j = i; j > 0 && x.strides[red_idx[j - 1]] > x.strides[red_idx[j]]; --j) {
      int t = red_idx[j - 1];
      red_idx[j - 1] = red_idx[j];
      red_idx[j] = t;
    }
  for (int i = 0; i < p.n_red; ++i) {
    p.red_dims[i] = x.dims[red_idx[i]];
    p.red_xstr[i] = x.strides[red_idx[i]];
  }
  cudaStream_t st = cx.dev->stream;
  // Row fast path: the reduced dims form one dense trailing block of memory and the
  // kept dims enumerate rows in order.
  bool rows_ok = !p.integer_math && p.n_red > 0;
  {
    int64_t expect = 1;
    for (int i = 0; i < p.n_red && rows_ok; ++i) {
      if (p.red_xstr[i] != expect) rows_ok = false;
      expect *= p.red_dims[i];
    }
    int64_t cols = expect;
    int64_t kexpect = cols;
    for (int i = p.n_keep - 1; i >= 0 && rows_ok; --i) {
      if (p.keep_xstr[i] != kexpect) rows_ok = false;
      kexpect *= p.keep_dims[i];
    }
    // output rows must be enumerated with a uniform stride
    int64_t ystride = p.n_keep > 0 ? p.keep_ystr[p.n_keep - 1] : 1;
    int64_t yexpect = ystride;
    for (int i = p.n_keep - 1; i >= 0 && rows_ok; --i) {
      if (p.keep_ystr[i] != yexpect) rows_ok = false;
      yexpect *= p.keep_dims[i];
    }
    size_t esz = dtype_size(x.dtype);
    if (rows_ok && cols >= 1024 && (cols * esz) % 16 == 0 && ((uintptr_t)p.x % 16 == 0)) {
      int64_t rows = p.n_out;
      int blocks = (int)std::min<int64_t>(rows, (int64_t)cx.dev->sm_count * 64);
      if (x.dtype == FB_DT_FLOAT)
        reduce_rows_kernel<float><<<blocks, 128, 0, st>>>((const float *)p.x, p.y, y.dtype, ystride, rows, cols, p.mode);
      else if (x.dtype == FB_DT_HALF)
        reduce_rows_kernel<__half><<<blocks, 128, 0, st>>>((const __half *)p.x, p.y, y.dtype, ystride, rows, cols, p.mode);
      else
        reduce_rows_kernel<__nv_bfloat16><<<blocks, 128, 0, st>>>((const __nv_bfloat16 *)p.x, p.y, y.dtype, ystride, rows, cols, p.mode);
      return FB_OK;
    }
  }
  int G = p.n_red_elems >= 2048 ? 256 : (p.n_red_elems >= 64 ? 32 : 1);
  int per_block = 256 / G;
  int64_t blocks64 = (p.n_out + per_block - 1) / per_block;
  FB_REQUIRE(blocks64 <= 0x7fffffff, FB_NOT_IMPLEMENTED, "reduction: output too large for one launch");
  int blocks = (int)blocks64;
#define FB_LAUNCH_RED(A)                                                        \
  do {                                                                          \
    if (G == 256) reduce_generic_kernel<A, 256><<<blocks, 256, 0, st>>>(p);     \
    else if (G == 32) reduce_generic_kernel<A, 32><<<blocks, 256, 0, st>>>(p);  \
    else reduce_generic_kernel<A, 1><<<blocks, 256, 0, st>>>(p);                \
  } while (0)
  if (p.integer_math) FB_LAUNCH_RED(int64_t);
  else FB_LAUNCH_RED(float);
#undef FB_LAUNCH_RED
  return FB_OK;
}

} // namespace fb

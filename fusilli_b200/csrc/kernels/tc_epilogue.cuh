// Register-resident epilogue shared by the tensor-core kernels. Each epilogue thread
// owns one accumulator row and works on 32 consecutive columns at a time: round to the
// contraction's declared dtype, apply the fused pointwise chain, convert, store.
// All mode / dtype switches sit OUTSIDE the 32-wide loops so the loops unroll into
// straight-line register code.
#ifndef FB_TC_EPILOGUE_CUH
#define FB_TC_EPILOGUE_CUH

#include "device_types.h"

namespace fb {

struct TcEpiOp {
  int32_t mode;
  int32_t kind; // 0 unary, 1 per-column vector, 2 scalar, 3 full tensor laid out like the output
  int32_t value_is_in1;
  int32_t round_dtype;
  int32_t dtype;
  float scalar;
  const void *ptr;
  float prm[4];
};

struct TcEpilogue {
  int32_t num_ops;
  int32_t acc_round_dtype;
  int32_t out_dtype;
  TcEpiOp ops[kMaxEpiOps];
};

#if defined(__CUDACC__)

// Rounds 32 values to a 16-bit type and back, two per conversion instruction.
__device__ __forceinline__ void epi_round_vec(float (&v)[32], int dt) {
  if (dt == FB_DT_BFLOAT16) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
      const uint32_t w = *reinterpret_cast<uint32_t *>(&h);
      v[2 * j] = __uint_as_float(w << 16);
      v[2 * j + 1] = __uint_as_float(w & 0xffff0000u);
    }
  } else if (dt == FB_DT_HALF) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float2 f = __half22float2(__floats2half2_rn(v[2 * j], v[2 * j + 1]));
      v[2 * j] = f.x;
      v[2 * j + 1] = f.y;
    }
  }
}

// 32 consecutive operand values starting at element `off` (vector loads when aligned).
__device__ __forceinline__ void epi_load32(const void *ptr, int dt, int64_t off, int valid, float (&o)[32]) {
  if (dt == FB_DT_FLOAT) {
    const float *q = static_cast<const float *>(ptr) + off;
    if (valid == 32 && (reinterpret_cast<uintptr_t>(q) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 t = __ldg(reinterpret_cast<const float4 *>(q) + j);
        o[4 * j] = t.x; o[4 * j + 1] = t.y; o[4 * j + 2] = t.z; o[4 * j + 3] = t.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) o[j] = j < valid ? __ldg(q + j) : 0.f;
    }
    return;
  }
  const uint16_t *q = static_cast<const uint16_t *>(ptr) + off;
  if (valid == 32 && (reinterpret_cast<uintptr_t>(q) & 15) == 0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 t = __ldg(reinterpret_cast<const uint4 *>(q) + j);
      const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (dt == FB_DT_BFLOAT16) {
          o[8 * j + 2 * e] = __uint_as_float(w[e] << 16);
          o[8 * j + 2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
        } else {
          __half2 h = *reinterpret_cast<const __half2 *>(&w[e]);
          float2 f = __half22float2(h);
          o[8 * j + 2 * e] = f.x;
          o[8 * j + 2 * e + 1] = f.y;
        }
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      uint16_t bits = j < valid ? __ldg(q + j) : (uint16_t)0;
      o[j] = dt == FB_DT_BFLOAT16 ? __uint_as_float((uint32_t)bits << 16)
                                  : __half2float(*reinterpret_cast<const __half *>(&bits));
    }
  }
}

#define FB_EPI_LOOP(expr)                                                                          \
  _Pragma("unroll") for (int j = 0; j < 32; ++j) {                                                 \
    const float a = in1 ? o[j] : v[j];                                                             \
    const float b = in1 ? v[j] : o[j];                                                             \
    (void)a; (void)b;                                                                              \
    v[j] = (expr);                                                                                 \
  }

// v = op(v, o) elementwise; the common modes get their own straight-line loop.
__device__ __forceinline__ void epi_apply_vec(const TcEpiOp &op, float (&v)[32], const float (&o)[32]) {
  const bool in1 = op.value_is_in1 != 0;
  switch (op.mode) {
  case FB_PW_ADD: FB_EPI_LOOP(a + b) break;
  case FB_PW_SUB: FB_EPI_LOOP(a - b) break;
  case FB_PW_MUL: FB_EPI_LOOP(a * b) break;
  case FB_PW_DIV: FB_EPI_LOOP(a / b) break;
  case FB_PW_MAX_OP: FB_EPI_LOOP(fmaxf(a, b)) break;
  case FB_PW_MIN_OP: FB_EPI_LOOP(fminf(a, b)) break;
  case FB_PW_RELU_FWD: FB_EPI_LOOP(fmaxf(a, 0.f)) break;
  case FB_PW_IDENTITY: break;
  case FB_PW_NEG: FB_EPI_LOOP(-a) break;
  case FB_PW_ABS: FB_EPI_LOOP(fabsf(a)) break;
  case FB_PW_SIGMOID_FWD: FB_EPI_LOOP(sigmoid_f(a)) break;
  case FB_PW_TANH_FWD: FB_EPI_LOOP(tanhf(a)) break;
  case FB_PW_GELU_FWD: FB_EPI_LOOP(0.5f * a * (1.f + erff(a * 0.7071067811865476f))) break;
  case FB_PW_SWISH_FWD: FB_EPI_LOOP(a * sigmoid_f(op.prm[3] * a)) break;
  default:
    // fully unrolled on purpose: a dynamic index would push v[] and o[] to local memory
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float a = in1 ? o[j] : v[j];
      const float b = in1 ? v[j] : o[j];
      v[j] = pw_apply_f(op.mode, a, b, 0.f, op.prm);
    }
    break;
  }
}
#undef FB_EPI_LOOP

// Full epilogue for 32 columns [nc, nc+32) of one output row; `row_off` is the element
// offset of the row start in the output (and in same-layout operands).
__device__ __forceinline__ void epi_run32(const TcEpilogue &e, float (&v)[32], int64_t row_off, int nc, int valid) {
  // Every stage rounds to its declared dtype, except a last stage whose dtype is the stored one:
  // the store performs that very rounding (rounding twice to one type changes nothing).
  if (!(e.num_ops == 0 && e.acc_round_dtype == e.out_dtype)) epi_round_vec(v, e.acc_round_dtype);
#pragma unroll 1
  for (int i = 0; i < e.num_ops; ++i) {
    const TcEpiOp &op = e.ops[i];
    float o[32];
    if (op.kind == 1) epi_load32(op.ptr, op.dtype, nc, valid, o);
    else if (op.kind == 3) epi_load32(op.ptr, op.dtype, row_off + nc, valid, o);
    else {
#pragma unroll
      for (int j = 0; j < 32; ++j) o[j] = op.scalar;
    }
    epi_apply_vec(op, v, o);
    if (!(i == e.num_ops - 1 && op.round_dtype == e.out_dtype)) epi_round_vec(v, op.round_dtype);
  }
}

// Converts and stores 32 consecutive outputs of one row (16-byte stores when aligned).
__device__ __forceinline__ void epi_store32(void *out, int out_dtype, int64_t off, const float (&v)[32], int valid) {
  if (out_dtype == FB_DT_FLOAT) {
    float *o = static_cast<float *>(out) + off;
    if (valid == 32 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        reinterpret_cast<float4 *>(o)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < valid) o[j] = v[j];
    }
    return;
  }
  uint16_t *o = static_cast<uint16_t *>(out) + off;
  const bool bf = out_dtype == FB_DT_BFLOAT16;
  if (valid == 32 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float lo = v[8 * j + 2 * e], hi = v[8 * j + 2 * e + 1];
        if (bf) {
          __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
          w[e] = *reinterpret_cast<uint32_t *>(&h);
        } else {
          __half2 h = __floats2half2_rn(lo, hi);
          w[e] = *reinterpret_cast<uint32_t *>(&h);
        }
      }
      reinterpret_cast<uint4 *>(o)[j] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (j < valid) {
        if (bf) {
          __nv_bfloat16 h = __float2bfloat16_rn(v[j]);
          o[j] = *reinterpret_cast<uint16_t *>(&h);
        } else {
          __half h = __float2half_rn(v[j]);
          o[j] = *reinterpret_cast<uint16_t *>(&h);
        }
      }
    }
  }
}

#endif // __CUDACC__

} // namespace fb

#endif // FB_TC_EPILOGUE_CUH

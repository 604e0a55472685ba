// POD types passed by value to kernels, typed element access, and the pointwise
// functor shared by the standalone elementwise kernel and every fused epilogue.
#ifndef FB_DEVICE_TYPES_H
#define FB_DEVICE_TYPES_H

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../../include/fusilli_b200.h"

namespace fb {

// A tensor as kernels see it: base pointer, element type, logical dims and
// element strides (0 = broadcast).
struct TensorRef {
  void *ptr;
  int32_t dtype;
  int32_t rank;
  int64_t dims[FB_MAX_RANK];
  int64_t strides[FB_MAX_RANK];
};

constexpr int kMaxEpiOps = 6;

// One fused pointwise op. The operand (if any) is addressed with the logical
// index of the output element: offset = sum(idx[d] * strides[d]), strides
// right-aligned to the output rank, 0 on broadcast dims.
struct EpiOpDev {
  int32_t mode;        // FB_PW_*
  int32_t operand_kind; // 0 none, 1 tensor, 2 scalar constant
  int32_t value_is_in1;
  int32_t round_dtype; // declared dtype of this op's result
  const void *operand;
  int32_t operand_dtype;
  float scalar;
  int64_t strides[FB_MAX_RANK];
  float fparams[4];
};

struct EpilogueDev {
  int32_t num_ops;
  int32_t acc_round_dtype; // declared dtype of the contraction's own result
  int32_t out_dtype;
  int32_t out_rank;
  EpiOpDev ops[kMaxEpiOps];
};

#if defined(__CUDACC__)

__device__ __forceinline__ bool dt_is_float(int dt) {
  return dt == FB_DT_HALF || dt == FB_DT_BFLOAT16 || dt == FB_DT_FLOAT;
}

__device__ __forceinline__ float load_f(const void *p, int dt, int64_t i) {
  switch (dt) {
  case FB_DT_FLOAT: return static_cast<const float *>(p)[i];
  case FB_DT_HALF: return __half2float(static_cast<const __half *>(p)[i]);
  case FB_DT_BFLOAT16: return __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]);
  case FB_DT_INT32: return (float)static_cast<const int32_t *>(p)[i];
  case FB_DT_INT64: return (float)static_cast<const int64_t *>(p)[i];
  case FB_DT_INT16: return (float)static_cast<const int16_t *>(p)[i];
  case FB_DT_INT8: return (float)static_cast<const int8_t *>(p)[i];
  case FB_DT_UINT8:
  case FB_DT_BOOLEAN: return (float)static_cast<const uint8_t *>(p)[i];
  case FB_DT_INT4: {
    // two's-complement nibbles, element 2k in the low half of byte k (reference
    // include/fusilli/support/int_types.h:56-66)
    const uint32_t byte = static_cast<const uint8_t *>(p)[i >> 1];
    const int v = (int)((byte >> ((i & 1) * 4)) & 0xFu);
    return (float)((v ^ 8) - 8);
  }
  default: return 0.f;
  }
}

__device__ __forceinline__ int64_t load_i(const void *p, int dt, int64_t i) {
  switch (dt) {
  case FB_DT_INT32: return static_cast<const int32_t *>(p)[i];
  case FB_DT_INT64: return static_cast<const int64_t *>(p)[i];
  case FB_DT_INT16: return static_cast<const int16_t *>(p)[i];
  case FB_DT_INT8: return static_cast<const int8_t *>(p)[i];
  case FB_DT_UINT8: return static_cast<const uint8_t *>(p)[i];
  case FB_DT_BOOLEAN: return static_cast<const uint8_t *>(p)[i] != 0;
  case FB_DT_FLOAT: return (int64_t) static_cast<const float *>(p)[i];
  case FB_DT_HALF: return (int64_t)__half2float(static_cast<const __half *>(p)[i]);
  case FB_DT_BFLOAT16: return (int64_t)__bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]);
  default: return 0;
  }
}

__device__ __forceinline__ void store_f(void *p, int dt, int64_t i, float v) {
  switch (dt) {
  case FB_DT_FLOAT: static_cast<float *>(p)[i] = v; break;
  case FB_DT_HALF: static_cast<__half *>(p)[i] = __float2half_rn(v); break;
  case FB_DT_BFLOAT16: static_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v); break;
  case FB_DT_INT32: static_cast<int32_t *>(p)[i] = (int32_t)v; break;
  case FB_DT_INT64: static_cast<int64_t *>(p)[i] = (int64_t)v; break;
  case FB_DT_INT16: static_cast<int16_t *>(p)[i] = (int16_t)v; break;
  case FB_DT_INT8: static_cast<int8_t *>(p)[i] = (int8_t)v; break;
  case FB_DT_UINT8: static_cast<uint8_t *>(p)[i] = (uint8_t)v; break;
  case FB_DT_BOOLEAN: static_cast<uint8_t *>(p)[i] = (v != 0.f) ? 1 : 0; break;
  default: break;
  }
}

__device__ __forceinline__ void store_i(void *p, int dt, int64_t i, int64_t v) {
  switch (dt) {
  case FB_DT_INT32: static_cast<int32_t *>(p)[i] = (int32_t)v; break;
  case FB_DT_INT64: static_cast<int64_t *>(p)[i] = v; break;
  case FB_DT_INT16: static_cast<int16_t *>(p)[i] = (int16_t)v; break;
  case FB_DT_INT8: static_cast<int8_t *>(p)[i] = (int8_t)v; break;
  case FB_DT_UINT8: static_cast<uint8_t *>(p)[i] = (uint8_t)v; break;
  case FB_DT_BOOLEAN: static_cast<uint8_t *>(p)[i] = v != 0; break;
  case FB_DT_FLOAT: static_cast<float *>(p)[i] = (float)v; break;
  case FB_DT_HALF: static_cast<__half *>(p)[i] = __float2half_rn((float)v); break;
  case FB_DT_BFLOAT16: static_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn((float)v); break;
  default: break;
  }
}

// Rounds a float to what a tensor of type `dt` would hold, back as float: the
// rounding the reference performs at a virtual tensor between two fused ops.
__device__ __forceinline__ float round_to(float v, int dt) {
  switch (dt) {
  case FB_DT_HALF: return __half2float(__float2half_rn(v));
  case FB_DT_BFLOAT16: return __bfloat162float(__float2bfloat16_rn(v));
  case FB_DT_FLOAT: return v;
  case FB_DT_BOOLEAN: return v != 0.f ? 1.f : 0.f;
  case FB_DT_INT32:
  case FB_DT_INT64:
  case FB_DT_INT16:
  case FB_DT_INT8:
  case FB_DT_UINT8: return truncf(v);
  default: return v;
  }
}

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

// Floating pointwise op: `a`,`b`,`c` are IN_0, IN_1, IN_2
// (semantics: include/fusilli/support/asm_emitter.h:1959-2116 of the reference).
__device__ __forceinline__ float pw_apply_f(int mode, float a, float b, float c, const float *prm) {
  const float kSqrt2OverPi = 0.7978845608028654f;
  const float kInvSqrt2 = 0.7071067811865476f;
  const float kInvSqrt2Pi = 0.3989422804014327f;
  switch (mode) {
  case FB_PW_ABS: return fabsf(a);
  case FB_PW_ADD: return a + b;
  case FB_PW_ADD_SQUARE: return a + b * b;
  case FB_PW_BINARY_SELECT: return a != 0.f ? b : c;
  case FB_PW_CEIL: return ceilf(a);
  case FB_PW_CMP_EQ: return a == b;
  case FB_PW_CMP_GE: return a >= b;
  case FB_PW_CMP_GT: return a > b;
  case FB_PW_CMP_LE: return a <= b;
  case FB_PW_CMP_LT: return a < b;
  case FB_PW_CMP_NEQ: return a != b;
  case FB_PW_DIV: return a / b;
  case FB_PW_ELU_FWD: return a > 0.f ? a : prm[0] * expm1f(a);
  case FB_PW_ERF: return erff(a);
  case FB_PW_EXP: return expf(a);
  case FB_PW_FLOOR: return floorf(a);
  case FB_PW_GELU_FWD: return 0.5f * a * (1.f + erff(a * kInvSqrt2));
  case FB_PW_GELU_APPROX_TANH_FWD:
    return 0.5f * a * (1.f + tanhf(kSqrt2OverPi * (a + 0.044715f * a * a * a)));
  case FB_PW_GELU_BWD: {
    float cdf = 0.5f * (1.f + erff(b * kInvSqrt2));
    float pdf = kInvSqrt2Pi * expf(-0.5f * b * b);
    return a * (cdf + b * pdf);
  }
  case FB_PW_GELU_APPROX_TANH_BWD: {
    float u = kSqrt2OverPi * (b + 0.044715f * b * b * b);
    float t = tanhf(u);
    float du = kSqrt2OverPi * (1.f + 3.f * 0.044715f * b * b);
    return a * (0.5f * (1.f + t) + 0.5f * b * (1.f - t * t) * du);
  }
  case FB_PW_IDENTITY: return a;
  case FB_PW_LOG: return logf(a);
  case FB_PW_LOGICAL_AND: return (a != 0.f) && (b != 0.f);
  case FB_PW_LOGICAL_NOT: return !(a != 0.f);
  case FB_PW_LOGICAL_OR: return (a != 0.f) || (b != 0.f);
  case FB_PW_MAX_OP: return (a > b || a != a) ? a : b;
  case FB_PW_MIN_OP: return (a < b || a != a) ? a : b;
  case FB_PW_MUL: return a * b;
  case FB_PW_NEG: return -a;
  case FB_PW_RECIPROCAL: return 1.f / a;
  case FB_PW_RELU_BWD: return b > 0.f ? a : 0.f;
  case FB_PW_RELU_FWD: return a > 0.f ? a : 0.f;
  case FB_PW_RSQRT: return rsqrtf(a);
  case FB_PW_SIGMOID_FWD: return sigmoid_f(a);
  case FB_PW_SIN: return sinf(a);
  case FB_PW_SOFTPLUS_FWD: return (a * prm[1] > prm[2]) ? a : log1pf(expf(a * prm[1])) / prm[1];
  case FB_PW_SQRT: return sqrtf(a);
  case FB_PW_SUB: return a - b;
  case FB_PW_SWISH_FWD: return a * sigmoid_f(prm[3] * a);
  case FB_PW_SWISH_BWD: {
    float s = sigmoid_f(prm[3] * b);
    return a * (s + prm[3] * b * s * (1.f - s));
  }
  case FB_PW_TAN: return tanf(a);
  case FB_PW_TANH_BWD: {
    float t = tanhf(b);
    return a * (1.f - t * t);
  }
  case FB_PW_TANH_FWD: return tanhf(a);
  default: return 0.f;
  }
}

// Integer pointwise op (exact; division truncates toward zero).
__device__ __forceinline__ int64_t pw_apply_i(int mode, int64_t a, int64_t b, int64_t c) {
  switch (mode) {
  case FB_PW_ABS: return a < 0 ? -a : a;
  case FB_PW_ADD: return a + b;
  case FB_PW_ADD_SQUARE: return a + b * b;
  case FB_PW_BINARY_SELECT: return a != 0 ? b : c;
  case FB_PW_CMP_EQ: return a == b;
  case FB_PW_CMP_GE: return a >= b;
  case FB_PW_CMP_GT: return a > b;
  case FB_PW_CMP_LE: return a <= b;
  case FB_PW_CMP_LT: return a < b;
  case FB_PW_CMP_NEQ: return a != b;
  case FB_PW_DIV: return b == 0 ? 0 : a / b;
  case FB_PW_IDENTITY:
  case FB_PW_CEIL:
  case FB_PW_FLOOR: return a;
  case FB_PW_LOGICAL_AND: return (a != 0) && (b != 0);
  case FB_PW_LOGICAL_NOT: return !(a != 0);
  case FB_PW_LOGICAL_OR: return (a != 0) || (b != 0);
  case FB_PW_MAX_OP: return a > b ? a : b;
  case FB_PW_MIN_OP: return a < b ? a : b;
  case FB_PW_MUL: return a * b;
  case FB_PW_NEG: return -a;
  case FB_PW_RELU_BWD: return b > 0 ? a : 0;
  case FB_PW_RELU_FWD: return a > 0 ? a : 0;
  case FB_PW_SUB: return a - b;
  default: return 0;
  }
}

// Applies a fused epilogue to the fp32 accumulator of the output element whose
// logical index is idx[0..rank).
__device__ __forceinline__ float apply_epilogue(const EpilogueDev &e, float v, const int64_t *idx) {
  v = round_to(v, e.acc_round_dtype);
#pragma unroll 1
  for (int i = 0; i < e.num_ops; ++i) {
    const EpiOpDev &op = e.ops[i];
    float other = 0.f;
    if (op.operand_kind == 1) {
      int64_t off = 0;
      for (int d = 0; d < e.out_rank; ++d) off += idx[d] * op.strides[d];
      other = load_f(op.operand, op.operand_dtype, off);
    } else if (op.operand_kind == 2) {
      other = op.scalar;
    }
    float a = op.value_is_in1 ? other : v;
    float b = op.value_is_in1 ? v : other;
    v = round_to(pw_apply_f(op.mode, a, b, 0.f, op.fparams), op.round_dtype);
  }
  return v;
}

#endif // __CUDACC__

} // namespace fb

#endif // FB_DEVICE_TYPES_H

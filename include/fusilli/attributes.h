// Per-op attribute bags of the graph builders: same class names, setters and getters as the
// reference's include/fusilli/attributes/{conv,matmul,sdpa,layernorm,rmsnorm,reduction,
// pointwise}_attributes.h. 
#ifndef FUSILLI_ATTRIBUTES_H
#define FUSILLI_ATTRIBUTES_H

#include <array>
#include <memory>
#include <optional>
#include <string>
#include <unordered_map>
#include <vector>

#include "../fusilli_b200.h"
#include "tensor.h"

namespace fusilli {

using TensorPtr = std::shared_ptr<TensorAttr>;

enum class NormFwdPhase : uint8_t { NOT_SET, TRAINING, INFERENCE };

// Common part of every bag (reference attributes/attributes.h:30-126): name, compute type, and
// tensors kept in the derived class's `inputs` / `outputs` maps, keyed by its InputNames /
// OutputNames enums.
template <typename Derived> class AttributesCRTP {
public:
  DataType computeDataType = DataType::NotSet;
  const std::string &getName() const { return name_; }
  Derived &setName(const std::string &n) { name_ = n; return self(); }
  Derived &setComputeDataType(DataType t) { computeDataType = t; return self(); }

  template <typename K> Derived &setInput(const K &key, const TensorPtr &t) {
    self().inputs[key] = t;
    return self();
  }
  template <typename K> Derived &setOutput(const K &key, const TensorPtr &t) {
    self().outputs[key] = t;
    return self();
  }
  template <typename K> TensorPtr getInput(const K &key) const {
    auto it = self().inputs.find(key);
    return it == self().inputs.end() ? nullptr : it->second;
  }
  template <typename K> TensorPtr getOutput(const K &key) const {
    auto it = self().outputs.find(key);
    return it == self().outputs.end() ? nullptr : it->second;
  }

  // Unset compute type and unset tensor dtypes take the graph context's defaults.
  void fillFromContext(const Context &ctx) {
    if (computeDataType == DataType::NotSet) computeDataType = ctx.getComputeDataType();
    for (auto &kv : self().inputs)
      if (kv.second) kv.second->fillFromContext(ctx);
    for (auto &kv : self().outputs)
      if (kv.second) kv.second->fillFromContext(ctx);
  }

protected:
  Derived &self() { return static_cast<Derived &>(*this); }
  const Derived &self() const { return static_cast<const Derived &>(*this); }
  std::string name_;
};

#define FUSILLI_TENSOR_MAPS                                                                          \
  std::unordered_map<InputNames, TensorPtr> inputs;                                                  \
  std::unordered_map<OutputNames, TensorPtr> outputs;
#define FUSILLI_IN(CLASS, KEY, NAME)                                                                 \
  CLASS &set##NAME(const TensorPtr &t) { return setInput(InputNames::KEY, t); }                      \
  TensorPtr get##NAME() const { return getInput(InputNames::KEY); }
#define FUSILLI_OUT(CLASS, KEY, NAME)                                                                \
  CLASS &set##NAME(const TensorPtr &t) { return setOutput(OutputNames::KEY, t); }                    \
  TensorPtr get##NAME() const { return getOutput(OutputNames::KEY); }

#define FUSILLI_CONV_GEOMETRY(CLASS)                                                                 \
  CLASS &setPadding(const std::vector<int64_t> &v) { padding_ = v; return *this; }                  \
  CLASS &setStride(const std::vector<int64_t> &v) { stride_ = v; return *this; }                    \
  CLASS &setDilation(const std::vector<int64_t> &v) { dilation_ = v; return *this; }                \
  template <Int64Range R> CLASS &setPadding(R &&v) { padding_.assign(v.begin(), v.end()); return *this; }  \
  template <Int64Range R> CLASS &setStride(R &&v) { stride_.assign(v.begin(), v.end()); return *this; }    \
  template <Int64Range R> CLASS &setDilation(R &&v) { dilation_.assign(v.begin(), v.end()); return *this; } \
  const std::vector<int64_t> &getPadding() const { return padding_; }                               \
  const std::vector<int64_t> &getStride() const { return stride_; }                                 \
  const std::vector<int64_t> &getDilation() const { return dilation_; }                             \
                                                                                                     \
private:                                                                                             \
  std::vector<int64_t> padding_, stride_, dilation_;                                                 \
                                                                                                     \
public:

class ConvFPropAttr : public AttributesCRTP<ConvFPropAttr> {
public:
  enum class InputNames : uint8_t { X, W };
  enum class OutputNames : uint8_t { Y };
  FUSILLI_TENSOR_MAPS
  FUSILLI_IN(ConvFPropAttr, X, X)
  FUSILLI_IN(ConvFPropAttr, W, W)
  FUSILLI_OUT(ConvFPropAttr, Y, Y)
  FUSILLI_CONV_GEOMETRY(ConvFPropAttr)
};

class ConvWGradAttr : public AttributesCRTP<ConvWGradAttr> {
public:
  enum class InputNames : uint8_t { DY, X };
  enum class OutputNames : uint8_t { DW };
  FUSILLI_TENSOR_MAPS
  FUSILLI_IN(ConvWGradAttr, DY, DY)
  FUSILLI_IN(ConvWGradAttr, X, X)
  FUSILLI_OUT(ConvWGradAttr, DW, DW)
  FUSILLI_CONV_GEOMETRY(ConvWGradAttr)
};

class ConvDGradAttr : public AttributesCRTP<ConvDGradAttr> {
public:
  enum class InputNames : uint8_t { DY, W };
  enum class OutputNames : uint8_t { DX };
  FUSILLI_TENSOR_MAPS
  FUSILLI_IN(ConvDGradAttr, DY, DY)
  FUSILLI_IN(ConvDGradAttr, W, W)
  FUSILLI_OUT(ConvDGradAttr, DX, DX)
  FUSILLI_CONV_GEOMETRY(ConvDGradAttr)
};

class MatmulAttr : public AttributesCRTP<MatmulAttr> {
public:
  enum class InputNames : uint8_t { A, B };
  enum class OutputNames : uint8_t { C };
  FUSILLI_TENSOR_MAPS
  FUSILLI_IN(MatmulAttr, A, A)
  FUSILLI_IN(MatmulAttr, B, B)
  FUSILLI_OUT(MatmulAttr, C, C)
};

class SdpaAttr : public AttributesCRTP<SdpaAttr> {
public:
  enum class InputNames : uint8_t { Q, K, V, MASK };
  enum class OutputNames : uint8_t { O };
  FUSILLI_TENSOR_MAPS
  FUSILLI_IN(SdpaAttr, Q, Q)
  FUSILLI_IN(SdpaAttr, K, K)
  FUSILLI_IN(SdpaAttr, V, V)
  FUSILLI_IN(SdpaAttr, MASK, MASK)
  FUSILLI_OUT(SdpaAttr, O, O)
  SdpaAttr &setDropout(float p) { dropout_ = p; return *this; }
  SdpaAttr &setIsCausal(bool v) { causal_ = v; return *this; }
  SdpaAttr &setScale(std::optional<float> s) { scale_ = s; return *this; }
  SdpaAttr &setEnableGqa(bool v) { gqa_ = v; return *this; }
  float getDropout() const { return dropout_; }
  bool getIsCausal() const { return causal_; }
  std::optional<float> getScale() const { return scale_; }
  bool getEnableGqa() const { return gqa_; }

private:
  float dropout_ = 0.f;
  bool causal_ = false, gqa_ = false;
  std::optional<float> scale_;
};

class LayernormAttr : public AttributesCRTP<LayernormAttr> {
public:
  enum class InputNames : uint8_t { X, SCALE, BIAS, EPSILON };
  enum class OutputNames : uint8_t { Y, MEAN, INV_VARIANCE };
  FUSILLI_TENSOR_MAPS
  FUSILLI_IN(LayernormAttr, X, X)
  FUSILLI_IN(LayernormAttr, SCALE, SCALE)
  FUSILLI_IN(LayernormAttr, BIAS, BIAS)
  FUSILLI_IN(LayernormAttr, EPSILON, Epsilon)
  FUSILLI_OUT(LayernormAttr, Y, Y)
  FUSILLI_OUT(LayernormAttr, MEAN, MEAN)
  FUSILLI_OUT(LayernormAttr, INV_VARIANCE, INV_VARIANCE)
  LayernormAttr &setForwardPhase(NormFwdPhase p) { phase_ = p; return *this; }
  NormFwdPhase getForwardPhase() const { return phase_; }

private:
  NormFwdPhase phase_ = NormFwdPhase::NOT_SET;
};

// reference attributes/batchnorm_attributes.h:27-90
class BatchnormAttr : public AttributesCRTP<BatchnormAttr> {
public:
  enum class InputNames : uint8_t { X, SCALE, BIAS, MEAN, VAR, EPSILON, MOMENTUM };
  enum class OutputNames : uint8_t { Y, SAVED_MEAN, SAVED_INV_VARIANCE };
  FUSILLI_TENSOR_MAPS
  FUSILLI_IN(BatchnormAttr, X, X)
  FUSILLI_IN(BatchnormAttr, SCALE, SCALE)
  FUSILLI_IN(BatchnormAttr, BIAS, BIAS)
  FUSILLI_IN(BatchnormAttr, MEAN, MEAN)
  FUSILLI_IN(BatchnormAttr, VAR, VAR)
  FUSILLI_IN(BatchnormAttr, EPSILON, Epsilon)
  FUSILLI_IN(BatchnormAttr, MOMENTUM, Momentum)
  FUSILLI_OUT(BatchnormAttr, Y, Y)
  FUSILLI_OUT(BatchnormAttr, SAVED_MEAN, SAVED_MEAN)
  FUSILLI_OUT(BatchnormAttr, SAVED_INV_VARIANCE, SAVED_INV_VARIANCE)
  BatchnormAttr &setForwardPhase(NormFwdPhase p) { phase_ = p; return *this; }
  NormFwdPhase getForwardPhase() const { return phase_; }

private:
  NormFwdPhase phase_ = NormFwdPhase::NOT_SET;
};

class RmsnormAttr : public AttributesCRTP<RmsnormAttr> {
public:
  enum class InputNames : uint8_t { X, SCALE, EPSILON };
  enum class OutputNames : uint8_t { Y, INV_RMS };
  FUSILLI_TENSOR_MAPS
  FUSILLI_IN(RmsnormAttr, X, X)
  FUSILLI_IN(RmsnormAttr, SCALE, SCALE)
  FUSILLI_IN(RmsnormAttr, EPSILON, Epsilon)
  FUSILLI_OUT(RmsnormAttr, Y, Y)
  FUSILLI_OUT(RmsnormAttr, INV_RMS, INV_RMS)
  RmsnormAttr &setForwardPhase(NormFwdPhase p) { phase_ = p; return *this; }
  NormFwdPhase getForwardPhase() const { return phase_; }

private:
  NormFwdPhase phase_ = NormFwdPhase::NOT_SET;
};

class ReductionAttr : public AttributesCRTP<ReductionAttr> {
public:
  enum class InputNames : uint8_t { X };
  enum class OutputNames : uint8_t { Y };
  FUSILLI_TENSOR_MAPS
  // Same order as the C ABI's FB_RED_* values.
  enum class Mode : uint8_t { NOT_SET, ADD, SUM, MUL, MIN, MAX, AMAX, AVG, NORM1, NORM2, MUL_NO_ZEROS };
  FUSILLI_IN(ReductionAttr, X, X)
  FUSILLI_OUT(ReductionAttr, Y, Y)
  ReductionAttr &setMode(Mode m) { mode_ = m; return *this; }
  Mode getMode() const { return mode_; }
  static const char *modeName(Mode m) {
    static const char *names[] = {"NOT_SET", "ADD", "SUM", "MUL", "MIN", "MAX", "AMAX", "AVG", "NORM1", "NORM2",
                                  "MUL_NO_ZEROS"};
    return names[static_cast<int>(m)];
  }
  // Mode -> spelling, under the name the reference's samples use (reduction_attributes.h:71).
  static const std::unordered_map<Mode, std::string> kModeToStr;

private:
  Mode mode_ = Mode::NOT_SET;
};

class PointwiseAttr : public AttributesCRTP<PointwiseAttr> {
public:
  enum class InputNames : uint8_t { IN_0, IN_1, IN_2 };
  enum class OutputNames : uint8_t { OUT_0 };
  FUSILLI_TENSOR_MAPS
  // Same order as the C ABI's FB_PW_* values.
  enum class Mode : uint8_t {
    NOT_SET, ABS, ADD, ADD_SQUARE, BINARY_SELECT, CEIL, CMP_EQ, CMP_GE, CMP_GT, CMP_LE, CMP_LT, CMP_NEQ, DIV,
    ELU_FWD, ERF, EXP, FLOOR, GELU_APPROX_TANH_BWD, GELU_APPROX_TANH_FWD, GELU_BWD, GELU_FWD, IDENTITY, LOG,
    LOGICAL_AND, LOGICAL_NOT, LOGICAL_OR, MAX_OP, MIN_OP, MUL, NEG, RECIPROCAL, RELU_BWD, RELU_FWD, RSQRT,
    SIGMOID_FWD, SIN, SOFTPLUS_FWD, SQRT, SUB, SWISH_BWD, SWISH_FWD, TAN, TANH_BWD, TANH_FWD
  };
  FUSILLI_IN(PointwiseAttr, IN_0, IN_0)
  FUSILLI_IN(PointwiseAttr, IN_1, IN_1)
  FUSILLI_IN(PointwiseAttr, IN_2, IN_2)
  FUSILLI_OUT(PointwiseAttr, OUT_0, OUT_0)
  PointwiseAttr &setMode(Mode m) { mode_ = m; return *this; }
  PointwiseAttr &setEluAlpha(float v) { eluAlpha_ = v; return *this; }
  PointwiseAttr &setSoftplusBeta(float v) { softplusBeta_ = v; return *this; }
  PointwiseAttr &setSoftplusThreshold(float v) { softplusThreshold_ = v; return *this; }
  PointwiseAttr &setSwishBeta(float v) { swishBeta_ = v; return *this; }
  Mode getMode() const { return mode_; }
  float getEluAlpha() const { return eluAlpha_; }
  float getSoftplusBeta() const { return softplusBeta_; }
  float getSoftplusThreshold() const { return softplusThreshold_; }
  float getSwishBeta() const { return swishBeta_; }

  // Number of inputs a mode takes (reference pointwise_attributes.h:157-201).
  static int requiredInputCount(Mode m) {
    switch (m) {
    case Mode::BINARY_SELECT: return 3;
    case Mode::ADD: case Mode::ADD_SQUARE: case Mode::CMP_EQ: case Mode::CMP_GE: case Mode::CMP_GT:
    case Mode::CMP_LE: case Mode::CMP_LT: case Mode::CMP_NEQ: case Mode::DIV:
    case Mode::GELU_APPROX_TANH_BWD: case Mode::GELU_BWD: case Mode::LOGICAL_AND: case Mode::LOGICAL_OR:
    case Mode::MAX_OP: case Mode::MIN_OP: case Mode::MUL: case Mode::RELU_BWD: case Mode::SUB:
    case Mode::SWISH_BWD: case Mode::TANH_BWD: return 2;
    default: return 1;
    }
  }
  // Compare and logical modes always produce Boolean (reference pointwise_node.h:31-42).
  static bool forcesBooleanOutput(Mode m) {
    switch (m) {
    case Mode::CMP_EQ: case Mode::CMP_NEQ: case Mode::CMP_LT: case Mode::CMP_LE: case Mode::CMP_GT:
    case Mode::CMP_GE: case Mode::LOGICAL_AND: case Mode::LOGICAL_NOT: case Mode::LOGICAL_OR: return true;
    default: return false;
    }
  }
  static const char *modeName(Mode m) {
    static const char *names[] = {
        "NOT_SET", "ABS", "ADD", "ADD_SQUARE", "BINARY_SELECT", "CEIL", "CMP_EQ", "CMP_GE", "CMP_GT", "CMP_LE",
        "CMP_LT", "CMP_NEQ", "DIV", "ELU_FWD", "ERF", "EXP", "FLOOR", "GELU_APPROX_TANH_BWD",
        "GELU_APPROX_TANH_FWD", "GELU_BWD", "GELU_FWD", "IDENTITY", "LOG", "LOGICAL_AND", "LOGICAL_NOT",
        "LOGICAL_OR", "MAX_OP", "MIN_OP", "MUL", "NEG", "RECIPROCAL", "RELU_BWD", "RELU_FWD", "RSQRT",
        "SIGMOID_FWD", "SIN", "SOFTPLUS_FWD", "SQRT", "SUB", "SWISH_BWD", "SWISH_FWD", "TAN", "TANH_BWD",
        "TANH_FWD"};
    return names[static_cast<int>(m)];
  }
  // Mode -> spelling, under the name the reference's samples use (pointwise_attributes.h:137).
  static const std::unordered_map<Mode, std::string> kModeToStr;

private:
  Mode mode_ = Mode::NOT_SET;
  float eluAlpha_ = 1.f, softplusBeta_ = 1.f, softplusThreshold_ = 20.f, swishBeta_ = 1.f;
};

namespace detail {
template <typename Attr, int Last> inline std::unordered_map<typename Attr::Mode, std::string> modeTable() {
  std::unordered_map<typename Attr::Mode, std::string> m;
  for (int i = 0; i <= Last; ++i) m.emplace(static_cast<typename Attr::Mode>(i), Attr::modeName(static_cast<typename Attr::Mode>(i)));
  return m;
}
} // namespace detail
inline const std::unordered_map<PointwiseAttr::Mode, std::string> PointwiseAttr::kModeToStr =
    detail::modeTable<PointwiseAttr, FB_PW_TANH_FWD>();
inline const std::unordered_map<ReductionAttr::Mode, std::string> ReductionAttr::kModeToStr =
    detail::modeTable<ReductionAttr, FB_RED_MUL_NO_ZEROS>();

static_assert(static_cast<int>(PointwiseAttr::Mode::TANH_FWD) == FB_PW_TANH_FWD, "pointwise modes out of step with the C ABI");
static_assert(static_cast<int>(ReductionAttr::Mode::MUL_NO_ZEROS) == FB_RED_MUL_NO_ZEROS, "reduction modes out of step with the C ABI");

#undef FUSILLI_IN
#undef FUSILLI_OUT
#undef FUSILLI_TENSOR_MAPS
#undef FUSILLI_CONV_GEOMETRY

} // namespace fusilli

#endif // FUSILLI_ATTRIBUTES_H

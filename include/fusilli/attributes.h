// Per-op attribute bags of the graph builders: same class names, setters and getters as the
// reference's include/fusilli/attributes/{conv,matmul,sdpa,layernorm,rmsnorm,reduction,
// pointwise}_attributes.h. Tensors are held in fixed slots (an array per bag) rather than maps.
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

// Common part of every bag: name, compute type, NIN input slots, NOUT output slots.
template <typename Derived, int NIN, int NOUT> class AttrBase {
public:
  DataType computeDataType = DataType::NotSet;
  const std::string &getName() const { return name_; }
  Derived &setName(const std::string &n) { name_ = n; return self(); }
  Derived &setComputeDataType(DataType t) { computeDataType = t; return self(); }

  void fillFromContext(const Context &ctx) {
    if (computeDataType == DataType::NotSet) computeDataType = ctx.getComputeDataType();
    for (auto &t : in_) if (t) t->fillFromContext(ctx);
    for (auto &t : out_) if (t) t->fillFromContext(ctx);
  }
  const std::array<TensorPtr, NIN> &inputSlots() const { return in_; }
  const std::array<TensorPtr, NOUT> &outputSlots() const { return out_; }

protected:
  Derived &self() { return static_cast<Derived &>(*this); }
  std::array<TensorPtr, NIN> in_{};
  std::array<TensorPtr, NOUT> out_{};
  std::string name_;
};

#define FUSILLI_SLOT(CLASS, ARR, IDX, NAME)                                                          \
  CLASS &set##NAME(const TensorPtr &t) { ARR[IDX] = t; return *this; }                               \
  TensorPtr get##NAME() const { return ARR[IDX]; }

#define FUSILLI_CONV_GEOMETRY(CLASS)                                                                 \
  CLASS &setPadding(const std::vector<int64_t> &v) { padding_ = v; return *this; }                  \
  CLASS &setStride(const std::vector<int64_t> &v) { stride_ = v; return *this; }                    \
  CLASS &setDilation(const std::vector<int64_t> &v) { dilation_ = v; return *this; }                \
  const std::vector<int64_t> &getPadding() const { return padding_; }                               \
  const std::vector<int64_t> &getStride() const { return stride_; }                                 \
  const std::vector<int64_t> &getDilation() const { return dilation_; }                             \
                                                                                                     \
private:                                                                                             \
  std::vector<int64_t> padding_, stride_, dilation_;                                                 \
                                                                                                     \
public:

class ConvFPropAttr : public AttrBase<ConvFPropAttr, 2, 1> {
public:
  FUSILLI_SLOT(ConvFPropAttr, in_, 0, X)
  FUSILLI_SLOT(ConvFPropAttr, in_, 1, W)
  FUSILLI_SLOT(ConvFPropAttr, out_, 0, Y)
  FUSILLI_CONV_GEOMETRY(ConvFPropAttr)
};

class ConvWGradAttr : public AttrBase<ConvWGradAttr, 2, 1> {
public:
  FUSILLI_SLOT(ConvWGradAttr, in_, 0, DY)
  FUSILLI_SLOT(ConvWGradAttr, in_, 1, X)
  FUSILLI_SLOT(ConvWGradAttr, out_, 0, DW)
  FUSILLI_CONV_GEOMETRY(ConvWGradAttr)
};

class ConvDGradAttr : public AttrBase<ConvDGradAttr, 2, 1> {
public:
  FUSILLI_SLOT(ConvDGradAttr, in_, 0, DY)
  FUSILLI_SLOT(ConvDGradAttr, in_, 1, W)
  FUSILLI_SLOT(ConvDGradAttr, out_, 0, DX)
  FUSILLI_CONV_GEOMETRY(ConvDGradAttr)
};

class MatmulAttr : public AttrBase<MatmulAttr, 2, 1> {
public:
  FUSILLI_SLOT(MatmulAttr, in_, 0, A)
  FUSILLI_SLOT(MatmulAttr, in_, 1, B)
  FUSILLI_SLOT(MatmulAttr, out_, 0, C)
};

class SdpaAttr : public AttrBase<SdpaAttr, 4, 1> {
public:
  FUSILLI_SLOT(SdpaAttr, in_, 0, Q)
  FUSILLI_SLOT(SdpaAttr, in_, 1, K)
  FUSILLI_SLOT(SdpaAttr, in_, 2, V)
  FUSILLI_SLOT(SdpaAttr, in_, 3, MASK)
  FUSILLI_SLOT(SdpaAttr, out_, 0, O)
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

class LayernormAttr : public AttrBase<LayernormAttr, 4, 3> {
public:
  FUSILLI_SLOT(LayernormAttr, in_, 0, X)
  FUSILLI_SLOT(LayernormAttr, in_, 1, SCALE)
  FUSILLI_SLOT(LayernormAttr, in_, 2, BIAS)
  FUSILLI_SLOT(LayernormAttr, in_, 3, Epsilon)
  FUSILLI_SLOT(LayernormAttr, out_, 0, Y)
  FUSILLI_SLOT(LayernormAttr, out_, 1, MEAN)
  FUSILLI_SLOT(LayernormAttr, out_, 2, INV_VARIANCE)
  LayernormAttr &setForwardPhase(NormFwdPhase p) { phase_ = p; return *this; }
  NormFwdPhase getForwardPhase() const { return phase_; }

private:
  NormFwdPhase phase_ = NormFwdPhase::NOT_SET;
};

class RmsnormAttr : public AttrBase<RmsnormAttr, 3, 2> {
public:
  FUSILLI_SLOT(RmsnormAttr, in_, 0, X)
  FUSILLI_SLOT(RmsnormAttr, in_, 1, SCALE)
  FUSILLI_SLOT(RmsnormAttr, in_, 2, Epsilon)
  FUSILLI_SLOT(RmsnormAttr, out_, 0, Y)
  FUSILLI_SLOT(RmsnormAttr, out_, 1, INV_RMS)
  RmsnormAttr &setForwardPhase(NormFwdPhase p) { phase_ = p; return *this; }
  NormFwdPhase getForwardPhase() const { return phase_; }

private:
  NormFwdPhase phase_ = NormFwdPhase::NOT_SET;
};

class ReductionAttr : public AttrBase<ReductionAttr, 1, 1> {
public:
  // Same order as the C ABI's FB_RED_* values.
  enum class Mode : uint8_t { NOT_SET, ADD, SUM, MUL, MIN, MAX, AMAX, AVG, NORM1, NORM2, MUL_NO_ZEROS };
  FUSILLI_SLOT(ReductionAttr, in_, 0, X)
  FUSILLI_SLOT(ReductionAttr, out_, 0, Y)
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

class PointwiseAttr : public AttrBase<PointwiseAttr, 3, 1> {
public:
  // Same order as the C ABI's FB_PW_* values.
  enum class Mode : uint8_t {
    NOT_SET, ABS, ADD, ADD_SQUARE, BINARY_SELECT, CEIL, CMP_EQ, CMP_GE, CMP_GT, CMP_LE, CMP_LT, CMP_NEQ, DIV,
    ELU_FWD, ERF, EXP, FLOOR, GELU_APPROX_TANH_BWD, GELU_APPROX_TANH_FWD, GELU_BWD, GELU_FWD, IDENTITY, LOG,
    LOGICAL_AND, LOGICAL_NOT, LOGICAL_OR, MAX_OP, MIN_OP, MUL, NEG, RECIPROCAL, RELU_BWD, RELU_FWD, RSQRT,
    SIGMOID_FWD, SIN, SOFTPLUS_FWD, SQRT, SUB, SWISH_BWD, SWISH_FWD, TAN, TANH_BWD, TANH_FWD
  };
  FUSILLI_SLOT(PointwiseAttr, in_, 0, IN_0)
  FUSILLI_SLOT(PointwiseAttr, in_, 1, IN_1)
  FUSILLI_SLOT(PointwiseAttr, in_, 2, IN_2)
  FUSILLI_SLOT(PointwiseAttr, out_, 0, OUT_0)
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

#undef FUSILLI_SLOT
#undef FUSILLI_CONV_GEOMETRY

} // namespace fusilli

#endif // FUSILLI_ATTRIBUTES_H

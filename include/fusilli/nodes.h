// Graph nodes: one class per op, each with the reference's validation rules and dim / stride /
// dtype inference (reference include/fusilli/node/{conv,matmul,sdpa,layernorm,rmsnorm,reduction,
// pointwise}_node.h and norm_utils.h), plus `describe()`, which writes the node into the POD
// descriptor the C ABI's fb_plan_build consumes. Where the reference's nodes emit MLIR text,
// these emit an fb_node_desc.
#ifndef FUSILLI_NODES_H
#define FUSILLI_NODES_H

#include <cstring>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "attributes.h"

namespace fusilli {

// Output extent of a convolution (reference conv_node.h:38-56).
inline std::vector<int64_t> getConvInferredOutputShape(const std::vector<int64_t> &xDim,
                                                       const std::vector<int64_t> &wDim,
                                                       const std::vector<int64_t> &dilation,
                                                       const std::vector<int64_t> &padding,
                                                       const std::vector<int64_t> &stride) {
  std::vector<int64_t> y(xDim.size());
  y[0] = xDim[0];
  y[1] = wDim[0];
  for (size_t i = 2; i < xDim.size(); ++i)
    y[i] = 1 + (xDim[i] - (wDim[i] - 1) * dilation[i - 2] + 2 * padding[i - 2] - 1) / stride[i - 2];
  return y;
}

// Output shape of a (batch-broadcast) matmul (reference matmul_node.h:40-66).
inline std::vector<int64_t> getMatmulInferredOutputShape(const std::vector<int64_t> &a,
                                                         const std::vector<int64_t> &b) {
  const size_t r = a.size();
  std::vector<int64_t> c(r);
  for (size_t i = 0; i + 2 < r; ++i) c[i] = std::max(a[i], b[i]);
  c[r - 2] = a[r - 2];
  c[r - 1] = b[r - 1];
  return c;
}

class INode {
public:
  enum class Type : uint8_t { Composite, Convolution, Pointwise, WGrad, DGrad, LayerNorm, BatchNorm, RmsNorm,
                              Matmul, Reduction, Custom, Sdpa };
  using TensorId = std::function<int32_t(const TensorPtr &)>;
  // A node keeps its own copy of the graph context as it was when the node was added
  // (reference node.h:47).
  explicit INode(const Context &ctx) : context(ctx) {}
  virtual ~INode() = default;
  virtual const std::string &getName() const = 0;
  virtual Type getType() const = 0;
  Context context;

  // Three phases, as in the reference (node.h:63-65): checks that need only what the user set,
  // inference of unset dims / strides / dtypes, checks on the completed node.
  virtual ErrorObject preValidateNode() const { return ok(); }
  virtual ErrorObject inferPropertiesNode() = 0;
  virtual ErrorObject postValidateNode() const { return ok(); }
  ErrorObject validateNode() {
    FUSILLI_CHECK_ERROR(preValidateNode());
    FUSILLI_CHECK_ERROR(inferPropertiesNode());
    FUSILLI_CHECK_ERROR(postValidateNode());
    return ok();
  }
  // Writes the node into the C ABI's POD descriptor; op = -1 marks a node kind the B200 backend
  // cannot run, which fb_plan_build rejects.
  virtual void describe(fb_node_desc &d, const TensorId &) const {
    std::memset(&d, 0, sizeof(d));
    d.op = -1;
  }
};

namespace detail {

inline bool layoutOk(const TensorPtr &t) { return t->isContiguous() || t->isChannelsLast(); }
inline std::string notChannelsLastMsg(const TensorPtr &t) {
  return "Tensor '" + t->getName() + "' is neither contiguous nor channels-last as defined by its stride";
}
inline std::vector<int64_t> strideLike(const TensorPtr &ref, const std::vector<int64_t> &dim) {
  return ref->isContiguous() ? generateStrideFromDim(dim, getContiguousStrideOrder(dim.size()))
                             : generateStrideFromDim(dim, getChannelsLastStrideOrder(dim.size()));
}
inline void initDesc(fb_node_desc &d, int op) {
  std::memset(&d, 0, sizeof(d));
  d.op = op;
  for (int &v : d.inputs) v = -1;
  for (int &v : d.outputs) v = -1;
}
template <typename A> void convGeometry(fb_node_desc &d, const A &a) {
  d.num_spatial = static_cast<int32_t>(a.getPadding().size());
  for (size_t i = 0; i < a.getPadding().size() && i < 3; ++i) {
    d.padding[i] = a.getPadding()[i];
    d.stride[i] = a.getStride()[i];
    d.dilation[i] = a.getDilation()[i];
  }
}
template <typename A> ErrorObject checkConvGeometrySet(const std::string &who, const A &a) {
  FUSILLI_RETURN_ERROR_IF(a.getPadding().empty(), ErrorCode::AttributeNotSet, who + " padding not set");
  FUSILLI_RETURN_ERROR_IF(a.getStride().empty(), ErrorCode::AttributeNotSet, who + " stride not set");
  FUSILLI_RETURN_ERROR_IF(a.getDilation().empty(), ErrorCode::AttributeNotSet, who + " dilation not set");
  return ok();
}
template <typename A> ErrorObject checkConvGeometryRank(const std::string &who, const A &a, size_t rank) {
  const size_t ns = rank - 2;
  FUSILLI_RETURN_ERROR_IF(a.getPadding().size() != ns, ErrorCode::InvalidAttribute,
                          who + " padding size does not match number of spatial dimensions");
  FUSILLI_RETURN_ERROR_IF(a.getStride().size() != ns, ErrorCode::InvalidAttribute,
                          who + " stride size does not match number of spatial dimensions");
  FUSILLI_RETURN_ERROR_IF(a.getDilation().size() != ns, ErrorCode::InvalidAttribute,
                          who + " dilation size does not match number of spatial dimensions");
  return ok();
}
// `inName` / `outName` are how the message names the two channel counts.
inline ErrorObject checkGroups(const std::string &who, const std::string &inName, const std::string &outName,
                               int64_t inC, int64_t outC, int64_t filterC) {
  FUSILLI_RETURN_ERROR_IF(filterC <= 0 || inC % filterC != 0, ErrorCode::InvalidAttribute,
                          who + " " + inName + " channels must be divisible by the filter" +
                              (inName == "input" ? "" : " (W)") + " channels");
  const int64_t groups = inC / filterC;
  FUSILLI_RETURN_ERROR_IF(groups <= 0 || groups > inC || groups > outC, ErrorCode::InvalidAttribute,
                          who + " group count must be greater than 0 and less than or equal to the "
                                "numbers of input and outputs channels");
  FUSILLI_RETURN_ERROR_IF(outC % groups != 0, ErrorCode::InvalidAttribute,
                          who + " " + outName + " channels must be divisible by the group count");
  return ok();
}
inline ErrorObject requireLayout(const TensorPtr &t) {
  FUSILLI_RETURN_ERROR_IF(!layoutOk(t), ErrorCode::NotImplemented, notChannelsLastMsg(t));
  return ok();
}

} // namespace detail

class ConvFPropNode : public INode {
public:
  ConvFPropAttr convFPropAttr;
  ConvFPropNode(ConvFPropAttr &&a, const Context &ctx) : INode(ctx), convFPropAttr(std::move(a)) {}
  const std::string &getName() const override { return convFPropAttr.getName(); }
  Type getType() const override { return Type::Convolution; }

  ErrorObject preValidateNode() const override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Pre-Validating ConvFPropNode '" << getName() << "'");
    const auto &a = convFPropAttr;
    FUSILLI_CHECK_ERROR(detail::checkConvGeometrySet("Conv", a));
    TensorPtr x = a.getX(), w = a.getW(), y = a.getY();
    FUSILLI_RETURN_ERROR_IF(!x, ErrorCode::AttributeNotSet, "Conv input tensor X not set");
    FUSILLI_RETURN_ERROR_IF(!w, ErrorCode::AttributeNotSet, "Conv weight tensor W not set");
    FUSILLI_RETURN_ERROR_IF(!y, ErrorCode::AttributeNotSet, "Conv output tensor Y not set");
    FUSILLI_RETURN_ERROR_IF(x->getDim().size() < 3, ErrorCode::InvalidAttribute,
                            "Conv input tensor X must have a rank of at least 3");
    FUSILLI_RETURN_ERROR_IF(x->getDim().size() != w->getDim().size(), ErrorCode::InvalidAttribute,
                            "Conv input tensor X and weight tensor W have different ranks");
    FUSILLI_CHECK_ERROR(detail::checkConvGeometryRank("Conv", a, x->getDim().size()));
    FUSILLI_CHECK_ERROR(detail::requireLayout(x));
    FUSILLI_CHECK_ERROR(detail::requireLayout(w));
    return detail::checkGroups("Conv", "input", "output", x->getDim()[1], w->getDim()[0], w->getDim()[1]);
  }
  ErrorObject inferPropertiesNode() override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Inferring properties for ConvFPropNode '" << getName() << "'");
    auto &a = convFPropAttr;
    a.fillFromContext(context);
    TensorPtr x = a.getX(), w = a.getW(), y = a.getY();
    if (y->getDim().empty())
      y->setDim(getConvInferredOutputShape(x->getDim(), w->getDim(), a.getDilation(), a.getPadding(), a.getStride()));
    if (y->getStride().empty()) y->setStride(detail::strideLike(x, y->getDim()));
    return ok();
  }
  ErrorObject postValidateNode() const override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Post-Validating ConvFPropNode '" << getName() << "'");
    const auto &a = convFPropAttr;
    TensorPtr x = a.getX(), w = a.getW(), y = a.getY();
    FUSILLI_RETURN_ERROR_IF(y->getDim().size() < 3, ErrorCode::InvalidAttribute,
                            "Conv output tensor Y must have a rank of at least 3");
    FUSILLI_RETURN_ERROR_IF(x->getDim().size() != y->getDim().size(), ErrorCode::InvalidAttribute,
                            "Conv input tensor X and output tensor Y have different ranks");
    FUSILLI_RETURN_ERROR_IF(y->getDim() != getConvInferredOutputShape(x->getDim(), w->getDim(), a.getDilation(),
                                                                      a.getPadding(), a.getStride()),
                            ErrorCode::InvalidAttribute,
                            "Conv output tensor Y dimensions do not match the expected shapes inferred "
                            "based on the input and weight dimensions");
    return detail::requireLayout(y);
  }
  void describe(fb_node_desc &d, const TensorId &id) const override {
    detail::initDesc(d, FB_OP_CONV_FPROP);
    d.inputs[0] = id(convFPropAttr.getX());
    d.inputs[1] = id(convFPropAttr.getW());
    d.outputs[0] = id(convFPropAttr.getY());
    detail::convGeometry(d, convFPropAttr);
  }
};

class ConvWGradNode : public INode {
public:
  ConvWGradAttr convWGradAttr;
  ConvWGradNode(ConvWGradAttr &&a, const Context &ctx) : INode(ctx), convWGradAttr(std::move(a)) {}
  const std::string &getName() const override { return convWGradAttr.getName(); }
  Type getType() const override { return Type::WGrad; }

  ErrorObject preValidateNode() const override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Pre-Validating ConvWGradNode '" << getName() << "'");
    const auto &a = convWGradAttr;
    FUSILLI_CHECK_ERROR(detail::checkConvGeometrySet("ConvWGrad", a));
    TensorPtr dy = a.getDY(), x = a.getX(), dw = a.getDW();
    FUSILLI_RETURN_ERROR_IF(!dy, ErrorCode::AttributeNotSet, "ConvWGrad gradient tensor DY not set");
    FUSILLI_RETURN_ERROR_IF(!x, ErrorCode::AttributeNotSet, "ConvWGrad input tensor X not set");
    FUSILLI_RETURN_ERROR_IF(!dw, ErrorCode::AttributeNotSet, "ConvWGrad output tensor DW not set");
    FUSILLI_RETURN_ERROR_IF(dy->getDim().size() < 3 || x->getDim().size() < 3, ErrorCode::InvalidAttribute,
                            "ConvWGrad input tensors DY/X must have a rank of at least 3");
    FUSILLI_RETURN_ERROR_IF(dy->getDim().size() != x->getDim().size(), ErrorCode::InvalidAttribute,
                            "ConvWGrad tensors DY and X have different ranks");
    FUSILLI_CHECK_ERROR(detail::checkConvGeometryRank("ConvWGrad", a, dy->getDim().size()));
    FUSILLI_CHECK_ERROR(detail::requireLayout(dy));
    FUSILLI_CHECK_ERROR(detail::requireLayout(x));
    // The filter extent cannot be inferred (the group count is unknown), so DW's dims are an input.
    FUSILLI_RETURN_ERROR_IF(dw->getDim().size() < 2, ErrorCode::InvalidAttribute,
                            "ConvWGrad weight gradient tensor DW must have a rank of at least 3");
    return detail::checkGroups("ConvWGrad", "input (X)", "output (DY)", x->getDim()[1], dy->getDim()[1],
                               dw->getDim()[1]);
  }
  ErrorObject inferPropertiesNode() override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Inferring properties for ConvWGradNode '" << getName() << "'");
    auto &a = convWGradAttr;
    a.fillFromContext(context);
    TensorPtr dy = a.getDY(), dw = a.getDW();
    if (dw->getStride().empty()) dw->setStride(detail::strideLike(dy, dw->getDim()));
    return ok();
  }
  ErrorObject postValidateNode() const override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Post-Validating ConvWGradNode '" << getName() << "'");
    const auto &a = convWGradAttr;
    TensorPtr dy = a.getDY(), x = a.getX(), dw = a.getDW();
    FUSILLI_RETURN_ERROR_IF(dw->getDim().size() < 3, ErrorCode::InvalidAttribute,
                            "ConvWGrad weight gradient tensor DW must have a rank of at least 3");
    FUSILLI_RETURN_ERROR_IF(dy->getDim() != getConvInferredOutputShape(x->getDim(), dw->getDim(), a.getDilation(),
                                                                       a.getPadding(), a.getStride()),
                            ErrorCode::InvalidAttribute,
                            "ConvWGrad output DW dimensions do not match the expected shapes inferred based on "
                            "input dimensions");
    return detail::requireLayout(dw);
  }
  void describe(fb_node_desc &d, const TensorId &id) const override {
    detail::initDesc(d, FB_OP_CONV_WGRAD);
    d.inputs[0] = id(convWGradAttr.getDY());
    d.inputs[1] = id(convWGradAttr.getX());
    d.outputs[0] = id(convWGradAttr.getDW());
    detail::convGeometry(d, convWGradAttr);
  }
};

class ConvDGradNode : public INode {
public:
  ConvDGradAttr convDGradAttr;
  ConvDGradNode(ConvDGradAttr &&a, const Context &ctx) : INode(ctx), convDGradAttr(std::move(a)) {}
  const std::string &getName() const override { return convDGradAttr.getName(); }
  Type getType() const override { return Type::DGrad; }

  ErrorObject preValidateNode() const override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Pre-Validating ConvDGradNode '" << getName() << "'");
    const auto &a = convDGradAttr;
    FUSILLI_CHECK_ERROR(detail::checkConvGeometrySet("ConvDGrad", a));
    TensorPtr dy = a.getDY(), w = a.getW(), dx = a.getDX();
    FUSILLI_RETURN_ERROR_IF(!dy, ErrorCode::AttributeNotSet, "ConvDGrad gradient tensor DY not set");
    FUSILLI_RETURN_ERROR_IF(!w, ErrorCode::AttributeNotSet, "ConvDGrad input tensor W not set");
    FUSILLI_RETURN_ERROR_IF(!dx, ErrorCode::AttributeNotSet, "ConvDGrad output tensor DX not set");
    FUSILLI_RETURN_ERROR_IF(dy->getDim().size() < 3 || w->getDim().size() < 3, ErrorCode::InvalidAttribute,
                            "ConvDGrad input tensors DY/W must have a rank of at least 3");
    FUSILLI_CHECK_ERROR(detail::checkConvGeometryRank("ConvDGrad", a, dy->getDim().size()));
    FUSILLI_CHECK_ERROR(detail::requireLayout(dy));
    FUSILLI_CHECK_ERROR(detail::requireLayout(w));
    // DX's extent cannot be inferred (the group count is unknown), so its dims are an input.
    FUSILLI_RETURN_ERROR_IF(dx->getDim().size() < 2, ErrorCode::InvalidAttribute,
                            "ConvDGrad input gradient DX must have a rank of at least 3");
    return detail::checkGroups("ConvDGrad", "input (DX)", "output (DY)", dx->getDim()[1], w->getDim()[0],
                               w->getDim()[1]);
  }
  ErrorObject inferPropertiesNode() override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Inferring properties for ConvDGradNode '" << getName() << "'");
    auto &a = convDGradAttr;
    a.fillFromContext(context);
    TensorPtr dy = a.getDY(), dx = a.getDX();
    if (dx->getStride().empty()) dx->setStride(detail::strideLike(dy, dx->getDim()));
    return ok();
  }
  ErrorObject postValidateNode() const override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Post-Validating ConvDGradNode '" << getName() << "'");
    const auto &a = convDGradAttr;
    TensorPtr dy = a.getDY(), w = a.getW(), dx = a.getDX();
    FUSILLI_RETURN_ERROR_IF(dx->getDim().size() < 3, ErrorCode::InvalidAttribute,
                            "ConvDGrad input gradient DX must have a rank of at least 3");
    FUSILLI_RETURN_ERROR_IF(dy->getDim().size() != dx->getDim().size(), ErrorCode::InvalidAttribute,
                            "ConvDGrad tensors DY and DX have different ranks");
    FUSILLI_RETURN_ERROR_IF(dy->getDim() != getConvInferredOutputShape(dx->getDim(), w->getDim(), a.getDilation(),
                                                                       a.getPadding(), a.getStride()),
                            ErrorCode::InvalidAttribute,
                            "ConvDGrad DY dimensions do not match the expected shapes inferred based on DX and W");
    return detail::requireLayout(dx);
  }
  void describe(fb_node_desc &d, const TensorId &id) const override {
    detail::initDesc(d, FB_OP_CONV_DGRAD);
    d.inputs[0] = id(convDGradAttr.getDY());
    d.inputs[1] = id(convDGradAttr.getW());
    d.outputs[0] = id(convDGradAttr.getDX());
    detail::convGeometry(d, convDGradAttr);
  }
};

} // namespace fusilli

#include "nodes_more.h"

#endif // FUSILLI_NODES_H

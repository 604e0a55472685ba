// Matmul, SDPA, LayerNorm, RMSNorm, reduction and pointwise nodes (continuation of nodes.h;
// include that file, not this one).
#ifndef FUSILLI_NODES_MORE_H
#define FUSILLI_NODES_MORE_H

namespace fusilli {

class MatmulNode : public INode {
public:
  MatmulAttr matmulAttr;
  MatmulNode(MatmulAttr &&a, const Context &ctx) : INode(ctx), matmulAttr(std::move(a)) {}
  const std::string &getName() const override { return matmulAttr.getName(); }
  Type getType() const override { return Type::Matmul; }

  ErrorObject preValidateNode() const override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Pre-Validating MatmulNode '" << getName() << "'");
    const auto &m = matmulAttr;
    TensorPtr a = m.getA(), b = m.getB(), c = m.getC();
    FUSILLI_RETURN_ERROR_IF(!a, ErrorCode::AttributeNotSet, "Matmul input tensor A not set");
    FUSILLI_RETURN_ERROR_IF(!b, ErrorCode::AttributeNotSet, "Matmul input tensor B not set");
    FUSILLI_RETURN_ERROR_IF(!c, ErrorCode::AttributeNotSet, "Matmul output tensor C not set");
    const auto &ad = a->getDim(), &bd = b->getDim();
    const size_t ra = ad.size(), rb = bd.size();
    FUSILLI_RETURN_ERROR_IF(ra < 2, ErrorCode::InvalidAttribute, "Matmul input tensor A must have a rank of at least 2");
    FUSILLI_RETURN_ERROR_IF(rb < 2, ErrorCode::InvalidAttribute, "Matmul input tensor B must have a rank of at least 2");
    FUSILLI_RETURN_ERROR_IF(ra != rb, ErrorCode::InvalidAttribute,
                            "Matmul input tensors A and B must have the same rank: A has rank=" +
                                std::to_string(ra) + ", B has rank=" + std::to_string(rb));
    FUSILLI_RETURN_ERROR_IF(ad[ra - 1] != bd[rb - 2], ErrorCode::InvalidAttribute,
                            "Matmul input tensors A and B have incompatible inner dimensions (K): A has K=" +
                                std::to_string(ad[ra - 1]) + ", B has K=" + std::to_string(bd[rb - 2]));
    for (size_t i = 0; i + 2 < ra; ++i)
      FUSILLI_RETURN_ERROR_IF(!(ad[i] % bd[i] == 0 || bd[i] % ad[i] == 0), ErrorCode::InvalidAttribute,
                              "Matmul input tensors A and B have incompatible batch dimensions for "
                              "broadcasting at index " + std::to_string(i) + ": A has dim=" +
                                  std::to_string(ad[i]) + ", B has dim=" + std::to_string(bd[i]));
    FUSILLI_CHECK_ERROR(batchDimsOutermost(a, "A"));
    FUSILLI_CHECK_ERROR(batchDimsOutermost(b, "B"));
    // Operands of different element types: one batch dim, equal on both sides.
    if (a->getDataType() != b->getDataType()) {
      FUSILLI_RETURN_ERROR_IF(ra != 3, ErrorCode::InvalidAttribute,
                              "Mixed precision matmul is only supported when input tensors A and B are of "
                              "rank 3 (single batch dim): A and B have rank=" + std::to_string(ra));
      FUSILLI_RETURN_ERROR_IF(ad[0] != bd[0], ErrorCode::InvalidAttribute,
                              "Mixed precision matmul input tensors A and B must have exactly equal batch "
                              "dimensions (no broadcast): A has batch dim=" + std::to_string(ad[0]) +
                                  ", B has batch dim=" + std::to_string(bd[0]));
    }
    return ok();
  }
  ErrorObject inferPropertiesNode() override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Inferring properties for MatmulNode '" << getName() << "'");
    auto &m = matmulAttr;
    m.fillFromContext(context);
    TensorPtr a = m.getA(), b = m.getB(), c = m.getC();
    if (c->getDim().empty()) c->setDim(getMatmulInferredOutputShape(a->getDim(), b->getDim()));
    if (c->getStride().empty())
      c->setStride(generateStrideFromDim(c->getDim(), getContiguousStrideOrder(c->getDim().size())));
    return ok();
  }
  ErrorObject postValidateNode() const override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Post-Validating MatmulNode '" << getName() << "'");
    const auto &m = matmulAttr;
    TensorPtr a = m.getA(), b = m.getB(), c = m.getC();
    FUSILLI_RETURN_ERROR_IF(c->getDim().size() < 2, ErrorCode::InvalidAttribute,
                            "Matmul output tensor C must have a rank of at least 2");
    FUSILLI_RETURN_ERROR_IF(c->getDim() != getMatmulInferredOutputShape(a->getDim(), b->getDim()),
                            ErrorCode::InvalidAttribute,
                            "Matmul output tensor C dimensions do not match the expected shapes inferred "
                            "based on the input dimensions");
    return batchDimsOutermost(c, "C");
  }
  void describe(fb_node_desc &d, const TensorId &id) const override {
    detail::initDesc(d, FB_OP_MATMUL);
    d.inputs[0] = id(matmulAttr.getA());
    d.inputs[1] = id(matmulAttr.getB());
    d.outputs[0] = id(matmulAttr.getC());
  }

private:
  static ErrorObject batchDimsOutermost(const TensorPtr &t, const std::string &which) {
    const auto perm = t->getLogicalToPhysicalPermuteOrder();
    for (size_t i = 0; i + 2 < t->getDim().size(); ++i)
      FUSILLI_RETURN_ERROR_IF(perm[i] != static_cast<int64_t>(i), ErrorCode::InvalidAttribute,
                              "Matmul tensor " + which + " has batch dimensions that are not outermost or "
                              "are transposed");
    return ok();
  }
};

class SdpaNode : public INode {
public:
  SdpaAttr sdpaAttr;
  SdpaNode(SdpaAttr &&a, const Context &ctx) : INode(ctx), sdpaAttr(std::move(a)) {}
  const std::string &getName() const override { return sdpaAttr.getName(); }
  Type getType() const override { return Type::Sdpa; }

  ErrorObject preValidateNode() const override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Pre-Validating SdpaNode '" << getName() << "'");
    const auto &a = sdpaAttr;
    TensorPtr q = a.getQ(), k = a.getK(), v = a.getV(), o = a.getO(), mask = a.getMASK();
    FUSILLI_RETURN_ERROR_IF(!q, ErrorCode::AttributeNotSet, "SDPA input tensor Q not set");
    FUSILLI_RETURN_ERROR_IF(!k, ErrorCode::AttributeNotSet, "SDPA input tensor K not set");
    FUSILLI_RETURN_ERROR_IF(!v, ErrorCode::AttributeNotSet, "SDPA input tensor V not set");
    FUSILLI_RETURN_ERROR_IF(!o, ErrorCode::AttributeNotSet, "SDPA output tensor O not set");
    FUSILLI_RETURN_ERROR_IF(q->getDim().size() != 4, ErrorCode::InvalidAttribute,
                            "SDPA input tensor Q must be rank 4 [batch, heads_q, seq_q, head_dim]");
    FUSILLI_RETURN_ERROR_IF(k->getDim().size() != 4, ErrorCode::InvalidAttribute,
                            "SDPA input tensor K must be rank 4 [batch, heads_kv, seq_kv, head_dim]");
    FUSILLI_RETURN_ERROR_IF(v->getDim().size() != 4, ErrorCode::InvalidAttribute,
                            "SDPA input tensor V must be rank 4 [batch, heads_kv, seq_kv, head_dim]");
    const auto &qd = q->getDim(), &kd = k->getDim(), &vd = v->getDim();
    FUSILLI_RETURN_ERROR_IF(qd[0] != kd[0] || qd[0] != vd[0], ErrorCode::InvalidAttribute,
                            "SDPA input tensors Q, K, V must have matching batch dimension");
    FUSILLI_RETURN_ERROR_IF(qd[3] != kd[3], ErrorCode::InvalidAttribute,
                            "SDPA input tensors Q and K must have matching head_dim");
    FUSILLI_RETURN_ERROR_IF(kd[2] != vd[2], ErrorCode::InvalidAttribute,
                            "SDPA input tensors K and V must have matching sequence length");
    const int64_t hq = qd[1], hk = kd[1], hv = vd[1];
    auto heads = [](int64_t a_, int64_t b_, const char *rel, const char *what) {
      return std::string("SDPA ") + what + " Q heads (" + std::to_string(a_) + ") " + rel + " heads (" +
             std::to_string(b_) + ")";
    };
    if (a.getEnableGqa()) {
      FUSILLI_RETURN_ERROR_IF(hq % hk != 0, ErrorCode::InvalidAttribute,
                              heads(hq, hk, "to be a multiple of K", "with GQA requires"));
      FUSILLI_RETURN_ERROR_IF(hq % hv != 0, ErrorCode::InvalidAttribute,
                              heads(hq, hv, "to be a multiple of V", "with GQA requires"));
    } else {
      FUSILLI_RETURN_ERROR_IF(hq != hk, ErrorCode::InvalidAttribute,
                              heads(hq, hk, "to equal K", "without GQA requires"));
      FUSILLI_RETURN_ERROR_IF(hq != hv, ErrorCode::InvalidAttribute,
                              heads(hq, hv, "to equal V", "without GQA requires"));
    }
    FUSILLI_RETURN_ERROR_IF(mask && a.getIsCausal(), ErrorCode::InvalidAttribute,
                            "SDPA attention mask and is_causal are mutually exclusive");
    if (mask) {
      const auto &md = mask->getDim();
      FUSILLI_RETURN_ERROR_IF(md.size() != 4, ErrorCode::InvalidAttribute, "SDPA attention mask must be rank 4");
      const int64_t full[4] = {qd[0], hq, qd[2], kd[2]};
      const char *what[4] = {"batch dim", "heads dim", "seq_q dim", "seq_kv dim"};
      const char *match[4] = {"input batch", "Q heads", "Q sequence length", "KV sequence length"};
      for (int i = 0; i < 4; ++i)
        FUSILLI_RETURN_ERROR_IF(md[i] != 1 && md[i] != full[i], ErrorCode::InvalidAttribute,
                                std::string("SDPA attention mask ") + what[i] + " (" + std::to_string(md[i]) +
                                    ") must be 1 or match " + match[i] + " (" + std::to_string(full[i]) + ")");
    }
    FUSILLI_RETURN_ERROR_IF(a.getDropout() < 0.f || a.getDropout() >= 1.f, ErrorCode::InvalidAttribute,
                            "SDPA dropout probability must be in [0, 1)");
    return ok();
  }
  ErrorObject inferPropertiesNode() override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Inferring properties for SdpaNode '" << getName() << "'");
    auto &a = sdpaAttr;
    a.fillFromContext(context);
    TensorPtr q = a.getQ(), v = a.getV(), o = a.getO();
    const std::vector<int64_t> od = {q->getDim()[0], q->getDim()[1], q->getDim()[2], v->getDim()[3]};
    if (o->getDim().empty()) o->setDim(od);
    if (o->getStride().empty())
      o->setStride(generateStrideFromDim(o->getDim(), getContiguousStrideOrder(o->getDim().size())));
    return ok();
  }
  ErrorObject postValidateNode() const override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Post-Validating SdpaNode '" << getName() << "'");
    const auto &a = sdpaAttr;
    TensorPtr q = a.getQ(), v = a.getV(), o = a.getO();
    const std::vector<int64_t> od = {q->getDim()[0], q->getDim()[1], q->getDim()[2], v->getDim()[3]};
    FUSILLI_RETURN_ERROR_IF(o->getDim() != od, ErrorCode::InvalidAttribute,
                            "SDPA output tensor O dimensions do not match expected shape "
                            "[batch, headsQ, seqQ, headDim]");
    return ok();
  }
  void describe(fb_node_desc &d, const TensorId &id) const override {
    detail::initDesc(d, FB_OP_SDPA);
    d.inputs[0] = id(sdpaAttr.getQ());
    d.inputs[1] = id(sdpaAttr.getK());
    d.inputs[2] = id(sdpaAttr.getV());
    d.inputs[3] = id(sdpaAttr.getMASK());
    d.outputs[0] = id(sdpaAttr.getO());
    if (sdpaAttr.getIsCausal()) d.flags |= FB_FLAG_SDPA_CAUSAL;
    if (sdpaAttr.getEnableGqa()) d.flags |= FB_FLAG_SDPA_GQA;
    if (sdpaAttr.getScale()) {
      d.flags |= FB_FLAG_SDPA_HAS_SCALE;
      d.fparams[0] = *sdpaAttr.getScale();
    }
    d.fparams[1] = sdpaAttr.getDropout();
  }
};

// Shape helpers shared by the norms (reference node/norm_utils.h:40-99).
namespace norm_utils {
// [B, 1, ..., 1] and its contiguous strides: the shape of MEAN / INV_VARIANCE / INV_RMS.
inline std::pair<std::vector<int64_t>, std::vector<int64_t>>
getTrainingForwardOutputDimAndStride(const std::vector<int64_t> &xDim, size_t batchDim = 0) {
  std::vector<int64_t> dim(xDim.size(), 1);
  dim[batchDim] = xDim[batchDim];
  return {dim, generateStrideFromDim(dim, getContiguousStrideOrder(dim.size()))};
}
// X's shape with the batch dim set to 1: the shape of SCALE / BIAS.
inline std::vector<int64_t> getScaleBiasDim(const std::vector<int64_t> &xDim, size_t batchDim = 0) {
  auto dim = xDim;
  dim[batchDim] = 1;
  return dim;
}
inline std::vector<int64_t> getScaleBiasStride(const std::vector<int64_t> &dim, const std::vector<int64_t> &xStride) {
  return generateStrideFromDim(dim, generateStrideOrderPreservingFormat(xStride, dim.size()));
}
inline void inferDimAndStride(const TensorPtr &t, const std::vector<int64_t> &dim, const std::vector<int64_t> &stride) {
  if (t->getDim().empty()) t->setDim(dim);
  if (t->getStride().empty()) t->setStride(stride);
}
inline void inferScaleBiasDimAndStride(const TensorPtr &t, const std::vector<int64_t> &xDim,
                                       const std::vector<int64_t> &xStride) {
  if (t->getDim().empty()) t->setDim(getScaleBiasDim(xDim));
  if (t->getStride().empty()) t->setStride(getScaleBiasStride(t->getDim(), xStride));
}
} // namespace norm_utils

namespace detail {
inline ErrorObject checkScaleBias(const std::string &who, const char *which, const TensorPtr &t, const TensorPtr &x) {
  if (!t) return ok();
  if (!t->getDim().empty())
    FUSILLI_RETURN_ERROR_IF(t->getDim() != norm_utils::getScaleBiasDim(x->getDim()), ErrorCode::InvalidAttribute,
                            who + " input tensor " + which + " must have shape as tensor X with single batch");
  if (!t->getStride().empty()) FUSILLI_CHECK_ERROR(requireLayout(t));
  return ok();
}
} // namespace detail

class LayerNormNode : public INode {
public:
  LayernormAttr layernormAttr;
  LayerNormNode(LayernormAttr &&a, const Context &ctx) : INode(ctx), layernormAttr(std::move(a)) {}
  const std::string &getName() const override { return layernormAttr.getName(); }
  Type getType() const override { return Type::LayerNorm; }
  bool isTrainingForwardPhase() const { return layernormAttr.getForwardPhase() == NormFwdPhase::TRAINING; }

  ErrorObject preValidateNode() const override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Pre-Validating LayerNormNode '" << getName() << "'");
    const auto &a = layernormAttr;
    FUSILLI_RETURN_ERROR_IF(a.getForwardPhase() == NormFwdPhase::NOT_SET, ErrorCode::AttributeNotSet,
                            "LayerNorm forward phase not set");
    TensorPtr x = a.getX(), s = a.getSCALE(), b = a.getBIAS(), y = a.getY(), m = a.getMEAN(),
              v = a.getINV_VARIANCE(), e = a.getEpsilon();
    FUSILLI_RETURN_ERROR_IF(!x, ErrorCode::AttributeNotSet, "LayerNorm input tensor X not set");
    FUSILLI_RETURN_ERROR_IF(!y, ErrorCode::AttributeNotSet, "LayerNorm output tensor Y not set");
    FUSILLI_RETURN_ERROR_IF(x->getDim().size() < 2, ErrorCode::InvalidAttribute,
                            "LayerNorm input tensor X must have a rank of at least 2");
    FUSILLI_CHECK_ERROR(detail::requireLayout(x));
    FUSILLI_CHECK_ERROR(detail::checkScaleBias("LayerNorm", "SCALE", s, x));
    FUSILLI_CHECK_ERROR(detail::checkScaleBias("LayerNorm", "BIAS", b, x));
    if (isTrainingForwardPhase()) {
      FUSILLI_RETURN_ERROR_IF(!m, ErrorCode::AttributeNotSet, "LayerNorm output tensor MEAN not set");
      FUSILLI_RETURN_ERROR_IF(!v, ErrorCode::AttributeNotSet, "LayerNorm output tensor INV_VARIANCE not set");
    } else {
      FUSILLI_RETURN_ERROR_IF(m != nullptr, ErrorCode::InvalidAttribute, "LayerNorm output tensor MEAN should not be set");
      FUSILLI_RETURN_ERROR_IF(v != nullptr, ErrorCode::InvalidAttribute,
                              "LayerNorm output tensor INV_VARIANCE should not be set");
    }
    FUSILLI_RETURN_ERROR_IF(!e, ErrorCode::AttributeNotSet, "LayerNorm epsilon not set");
    FUSILLI_RETURN_ERROR_IF(!e->isScalar(), ErrorCode::InvalidAttribute, "LayerNorm epsilon must be a scalar constant");
    return ok();
  }
  ErrorObject inferPropertiesNode() override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Inferring properties for LayerNormNode '" << getName() << "'");
    auto &a = layernormAttr;
    a.fillFromContext(context);
    TensorPtr x = a.getX(), s = a.getSCALE(), b = a.getBIAS(), y = a.getY();
    if (s) norm_utils::inferScaleBiasDimAndStride(s, x->getDim(), x->getStride());
    if (b) norm_utils::inferScaleBiasDimAndStride(b, x->getDim(), x->getStride());
    norm_utils::inferDimAndStride(y, x->getDim(), x->getStride());
    if (isTrainingForwardPhase()) {
      const auto [dim, stride] = norm_utils::getTrainingForwardOutputDimAndStride(x->getDim());
      norm_utils::inferDimAndStride(a.getMEAN(), dim, stride);
      norm_utils::inferDimAndStride(a.getINV_VARIANCE(), dim, stride);
    }
    return ok();
  }
  ErrorObject postValidateNode() const override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Post-Validating LayerNormNode '" << getName() << "'");
    const auto &a = layernormAttr;
    TensorPtr x = a.getX(), y = a.getY();
    FUSILLI_RETURN_ERROR_IF(x->getDim() != y->getDim(), ErrorCode::InvalidAttribute,
                            "LayerNorm output Y tensor must have the same shape as input X tensor");
    FUSILLI_CHECK_ERROR(detail::requireLayout(y));
    if (isTrainingForwardPhase()) {
      const auto [dim, stride] = norm_utils::getTrainingForwardOutputDimAndStride(x->getDim());
      TensorPtr m = a.getMEAN(), v = a.getINV_VARIANCE();
      FUSILLI_RETURN_ERROR_IF(m->getDim() != dim, ErrorCode::InvalidAttribute,
                              "Layernorm output MEAN tensor must have shape [B, 1, ..., 1] with rank equal to "
                              "input X tensor's rank, and batch dimension equal to input X tensor's batch dimension");
      FUSILLI_RETURN_ERROR_IF(v->getDim() != dim, ErrorCode::InvalidAttribute,
                              "LayerNorm output INV_VARIANCE tensor must have shape [B, 1, ..., 1] with  rank equal "
                              "to input X tensor's rank, and batch dimension equal to input X tensor's batch dimension");
      FUSILLI_RETURN_ERROR_IF(m->getStride() != stride, ErrorCode::InvalidAttribute,
                              "LayerNorm output MEAN tensor must have unit strides");
      FUSILLI_RETURN_ERROR_IF(v->getStride() != stride, ErrorCode::InvalidAttribute,
                              "LayerNorm output INV_VARIANCE tensor must have unit strides");
    }
    return ok();
  }
  void describe(fb_node_desc &d, const TensorId &id) const override {
    detail::initDesc(d, FB_OP_LAYERNORM);
    d.inputs[0] = id(layernormAttr.getX());
    d.inputs[1] = id(layernormAttr.getSCALE());
    d.inputs[2] = id(layernormAttr.getBIAS());
    d.inputs[3] = id(layernormAttr.getEpsilon());
    d.outputs[0] = id(layernormAttr.getY());
    d.outputs[1] = id(layernormAttr.getMEAN());
    d.outputs[2] = id(layernormAttr.getINV_VARIANCE());
    if (isTrainingForwardPhase()) d.flags |= FB_FLAG_NORM_TRAINING;
  }
};

class RmsNormNode : public INode {
public:
  RmsnormAttr rmsnormAttr;
  RmsNormNode(RmsnormAttr &&a, const Context &ctx) : INode(ctx), rmsnormAttr(std::move(a)) {}
  const std::string &getName() const override { return rmsnormAttr.getName(); }
  Type getType() const override { return Type::RmsNorm; }
  bool isTrainingForwardPhase() const { return rmsnormAttr.getForwardPhase() == NormFwdPhase::TRAINING; }

  ErrorObject preValidateNode() const override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Pre-Validating RmsNormNode '" << getName() << "'");
    const auto &a = rmsnormAttr;
    FUSILLI_RETURN_ERROR_IF(a.getForwardPhase() == NormFwdPhase::NOT_SET, ErrorCode::AttributeNotSet,
                            "RmsNorm forward phase not set");
    TensorPtr x = a.getX(), s = a.getSCALE(), y = a.getY(), r = a.getINV_RMS(), e = a.getEpsilon();
    FUSILLI_RETURN_ERROR_IF(!x, ErrorCode::AttributeNotSet, "RmsNorm input tensor X not set");
    FUSILLI_RETURN_ERROR_IF(!y, ErrorCode::AttributeNotSet, "RmsNorm output tensor Y not set");
    FUSILLI_RETURN_ERROR_IF(x->getDim().size() < 2, ErrorCode::InvalidAttribute,
                            "RmsNorm input tensor X must have a rank of at least 2");
    FUSILLI_CHECK_ERROR(detail::requireLayout(x));
    FUSILLI_CHECK_ERROR(detail::checkScaleBias("RmsNorm", "SCALE", s, x));
    if (isTrainingForwardPhase())
      FUSILLI_RETURN_ERROR_IF(!r, ErrorCode::AttributeNotSet, "RmsNorm output tensor INV_RMS not set");
    else
      FUSILLI_RETURN_ERROR_IF(r != nullptr, ErrorCode::InvalidAttribute, "RmsNorm output tensor INV_RMS should not be set");
    FUSILLI_RETURN_ERROR_IF(!e, ErrorCode::AttributeNotSet, "RmsNorm epsilon not set");
    FUSILLI_RETURN_ERROR_IF(!e->isScalar(), ErrorCode::InvalidAttribute, "RmsNorm epsilon must be a scalar constant");
    return ok();
  }
  ErrorObject inferPropertiesNode() override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Inferring properties for RmsNormNode '" << getName() << "'");
    auto &a = rmsnormAttr;
    a.fillFromContext(context);
    TensorPtr x = a.getX(), s = a.getSCALE(), y = a.getY();
    if (s) norm_utils::inferScaleBiasDimAndStride(s, x->getDim(), x->getStride());
    norm_utils::inferDimAndStride(y, x->getDim(), x->getStride());
    if (isTrainingForwardPhase()) {
      const auto [dim, stride] = norm_utils::getTrainingForwardOutputDimAndStride(x->getDim());
      norm_utils::inferDimAndStride(a.getINV_RMS(), dim, stride);
    }
    return ok();
  }
  ErrorObject postValidateNode() const override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Post-Validating RmsNormNode '" << getName() << "'");
    const auto &a = rmsnormAttr;
    TensorPtr x = a.getX(), y = a.getY();
    FUSILLI_RETURN_ERROR_IF(x->getDim() != y->getDim(), ErrorCode::InvalidAttribute,
                            "RmsNorm output Y tensor must have the same shape as input X tensor");
    FUSILLI_CHECK_ERROR(detail::requireLayout(y));
    if (isTrainingForwardPhase()) {
      const auto [dim, stride] = norm_utils::getTrainingForwardOutputDimAndStride(x->getDim());
      TensorPtr r = a.getINV_RMS();
      FUSILLI_RETURN_ERROR_IF(r->getDim() != dim, ErrorCode::InvalidAttribute,
                              "RmsNorm output INV_RMS tensor must have shape [B, 1, ..., 1] with rank equal to "
                              "input X tensor's rank, and batch dimension equal to input X tensor's batch dimension");
      FUSILLI_RETURN_ERROR_IF(r->getStride() != stride, ErrorCode::InvalidAttribute,
                              "RmsNorm output INV_RMS tensor must have unit strides");
    }
    // As in the reference (rmsnorm_node.h:203-206) the training variant is declared but refused.
    FUSILLI_RETURN_ERROR_IF(isTrainingForwardPhase(), ErrorCode::NotImplemented,
                            "RmsNorm training mode is not yet supported: torch-mlir does not lower the "
                            "training variant");
    return ok();
  }
  void describe(fb_node_desc &d, const TensorId &id) const override {
    detail::initDesc(d, FB_OP_RMSNORM);
    d.inputs[0] = id(rmsnormAttr.getX());
    d.inputs[1] = id(rmsnormAttr.getSCALE());
    d.inputs[2] = id(rmsnormAttr.getEpsilon());
    d.outputs[0] = id(rmsnormAttr.getY());
  }
};

class ReductionNode : public INode {
public:
  ReductionAttr reductionAttr;
  ReductionNode(ReductionAttr &&a, const Context &ctx) : INode(ctx), reductionAttr(std::move(a)) {}
  const std::string &getName() const override { return reductionAttr.getName(); }
  Type getType() const override { return Type::Reduction; }
  // dims i with Y[i] == 1 and X[i] > 1
  std::vector<int64_t> getReductionDims() const {
    std::vector<int64_t> dims;
    const auto &xd = reductionAttr.getX()->getDim(), &yd = reductionAttr.getY()->getDim();
    for (size_t i = 0; i < xd.size(); ++i)
      if (yd[i] == 1 && xd[i] > 1) dims.push_back(static_cast<int64_t>(i));
    return dims;
  }

  ErrorObject preValidateNode() const override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Pre-Validating ReductionNode '" << getName() << "'");
    const auto &a = reductionAttr;
    FUSILLI_RETURN_ERROR_IF(a.getMode() == ReductionAttr::Mode::NOT_SET, ErrorCode::AttributeNotSet,
                            "Reduction mode not set");
    FUSILLI_RETURN_ERROR_IF(!a.getX(), ErrorCode::AttributeNotSet, "Reduction operation requires X input");
    FUSILLI_RETURN_ERROR_IF(!a.getY(), ErrorCode::AttributeNotSet, "Reduction operation requires Y output");
    FUSILLI_RETURN_ERROR_IF(a.getX()->getDim().empty(), ErrorCode::AttributeNotSet,
                            "Reduction input X dimensions not set");
    return ok();
  }
  ErrorObject inferPropertiesNode() override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Inferring properties for ReductionNode '" << getName() << "'");
    auto &a = reductionAttr;
    a.fillFromContext(context);
    TensorPtr x = a.getX(), y = a.getY();
    if (y->getDim().empty()) y->setDim(x->getDim());
    if (y->getStride().empty())
      y->setStride(generateStrideFromDim(y->getDim(), getContiguousStrideOrder(y->getDim().size())));
    return ok();
  }
  ErrorObject postValidateNode() const override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Post-Validating ReductionNode '" << getName() << "'");
    const auto &a = reductionAttr;
    TensorPtr x = a.getX(), y = a.getY();
    FUSILLI_RETURN_ERROR_IF(x->getDim().size() != y->getDim().size(), ErrorCode::InvalidAttribute,
                            "Reduction input and output must have the same rank");
    FUSILLI_RETURN_ERROR_IF(a.getMode() == ReductionAttr::Mode::AVG &&
                                (isIntegralOrBoolType(x->getDataType()) || isIntegralOrBoolType(y->getDataType())),
                            ErrorCode::InvalidAttribute,
                            "Reduction AVG is not supported for integral or boolean tensors");
    for (size_t i = 0; i < x->getDim().size(); ++i)
      FUSILLI_RETURN_ERROR_IF(y->getDim()[i] != 1 && y->getDim()[i] != x->getDim()[i], ErrorCode::InvalidAttribute,
                              "Reduction output dimension " + std::to_string(i) +
                                  " must be 1 or match input dimension");
    FUSILLI_RETURN_ERROR_IF(getReductionDims().empty(), ErrorCode::InvalidAttribute,
                            "Reduction requires at least one dimension to reduce (Y[i] == 1 where X[i] > 1)");
    return ok();
  }
  void describe(fb_node_desc &d, const TensorId &id) const override {
    detail::initDesc(d, FB_OP_REDUCTION);
    d.mode = static_cast<int32_t>(reductionAttr.getMode());
    d.inputs[0] = id(reductionAttr.getX());
    d.outputs[0] = id(reductionAttr.getY());
  }
};

class PointwiseNode : public INode {
public:
  PointwiseAttr pointwiseAttr;
  PointwiseNode(PointwiseAttr &&a, const Context &ctx) : INode(ctx), pointwiseAttr(std::move(a)) {}
  const std::string &getName() const override { return pointwiseAttr.getName(); }
  Type getType() const override { return Type::Pointwise; }

  ErrorObject preValidateNode() const override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Pre-Validating PointwiseNode '" << getName() << "'");
    const auto &a = pointwiseAttr;
    const auto mode = a.getMode();
    FUSILLI_RETURN_ERROR_IF(mode == PointwiseAttr::Mode::NOT_SET, ErrorCode::AttributeNotSet, "Pointwise mode not set");
    const TensorPtr ins[3] = {a.getIN_0(), a.getIN_1(), a.getIN_2()};
    const int need = PointwiseAttr::requiredInputCount(mode);
    const std::string nm = PointwiseAttr::modeName(mode);
    for (int i = 0; i < 3; ++i) {
      if (i < need)
        FUSILLI_RETURN_ERROR_IF(!ins[i], ErrorCode::AttributeNotSet,
                                nm + " mode requires IN_" + std::to_string(i) + " input");
      else
        FUSILLI_RETURN_ERROR_IF(ins[i] != nullptr, ErrorCode::InvalidAttribute,
                                nm + " mode should not have IN_" + std::to_string(i) + " input set");
    }
    FUSILLI_RETURN_ERROR_IF(!a.getOUT_0(), ErrorCode::AttributeNotSet, "Pointwise operation requires output");
    return ok();
  }
  ErrorObject inferPropertiesNode() override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Inferring properties for PointwiseNode '" << getName() << "'");
    auto &a = pointwiseAttr;
    TensorPtr out = a.getOUT_0();
    if (PointwiseAttr::forcesBooleanOutput(a.getMode())) out->setDataType(DataType::Boolean);
    a.fillFromContext(context);
    const TensorPtr ins[3] = {a.getIN_0(), a.getIN_1(), a.getIN_2()};
    if (out->getDim().empty()) {
      std::vector<std::vector<int64_t>> shapes;
      for (const auto &t : ins)
        if (t) shapes.push_back(t->getDim());
      FUSILLI_ASSIGN_OR_RETURN(auto shape, computeBroadcastShape(shapes));
      out->setDim(shape);
    }
    if (out->getStride().empty()) {
      // the first input of the output's shape lends its strides; a virtual output otherwise keeps
      // IN_0's memory format
      for (const auto &t : ins)
        if (t && t->getDim() == out->getDim()) {
          out->setStride(t->getStride());
          break;
        }
      if (out->getStride().empty() && out->isVirtual())
        out->setStride(generateStrideFromDim(
            out->getDim(), generateStrideOrderPreservingFormat(ins[0]->getStride(), out->getDim().size())));
      FUSILLI_RETURN_ERROR_IF(out->getStride().empty(), ErrorCode::InvalidAttribute,
                              "Pointwise output strides could not be computed");
    }
    return ok();
  }
  void describe(fb_node_desc &d, const TensorId &id) const override {
    detail::initDesc(d, FB_OP_POINTWISE);
    d.mode = static_cast<int32_t>(pointwiseAttr.getMode());
    d.inputs[0] = id(pointwiseAttr.getIN_0());
    d.inputs[1] = id(pointwiseAttr.getIN_1());
    d.inputs[2] = id(pointwiseAttr.getIN_2());
    d.outputs[0] = id(pointwiseAttr.getOUT_0());
    d.fparams[0] = pointwiseAttr.getEluAlpha();
    d.fparams[1] = pointwiseAttr.getSoftplusBeta();
    d.fparams[2] = pointwiseAttr.getSoftplusThreshold();
    d.fparams[3] = pointwiseAttr.getSwishBeta();
  }
};

// ---- batch normalisation (reference node/batchnorm_node.h:33-247) ------------------------------
class BatchNormNode : public INode {
public:
  BatchnormAttr batchnormAttr;
  BatchNormNode(BatchnormAttr &&a, const Context &ctx) : INode(ctx), batchnormAttr(std::move(a)) {}
  const std::string &getName() const override { return batchnormAttr.getName(); }
  Type getType() const override { return Type::BatchNorm; }
  bool isTrainingForwardPhase() const { return batchnormAttr.getForwardPhase() == NormFwdPhase::TRAINING; }

  ErrorObject preValidateNode() const override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Pre-Validating BatchNormNode '" << getName() << "'");
    const auto &a = batchnormAttr;
    FUSILLI_RETURN_ERROR_IF(a.getForwardPhase() == NormFwdPhase::NOT_SET, ErrorCode::AttributeNotSet,
                            "BatchNorm forward phase not set");
    TensorPtr x = a.getX(), y = a.getY();
    FUSILLI_RETURN_ERROR_IF(!x, ErrorCode::AttributeNotSet, "BatchNorm input tensor X not set");
    FUSILLI_RETURN_ERROR_IF(!y, ErrorCode::AttributeNotSet, "BatchNorm output tensor Y not set");
    FUSILLI_RETURN_ERROR_IF(x->getDim().size() < 2, ErrorCode::InvalidAttribute,
                            "BatchNorm input tensor X must have a rank of at least 2");
    FUSILLI_CHECK_ERROR(detail::requireLayout(x));
    if (!isTrainingForwardPhase()) {
      FUSILLI_RETURN_ERROR_IF(!a.getMEAN(), ErrorCode::AttributeNotSet, "BatchNorm inference requires running MEAN");
      FUSILLI_RETURN_ERROR_IF(!a.getVAR(), ErrorCode::AttributeNotSet, "BatchNorm inference requires running VAR");
      FUSILLI_RETURN_ERROR_IF(a.getSAVED_MEAN() != nullptr, ErrorCode::InvalidAttribute,
                              "BatchNorm SAVED_MEAN should not be set in inference mode");
      FUSILLI_RETURN_ERROR_IF(a.getSAVED_INV_VARIANCE() != nullptr, ErrorCode::InvalidAttribute,
                              "BatchNorm SAVED_INV_VARIANCE should not be set in inference mode");
    } else {
      FUSILLI_RETURN_ERROR_IF(!a.getSAVED_MEAN(), ErrorCode::AttributeNotSet,
                              "BatchNorm training requires SAVED_MEAN output");
      FUSILLI_RETURN_ERROR_IF(!a.getSAVED_INV_VARIANCE(), ErrorCode::AttributeNotSet,
                              "BatchNorm training requires SAVED_INV_VARIANCE output");
    }
    TensorPtr e = a.getEpsilon(), m = a.getMomentum();
    FUSILLI_RETURN_ERROR_IF(!e, ErrorCode::AttributeNotSet, "BatchNorm epsilon not set");
    FUSILLI_RETURN_ERROR_IF(!e->isScalar(), ErrorCode::InvalidAttribute, "BatchNorm epsilon must be a scalar constant");
    FUSILLI_RETURN_ERROR_IF(!m, ErrorCode::AttributeNotSet, "BatchNorm momentum not set");
    FUSILLI_RETURN_ERROR_IF(!m->isScalar(), ErrorCode::InvalidAttribute, "BatchNorm momentum must be a scalar constant");
    return ok();
  }
  ErrorObject inferPropertiesNode() override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Inferring properties for BatchNormNode '" << getName() << "'");
    auto &a = batchnormAttr;
    a.fillFromContext(context);
    TensorPtr x = a.getX(), y = a.getY();
    const std::vector<int64_t> perChannel = {x->getDim()[1]}, unit = {1};
    for (const TensorPtr &t : perChannelTensors()) {
      if (!t) continue;
      if (t->getDim().empty()) t->setDim(perChannel);
      if (t->getStride().empty()) t->setStride(unit);
    }
    if (y->getDim().empty()) y->setDim(x->getDim());
    if (y->getStride().empty()) y->setStride(x->getStride());
    return ok();
  }
  ErrorObject postValidateNode() const override {
    FUSILLI_LOG_LABEL_ENDL("INFO: Post-Validating BatchNormNode '" << getName() << "'");
    const auto &a = batchnormAttr;
    TensorPtr x = a.getX(), y = a.getY();
    FUSILLI_RETURN_ERROR_IF(x->getDim() != y->getDim(), ErrorCode::InvalidAttribute,
                            "BatchNorm output Y tensor must have the same shape as input X tensor");
    FUSILLI_CHECK_ERROR(detail::requireLayout(y));
    static const char *const names[] = {"SCALE", "BIAS", "MEAN", "VAR", "SAVED_MEAN", "SAVED_INV_VARIANCE"};
    const std::vector<int64_t> perChannel = {x->getDim()[1]}, unit = {1};
    const auto tensors = perChannelTensors();
    for (size_t i = 0; i < tensors.size(); ++i) {
      if (!tensors[i]) continue;
      FUSILLI_RETURN_ERROR_IF(tensors[i]->getDim() != perChannel, ErrorCode::InvalidAttribute,
                              std::string("BatchNorm tensor ") + names[i] +
                                  " must be 1D with size equal to channel dimension C");
      FUSILLI_RETURN_ERROR_IF(tensors[i]->getStride() != unit, ErrorCode::InvalidAttribute,
                              std::string("BatchNorm tensor ") + names[i] + " must have unit stride");
    }
    return ok();
  }
  void describe(fb_node_desc &d, const TensorId &id) const override {
    detail::initDesc(d, FB_OP_BATCHNORM);
    const auto &a = batchnormAttr;
    d.inputs[0] = id(a.getX());
    d.inputs[1] = id(a.getSCALE());
    d.inputs[2] = id(a.getBIAS());
    d.inputs[3] = id(a.getMEAN());
    d.inputs[4] = id(a.getVAR());
    d.inputs[5] = id(a.getEpsilon());
    d.outputs[0] = id(a.getY());
    d.outputs[1] = id(a.getSAVED_MEAN());
    d.outputs[2] = id(a.getSAVED_INV_VARIANCE());
    if (isTrainingForwardPhase()) d.flags |= FB_FLAG_NORM_TRAINING;
    // functional op: momentum reaches no output; kept in the plan for the record
    if (a.getMomentum()) d.fparams[0] = static_cast<float>(a.getMomentum()->scalarAsDouble());
  }

private:
  // SCALE, BIAS, MEAN, VAR and, in training, the two saved statistics: all [C] with unit stride
  std::vector<TensorPtr> perChannelTensors() const {
    const auto &a = batchnormAttr;
    std::vector<TensorPtr> t = {a.getSCALE(), a.getBIAS(), a.getMEAN(), a.getVAR()};
    if (isTrainingForwardPhase()) {
      t.push_back(a.getSAVED_MEAN());
      t.push_back(a.getSAVED_INV_VARIANCE());
    }
    return t;
  }
};

// ---- custom op (reference attributes/custom_op_attributes.h:23-110, node/custom_op_node.h) ------
// A node whose body is a piece of torch-dialect MLIR supplied by the user. The builders and
// validate() accept it as the reference does (its checks need no compiler); this backend has no
// MLIR compiler, so building a plan for a graph that holds one is refused with NotImplemented.
class CustomOpAttr {
public:
  CustomOpAttr &setName(const std::string &name) { name_ = name; return *this; }
  CustomOpAttr &setMlir(const std::string &mlir) { mlir_ = mlir; return *this; }
  CustomOpAttr &setNumOutputs(size_t n) { numOutputs_ = n; return *this; }
  const std::string &getName() const { return name_; }
  const std::string &getMlir() const { return mlir_; }
  size_t getNumOutputs() const { return numOutputs_; }

private:
  std::string name_, mlir_;
  size_t numOutputs_ = 0;
};

class CustomOpNode : public INode {
public:
  CustomOpAttr customOpAttr;
  std::vector<TensorPtr> inputs, outputs;
  CustomOpNode(CustomOpAttr &&a, const Context &ctx) : INode(ctx), customOpAttr(std::move(a)) {}
  const std::string &getName() const override { return customOpAttr.getName(); }
  Type getType() const override { return Type::Custom; }
  ErrorObject preValidateNode() const override {
    FUSILLI_RETURN_ERROR_IF(customOpAttr.getMlir().empty(), ErrorCode::AttributeNotSet, "CustomOp MLIR not set");
    FUSILLI_RETURN_ERROR_IF(inputs.empty(), ErrorCode::AttributeNotSet, "CustomOp inputs not set");
    FUSILLI_RETURN_ERROR_IF(outputs.empty(), ErrorCode::AttributeNotSet, "CustomOp outputs not set");
    for (size_t i = 0; i < inputs.size(); ++i) {
      FUSILLI_RETURN_ERROR_IF(!inputs[i], ErrorCode::AttributeNotSet, "CustomOp input " + std::to_string(i) + " is null");
      FUSILLI_RETURN_ERROR_IF(inputs[i]->isScalar(), ErrorCode::InvalidAttribute,
                              "CustomOp input " + std::to_string(i) + " is scalar (not supported)");
    }
    for (size_t i = 0; i < outputs.size(); ++i)
      FUSILLI_RETURN_ERROR_IF(outputs[i]->isScalar(), ErrorCode::InvalidAttribute,
                              "CustomOp output " + std::to_string(i) + " is scalar (not supported)");
    return ok();
  }
  ErrorObject inferPropertiesNode() override {
    for (auto &t : inputs) t->fillFromContext(context);
    return ok();
  }
};

} // namespace fusilli

#endif // FUSILLI_NODES_MORE_H

// TensorAttr: tensor metadata (name, dtype, logical dims, element strides, virtual / scalar
// flags) and the stride / layout algebra of the front end. Same names and behaviour as the
// reference's include/fusilli/attributes/tensor_attributes.h (stride helpers :159-254,
// computeBroadcastShape :334, TensorAttr :374-809) and include/fusilli/graph/context.h.
#ifndef FUSILLI_TENSOR_H
#define FUSILLI_TENSOR_H

#include <algorithm>
#include <cstdint>
#include <memory>
#include <numeric>
#include <optional>
#include <ranges>
#include <span>
#include <string>
#include <utility>
#include <variant>
#include <vector>

#include "error.h"
#include "types.h"

namespace fusilli {

// Graph-wide defaults that tensors and nodes inherit when they leave a field unset.
class Context {
public:
  Context &setIntermediateDataType(DataType t) { intermediate_ = t; return *this; }
  Context &setIODataType(DataType t) { io_ = t; return *this; }
  Context &setComputeDataType(DataType t) { compute_ = t; return *this; }
  Context &setName(const std::string &n) { name_ = n; return *this; }
  DataType getIODataType() const { return io_; }
  DataType getIntermediateDataType() const { return intermediate_; }
  DataType getComputeDataType() const { return compute_; }
  const std::string &getName() const { return name_; }

private:
  DataType compute_ = DataType::NotSet, intermediate_ = DataType::NotSet, io_ = DataType::NotSet;
  std::string name_;
};

// Rank of each dim in memory, 0 = fastest. Contiguous: last dim fastest.
inline std::vector<size_t> getContiguousStrideOrder(size_t rank) {
  std::vector<size_t> order(rank);
  for (size_t i = 0; i < rank; ++i) order[i] = rank - 1 - i;
  return order;
}

// Channels-last: dim 1 fastest, then the spatial dims from the last one, dim 0 slowest.
inline std::vector<size_t> getChannelsLastStrideOrder(size_t rank) {
  if (rank < 3) return getContiguousStrideOrder(rank);
  std::vector<size_t> order(rank, 0);
  size_t next = 1;
  for (size_t i = rank - 1; i > 1; --i) order[i] = next++;
  if (rank > 0) order[0] = next;
  if (rank > 1) order[1] = 0;
  return order;
}

// Stride order that keeps the memory ordering of `inputStride`, padded to `outputRank` dims.
inline std::vector<size_t> generateStrideOrderPreservingFormat(const std::vector<int64_t> &inputStride,
                                                               size_t outputRank) {
  std::vector<size_t> idx(inputStride.size());
  std::iota(idx.begin(), idx.end(), 0);
  std::stable_sort(idx.begin(), idx.end(), [&](size_t a, size_t b) { return inputStride[a] < inputStride[b]; });
  std::vector<size_t> order(std::max(outputRank, inputStride.size()));
  for (size_t r = 0; r < idx.size(); ++r) order[idx[r]] = r;
  for (size_t i = inputStride.size(); i < order.size(); ++i) order[i] = i;
  return order;
}

inline std::vector<int64_t> generateStrideFromDim(const std::vector<int64_t> &dim,
                                                  const std::vector<size_t> &strideOrder) {
  const size_t rank = dim.size();
  std::vector<size_t> byRank(rank);
  for (size_t i = 0; i < rank; ++i) byRank[strideOrder[i]] = i;
  std::vector<int64_t> stride(rank);
  int64_t acc = 1;
  for (size_t r = 0; r < rank; ++r) {
    stride[byRank[r]] = acc;
    acc *= dim[byRank[r]];
  }
  return stride;
}

inline ErrorOr<std::vector<int64_t>> generateStrideFromLayout(const std::vector<int64_t> &dims,
                                                              const std::string &layout) {
  FUSILLI_RETURN_ERROR_IF(dims.size() != layout.size(), ErrorCode::InvalidArgument,
                          "Invalid input dimensions and layout: they must have the same rank");
  if (layout == "NHC" || layout == "NHWC" || layout == "NDHWC")
    return ok(generateStrideFromDim(dims, getChannelsLastStrideOrder(dims.size())));
  if (layout == "N" || layout == "NC" || layout == "NCH" || layout == "NCHW" || layout == "NCDHW")
    return ok(generateStrideFromDim(dims, getContiguousStrideOrder(dims.size())));
  return error(ErrorCode::InvalidArgument, "Invalid layout string: " + layout);
}

// Permutations between the two supported memory formats, as dimension orders
// (reference attributes/tensor_attributes.h:274-311).
inline std::vector<int64_t> getPreserveContiguousPermuteOrder(size_t numDims) {
  std::vector<int64_t> p(numDims);
  std::iota(p.begin(), p.end(), 0);
  return p;
}
inline std::vector<int64_t> getChannelsLastToContiguousPermuteOrder(size_t numDims) {
  // N, then the spatial dims, then C
  std::vector<int64_t> p(numDims);
  p[0] = 0;
  for (size_t i = 2; i < numDims; ++i) p[i] = static_cast<int64_t>(i - 1);
  p[1] = static_cast<int64_t>(numDims - 1);
  return p;
}
inline std::vector<int64_t> getContiguousToChannelsLastPermuteOrder(size_t numDims) {
  // N, then C moved to the end of the spatial dims
  std::vector<int64_t> p(numDims);
  p[0] = 0;
  p[numDims - 1] = 1;
  for (size_t i = 1; i + 1 < numDims; ++i) p[i] = static_cast<int64_t>(i + 1);
  return p;
}

// Any range of integers convertible to int64_t that is not already a std::vector<int64_t>.
template <typename R>
concept Int64Range = std::ranges::input_range<R> &&
                     std::convertible_to<std::ranges::range_value_t<R>, int64_t> &&
                     !std::same_as<std::remove_cvref_t<R>, std::vector<int64_t>>;

inline std::vector<int64_t> inversePermutation(const std::vector<int64_t> &perm) {
  std::vector<int64_t> inv(perm.size());
  for (size_t i = 0; i < perm.size(); ++i) inv[perm[i]] = static_cast<int64_t>(i);
  return inv;
}

// Right-aligned (PyTorch-style) broadcast of a set of shapes.
inline ErrorOr<std::vector<int64_t>> computeBroadcastShape(const std::vector<std::vector<int64_t>> &shapes) {
  size_t rank = 0;
  for (const auto &s : shapes) rank = std::max(rank, s.size());
  FUSILLI_RETURN_ERROR_IF(rank == 0, ErrorCode::InvalidAttribute, "All input shapes are empty");
  std::vector<int64_t> out(rank, 1);
  for (const auto &s : shapes) {
    for (size_t off = 0; off < s.size(); ++off) {
      int64_t &o = out[rank - 1 - off];
      const int64_t d = s[s.size() - 1 - off];
      if (o == 1) o = d;
      FUSILLI_RETURN_ERROR_IF(d != 1 && o != d, ErrorCode::InvalidAttribute,
                              "Cannot broadcast two non unit dimensions");
    }
  }
  return ok(std::move(out));
}

class TensorAttr {
public:
  using scalar_t = std::variant<int64_t, int32_t, float, double>;

  TensorAttr() = default;
  explicit TensorAttr(float v) { initScalar(v, DataType::Float); }
  explicit TensorAttr(double v) { initScalar(v, DataType::Double); }
  explicit TensorAttr(int32_t v) { initScalar(v, DataType::Int32); }
  explicit TensorAttr(int64_t v) { initScalar(v, DataType::Int64); }

  // setters (chainable)
  TensorAttr &setName(const std::string &n) { name_ = n; return *this; }
  TensorAttr &setDataType(DataType t) { dtype_ = t; return *this; }
  TensorAttr &setDim(const std::vector<int64_t> &d) { dim_ = d; return *this; }
  TensorAttr &setStride(const std::vector<int64_t> &s) { stride_ = s; return *this; }
  template <Int64Range R> TensorAttr &setDim(R &&d) { dim_.assign(d.begin(), d.end()); return *this; }
  template <Int64Range R> TensorAttr &setStride(R &&s) { stride_.assign(s.begin(), s.end()); return *this; }
  // Dynamic dims are part of the reference's tensor description (tensor_attributes.h:512-570);
  // the B200 backend builds plans for static shapes only and refuses graphs that use them.
  TensorAttr &setDynamicDim(size_t index) {
    dynamic_.push_back(index);
    canonicalizeDynamicDims();
    return *this;
  }
  TensorAttr &setDynamicDims(std::span<const size_t> indices) {
    dynamic_.assign(indices.begin(), indices.end());
    canonicalizeDynamicDims();
    return *this;
  }
  TensorAttr &setDynamicDims(std::initializer_list<size_t> indices) {
    return setDynamicDims(std::span<const size_t>(indices.begin(), indices.size()));
  }
  TensorAttr &clearDynamicDims() { dynamic_.clear(); return *this; }
  TensorAttr &setIsVirtual(bool v) { virtual_ = v; return *this; }
  TensorAttr &setOutput(bool isOutput) { return setIsVirtual(!isOutput); }
  TensorAttr &setIsScalar(bool v) { scalar_ = v; return *this; }

  // getters
  const std::string &getName() const { return name_; }
  DataType getDataType() const { return dtype_; }
  const std::vector<int64_t> &getDim() const { return dim_; }
  const std::vector<int64_t> &getStride() const { return stride_; }
  bool isVirtual() const { return virtual_; }
  bool isScalar() const { return scalar_; }
  bool isDynamicDim(size_t index) const { return std::binary_search(dynamic_.begin(), dynamic_.end(), index); }
  bool hasDynamicDims() const { return !dynamic_.empty(); }
  const std::vector<size_t> &getDynamicDims() const { return dynamic_; }
  std::optional<scalar_t> getScalarValue() const { return value_; }
  double scalarAsDouble() const {
    return value_ ? std::visit([](auto v) { return static_cast<double>(v); }, *value_) : 0.0;
  }

  int64_t getVolume() const {
    int64_t v = 1;
    for (int64_t d : dim_) v *= d;
    return v;
  }
  bool isContiguous() const {
    return !dim_.empty() && stride_ == generateStrideFromDim(dim_, getContiguousStrideOrder(dim_.size()));
  }
  bool isChannelsLast() const {
    return dim_.size() >= 3 && stride_ == generateStrideFromDim(dim_, getChannelsLastStrideOrder(dim_.size()));
  }
  bool hasBroadcastDims() const {
    for (size_t i = 0; i < dim_.size() && i < stride_.size(); ++i)
      if (dim_[i] > 1 && stride_[i] == 0) return true;
    return false;
  }
  std::vector<int64_t> getUnexpandedDim() const {
    std::vector<int64_t> d = dim_;
    for (size_t i = 0; i < d.size() && i < stride_.size(); ++i)
      if (d[i] > 1 && stride_[i] == 0) d[i] = 1;
    return d;
  }

  // True when the strides describe a dense permutation of the dims (unit and broadcast dims
  // do not take part).
  bool hasValidPhysicalRepresentation() const {
    if (dim_.size() != stride_.size()) return false;
    std::vector<std::pair<int64_t, int64_t>> sd;
    for (size_t i = 0; i < dim_.size(); ++i) {
      if (stride_[i] < 0) return false;
      sd.emplace_back(stride_[i], dim_[i]);
    }
    std::stable_sort(sd.begin(), sd.end(), [](const auto &a, const auto &b) { return a.first < b.first; });
    int64_t expect = 1;
    for (const auto &[s, d] : sd) {
      if (d == 1 || s == 0) continue;
      if (s != expect) return false;
      expect = s * d;
    }
    return true;
  }

  // perm[i] = logical dim stored at physical position i; unit and broadcast dims stay put.
  std::vector<int64_t> getLogicalToPhysicalPermuteOrder() const {
    const size_t rank = dim_.size();
    std::vector<int64_t> perm(rank);
    std::iota(perm.begin(), perm.end(), 0);
    std::vector<size_t> movable;
    for (size_t i = 0; i < rank; ++i)
      if (dim_[i] != 1 && stride_[i] != 0) movable.push_back(i);
    std::vector<size_t> byStride = movable;
    std::stable_sort(byStride.begin(), byStride.end(), [&](size_t a, size_t b) { return stride_[a] > stride_[b]; });
    for (size_t k = 0; k < movable.size(); ++k) perm[movable[k]] = static_cast<int64_t>(byStride[k]);
    return perm;
  }
  std::vector<int64_t> getPhysicalToLogicalPermuteOrder() const {
    return inversePermutation(getLogicalToPhysicalPermuteOrder());
  }
  // Dims of the dense buffer that backs the tensor (broadcast dims collapse to 1).
  std::vector<int64_t> getPhysicalDim() const {
    const auto perm = getLogicalToPhysicalPermuteOrder();
    std::vector<int64_t> phys(perm.size());
    for (size_t i = 0; i < perm.size(); ++i) {
      const size_t src = static_cast<size_t>(perm[i]);
      phys[i] = (dim_[src] > 1 && stride_[src] == 0) ? 1 : dim_[src];
    }
    return phys;
  }

  TensorAttr &fillFromContext(const Context &ctx) {
    if (dtype_ == DataType::NotSet) dtype_ = virtual_ ? ctx.getIntermediateDataType() : ctx.getIODataType();
    return *this;
  }

  ErrorObject validate() const {
    const std::string who = "Tensor '" + name_ + "'";
    FUSILLI_RETURN_ERROR_IF(dim_.empty(), ErrorCode::AttributeNotSet, who + " dims not set");
    FUSILLI_RETURN_ERROR_IF(stride_.empty(), ErrorCode::AttributeNotSet, who + " strides not set");
    FUSILLI_RETURN_ERROR_IF(dim_.size() != stride_.size(), ErrorCode::InvalidAttribute,
                            who + " uses dim and stride of different dimensionality");
    for (size_t d : dynamic_) {
      FUSILLI_RETURN_ERROR_IF(d >= dim_.size(), ErrorCode::InvalidAttribute,
                              who + " has dynamic dim index " + std::to_string(d) + " out of range for rank " +
                                  std::to_string(dim_.size()));
      FUSILLI_RETURN_ERROR_IF(stride_[d] == 0, ErrorCode::InvalidAttribute,
                              who + " has dynamic dim at index " + std::to_string(d) +
                                  " with stride 0 (broadcast stride), which is not supported");
      FUSILLI_RETURN_ERROR_IF(dim_[d] == 1, ErrorCode::InvalidAttribute,
                              who + " has dynamic dim at index " + std::to_string(d) +
                                  " with representative size 1, which is not supported");
    }
    FUSILLI_RETURN_ERROR_IF(hasBroadcastDims() && hasDynamicDims(), ErrorCode::InvalidAttribute,
                            who + " has dynamic dimensions on a tensor with broadcast strides, which is not "
                                  "supported");
    FUSILLI_RETURN_ERROR_IF(!hasValidPhysicalRepresentation(), ErrorCode::InvalidAttribute,
                            who + " has invalid physical representation. It must be a valid "
                                  "permutation of the logical dimensions");
    FUSILLI_RETURN_ERROR_IF(dtype_ == DataType::NotSet, ErrorCode::AttributeNotSet, who + " data type not set");
    FUSILLI_RETURN_ERROR_IF(virtual_ && scalar_, ErrorCode::InvalidAttribute,
                            who + " cannot be both virtual (intermediate) and a scalar constant");
    FUSILLI_RETURN_ERROR_IF(value_.has_value() && !scalar_, ErrorCode::InvalidAttribute,
                            who + " has a scalar value set but is not marked as a scalar");
    FUSILLI_RETURN_ERROR_IF(!value_.has_value() && scalar_, ErrorCode::InvalidAttribute,
                            who + " is marked as a scalar but does not have a scalar value set");
    return ok();
  }

private:
  template <typename V> void initScalar(V v, DataType t) {
    value_ = v;
    scalar_ = true;
    dim_ = stride_ = {1};
    dtype_ = t;
  }
  std::string name_;
  DataType dtype_ = DataType::NotSet;
  std::vector<int64_t> dim_, stride_;
  std::vector<size_t> dynamic_;
  void canonicalizeDynamicDims() {
    std::sort(dynamic_.begin(), dynamic_.end());
    dynamic_.erase(std::unique(dynamic_.begin(), dynamic_.end()), dynamic_.end());
  }
  bool virtual_ = false, scalar_ = false;
  std::optional<scalar_t> value_;
};

struct TensorAttrSortByName {
  bool operator()(const std::shared_ptr<TensorAttr> &a, const std::shared_ptr<TensorAttr> &b) const {
    return a->getName() < b->getName();
  }
};

} // namespace fusilli

#endif // FUSILLI_TENSOR_H

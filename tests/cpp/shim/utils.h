// Test helpers with the names the reference's samples and tests expect from their
// `utils.h` (reference tests/utils.h): FUSILLI_REQUIRE_OK / FUSILLI_REQUIRE_ASSIGN,
// castToSizeT, kDefaultBackend, allocateBufferOfType, allocateWorkspace. The default backend
// of this build is Backend::CUDA.
#ifndef FUSILLI_B200_TESTS_UTILS_H
#define FUSILLI_B200_TESTS_UTILS_H

#include <fusilli.h>

#include <catch2/catch_test_macros.hpp>

#include <cstdint>
#include <functional>
#include <memory>
#include <optional>
#include <span>
#include <vector>

// Runs a clean-up callback when the scope ends, also when a REQUIRE aborts the test case.
class [[nodiscard]] ScopeExit {
public:
  explicit ScopeExit(std::function<void()> &&f) : fn_(std::move(f)) {}
  ScopeExit(ScopeExit &&o) noexcept : fn_(std::move(o.fn_)) { o.release(); }
  ScopeExit(const ScopeExit &) = delete;
  ScopeExit &operator=(const ScopeExit &) = delete;
  ScopeExit &operator=(ScopeExit &&) = delete;
  void release() { fn_ = nullptr; }
  ~ScopeExit() {
    if (fn_) fn_();
  }

private:
  std::function<void()> fn_;
};

#define FUSILLI_REQUIRE_OK(expr)                                                                     \
  do {                                                                                               \
    const fusilli::ErrorObject fusilli_req_err = (expr);                                             \
    if (fusilli::isError(fusilli_req_err)) std::cerr << "  " << fusilli_req_err << std::endl;        \
    REQUIRE(fusilli::isOk(fusilli_req_err));                                                         \
  } while (false)

#define FUSILLI_REQUIRE_ASSIGN_IMPL(tmp, decl, expr)                                                 \
  auto tmp = (expr);                                                                                 \
  FUSILLI_REQUIRE_OK(tmp);                                                                           \
  decl = std::move(*tmp);
#define FUSILLI_REQUIRE_ASSIGN(decl, expr) FUSILLI_REQUIRE_ASSIGN_IMPL(FUSILLI_ERROR_VAR(_errorOr), decl, expr)

inline std::vector<size_t> castToSizeT(const std::vector<int64_t> &v) { return std::vector<size_t>(v.begin(), v.end()); }

namespace fusilli {

constexpr Backend kDefaultBackend = Backend::CUDA;

template <typename T>
inline ErrorOr<std::shared_ptr<Buffer>> allocateBufferOfType(Handle &handle, const std::shared_ptr<TensorAttr> &tensor,
                                                            const std::vector<T> &data) {
  FUSILLI_RETURN_ERROR_IF(!tensor, ErrorCode::AttributeNotSet, "Tensor is not set");
  FUSILLI_ASSIGN_OR_RETURN(auto buf, Buffer::allocate(handle, castToSizeT(tensor->getPhysicalDim()), data));
  return ok(std::make_shared<Buffer>(std::move(buf)));
}

// A buffer shaped like `tensor`, every element set to `initVal` converted to `type`.
inline ErrorOr<std::shared_ptr<Buffer>> allocateBufferOfType(Handle &handle, const std::shared_ptr<TensorAttr> &tensor,
                                                            DataType type, double initVal) {
  FUSILLI_RETURN_ERROR_IF(!tensor, ErrorCode::AttributeNotSet, "Tensor is not set");
  const size_t n = static_cast<size_t>(tensor->getVolume());
  switch (type) {
  case DataType::Float: return allocateBufferOfType(handle, tensor, std::vector<float>(n, float(initVal)));
  case DataType::Int32: return allocateBufferOfType(handle, tensor, std::vector<int32_t>(n, int32_t(initVal)));
  case DataType::Int64: return allocateBufferOfType(handle, tensor, std::vector<int64_t>(n, int64_t(initVal)));
  case DataType::Half: return allocateBufferOfType(handle, tensor, std::vector<half>(n, half(initVal)));
  case DataType::BFloat16: return allocateBufferOfType(handle, tensor, std::vector<bf16>(n, bf16(initVal)));
  case DataType::Int16: return allocateBufferOfType(handle, tensor, std::vector<int16_t>(n, int16_t(initVal)));
  case DataType::Int8:
  case DataType::Boolean: return allocateBufferOfType(handle, tensor, std::vector<int8_t>(n, int8_t(initVal)));
  case DataType::Uint8: return allocateBufferOfType(handle, tensor, std::vector<uint8_t>(n, uint8_t(initVal)));
  case DataType::Int4: return allocateBufferOfType(handle, tensor, std::vector<int4>(n, int4(int8_t(initVal))));
  default: return error(ErrorCode::InvalidAttribute, "Unsupported DataType");
  }
}

inline ErrorOr<std::shared_ptr<Buffer>> allocateWorkspace(const Handle &handle, std::optional<size_t> workspaceSize) {
  if (!workspaceSize.has_value() || *workspaceSize == 0) return ok(std::shared_ptr<Buffer>(nullptr));
  FUSILLI_ASSIGN_OR_RETURN(auto buf, Buffer::allocateRaw(handle, *workspaceSize));
  return ok(std::make_shared<Buffer>(std::move(buf)));
}

inline TensorAttr createTestTensorAttr(const std::string &name, std::span<const int64_t> dim) {
  std::vector<int64_t> d(dim.begin(), dim.end());
  TensorAttr t;
  t.setName(name).setDim(d).setStride(generateStrideFromDim(d, getContiguousStrideOrder(d.size())));
  return t;
}

inline std::shared_ptr<TensorAttr> createTestTensor(const std::string &name, std::span<const int64_t> dim, Graph *graph) {
  return graph->tensor(createTestTensorAttr(name, dim));
}

} // namespace fusilli

#endif // FUSILLI_B200_TESTS_UTILS_H

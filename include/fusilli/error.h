// Error-as-value plumbing and the env-driven logger of the Fusilli front end.
//
// Same public names and behaviour as the reference's
// include/fusilli/support/logging.h (ErrorCode :58-71, ErrorObject :88,
// ErrorOr<T> :150, FUSILLI_RETURN_ERROR_IF :383, FUSILLI_CHECK_ERROR :407,
// FUSILLI_ASSIGN_OR_RETURN :468, FUSILLI_LOG_INFO / FUSILLI_LOG_FILE :294-332),
// written against the C ABI's status codes instead of iree_status_t.
#ifndef FUSILLI_ERROR_H
#define FUSILLI_ERROR_H

#include <cstdint>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <optional>
#include <string>
#include <type_traits>
#include <utility>

namespace fusilli {

enum class [[nodiscard]] ErrorCode : uint8_t {
  OK = 0,
  NotImplemented,
  NotValidated,
  NotCompiled,
  AttributeNotSet,
  InternalError,
  InvalidAttribute,
  InvalidArgument,
  VariantPackError,
  CompileFailure,
  RuntimeFailure,
  FileSystemFailure,
};

inline const char *errorCodeName(ErrorCode c) {
  switch (c) {
  case ErrorCode::OK: return "OK";
  case ErrorCode::NotImplemented: return "NOT_IMPLEMENTED";
  case ErrorCode::NotValidated: return "NOT_VALIDATED";
  case ErrorCode::NotCompiled: return "NOT_COMPILED";
  case ErrorCode::AttributeNotSet: return "ATTRIBUTE_NOT_SET";
  case ErrorCode::InternalError: return "INTERNAL_ERROR";
  case ErrorCode::InvalidAttribute: return "INVALID_ATTRIBUTE";
  case ErrorCode::InvalidArgument: return "INVALID_ARGUMENT";
  case ErrorCode::VariantPackError: return "VARIANT_PACK_ERROR";
  case ErrorCode::CompileFailure: return "COMPILE_FAILURE";
  case ErrorCode::RuntimeFailure: return "RUNTIME_FAILURE";
  case ErrorCode::FileSystemFailure: return "FILE_SYSTEM_FAILURE";
  }
  return "UNKNOWN_ERROR_CODE";
}

struct [[nodiscard]] ErrorObject {
  ErrorCode code = ErrorCode::OK;
  std::string errMsg;

  ErrorObject() = default;
  ErrorObject(ErrorCode c, std::string msg) : code(c), errMsg(std::move(msg)) {}

  ErrorCode getCode() const { return code; }
  const std::string &getMessage() const { return errMsg; }
  bool isOk() const { return code == ErrorCode::OK; }
  bool isError() const { return !isOk(); }
  bool operator==(ErrorCode other) const { return code == other; }
  bool operator!=(ErrorCode other) const { return code != other; }
};

inline bool isOk(const ErrorObject &e) { return e.isOk(); }
inline bool isError(const ErrorObject &e) { return e.isError(); }
inline ErrorObject ok() { return {}; }
inline ErrorObject error(ErrorCode c, std::string msg) { return ErrorObject(c, std::move(msg)); }

// Either a T or the error that prevented producing one.
template <typename T> class [[nodiscard]] ErrorOr {
public:
  template <typename U>
    requires std::is_constructible_v<T, U &&> && (!std::is_same_v<std::decay_t<U>, ErrorObject>) &&
             (!std::is_same_v<std::decay_t<U>, ErrorOr<T>>)
  ErrorOr(U &&value) : value_(std::in_place, std::forward<U>(value)) {}
  ErrorOr(ErrorObject err) : err_(std::move(err)) {}
  template <typename U>
    requires std::is_constructible_v<T, U>
  ErrorOr(ErrorOr<U> &&other) {
    if (other.hasValue()) value_.emplace(std::move(*other));
    else err_ = ErrorObject(other);
  }
  ErrorOr(ErrorOr &&) noexcept = default;
  ErrorOr(const ErrorOr &) = delete;
  ErrorOr &operator=(const ErrorOr &) = delete;

  operator ErrorObject() const { return value_ ? ErrorObject() : err_; }
  bool hasValue() const { return value_.has_value(); }

  T &operator*() { check(); return *value_; }
  const T &operator*() const { check(); return *value_; }
  T *operator->() { check(); return &*value_; }
  const T *operator->() const { check(); return &*value_; }

private:
  void check() const {
    if (!value_) {
      std::cerr << "ErrorOr<T> dereferenced while holding an error: " << errorCodeName(err_.code) << ": "
                << err_.errMsg << std::endl;
      std::abort();
    }
  }
  std::optional<T> value_;
  ErrorObject err_;
  template <typename U> friend class ErrorOr;
};

template <typename T> inline bool isOk(const ErrorOr<T> &e) { return e.hasValue(); }
template <typename T> inline bool isError(const ErrorOr<T> &e) { return !e.hasValue(); }
template <typename T> inline auto ok(T &&v) { return ErrorOr<std::decay_t<T>>(std::forward<T>(v)); }

inline std::ostream &operator<<(std::ostream &os, ErrorCode c) { return os << errorCodeName(c); }
inline std::ostream &operator<<(std::ostream &os, const ErrorObject &e) {
  return os << e.getCode() << ": " << e.getMessage();
}
template <typename T> inline std::ostream &operator<<(std::ostream &os, const ErrorOr<T> &e) {
  return os << ErrorObject(e);
}

// ---- logging: FUSILLI_LOG_INFO=1 enables, FUSILLI_LOG_FILE=stdout|stderr|<path> ------------
inline bool &isLoggingEnabled() {
  static bool enabled = [] {
    const char *v = std::getenv("FUSILLI_LOG_INFO");
    return v && v[0] != '\0' && v[0] != '0';
  }();
  return enabled;
}

inline std::ostream &getStream() {
  static std::ofstream file;
  static std::ostream *stream = [] () -> std::ostream * {
    const char *dest = std::getenv("FUSILLI_LOG_FILE");
    if (!dest) {
      isLoggingEnabled() = false;
      return &std::cout;
    }
    std::string d(dest);
    if (d == "stdout") return &std::cout;
    if (d == "stderr") return &std::cerr;
    file.open(d, std::ios::out);
    return &file;
  }();
  return *stream;
}

class ConditionalStreamer {
public:
  explicit ConditionalStreamer(std::ostream &s) : stream_(s) {}
  template <typename T> const ConditionalStreamer &operator<<(const T &t) const {
    if (isLoggingEnabled()) stream_ << t;
    return *this;
  }
  const ConditionalStreamer &operator<<(std::ostream &(*manip)(std::ostream &)) const {
    if (isLoggingEnabled()) stream_ << manip;
    return *this;
  }

private:
  std::ostream &stream_;
};

inline ConditionalStreamer &getLogger() {
  static ConditionalStreamer logger(getStream());
  return logger;
}

} // namespace fusilli

#define FUSILLI_COLOR_RED "\033[31m"
#define FUSILLI_COLOR_GREEN "\033[32m"
#define FUSILLI_COLOR_YELLOW "\033[33m"
#define FUSILLI_COLOR_RESET "\033[0m"

#define FUSILLI_LOG(X) fusilli::getLogger() << X
#define FUSILLI_LOG_ENDL(X) fusilli::getLogger() << X << std::endl
#define FUSILLI_LOG_LABEL_RED(X) fusilli::getLogger() << FUSILLI_COLOR_RED << "[FUSILLI] " << X << FUSILLI_COLOR_RESET
#define FUSILLI_LOG_LABEL_GREEN(X) fusilli::getLogger() << FUSILLI_COLOR_GREEN << "[FUSILLI] " << X << FUSILLI_COLOR_RESET
#define FUSILLI_LOG_LABEL_YELLOW(X) fusilli::getLogger() << FUSILLI_COLOR_YELLOW << "[FUSILLI] " << X << FUSILLI_COLOR_RESET
#define FUSILLI_LOG_LABEL_ENDL(X) fusilli::getLogger() << "[FUSILLI] " << X << std::endl

#define FUSILLI_RETURN_ERROR_IF(cond, retval, message)                                              \
  do {                                                                                              \
    if (cond) {                                                                                     \
      FUSILLI_LOG_LABEL_RED("ERROR: ");                                                             \
      FUSILLI_LOG_ENDL(retval << ": " << message << ": (" << #cond ") at " << __FILE__ << ":" << __LINE__); \
      return fusilli::error(retval, message);                                                       \
    }                                                                                               \
  } while (false)

#define FUSILLI_CHECK_ERROR(expr)                                                                   \
  do {                                                                                              \
    fusilli::ErrorObject _fusilli_err = (expr);                                                     \
    if (fusilli::isError(_fusilli_err)) {                                                           \
      FUSILLI_LOG_LABEL_RED("ERROR: " << _fusilli_err << " ");                                      \
      FUSILLI_LOG_ENDL(#expr << " at " << __FILE__ << ":" << __LINE__);                             \
      return _fusilli_err;                                                                          \
    }                                                                                               \
  } while (false)

#define FUSILLI_CONCAT_IMPL(a, b, c) a##_##b##_##c
#define FUSILLI_CONCAT(a, b, c) FUSILLI_CONCAT_IMPL(a, b, c)
#define FUSILLI_ERROR_VAR(name) FUSILLI_CONCAT(name, __LINE__, __COUNTER__)

#define FUSILLI_ASSIGN_OR_RETURN_IMPL(tmp, decl, expr)                                              \
  auto tmp = (expr);                                                                                \
  if (fusilli::isError(tmp)) {                                                                      \
    FUSILLI_LOG_LABEL_RED("ERROR: " << tmp << " ");                                                 \
    FUSILLI_LOG_ENDL(#expr << " at " << __FILE__ << ":" << __LINE__);                               \
    return fusilli::ErrorObject(tmp);                                                               \
  }                                                                                                 \
  decl = std::move(*tmp);

#define FUSILLI_ASSIGN_OR_RETURN(decl, expr) FUSILLI_ASSIGN_OR_RETURN_IMPL(FUSILLI_ERROR_VAR(_errorOr), decl, expr)

#endif // FUSILLI_ERROR_H

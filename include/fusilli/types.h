// Element types of the Fusilli front end (reference include/fusilli/attributes/types.h:27-47,
// include/fusilli/support/float_types.h:101-102). Numbering equals the FB_DT_* values of the C ABI.
#ifndef FUSILLI_TYPES_H
#define FUSILLI_TYPES_H

#include <cstddef>
#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

namespace fusilli {

enum class DataType : uint8_t {
  NotSet = 0,
  Half,
  BFloat16,
  Float,
  Double,
  Uint8,
  Int4,
  Int8,
  Int16,
  Int32,
  Int64,
  Boolean,
  FP8E5M2,
};

// Native 16-bit float types, as in the reference on Linux.
using half = _Float16;
using bf16 = __bf16;

// Signed 4-bit integer element (reference include/fusilli/support/int_types.h:26-88): values
// clamp to [-8, 7] on construction; in device buffers two elements share a byte, element 2k in
// the low half of byte k.
struct Int4 {
  static constexpr unsigned kBitWidth = 4;
  constexpr Int4() = default;
  Int4(int8_t v) : bits_(static_cast<uint8_t>((v < -8 ? -8 : (v > 7 ? 7 : v)) & 0x0F)) {}
  [[nodiscard]] constexpr uint8_t toBits() const { return bits_; }
  [[nodiscard]] constexpr int8_t toInt() const {
    return static_cast<int8_t>(bits_ & 0x08 ? static_cast<int>(bits_) - 16 : static_cast<int>(bits_));
  }
  [[nodiscard]] operator int8_t() const { return toInt(); }
  [[nodiscard]] static constexpr Int4 fromBits(uint8_t bits) {
    Int4 r;
    r.bits_ = bits & 0x0F;
    return r;
  }
  static std::vector<uint8_t> pack(const std::vector<Int4> &elements) {
    std::vector<uint8_t> bytes((elements.size() + 1) / 2, 0);
    for (size_t i = 0; i < elements.size(); ++i) bytes[i >> 1] |= static_cast<uint8_t>(elements[i].toBits() << (4 * (i & 1)));
    return bytes;
  }
  static std::vector<Int4> unpack(const uint8_t *bytes, size_t count) {
    std::vector<Int4> elements(count);
    for (size_t i = 0; i < count; ++i) elements[i] = fromBits(static_cast<uint8_t>(bytes[i >> 1] >> (4 * (i & 1))));
    return elements;
  }

private:
  uint8_t bits_ = 0;
};
using int4 = Int4;
template <typename T> inline constexpr bool kIsSubByteElement = false;
template <> inline constexpr bool kIsSubByteElement<Int4> = true;

inline bool isIntegerType(DataType t) {
  switch (t) {
  case DataType::Uint8:
  case DataType::Int4:
  case DataType::Int8:
  case DataType::Int16:
  case DataType::Int32:
  case DataType::Int64: return true;
  default: return false;
  }
}
inline bool isIntegralOrBoolType(DataType t) { return isIntegerType(t) || t == DataType::Boolean; }

// Storage bytes per element; 0 for types the B200 backend has no kernels for.
inline size_t dataTypeSize(DataType t) {
  switch (t) {
  case DataType::Half:
  case DataType::BFloat16:
  case DataType::Int16: return 2;
  case DataType::Float:
  case DataType::Int32: return 4;
  case DataType::Double:
  case DataType::Int64: return 8;
  case DataType::Uint8:
  case DataType::Int8:
  case DataType::Boolean:
  case DataType::FP8E5M2: return 1;
  default: return 0;
  }
}

inline const char *dataTypeName(DataType t) {
  static const char *names[] = {"notset", "f16",  "bf16", "f32",  "f64", "ui8",   "si4",
                                "si8",    "si16", "si32", "si64", "i1",  "f8E5M2"};
  return names[static_cast<int>(t)];
}

// DataType -> short type spelling, under the name the reference's samples use to build graph
// names (attributes/types.h:67).
inline const std::unordered_map<DataType, std::string> kDataTypeToMlirTypeAsm = [] {
  std::unordered_map<DataType, std::string> m;
  for (int i = 1; i <= static_cast<int>(DataType::FP8E5M2); ++i)
    m.emplace(static_cast<DataType>(i), dataTypeName(static_cast<DataType>(i)));
  return m;
}();

// C++ element type -> DataType, used by Buffer::allocate / read.
template <typename T> struct DataTypeOf;
template <> struct DataTypeOf<float> { static constexpr DataType value = DataType::Float; };
template <> struct DataTypeOf<double> { static constexpr DataType value = DataType::Double; };
template <> struct DataTypeOf<half> { static constexpr DataType value = DataType::Half; };
template <> struct DataTypeOf<bf16> { static constexpr DataType value = DataType::BFloat16; };
template <> struct DataTypeOf<int32_t> { static constexpr DataType value = DataType::Int32; };
template <> struct DataTypeOf<int64_t> { static constexpr DataType value = DataType::Int64; };
template <> struct DataTypeOf<int16_t> { static constexpr DataType value = DataType::Int16; };
template <> struct DataTypeOf<int8_t> { static constexpr DataType value = DataType::Int8; };
template <> struct DataTypeOf<uint8_t> { static constexpr DataType value = DataType::Uint8; };
template <> struct DataTypeOf<bool> { static constexpr DataType value = DataType::Boolean; };
template <> struct DataTypeOf<Int4> { static constexpr DataType value = DataType::Int4; };

} // namespace fusilli

#endif // FUSILLI_TYPES_H

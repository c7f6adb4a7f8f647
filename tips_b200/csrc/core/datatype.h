// Element types understood by the runtime, typed spans and the type-erased
// vector used as the parameter-server value / gradient type.
//
// Capability parity with the reference:
//   Datatype        tips/core/common/datatype.h:7-24  (fp32/fp64/int32/int64/int8/uint8;
//                   here also bf16 and fp16, and DatatypeNumBytes covers every member)
//   Vec<T>          tips/core/common/vec.h:13-259     (non-owning span, elementwise math, dot,
//                   text form "Vec:\t" + "<elem> " per element, vec.h:85-101)
//   AnyVec          tips/core/common/any_vec.h:12-184 (owning or borrowing, Copy/ShadowCopy,
//                   typed views, dtype-dispatched Mul/Add)
#pragma once

#include <cmath>
#include <cstdint>
#include <cstring>
#include <sstream>
#include <string>

#include "core/logging.h"

namespace tips {

// The numeric values are part of the wire and checkpoint formats.
enum class Datatype : int32_t {
  kUnknown = -1,
  kFp32    = 0,
  kFp64    = 1,
  kInt32   = 2,
  kInt64   = 3,
  kInt8    = 4,
  kUInt8   = 5,
  kBf16    = 6,
  kFp16    = 7,
};

const char* DatatypeName(Datatype t);
size_t DatatypeNumBytes(Datatype t);
Datatype DatatypeFromName(const std::string& name);

template <typename T>
struct DatatypeOf;
template <>
struct DatatypeOf<float> {
  static constexpr Datatype value = Datatype::kFp32;
};
template <>
struct DatatypeOf<double> {
  static constexpr Datatype value = Datatype::kFp64;
};
template <>
struct DatatypeOf<int32_t> {
  static constexpr Datatype value = Datatype::kInt32;
};
template <>
struct DatatypeOf<int64_t> {
  static constexpr Datatype value = Datatype::kInt64;
};
template <>
struct DatatypeOf<int8_t> {
  static constexpr Datatype value = Datatype::kInt8;
};
template <>
struct DatatypeOf<uint8_t> {
  static constexpr Datatype value = Datatype::kUInt8;
};

// bf16 / fp16 <-> fp32 conversions for host-side reductions (round to nearest even).
inline float Bf16ToFloat(uint16_t v) {
  uint32_t bits = static_cast<uint32_t>(v) << 16;
  float f;
  memcpy(&f, &bits, 4);
  return f;
}
inline uint16_t FloatToBf16(float f) {
  uint32_t bits;
  memcpy(&bits, &f, 4);
  if ((bits & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((bits >> 16) | 0x40);  // NaN
  uint32_t lsb = (bits >> 16) & 1u;
  bits += 0x7fffu + lsb;
  return static_cast<uint16_t>(bits >> 16);
}
float Fp16ToFloat(uint16_t v);
uint16_t FloatToFp16(float f);

// Non-owning typed span with elementwise arithmetic.
template <typename T>
class Vec {
 public:
  using value_type = T;
  Vec() = default;
  Vec(T* data, size_t n) : data_(data), size_(n) {}

  T* data() { return data_; }
  const T* data() const { return data_; }
  size_t size() const { return size_; }
  bool empty() const { return size_ == 0; }
  T& operator[](size_t i) { return data_[i]; }
  const T& operator[](size_t i) const { return data_[i]; }
  T* begin() { return data_; }
  T* end() { return data_ + size_; }
  const T* begin() const { return data_; }
  const T* end() const { return data_ + size_; }

  void Fill(T v) {
    for (size_t i = 0; i < size_; ++i) data_[i] = v;
  }

  Vec& operator+=(const Vec& o) { return Apply(o, [](T a, T b) { return a + b; }); }
  Vec& operator-=(const Vec& o) { return Apply(o, [](T a, T b) { return a - b; }); }
  Vec& operator*=(const Vec& o) { return Apply(o, [](T a, T b) { return a * b; }); }
  Vec& operator/=(const Vec& o) { return Apply(o, [](T a, T b) { return a / b; }); }
  Vec& operator+=(T s) { return ApplyScalar([s](T a) { return a + s; }); }
  Vec& operator-=(T s) { return ApplyScalar([s](T a) { return a - s; }); }
  Vec& operator*=(T s) { return ApplyScalar([s](T a) { return a * s; }); }
  Vec& operator/=(T s) { return ApplyScalar([s](T a) { return a / s; }); }

  T dot(const Vec& o) const {
    TIPS_CHECK_EQ(size_, o.size_);
    T acc = T();
    for (size_t i = 0; i < size_; ++i) acc += data_[i] * o.data_[i];
    return acc;
  }
  T sum() const {
    T acc = T();
    for (size_t i = 0; i < size_; ++i) acc += data_[i];
    return acc;
  }

  // out = a * b / out = a * scalar / out = a + b ; out may alias an input.
  static void Mul(const Vec& a, const Vec& b, Vec* out) {
    TIPS_CHECK_EQ(a.size(), b.size());
    TIPS_CHECK_EQ(a.size(), out->size());
    for (size_t i = 0; i < a.size(); ++i) (*out)[i] = a[i] * b[i];
  }
  static void Mul(const Vec& a, T s, Vec* out) {
    TIPS_CHECK_EQ(a.size(), out->size());
    for (size_t i = 0; i < a.size(); ++i) (*out)[i] = a[i] * s;
  }
  static void Add(const Vec& a, const Vec& b, Vec* out) {
    TIPS_CHECK_EQ(a.size(), b.size());
    TIPS_CHECK_EQ(a.size(), out->size());
    for (size_t i = 0; i < a.size(); ++i) (*out)[i] = a[i] + b[i];
  }

  // "Vec:\t" followed by every element and one space: the text form used in
  // the text table dump.
  std::string ToStr() const {
    std::ostringstream ss;
    ss << "Vec:\t";
    for (size_t i = 0; i < size_; ++i) {
      if (sizeof(T) == 1)
        ss << static_cast<int>(data_[i]) << " ";
      else
        ss << data_[i] << " ";
    }
    return ss.str();
  }

 private:
  template <typename F>
  Vec& Apply(const Vec& o, F f) {
    TIPS_CHECK_EQ(size_, o.size_);
    for (size_t i = 0; i < size_; ++i) data_[i] = f(data_[i], o.data_[i]);
    return *this;
  }
  template <typename F>
  Vec& ApplyScalar(F f) {
    for (size_t i = 0; i < size_; ++i) data_[i] = f(data_[i]);
    return *this;
  }

  T* data_{nullptr};
  size_t size_{0};
};

template <typename T>
std::ostream& operator<<(std::ostream& os, const Vec<T>& v) {
  return os << v.ToStr();
}

// Type-erased vector that either owns its storage or borrows it.
class AnyVec {
 public:
  AnyVec() = default;
  AnyVec(Datatype dtype, size_t n);                           // owning, zero-initialised
  AnyVec(Datatype dtype, size_t n, void* borrowed);           // borrowing
  AnyVec(const AnyVec& o);                                    // deep copy
  AnyVec(AnyVec&& o) noexcept;
  AnyVec& operator=(const AnyVec& o);
  AnyVec& operator=(AnyVec&& o) noexcept;
  ~AnyVec();

  Datatype dtype() const { return dtype_; }
  size_t size() const { return size_; }
  size_t num_bytes() const { return size_ * DatatypeNumBytes(dtype_); }
  bool own_data() const { return own_; }
  bool valid() const { return data_ != nullptr; }
  uint8_t* buffer() { return data_; }
  const uint8_t* buffer() const { return data_; }

  // Re-allocates owning zeroed storage.
  void Resize(Datatype dtype, size_t n);
  // Deep copy of `o` into owned storage.
  void CopyFrom(const AnyVec& o);
  // Borrow `o`'s storage (no ownership).
  void ShadowCopyFrom(const AnyVec& o);
  AnyVec ShadowCopy() const;
  AnyVec Copy() const { return AnyVec(*this); }
  // Copy raw bytes into the existing storage; sizes must match.
  void AssignBytes(const void* src, size_t nbytes);

  template <typename T>
  Vec<T> ToVec() {
    TIPS_CHECK(DatatypeOf<T>::value == dtype_) << "AnyVec holds " << DatatypeName(dtype_);
    return Vec<T>(reinterpret_cast<T*>(data_), size_);
  }
  template <typename T>
  Vec<T> ToVec() const {
    TIPS_CHECK(DatatypeOf<T>::value == dtype_) << "AnyVec holds " << DatatypeName(dtype_);
    return Vec<T>(reinterpret_cast<T*>(data_), size_);
  }

  // Element i converted to double / set from double, whatever the dtype.
  double GetAsDouble(size_t i) const;
  void SetFromDouble(size_t i, double v);

  // dtype-dispatched kernels; `out` must have the inputs' dtype and size.
  static void Mul(const AnyVec& a, const AnyVec& b, AnyVec* out);
  static void Mul(const AnyVec& a, double scalar, AnyVec* out);
  static void Add(const AnyVec& a, const AnyVec& b, AnyVec* out);
  // out += alpha * a
  static void Axpy(double alpha, const AnyVec& a, AnyVec* out);

  std::string ToStr() const;

 private:
  void Free();

  Datatype dtype_{Datatype::kUnknown};
  uint8_t* data_{nullptr};
  size_t size_{0};
  bool own_{false};
};

std::ostream& operator<<(std::ostream& os, const AnyVec& v);

}  // namespace tips

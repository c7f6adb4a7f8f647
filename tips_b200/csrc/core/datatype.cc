#include "core/datatype.h"

#include <cstdlib>

namespace tips {

const char* DatatypeName(Datatype t) {
  switch (t) {
    case Datatype::kFp32: return "fp32";
    case Datatype::kFp64: return "fp64";
    case Datatype::kInt32: return "int32";
    case Datatype::kInt64: return "int64";
    case Datatype::kInt8: return "int8";
    case Datatype::kUInt8: return "uint8";
    case Datatype::kBf16: return "bf16";
    case Datatype::kFp16: return "fp16";
    default: return "unknown";
  }
}

size_t DatatypeNumBytes(Datatype t) {
  switch (t) {
    case Datatype::kFp32: return 4;
    case Datatype::kFp64: return 8;
    case Datatype::kInt32: return 4;
    case Datatype::kInt64: return 8;
    case Datatype::kInt8: return 1;
    case Datatype::kUInt8: return 1;
    case Datatype::kBf16: return 2;
    case Datatype::kFp16: return 2;
    default: TIPS_LOG(FATAL) << "DatatypeNumBytes of unknown type"; return 0;
  }
}

Datatype DatatypeFromName(const std::string& name) {
  for (int i = 0; i <= 7; ++i)
    if (name == DatatypeName(static_cast<Datatype>(i))) return static_cast<Datatype>(i);
  return Datatype::kUnknown;
}

float Fp16ToFloat(uint16_t h) {
  uint32_t sign = (h & 0x8000u) << 16;
  uint32_t exp  = (h >> 10) & 0x1fu;
  uint32_t man  = h & 0x3ffu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do {
        ++e;
        man <<= 1;
      } while (!(man & 0x400u));
      bits = sign | ((127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

uint16_t FloatToFp16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  x &= 0x7fffffffu;
  if (x >= 0x7f800000u) return static_cast<uint16_t>(sign | 0x7c00u | (x > 0x7f800000u ? 0x200u : 0));
  if (x >= 0x477ff000u) return static_cast<uint16_t>(sign | 0x7c00u);  // overflow -> inf
  if (x < 0x33000001u) return static_cast<uint16_t>(sign);             // underflow -> 0
  int exp      = static_cast<int>(x >> 23) - 127 + 15;
  uint32_t man = x & 0x7fffffu;
  if (exp <= 0) {
    man |= 0x800000u;
    int shift     = 14 - exp;
    uint32_t half = man >> shift;
    uint32_t rem  = man & ((1u << shift) - 1);
    uint32_t mid  = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) ++half;
    return static_cast<uint16_t>(sign | half);
  }
  uint32_t half = (static_cast<uint32_t>(exp) << 10) | (man >> 13);
  uint32_t rem  = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) ++half;
  return static_cast<uint16_t>(sign | half);
}

AnyVec::AnyVec(Datatype dtype, size_t n) { Resize(dtype, n); }

AnyVec::AnyVec(Datatype dtype, size_t n, void* borrowed)
    : dtype_(dtype), data_(static_cast<uint8_t*>(borrowed)), size_(n), own_(false) {}

AnyVec::AnyVec(const AnyVec& o) { CopyFrom(o); }

AnyVec::AnyVec(AnyVec&& o) noexcept : dtype_(o.dtype_), data_(o.data_), size_(o.size_), own_(o.own_) {
  o.data_ = nullptr;
  o.size_ = 0;
  o.own_  = false;
}

AnyVec& AnyVec::operator=(const AnyVec& o) {
  if (this != &o) CopyFrom(o);
  return *this;
}

AnyVec& AnyVec::operator=(AnyVec&& o) noexcept {
  if (this != &o) {
    Free();
    dtype_  = o.dtype_;
    data_   = o.data_;
    size_   = o.size_;
    own_    = o.own_;
    o.data_ = nullptr;
    o.size_ = 0;
    o.own_  = false;
  }
  return *this;
}

AnyVec::~AnyVec() { Free(); }

void AnyVec::Free() {
  if (own_ && data_) delete[] data_;
  data_ = nullptr;
  size_ = 0;
  own_  = false;
}

void AnyVec::Resize(Datatype dtype, size_t n) {
  Free();
  dtype_ = dtype;
  size_  = n;
  own_   = true;
  data_  = new uint8_t[n * DatatypeNumBytes(dtype) + 1]();
}

void AnyVec::CopyFrom(const AnyVec& o) {
  if (!o.valid()) {
    Free();
    dtype_ = o.dtype_;
    return;
  }
  Resize(o.dtype_, o.size_);
  memcpy(data_, o.data_, o.num_bytes());
}

void AnyVec::ShadowCopyFrom(const AnyVec& o) {
  Free();
  dtype_ = o.dtype_;
  data_  = o.data_;
  size_  = o.size_;
  own_   = false;
}

AnyVec AnyVec::ShadowCopy() const {
  AnyVec v;
  v.ShadowCopyFrom(*this);
  return v;
}

void AnyVec::AssignBytes(const void* src, size_t nbytes) {
  TIPS_CHECK_EQ(nbytes, num_bytes());
  memcpy(data_, src, nbytes);
}

double AnyVec::GetAsDouble(size_t i) const {
  TIPS_CHECK_LT(i, size_);
  switch (dtype_) {
    case Datatype::kFp32: return reinterpret_cast<const float*>(data_)[i];
    case Datatype::kFp64: return reinterpret_cast<const double*>(data_)[i];
    case Datatype::kInt32: return reinterpret_cast<const int32_t*>(data_)[i];
    case Datatype::kInt64: return static_cast<double>(reinterpret_cast<const int64_t*>(data_)[i]);
    case Datatype::kInt8: return reinterpret_cast<const int8_t*>(data_)[i];
    case Datatype::kUInt8: return data_[i];
    case Datatype::kBf16: return Bf16ToFloat(reinterpret_cast<const uint16_t*>(data_)[i]);
    case Datatype::kFp16: return Fp16ToFloat(reinterpret_cast<const uint16_t*>(data_)[i]);
    default: TIPS_LOG(FATAL) << "unknown dtype"; return 0;
  }
}

void AnyVec::SetFromDouble(size_t i, double v) {
  TIPS_CHECK_LT(i, size_);
  switch (dtype_) {
    case Datatype::kFp32: reinterpret_cast<float*>(data_)[i] = static_cast<float>(v); break;
    case Datatype::kFp64: reinterpret_cast<double*>(data_)[i] = v; break;
    case Datatype::kInt32: reinterpret_cast<int32_t*>(data_)[i] = static_cast<int32_t>(v); break;
    case Datatype::kInt64: reinterpret_cast<int64_t*>(data_)[i] = static_cast<int64_t>(v); break;
    case Datatype::kInt8: reinterpret_cast<int8_t*>(data_)[i] = static_cast<int8_t>(v); break;
    case Datatype::kUInt8: data_[i] = static_cast<uint8_t>(v); break;
    case Datatype::kBf16: reinterpret_cast<uint16_t*>(data_)[i] = FloatToBf16(static_cast<float>(v)); break;
    case Datatype::kFp16: reinterpret_cast<uint16_t*>(data_)[i] = FloatToFp16(static_cast<float>(v)); break;
    default: TIPS_LOG(FATAL) << "unknown dtype";
  }
}

namespace {

template <typename F>
void Dispatch2(const AnyVec& a, const AnyVec& b, AnyVec* out, F f) {
  TIPS_CHECK(a.dtype() == b.dtype() && a.dtype() == out->dtype()) << "dtype mismatch";
  TIPS_CHECK_EQ(a.size(), b.size());
  TIPS_CHECK_EQ(a.size(), out->size());
  const size_t n = a.size();
  switch (a.dtype()) {
#define TIPS_CASE(DT, T)                                        \
  case Datatype::DT: {                                          \
    const T* pa = reinterpret_cast<const T*>(a.buffer());       \
    const T* pb = reinterpret_cast<const T*>(b.buffer());       \
    T* po       = reinterpret_cast<T*>(out->buffer());          \
    for (size_t i = 0; i < n; ++i) po[i] = static_cast<T>(f(pa[i], pb[i])); \
  } break;
    TIPS_CASE(kFp32, float)
    TIPS_CASE(kFp64, double)
    TIPS_CASE(kInt32, int32_t)
    TIPS_CASE(kInt64, int64_t)
    TIPS_CASE(kInt8, int8_t)
    TIPS_CASE(kUInt8, uint8_t)
#undef TIPS_CASE
    default:
      for (size_t i = 0; i < n; ++i) out->SetFromDouble(i, f(a.GetAsDouble(i), b.GetAsDouble(i)));
  }
}

}  // namespace

void AnyVec::Mul(const AnyVec& a, const AnyVec& b, AnyVec* out) {
  Dispatch2(a, b, out, [](auto x, auto y) { return x * y; });
}

void AnyVec::Add(const AnyVec& a, const AnyVec& b, AnyVec* out) {
  Dispatch2(a, b, out, [](auto x, auto y) { return x + y; });
}

void AnyVec::Mul(const AnyVec& a, double scalar, AnyVec* out) {
  TIPS_CHECK(a.dtype() == out->dtype()) << "dtype mismatch";
  TIPS_CHECK_EQ(a.size(), out->size());
  const size_t n = a.size();
  if (a.dtype() == Datatype::kFp32) {
    const float* pa = reinterpret_cast<const float*>(a.buffer());
    float* po       = reinterpret_cast<float*>(out->buffer());
    const float s   = static_cast<float>(scalar);
    for (size_t i = 0; i < n; ++i) po[i] = pa[i] * s;
    return;
  }
  for (size_t i = 0; i < n; ++i) out->SetFromDouble(i, a.GetAsDouble(i) * scalar);
}

void AnyVec::Axpy(double alpha, const AnyVec& a, AnyVec* out) {
  TIPS_CHECK(a.dtype() == out->dtype()) << "dtype mismatch";
  TIPS_CHECK_EQ(a.size(), out->size());
  const size_t n = a.size();
  if (a.dtype() == Datatype::kFp32) {
    const float* pa = reinterpret_cast<const float*>(a.buffer());
    float* po       = reinterpret_cast<float*>(out->buffer());
    const float s   = static_cast<float>(alpha);
    for (size_t i = 0; i < n; ++i) po[i] += pa[i] * s;
    return;
  }
  for (size_t i = 0; i < n; ++i) out->SetFromDouble(i, out->GetAsDouble(i) + alpha * a.GetAsDouble(i));
}

std::string AnyVec::ToStr() const {
  switch (dtype_) {
    case Datatype::kFp32: return ToVec<float>().ToStr();
    case Datatype::kFp64: return ToVec<double>().ToStr();
    case Datatype::kInt32: return ToVec<int32_t>().ToStr();
    case Datatype::kInt64: return ToVec<int64_t>().ToStr();
    case Datatype::kInt8: return ToVec<int8_t>().ToStr();
    case Datatype::kUInt8: return ToVec<uint8_t>().ToStr();
    default: {
      std::ostringstream ss;
      ss << "Vec:\t";
      for (size_t i = 0; i < size_; ++i) ss << GetAsDouble(i) << " ";
      return ss.str();
    }
  }
}

std::ostream& operator<<(std::ostream& os, const AnyVec& v) { return os << v.ToStr(); }

}  // namespace tips

// Append-only byte buffer with a read cursor, stream operators and typed field
// builders.  It is the wire format of every control-plane message in this
// runtime and of the binary table checkpoints.
//
// Wire-format parity with the reference (tips/core/common/naive_buffer.h:87-508,
// naive_buffer.cc:84-109): a POD is its sizeof(T) raw little-endian bytes; a
// string or a list is a uint64 element count followed by the raw elements.
// File helpers mirror SaveToFile / AppendToFile / LoadFromFile(offset, size)
// (naive_buffer.cc:35-75).
#pragma once

#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <type_traits>
#include <vector>

#include "core/logging.h"

namespace tips {

class NaiveBuffer {
 public:
  NaiveBuffer() = default;
  // Read mode over a copy of `size` bytes at `data`.
  NaiveBuffer(const void* data, size_t size) { LoadFromMemory(data, size); }

  // Grows the buffer so that `size` more bytes fit after the cursor.
  void Require(size_t size) {
    if (cursor_ + size > bytes_.size()) bytes_.resize(cursor_ + size);
  }
  // Advances the cursor.
  void Consume(size_t size) {
    TIPS_CHECK_LE(cursor_ + size, bytes_.size()) << "NaiveBuffer overrun";
    cursor_ += size;
  }
  void ToHead() { cursor_ = 0; }

  uint8_t* cursor() { return bytes_.data() + cursor_; }
  size_t cursor_pos() const { return cursor_; }
  const char* data() const { return reinterpret_cast<const char*>(bytes_.data()); }
  void* data() { return bytes_.data(); }
  size_t size() const { return bytes_.size(); }
  size_t free_size() const { return bytes_.size() - cursor_; }
  const std::vector<uint8_t>& bytes() const { return bytes_; }
  std::vector<uint8_t>&& TakeBytes() { return std::move(bytes_); }

  void WriteRaw(const void* src, size_t n) {
    Require(n);
    if (n) memcpy(cursor(), src, n);
    cursor_ += n;
  }
  void ReadRaw(void* dst, size_t n) {
    TIPS_CHECK_LE(cursor_ + n, bytes_.size()) << "NaiveBuffer underrun: need " << n << " bytes at " << cursor_;
    if (n) memcpy(dst, cursor(), n);
    cursor_ += n;
  }

  void SaveToFile(const std::string& path) const;
  void AppendToFile(const std::string& path) const;
  // size == 0 means "to the end of the file".
  void LoadFromFile(const std::string& path, size_t offset = 0, size_t size = 0);
  void LoadFromMemory(const void* data, size_t size) {
    bytes_.assign(static_cast<const uint8_t*>(data), static_cast<const uint8_t*>(data) + size);
    cursor_ = 0;
  }

 private:
  std::vector<uint8_t> bytes_;
  size_t cursor_{0};
};

template <typename T, typename = typename std::enable_if<std::is_trivially_copyable<T>::value>::type>
NaiveBuffer& operator<<(NaiveBuffer& buf, const T& v) {
  buf.WriteRaw(&v, sizeof(T));
  return buf;
}
template <typename T, typename = typename std::enable_if<std::is_trivially_copyable<T>::value>::type>
NaiveBuffer& operator>>(NaiveBuffer& buf, T& v) {
  buf.ReadRaw(&v, sizeof(T));
  return buf;
}
NaiveBuffer& operator<<(NaiveBuffer& buf, const std::string& s);
NaiveBuffer& operator>>(NaiveBuffer& buf, std::string& s);

template <typename T>
NaiveBuffer& operator<<(NaiveBuffer& buf, const std::vector<T>& v) {
  static_assert(std::is_trivially_copyable<T>::value, "vector element must be POD");
  uint64_t n = v.size();
  buf << n;
  buf.WriteRaw(v.data(), n * sizeof(T));
  return buf;
}
template <typename T>
NaiveBuffer& operator>>(NaiveBuffer& buf, std::vector<T>& v) {
  static_assert(std::is_trivially_copyable<T>::value, "vector element must be POD");
  uint64_t n = 0;
  buf >> n;
  TIPS_CHECK_LE(n * sizeof(T), buf.free_size()) << "corrupt list length " << n;
  v.resize(n);
  buf.ReadRaw(v.data(), n * sizeof(T));
  return buf;
}

// ---- typed field builders -------------------------------------------------
// A field is bound to a buffer; Flush() appends its value at the cursor and
// Load() reads it back.  StructBuilder composes named fields in declaration
// order, ListBuilder<F> holds a counted sequence of fields.

class FieldBuilder {
 public:
  explicit FieldBuilder(NaiveBuffer* table) : table_(table) {}
  virtual ~FieldBuilder() = default;
  virtual void Flush()           = 0;
  virtual void Load()            = 0;
  virtual const char* type_name() const = 0;
  NaiveBuffer* table() { return table_; }

 private:
  NaiveBuffer* table_;
};

template <typename P>
class PrimaryBuilder : public FieldBuilder {
 public:
  using value_type = P;
  explicit PrimaryBuilder(NaiveBuffer* table, P v = P()) : FieldBuilder(table), value_(v) {}
  void set(P v) { value_ = v; }
  P data() const { return value_; }
  void Flush() override { *table() << value_; }
  void Load() override { *table() >> value_; }
  const char* type_name() const override { return "primary"; }

 private:
  P value_;
};

using BoolBuilder    = PrimaryBuilder<bool>;
using CharBuilder    = PrimaryBuilder<char>;
using Int32Builder   = PrimaryBuilder<int32_t>;
using UInt32Builder  = PrimaryBuilder<uint32_t>;
using Int64Builder   = PrimaryBuilder<int64_t>;
using UInt64Builder  = PrimaryBuilder<uint64_t>;
using Float32Builder = PrimaryBuilder<float>;
using Float64Builder = PrimaryBuilder<double>;

template <typename E>
class EnumBuilder : public FieldBuilder {
  static_assert(std::is_enum<E>::value, "EnumBuilder needs an enum");

 public:
  explicit EnumBuilder(NaiveBuffer* table, E v = E()) : FieldBuilder(table), value_(v) {}
  void set(E v) { value_ = v; }
  E data() const { return value_; }
  void Flush() override { *table() << static_cast<int32_t>(value_); }
  void Load() override {
    int32_t raw = 0;
    *table() >> raw;
    value_ = static_cast<E>(raw);
  }
  const char* type_name() const override { return "enum"; }

 private:
  E value_;
};

template <typename P>
class PrimaryListBuilder : public FieldBuilder {
 public:
  explicit PrimaryListBuilder(NaiveBuffer* table) : FieldBuilder(table) {}
  void set(const P* data, size_t n) { values_.assign(data, data + n); }
  void set(const std::vector<P>& v) { values_ = v; }
  const std::vector<P>& data() const { return values_; }
  size_t size() const { return values_.size(); }
  void Flush() override { *table() << values_; }
  void Load() override { *table() >> values_; }
  const char* type_name() const override { return "primary_list"; }

 private:
  std::vector<P> values_;
};

class StringBuilder : public FieldBuilder {
 public:
  explicit StringBuilder(NaiveBuffer* table, std::string v = "") : FieldBuilder(table), value_(std::move(v)) {}
  void set(const std::string& v) { value_ = v; }
  const std::string& data() const { return value_; }
  void Flush() override { *table() << value_; }
  void Load() override { *table() >> value_; }
  const char* type_name() const override { return "string"; }

 private:
  std::string value_;
};

class StructBuilder : public FieldBuilder {
 public:
  explicit StructBuilder(NaiveBuffer* table) : FieldBuilder(table) {}

  // Creates a field of type F named `name`; fields are serialised in the
  // order in which they were created.
  template <typename F, typename... Args>
  F* NewField(const std::string& name, Args&&... args) {
    auto* f = new F(table(), std::forward<Args>(args)...);
    names_.push_back(name);
    fields_.emplace_back(f);
    return f;
  }

  template <typename F>
  F* GetField(const std::string& name) {
    for (size_t i = 0; i < names_.size(); ++i)
      if (names_[i] == name) return dynamic_cast<F*>(fields_[i].get());
    TIPS_LOG(FATAL) << "no field named " << name;
    return nullptr;
  }

  size_t num_fields() const { return fields_.size(); }
  void Flush() override {
    for (auto& f : fields_) f->Flush();
  }
  void Load() override {
    for (auto& f : fields_) f->Load();
  }
  const char* type_name() const override { return "struct"; }

 private:
  std::vector<std::string> names_;
  std::vector<std::unique_ptr<FieldBuilder>> fields_;
};

template <typename F>
class ListBuilder : public FieldBuilder {
 public:
  explicit ListBuilder(NaiveBuffer* table) : FieldBuilder(table) {}
  F* New() {
    items_.emplace_back(new F(table()));
    return items_.back().get();
  }
  F* Get(size_t i) { return items_.at(i).get(); }
  size_t size() const { return items_.size(); }
  void Clear() { items_.clear(); }
  void Flush() override {
    *table() << static_cast<uint64_t>(items_.size());
    for (auto& it : items_) it->Flush();
  }
  void Load() override {
    uint64_t n = 0;
    *table() >> n;
    items_.clear();
    for (uint64_t i = 0; i < n; ++i) New()->Load();
  }
  const char* type_name() const override { return "list"; }

 private:
  std::vector<std::unique_ptr<F>> items_;
};

}  // namespace tips

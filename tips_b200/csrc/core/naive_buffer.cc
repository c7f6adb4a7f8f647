#include "core/naive_buffer.h"

#include <cstdio>

namespace tips {

namespace {
void WriteFile(const std::string& path, const char* mode, const std::vector<uint8_t>& bytes) {
  FILE* f = fopen(path.c_str(), mode);
  TIPS_CHECK(f != nullptr) << "cannot open " << path;
  size_t n = bytes.empty() ? 0 : fwrite(bytes.data(), 1, bytes.size(), f);
  fclose(f);
  TIPS_CHECK_EQ(n, bytes.size()) << "short write to " << path;
}
}  // namespace

void NaiveBuffer::SaveToFile(const std::string& path) const { WriteFile(path, "wb", bytes_); }
void NaiveBuffer::AppendToFile(const std::string& path) const { WriteFile(path, "ab", bytes_); }

void NaiveBuffer::LoadFromFile(const std::string& path, size_t offset, size_t size) {
  FILE* f = fopen(path.c_str(), "rb");
  TIPS_CHECK(f != nullptr) << "cannot open " << path;
  fseek(f, 0, SEEK_END);
  size_t file_size = static_cast<size_t>(ftell(f));
  if (offset > file_size) {
    fclose(f);
    TIPS_LOG(FATAL) << "offset " << offset << " beyond the end of " << path << " (" << file_size << ")";
  }
  if (size == 0) size = file_size - offset;
  if (offset + size > file_size) {
    fclose(f);
    TIPS_LOG(FATAL) << "range [" << offset << ", " << offset + size << ") beyond the end of " << path;
  }
  fseek(f, static_cast<long>(offset), SEEK_SET);
  bytes_.resize(size);
  size_t n = size ? fread(bytes_.data(), 1, size, f) : 0;
  fclose(f);
  TIPS_CHECK_EQ(n, size) << "short read from " << path;
  cursor_ = 0;
}

NaiveBuffer& operator<<(NaiveBuffer& buf, const std::string& s) {
  uint64_t n = s.size();
  buf << n;
  buf.WriteRaw(s.data(), n);
  return buf;
}

NaiveBuffer& operator>>(NaiveBuffer& buf, std::string& s) {
  uint64_t n = 0;
  buf >> n;
  TIPS_CHECK_LE(n, buf.free_size()) << "corrupt string length " << n;
  s.resize(n);
  buf.ReadRaw(&s[0], n);
  return buf;
}

}  // namespace tips

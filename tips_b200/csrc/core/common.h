// Small shared utilities of the native runtime: Status, string helpers, an
// insertion-ordered map, EINTR-safe syscall retry and local-address discovery.
//
// Capability parity with the reference's tips/core/common/common.h:21-64
// (ZCHECK, ignore_signal_call, GetLocalIp, StringFormat, OrderedMap) and
// tips/core/utils/string.h:8-18 (ToString of a span).
#pragma once

#include <cerrno>
#include <cstdarg>
#include <cstdint>
#include <sstream>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "core/logging.h"

namespace tips {

// Error codes shared with the C API and the Python layer.
enum StatusCode : int32_t {
  kOk              = 0,
  kInProgress      = 1,
  kInvalidArgument = 2,
  kPrecondition    = 3,  // cross-rank mismatch found during negotiation
  kAborted         = 4,  // shutdown while in flight
  kTimeout         = 5,
  kUnavailable     = 6,  // transport failure
  kInternal        = 7,
  kDuplicateName   = 8,
};

class Status {
 public:
  Status() = default;
  Status(StatusCode code, std::string msg) : code_(code), msg_(std::move(msg)) {}
  static Status OK() { return Status(); }
  bool ok() const { return code_ == kOk; }
  StatusCode code() const { return code_; }
  const std::string& message() const { return msg_; }
  std::string ToString() const { return ok() ? "OK" : ("[" + std::to_string(code_) + "] " + msg_); }

 private:
  StatusCode code_{kOk};
  std::string msg_;
};

std::string StringFormat(const char* fmt, ...) __attribute__((format(printf, 1, 2)));

// First non-loopback IPv4 address of this host, "127.0.0.1" if there is none.
// TIPS_LOCAL_IP overrides the discovery.
std::string GetLocalIp();

// Calls f(args...) again while it fails with EINTR.
template <typename F, typename... Args>
auto ignore_signal_call(F&& f, Args&&... args) -> decltype(f(args...)) {
  for (;;) {
    auto r = f(args...);
    if (r != -1 || errno != EINTR) return r;
  }
}

// Checks the return value of a socket / system call.
#define TIPS_ZCHECK(expr) TIPS_CHECK((expr) == 0) << "errno=" << errno << " (" << strerror(errno) << ") "

template <typename It>
std::string ToString(It begin, It end, const char* sep = ", ") {
  std::ostringstream ss;
  ss << "[";
  for (It it = begin; it != end; ++it) {
    if (it != begin) ss << sep;
    ss << *it;
  }
  ss << "]";
  return ss.str();
}
template <typename T>
std::string ToString(const std::vector<T>& v) {
  return ToString(v.begin(), v.end());
}

// Map that remembers insertion order.
template <typename K, typename V>
class OrderedMap {
 public:
  bool Has(const K& k) const { return index_.count(k) > 0; }
  void Set(const K& k, V v) {
    auto it = index_.find(k);
    if (it != index_.end()) {
      items_[it->second].second = std::move(v);
      return;
    }
    index_[k] = items_.size();
    items_.emplace_back(k, std::move(v));
  }
  V& Get(const K& k) {
    auto it = index_.find(k);
    TIPS_CHECK(it != index_.end()) << "OrderedMap: missing key";
    return items_[it->second].second;
  }
  const V& Get(const K& k) const {
    auto it = index_.find(k);
    TIPS_CHECK(it != index_.end()) << "OrderedMap: missing key";
    return items_[it->second].second;
  }
  size_t size() const { return items_.size(); }
  const std::vector<std::pair<K, V>>& items() const { return items_; }
  void Clear() {
    items_.clear();
    index_.clear();
  }

 private:
  std::vector<std::pair<K, V>> items_;
  std::unordered_map<K, size_t> index_;
};

// 64-bit mix used for key -> shard / server placement (splitmix64 finaliser).
inline uint64_t HashKey(uint64_t x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}

int64_t NowMicros();

}  // namespace tips

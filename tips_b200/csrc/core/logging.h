// Stream-style logging and check macros for the native runtime.
//
// Capability parity with the reference's glog clone (tips/core/common/logging.h:37-163,
// logging.cc:7-31): severity levels, verbose logging gated by an environment
// variable, CHECK macros, and a FATAL level that throws instead of aborting so
// that a failed check inside a background thread can be turned into an error
// status for the caller.
//
// Differences: the minimum severity is configurable (TIPS_LOG_LEVEL, default
// WARNING) so hot paths stay silent, and every line carries the "#rank-[r/n]"
// prefix once the runtime knows its rank (reference: tips/core/mpi/tips_mpi.h:180-181).
#pragma once

#include <cstdint>
#include <cstdlib>
#include <sstream>
#include <stdexcept>
#include <string>

namespace tips {

enum class LogLevel : int { kInfo = 0, kWarning = 1, kError = 2, kFatal = 3 };

// Thrown by TIPS_LOG(FATAL) and failed TIPS_CHECK*.
class FatalError : public std::runtime_error {
 public:
  explicit FatalError(const std::string& what) : std::runtime_error(what) {}
};

// Process-wide logging configuration.
struct LogConfig {
  static int& MinLevel();      // from TIPS_LOG_LEVEL (0..3 or INFO/WARNING/ERROR/FATAL)
  static int& VerboseLevel();  // from TIPS_VLOG, else GLOG_v
  static void SetRank(int rank, int size);
  static std::string RankPrefix();
  static void Reload();  // re-read the environment
};

class LogMessage {
 public:
  LogMessage(const char* file, const char* func, int line, LogLevel level, bool enabled);
  ~LogMessage() noexcept(false);
  std::ostream& stream() { return os_; }

 private:
  std::ostringstream os_;
  LogLevel level_;
  bool enabled_;
};

// Swallows a stream expression when a log statement is disabled.
struct LogVoidify {
  void operator&(std::ostream&) {}
};

}  // namespace tips

#define TIPS_LOG_LEVEL_INFO ::tips::LogLevel::kInfo
#define TIPS_LOG_LEVEL_WARNING ::tips::LogLevel::kWarning
#define TIPS_LOG_LEVEL_ERROR ::tips::LogLevel::kError
#define TIPS_LOG_LEVEL_FATAL ::tips::LogLevel::kFatal

#define TIPS_LOG_ENABLED(level) \
  (static_cast<int>(TIPS_LOG_LEVEL_##level) >= ::tips::LogConfig::MinLevel())

#define TIPS_LOG(level)                                                                     \
  ::tips::LogMessage(__FILE__, __func__, __LINE__, TIPS_LOG_LEVEL_##level,                  \
                     TIPS_LOG_ENABLED(level) || TIPS_LOG_LEVEL_##level == ::tips::LogLevel::kFatal) \
      .stream()

#define TIPS_VLOG(n)                                    \
  !((n) <= ::tips::LogConfig::VerboseLevel())           \
      ? (void)0                                         \
      : ::tips::LogVoidify() &                          \
            ::tips::LogMessage(__FILE__, __func__, __LINE__, ::tips::LogLevel::kInfo, true).stream()

#define TIPS_CHECK(cond) \
  if (!(cond)) TIPS_LOG(FATAL) << "Check failed: " #cond " "

#define TIPS_CHECK_OP(a, b, op)                                                               \
  if (!((a)op(b)))                                                                            \
  TIPS_LOG(FATAL) << "Check failed: " #a " " #op " " #b " (" << (a) << " vs " << (b) << ") "

#define TIPS_CHECK_EQ(a, b) TIPS_CHECK_OP(a, b, ==)
#define TIPS_CHECK_NE(a, b) TIPS_CHECK_OP(a, b, !=)
#define TIPS_CHECK_LT(a, b) TIPS_CHECK_OP(a, b, <)
#define TIPS_CHECK_LE(a, b) TIPS_CHECK_OP(a, b, <=)
#define TIPS_CHECK_GT(a, b) TIPS_CHECK_OP(a, b, >)
#define TIPS_CHECK_GE(a, b) TIPS_CHECK_OP(a, b, >=)
#define TIPS_CHECK_NEAR(a, b, eps)                                  \
  if (!(((a) - (b)) <= (eps) && ((b) - (a)) <= (eps)))              \
  TIPS_LOG(FATAL) << "Check failed: |" #a " - " #b "| <= " #eps " (" << (a) << " vs " << (b) << ") "

#define TIPS_DISALLOW_COPY_AND_ASSIGN(T) \
  T(const T&) = delete;                  \
  T& operator=(const T&) = delete

#define TIPS_MUST_USE_RESULT __attribute__((warn_unused_result))

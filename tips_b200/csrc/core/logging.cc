#include "core/logging.h"

#include <sys/time.h>

#include <atomic>
#include <cstdio>
#include <cstring>
#include <ctime>
#include <mutex>

namespace tips {

namespace {

int ParseLevel(const char* s, int dflt) {
  if (!s || !*s) return dflt;
  if (!strcasecmp(s, "INFO")) return 0;
  if (!strcasecmp(s, "WARNING") || !strcasecmp(s, "WARN")) return 1;
  if (!strcasecmp(s, "ERROR")) return 2;
  if (!strcasecmp(s, "FATAL")) return 3;
  char* end = nullptr;
  long v = strtol(s, &end, 10);
  if (end == s) return dflt;
  return static_cast<int>(v);
}

std::atomic<int> g_rank{-1};
std::atomic<int> g_size{0};
std::mutex g_write_mu;

const char* Basename(const char* path) {
  const char* slash = strrchr(path, '/');
  return slash ? slash + 1 : path;
}

}  // namespace

int& LogConfig::MinLevel() {
  static int level = ParseLevel(getenv("TIPS_LOG_LEVEL"), 1);
  return level;
}

int& LogConfig::VerboseLevel() {
  static int v = ParseLevel(getenv("TIPS_VLOG") ? getenv("TIPS_VLOG") : getenv("GLOG_v"), 0);
  return v;
}

void LogConfig::Reload() {
  MinLevel()     = ParseLevel(getenv("TIPS_LOG_LEVEL"), 1);
  VerboseLevel() = ParseLevel(getenv("TIPS_VLOG") ? getenv("TIPS_VLOG") : getenv("GLOG_v"), 0);
}

void LogConfig::SetRank(int rank, int size) {
  g_rank = rank;
  g_size = size;
}

std::string LogConfig::RankPrefix() {
  int r = g_rank.load();
  if (r < 0) return "";
  char buf[48];
  snprintf(buf, sizeof(buf), "#rank-[%d/%d] ", r, g_size.load());
  return buf;
}

LogMessage::LogMessage(const char* file, const char* func, int line, LogLevel level, bool enabled)
    : level_(level), enabled_(enabled) {
  if (!enabled_) return;
  static const char kTags[] = {'I', 'W', 'E', 'F'};
  struct timeval tv;
  gettimeofday(&tv, nullptr);
  struct tm tm_buf;
  time_t secs = tv.tv_sec;
  localtime_r(&secs, &tm_buf);
  char head[96];
  snprintf(head, sizeof(head), "[%c %02d/%02d %02d:%02d:%02d.%03d ", kTags[static_cast<int>(level)],
           tm_buf.tm_mon + 1, tm_buf.tm_mday, tm_buf.tm_hour, tm_buf.tm_min, tm_buf.tm_sec,
           static_cast<int>(tv.tv_usec / 1000));
  os_ << head << Basename(file) << " " << func << ":" << line << "] " << LogConfig::RankPrefix();
}

LogMessage::~LogMessage() noexcept(false) {
  if (!enabled_) return;
  os_ << "\n";
  {
    std::lock_guard<std::mutex> lock(g_write_mu);
    const std::string s = os_.str();
    fwrite(s.data(), 1, s.size(), stderr);
    fflush(stderr);
  }
  if (level_ == LogLevel::kFatal) {
    throw FatalError(os_.str());
  }
}

}  // namespace tips

#include "native_log.h"

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <deque>
#include <mutex>

namespace fkv {

const char* const kCacheOpNames[kNumCacheOps] = {"hit", "miss", "match", "insert", "evict"};

namespace {

struct LogState {
  std::atomic<int> level{(int)LogLevel::kInfo};
  std::mutex mu;
  std::string prefix = "[FLEXKV]";
  std::deque<std::string> ring;
  LogState() {
    if (const char* p = std::getenv("FLEXKV_LOGGING_PREFIX")) prefix = p;
    if (const char* l = std::getenv("FLEXKV_LOG_LEVEL")) apply(l);
  }
  void apply(const std::string& name) {
    std::string s;
    for (char c : name) s.push_back((char)std::tolower((unsigned char)c));
    static const struct { const char* n; LogLevel l; } table[] = {
        {"trace", LogLevel::kTrace}, {"debug", LogLevel::kDebug}, {"info", LogLevel::kInfo},
        {"warn", LogLevel::kWarn},   {"warning", LogLevel::kWarn}, {"error", LogLevel::kError},
        {"critical", LogLevel::kError}, {"off", LogLevel::kOff}};
    for (auto& e : table)
      if (s == e.n) level.store((int)e.l, std::memory_order_relaxed);
  }
};

LogState& state() {
  static LogState s;
  return s;
}

constexpr size_t kRingLines = 256;
const char* const kLevelNames[] = {"TRACE", "DEBUG", "INFO", "WARN", "ERROR", "OFF"};

std::atomic<bool> g_metrics_enabled{false};

}  // namespace

LogLevel log_level() { return (LogLevel)state().level.load(std::memory_order_relaxed); }
void set_log_level(LogLevel l) { state().level.store((int)l, std::memory_order_relaxed); }
void set_log_level(const std::string& name) { state().apply(name); }
void set_log_prefix(const std::string& p) {
  std::lock_guard<std::mutex> g(state().mu);
  state().prefix = p;
}

void log_write(LogLevel l, const char* file, int line, const char* fmt, ...) {
  char msg[1024];
  va_list ap;
  va_start(ap, fmt);
  std::vsnprintf(msg, sizeof(msg), fmt, ap);
  va_end(ap);
  auto now = std::chrono::system_clock::now();
  std::time_t t = std::chrono::system_clock::to_time_t(now);
  int ms = (int)(std::chrono::duration_cast<std::chrono::milliseconds>(now.time_since_epoch()).count() % 1000);
  std::tm tmv;
  localtime_r(&t, &tmv);
  const char* base = std::strrchr(file, '/');
  base = base ? base + 1 : file;
  char out[1280];
  LogState& s = state();
  std::lock_guard<std::mutex> g(s.mu);
  std::snprintf(out, sizeof(out), "%s %s %02d-%02d %02d:%02d:%02d.%03d [%s:%d] %s", s.prefix.c_str(),
                kLevelNames[(int)l], tmv.tm_mon + 1, tmv.tm_mday, tmv.tm_hour, tmv.tm_min, tmv.tm_sec, ms, base, line,
                msg);
  std::fprintf(stdout, "%s\n", out);
  std::fflush(stdout);
  s.ring.emplace_back(out);
  if (s.ring.size() > kRingLines) s.ring.pop_front();
}

std::vector<std::string> log_recent(size_t max_lines) {
  LogState& s = state();
  std::lock_guard<std::mutex> g(s.mu);
  size_t n = std::min(max_lines, s.ring.size());
  return std::vector<std::string>(s.ring.end() - (long)n, s.ring.end());
}

CacheCounters& cache_counters() {
  static CacheCounters c{};
  return c;
}
bool metrics_enabled() { return g_metrics_enabled.load(std::memory_order_relaxed); }
void configure_metrics(bool enabled) { g_metrics_enabled.store(enabled, std::memory_order_relaxed); }
void reset_metrics() {
  auto& c = cache_counters();
  for (int i = 0; i < kNumCacheOps; ++i) {
    c.ops[i].store(0);
    c.blocks[i].store(0);
  }
}

}  // namespace fkv

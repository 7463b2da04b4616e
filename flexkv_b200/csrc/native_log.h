// Native logger and cache-operation counters for the C++ control plane.
//
// Same knobs as the reference's spdlog front end (csrc/logging.cpp:50-104):
// FLEXKV_LOG_LEVEL (trace|debug|info|warn|error|off) and FLEXKV_LOGGING_PREFIX.
// Counters mirror its Prometheus families flexkv_cpp_cache_ops_total{operation=..}
// and flexkv_cpp_cache_blocks_total{operation=..} (csrc/monitoring/metrics_manager.cpp:104-110,
// macros metrics_manager.h:211-235); here they are lock-free atomics that Python
// scrapes into its own registry and that metrics_exposer.{h,cpp} serves on a port of their own.
#pragma once
#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <string>
#include <vector>

namespace fkv {

enum class LogLevel : int { kTrace = 0, kDebug, kInfo, kWarn, kError, kOff };

LogLevel log_level();
void set_log_level(LogLevel l);
void set_log_level(const std::string& name);   // unknown names leave the level unchanged
void set_log_prefix(const std::string& p);
void log_write(LogLevel l, const char* file, int line, const char* fmt, ...) __attribute__((format(printf, 4, 5)));
// Messages are also kept in a small ring so tests (and crash reports) can read them back.
std::vector<std::string> log_recent(size_t max_lines);

#define FKV_LOG(level, ...)                                                             \
  do {                                                                                  \
    if ((int)(level) >= (int)::fkv::log_level()) ::fkv::log_write(level, __FILE__, __LINE__, __VA_ARGS__); \
  } while (0)
#define FKV_DEBUG(...) FKV_LOG(::fkv::LogLevel::kDebug, __VA_ARGS__)
#define FKV_INFO(...) FKV_LOG(::fkv::LogLevel::kInfo, __VA_ARGS__)
#define FKV_WARN(...) FKV_LOG(::fkv::LogLevel::kWarn, __VA_ARGS__)
#define FKV_ERROR(...) FKV_LOG(::fkv::LogLevel::kError, __VA_ARGS__)

enum CacheOp : int { kOpHit = 0, kOpMiss, kOpMatch, kOpInsert, kOpEvict, kNumCacheOps };
extern const char* const kCacheOpNames[kNumCacheOps];

struct CacheCounters {
  std::atomic<uint64_t> ops[kNumCacheOps];
  std::atomic<uint64_t> blocks[kNumCacheOps];
};

// One process-wide set; `enabled` is flipped from Python (configure_cpp_metrics).
CacheCounters& cache_counters();
bool metrics_enabled();
void configure_metrics(bool enabled);
void reset_metrics();

inline void count_cache_op(CacheOp op, uint64_t blocks) {
  if (!metrics_enabled()) return;
  auto& c = cache_counters();
  c.ops[op].fetch_add(1, std::memory_order_relaxed);
  c.blocks[op].fetch_add(blocks, std::memory_order_relaxed);
}

}  // namespace fkv

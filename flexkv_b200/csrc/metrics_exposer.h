// Prometheus text endpoint served from native code.
//
// The reference starts a prometheus-cpp Exposer on FLEXKV_CPP_METRICS_PORT (default 8081) for the counters of
// its C++ control plane (csrc/monitoring/metrics_manager.cpp:60-110). Here the same two families,
// flexkv_cpp_cache_ops_total{operation=..} and flexkv_cpp_cache_blocks_total{operation=..}, are written straight
// from the atomics in native_log.h by one small thread: poll() on the listening socket and on an eventfd that
// ends it, one request per connection, no library. The endpoint answers while the Python interpreter is busy
// or holds the GIL, which is the point of serving it here.
#pragma once
#include <string>

namespace fkv {

// Starts the endpoint (GET /metrics; every other path answers 404). port 0 takes a free one. Returns the bound
// port, or a negative errno. A second call while one runs returns the running port.
int metrics_exposer_start(int port, const std::string& bind_addr = "0.0.0.0");
void metrics_exposer_stop();
int metrics_exposer_port();                 // 0 when none runs
std::string metrics_text();                 // the body a scrape gets

}  // namespace fkv

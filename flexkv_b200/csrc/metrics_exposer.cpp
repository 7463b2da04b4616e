#include "metrics_exposer.h"

#include <arpa/inet.h>
#include <netinet/in.h>
#include <poll.h>
#include <sys/eventfd.h>
#include <sys/socket.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <mutex>
#include <thread>

#include "native_log.h"

namespace fkv {
namespace {

std::mutex g_mu;
std::thread* g_thread = nullptr;   // heap-held: a process that exits with the endpoint up must not run ~thread on a joinable one
int g_listen_fd = -1, g_stop_fd = -1, g_port = 0;

void send_all(int fd, const std::string& s) {
  size_t off = 0;
  while (off < s.size()) {
    ssize_t n = ::send(fd, s.data() + off, s.size() - off, MSG_NOSIGNAL);
    if (n <= 0) {
      if (n < 0 && errno == EINTR) continue;
      return;
    }
    off += (size_t)n;
  }
}

void serve_one(int fd) {
  // a scrape is one short GET; read until the blank line or 4 KiB, for at most a second
  char buf[4096];
  size_t have = 0;
  pollfd p{fd, POLLIN, 0};
  while (have < sizeof(buf) - 1) {
    if (::poll(&p, 1, 1000) <= 0) break;
    ssize_t n = ::recv(fd, buf + have, sizeof(buf) - 1 - have, 0);
    if (n <= 0) break;
    have += (size_t)n;
    buf[have] = 0;
    if (std::strstr(buf, "\r\n\r\n") || std::strstr(buf, "\n\n")) break;
  }
  buf[have] = 0;
  const bool is_get = std::strncmp(buf, "GET ", 4) == 0;
  const char* path = buf + 4;
  const bool is_metrics = is_get && (std::strncmp(path, "/metrics", 8) == 0 || std::strncmp(path, "/ ", 2) == 0);
  std::string body, head;
  if (is_metrics) {
    body = metrics_text();
    head = "HTTP/1.1 200 OK\r\nContent-Type: text/plain; version=0.0.4; charset=utf-8\r\n";
  } else {
    body = "not found\n";
    head = "HTTP/1.1 404 Not Found\r\nContent-Type: text/plain\r\n";
  }
  head += "Content-Length: " + std::to_string(body.size()) + "\r\nConnection: close\r\n\r\n";
  send_all(fd, head + body);
}

void loop(int listen_fd, int stop_fd) {
  pollfd fds[2] = {{listen_fd, POLLIN, 0}, {stop_fd, POLLIN, 0}};
  for (;;) {
    int r = ::poll(fds, 2, -1);
    if (r < 0) {
      if (errno == EINTR) continue;
      break;
    }
    if (fds[1].revents) break;
    if (fds[0].revents & POLLIN) {
      int c = ::accept4(listen_fd, nullptr, nullptr, SOCK_CLOEXEC);
      if (c >= 0) {
        serve_one(c);
        ::close(c);
      }
    }
  }
}

}  // namespace

std::string metrics_text() {
  auto& c = cache_counters();
  std::string s;
  s += "# HELP flexkv_cpp_cache_ops_total Index operations counted in native code\n";
  s += "# TYPE flexkv_cpp_cache_ops_total counter\n";
  for (int i = 0; i < kNumCacheOps; ++i)
    s += std::string("flexkv_cpp_cache_ops_total{operation=\"") + kCacheOpNames[i] + "\"} " +
         std::to_string(c.ops[i].load(std::memory_order_relaxed)) + "\n";
  s += "# HELP flexkv_cpp_cache_blocks_total Blocks touched by native index operations\n";
  s += "# TYPE flexkv_cpp_cache_blocks_total counter\n";
  for (int i = 0; i < kNumCacheOps; ++i)
    s += std::string("flexkv_cpp_cache_blocks_total{operation=\"") + kCacheOpNames[i] + "\"} " +
         std::to_string(c.blocks[i].load(std::memory_order_relaxed)) + "\n";
  return s;
}

int metrics_exposer_start(int port, const std::string& bind_addr) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_listen_fd >= 0) return g_port;
  int fd = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) return -errno;
  int one = 1;
  ::setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_port = htons((uint16_t)port);
  if (::inet_pton(AF_INET, bind_addr.c_str(), &a.sin_addr) != 1) {
    ::close(fd);
    return -EINVAL;
  }
  if (::bind(fd, (sockaddr*)&a, sizeof(a)) < 0 || ::listen(fd, 16) < 0) {
    int e = errno;
    ::close(fd);
    return -e;
  }
  socklen_t len = sizeof(a);
  ::getsockname(fd, (sockaddr*)&a, &len);
  int sfd = ::eventfd(0, EFD_CLOEXEC);
  if (sfd < 0) {
    int e = errno;
    ::close(fd);
    return -e;
  }
  g_listen_fd = fd;
  g_stop_fd = sfd;
  g_port = ntohs(a.sin_port);
  configure_metrics(true);
  g_thread = new std::thread(loop, fd, sfd);
  FKV_INFO("native metrics endpoint on %s:%d", bind_addr.c_str(), g_port);
  return g_port;
}

void metrics_exposer_stop() {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_listen_fd < 0) return;
  uint64_t v = 1;
  ssize_t w = ::write(g_stop_fd, &v, sizeof(v));
  (void)w;
  if (g_thread != nullptr) {
    if (g_thread->joinable()) g_thread->join();
    delete g_thread;
    g_thread = nullptr;
  }
  ::close(g_listen_fd);
  ::close(g_stop_fd);
  g_listen_fd = g_stop_fd = -1;
  g_port = 0;
}

int metrics_exposer_port() {
  std::lock_guard<std::mutex> lk(g_mu);
  return g_listen_fd >= 0 ? g_port : 0;
}

}  // namespace fkv

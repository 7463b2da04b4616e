#include "resp_client.h"

#include <arpa/inet.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstring>

namespace fkv {

RespClient::RespClient(std::string host, int port, int timeout_ms, std::string password, int db)
    : host_(std::move(host)), password_(std::move(password)), port_(port), timeout_ms_(timeout_ms), db_(db) {}

RespClient::~RespClient() { close(); }

void RespClient::close() {
  std::lock_guard<std::mutex> lk(mu_);
  close_locked();
}

bool RespClient::connected() {
  std::lock_guard<std::mutex> lk(mu_);
  return fd_ >= 0;
}

void RespClient::close_locked() {
  if (fd_ >= 0) ::close(fd_);
  fd_ = -1;
  rbuf_.clear();
  rpos_ = 0;
}

std::string RespClient::encode(const std::vector<std::string>& args) {
  std::string s = "*" + std::to_string(args.size()) + "\r\n";
  for (const auto& a : args) {
    s += "$" + std::to_string(a.size()) + "\r\n";
    s += a;
    s += "\r\n";
  }
  return s;
}

namespace {
// one line ending in CRLF starting at pos; returns false when incomplete
bool read_line(const std::string& buf, size_t pos, std::string& line, size_t& next) {
  size_t e = buf.find("\r\n", pos);
  if (e == std::string::npos) return false;
  line.assign(buf, pos, e - pos);
  next = e + 2;
  return true;
}
}  // namespace

bool RespClient::parse(const std::string& buf, size_t& pos, RespValue& out) {
  if (pos >= buf.size()) return false;
  const char t = buf[pos];
  std::string line;
  size_t next = 0;
  if (!read_line(buf, pos + 1, line, next)) return false;
  out = RespValue();
  switch (t) {
    case '+':
      out.type = RespValue::kString;
      out.str = line;
      break;
    case '-':
      out.type = RespValue::kError;
      out.str = line;
      break;
    case ':':
      out.type = RespValue::kInteger;
      out.integer = std::strtoll(line.c_str(), nullptr, 10);
      break;
    case '$': {
      const long long n = std::strtoll(line.c_str(), nullptr, 10);
      if (n < 0) {
        out.type = RespValue::kNil;
        break;
      }
      if (buf.size() < next + (size_t)n + 2) return false;
      out.type = RespValue::kBulk;
      out.str.assign(buf, next, (size_t)n);
      next += (size_t)n + 2;
      break;
    }
    case '*': {
      const long long n = std::strtoll(line.c_str(), nullptr, 10);
      if (n < 0) {
        out.type = RespValue::kNil;
        break;
      }
      out.type = RespValue::kArray;
      out.items.resize((size_t)n);
      size_t p = next;
      for (long long i = 0; i < n; ++i)
        if (!parse(buf, p, out.items[(size_t)i])) return false;
      next = p;
      break;
    }
    default:
      throw RespIoError(std::string("unexpected reply type byte '") + t + "'");
  }
  pos = next;
  return true;
}

void RespClient::ensure_connected_locked() {
  if (fd_ >= 0) return;
  addrinfo hints{}, *res = nullptr;
  hints.ai_family = AF_UNSPEC;
  hints.ai_socktype = SOCK_STREAM;
  const std::string port = std::to_string(port_);
  int rc = ::getaddrinfo(host_.c_str(), port.c_str(), &hints, &res);
  if (rc != 0) throw RespIoError("cannot resolve " + host_ + ": " + gai_strerror(rc));
  int fd = -1;
  std::string why = "no address";
  for (addrinfo* a = res; a != nullptr; a = a->ai_next) {
    fd = ::socket(a->ai_family, a->ai_socktype | SOCK_CLOEXEC, a->ai_protocol);
    if (fd < 0) continue;
    timeval tv{timeout_ms_ / 1000, (timeout_ms_ % 1000) * 1000};
    ::setsockopt(fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof(tv));
    ::setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
    int one = 1;
    ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    if (::connect(fd, a->ai_addr, a->ai_addrlen) == 0) break;
    why = std::strerror(errno);
    ::close(fd);
    fd = -1;
  }
  ::freeaddrinfo(res);
  if (fd < 0) throw RespIoError("cannot connect to " + host_ + ":" + port + ": " + why);
  fd_ = fd;
  // session set-up; a refusal is an IO-level failure of the connection
  std::vector<std::vector<std::string>> hello;
  if (!password_.empty()) hello.push_back({"AUTH", password_});
  if (db_ != 0) hello.push_back({"SELECT", std::to_string(db_)});
  for (const auto& c : hello) {
    write_all_locked(encode(c));
    RespValue v = read_reply_locked();
    if (v.type == RespValue::kError) {
      close_locked();
      throw RespIoError(c[0] + " refused: " + v.str);
    }
  }
}

void RespClient::write_all_locked(const std::string& s) {
  size_t off = 0;
  while (off < s.size()) {
    ssize_t n = ::send(fd_, s.data() + off, s.size() - off, MSG_NOSIGNAL);
    if (n < 0 && errno == EINTR) continue;
    if (n <= 0) {
      const std::string why = n == 0 ? "connection closed" : std::strerror(errno);
      close_locked();
      throw RespIoError("send failed: " + why);
    }
    off += (size_t)n;
  }
}

RespValue RespClient::read_reply_locked() {
  RespValue v;
  for (;;) {
    size_t p = rpos_;
    bool ok;
    try {
      ok = parse(rbuf_, p, v);
    } catch (const RespIoError&) {
      close_locked();
      throw;
    }
    if (ok) {
      rpos_ = p;
      if (rpos_ == rbuf_.size()) {
        rbuf_.clear();
        rpos_ = 0;
      }
      return v;
    }
    char tmp[16384];
    ssize_t n = ::recv(fd_, tmp, sizeof(tmp), 0);
    if (n < 0 && errno == EINTR) continue;
    if (n <= 0) {
      const std::string why = n == 0 ? "connection closed by the server"
                                     : (errno == EAGAIN || errno == EWOULDBLOCK ? "timed out" : std::strerror(errno));
      close_locked();
      throw RespIoError("receive failed: " + why);
    }
    rbuf_.append(tmp, (size_t)n);
  }
}

RespValue RespClient::command(const std::vector<std::string>& args) {
  std::lock_guard<std::mutex> lk(mu_);
  ensure_connected_locked();
  write_all_locked(encode(args));
  return read_reply_locked();
}

std::vector<RespValue> RespClient::pipeline(const std::vector<std::vector<std::string>>& cmds) {
  std::lock_guard<std::mutex> lk(mu_);
  ensure_connected_locked();
  std::vector<RespValue> out;
  out.reserve(cmds.size());
  // bounded batches: the server's replies must not fill both socket buffers while requests are still being written
  constexpr size_t kBatch = 256;
  for (size_t i = 0; i < cmds.size(); i += kBatch) {
    const size_t e = std::min(cmds.size(), i + kBatch);
    std::string req;
    for (size_t j = i; j < e; ++j) req += encode(cmds[j]);
    write_all_locked(req);
    for (size_t j = i; j < e; ++j) out.push_back(read_reply_locked());
  }
  return out;
}

}  // namespace fkv

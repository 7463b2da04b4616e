// A small Redis wire-protocol (RESP2) client: blocking TCP socket, request pipelining, typed replies.
//
// The reference reaches Redis through hiredis (csrc/dist/redis_meta_channel.cpp:60-215) and redis-py
// (flexkv/cache/redis_meta.py:158-290); neither is available here, and the command set the cross-node index
// needs is small (INCR, HSET, HGETALL, PEXPIRE, EXISTS, DEL, SCAN, AUTH, SELECT, PING), so the protocol is
// spoken directly. One connection per client, serialised by a mutex; an IO error closes the socket and the
// next call connects again.
#pragma once
#include <cstdint>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

namespace fkv {

struct RespValue {
  enum Type : int { kNil = 0, kString, kError, kInteger, kBulk, kArray };
  Type type = kNil;
  int64_t integer = 0;
  std::string str;                  // simple string, error text or bulk payload
  std::vector<RespValue> items;     // array elements
};

class RespIoError : public std::runtime_error {
 public:
  using std::runtime_error::runtime_error;
};

class RespClient {
 public:
  RespClient(std::string host, int port, int timeout_ms = 3000, std::string password = "", int db = 0);
  ~RespClient();
  RespClient(const RespClient&) = delete;
  RespClient& operator=(const RespClient&) = delete;

  // One command, one reply. A reply of type kError is returned, not thrown; RespIoError means the
  // connection broke (it is closed; the next call reconnects).
  RespValue command(const std::vector<std::string>& args);
  // All commands are written before the first reply is read.
  std::vector<RespValue> pipeline(const std::vector<std::vector<std::string>>& cmds);
  void close();
  bool connected();

  static std::string encode(const std::vector<std::string>& args);       // the bytes of one command
  // Parses one reply from buf[pos..]; returns false when more bytes are needed (pos unchanged).
  static bool parse(const std::string& buf, size_t& pos, RespValue& out);

 private:
  void ensure_connected_locked();
  void close_locked();
  void write_all_locked(const std::string& s);
  RespValue read_reply_locked();

  std::string host_, password_;
  int port_, timeout_ms_, db_;
  int fd_ = -1;
  std::string rbuf_;
  size_t rpos_ = 0;
  std::mutex mu_;
};

}  // namespace fkv

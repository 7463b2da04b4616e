// Self-contained XXH64 (one-shot and streaming), written from the public
// algorithm description. Block keys of the cache index are cumulative
// streaming XXH64 digests (seed 0) over int64 token ids; the digests must be
// bit-identical to the canonical xxHash library so that keys computed by
// other tools interoperate (reference behaviour: csrc/hash.cpp:47-66).
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstring>

namespace fkv {

struct XXH64 {
  static constexpr uint64_t P1 = 0x9E3779B185EBCA87ULL;
  static constexpr uint64_t P2 = 0xC2B2AE3D27D4EB4FULL;
  static constexpr uint64_t P3 = 0x165667B19E3779F9ULL;
  static constexpr uint64_t P4 = 0x85EBCA77C2B2AE63ULL;
  static constexpr uint64_t P5 = 0x27D4EB2F165667C5ULL;

  static inline uint64_t rotl(uint64_t x, int r) { return (x << r) | (x >> (64 - r)); }
  static inline uint64_t rd64(const uint8_t* p) { uint64_t v; std::memcpy(&v, p, 8); return v; }
  static inline uint32_t rd32(const uint8_t* p) { uint32_t v; std::memcpy(&v, p, 4); return v; }
  static inline uint64_t round(uint64_t acc, uint64_t in) {
    acc += in * P2; acc = rotl(acc, 31); return acc * P1;
  }
  static inline uint64_t merge(uint64_t h, uint64_t v) {
    v = round(0, v); h ^= v; return h * P1 + P4;
  }
  static inline uint64_t avalanche(uint64_t h) {
    h ^= h >> 33; h *= P2; h ^= h >> 29; h *= P3; h ^= h >> 32; return h;
  }
  static inline uint64_t tail(uint64_t h, const uint8_t* p, size_t len) {
    while (len >= 8) { h ^= round(0, rd64(p)); h = rotl(h, 27) * P1 + P4; p += 8; len -= 8; }
    if (len >= 4) { h ^= (uint64_t)rd32(p) * P1; h = rotl(h, 23) * P2 + P3; p += 4; len -= 4; }
    while (len > 0) { h ^= (uint64_t)(*p) * P5; h = rotl(h, 11) * P1; ++p; --len; }
    return avalanche(h);
  }

  // ---- streaming state ----
  uint64_t total = 0;
  uint64_t v[4];
  uint8_t mem[32];
  uint32_t memsize = 0;
  uint64_t seed_ = 0;

  explicit XXH64(uint64_t seed = 0) { reset(seed); }
  void reset(uint64_t seed = 0) {
    seed_ = seed; total = 0; memsize = 0;
    v[0] = seed + P1 + P2; v[1] = seed + P2; v[2] = seed; v[3] = seed - P1;
  }
  void update(const void* data, size_t len) {
    const uint8_t* p = static_cast<const uint8_t*>(data);
    total += len;
    if (memsize + len < 32) { std::memcpy(mem + memsize, p, len); memsize += (uint32_t)len; return; }
    if (memsize) {
      size_t fill = 32 - memsize;
      std::memcpy(mem + memsize, p, fill);
      v[0] = round(v[0], rd64(mem)); v[1] = round(v[1], rd64(mem + 8));
      v[2] = round(v[2], rd64(mem + 16)); v[3] = round(v[3], rd64(mem + 24));
      p += fill; len -= fill; memsize = 0;
    }
    uint64_t a = v[0], b = v[1], c = v[2], d = v[3];
    while (len >= 32) {
      a = round(a, rd64(p)); b = round(b, rd64(p + 8));
      c = round(c, rd64(p + 16)); d = round(d, rd64(p + 24));
      p += 32; len -= 32;
    }
    v[0] = a; v[1] = b; v[2] = c; v[3] = d;
    if (len) { std::memcpy(mem, p, len); memsize = (uint32_t)len; }
  }
  uint64_t digest() const {
    uint64_t h;
    if (total >= 32) {
      h = rotl(v[0], 1) + rotl(v[1], 7) + rotl(v[2], 12) + rotl(v[3], 18);
      h = merge(h, v[0]); h = merge(h, v[1]); h = merge(h, v[2]); h = merge(h, v[3]);
    } else {
      h = seed_ + P5;
    }
    h += total;
    return tail(h, mem, memsize);
  }
  static uint64_t hash(const void* data, size_t len, uint64_t seed = 0) {
    XXH64 s(seed); s.update(data, len); return s.digest();
  }
};

}  // namespace fkv
